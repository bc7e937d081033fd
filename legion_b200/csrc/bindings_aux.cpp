// Python bindings for the Gated DeltaNet, communication and block-scaled format kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.h"
#include "ep.h"
#include "gdn.h"
#include "gemm_nvfp4_sm100.h"
#include "kernels.h"
#include "quant.h"

namespace {
using torch::Tensor;
using OptT = c10::optional<Tensor>;
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
template <typename T>
const T* optp(const OptT& t) {
  return t.has_value() ? reinterpret_cast<const T*>(t->data_ptr()) : nullptr;
}
template <typename T>
T* optpm(const OptT& t) {
  return t.has_value() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

lb::CommPeers make_peers(const std::vector<int64_t>& buffers, const std::vector<int64_t>& signals, int64_t rank) {
  TORCH_CHECK(buffers.size() == signals.size() && buffers.size() <= LB_MAX_RANKS, "bad peer table");
  lb::CommPeers p{};
  p.world = int(buffers.size());
  p.rank = int(rank);
  for (size_t i = 0; i < buffers.size(); ++i) {
    p.buffer[i] = reinterpret_cast<void*>(buffers[i]);
    p.signal[i] = reinterpret_cast<void*>(signals[i]);
  }
  return p;
}
}  // namespace

void bind_gdn(pybind11::module_& m) {
  m.def("conv1d_silu", [](const Tensor& x, const Tensor& w, const OptT& bias, Tensor& conv_state, const Tensor& cu_seq,
                          const Tensor& slots, Tensor& out, bool write_state, int64_t max_len) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kFloat, "conv1d_silu dtypes");
    TORCH_CHECK(lb::conv1d_silu_launch(x.data_ptr(), x.stride(0), w.data_ptr<float>(), optp<float>(bias),
                                       conv_state.data_ptr<float>(), cu_seq.data_ptr<int>(), slots.data_ptr<int>(),
                                       int(slots.numel()), int(x.size(1)), int(w.size(1)), out.data_ptr(),
                                       out.stride(0), write_state ? 1 : 0, cur_stream(), int(max_len)) == 0,
                "conv1d_silu: unsupported kernel width");
  });
  m.def("gdn_recurrent", [](const Tensor& qkv, const Tensor& g, const Tensor& beta, Tensor& state,
                            const Tensor& cu_seq, const Tensor& slots, int64_t Hk, int64_t Hv, int64_t DK, int64_t DV,
                            bool tiled_heads, double scale, double l2_eps, Tensor& out, bool write_state,
                            bool write_out, bool prompt_rows) {
    c10::cuda::CUDAGuard guard(qkv.device());
    TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 && state.scalar_type() == at::kFloat, "gdn_recurrent dtypes");
    TORCH_CHECK(lb::gdn_recurrent_launch(qkv.data_ptr(), qkv.stride(0), g.data_ptr<float>(), beta.data_ptr<float>(),
                                         state.data_ptr<float>(), cu_seq.data_ptr<int>(), slots.data_ptr<int>(),
                                         int(slots.numel()), int(Hk), int(Hv), int(DK), int(DV), tiled_heads ? 1 : 0,
                                         float(scale), float(l2_eps), out.data_ptr(), write_state ? 1 : 0,
                                         write_out ? 1 : 0, prompt_rows ? 1 : 0, cur_stream()) == 0,
                "gdn_recurrent: unsupported head dims");
  });
  m.def("gdn_decode_fused", [](const Tensor& proj, const Tensor& conv_w, Tensor& conv_state, const Tensor& A,
                               const Tensor& dt_bias, const Tensor& norm_w, double eps, int64_t act, Tensor& state,
                               const Tensor& slots, int64_t Hk, int64_t Hv, int64_t DK, int64_t DV, bool tiled_heads,
                               double scale, double l2_eps, Tensor& out) {
    c10::cuda::CUDAGuard guard(proj.device());
    TORCH_CHECK(proj.scalar_type() == at::kBFloat16 && proj.dim() == 2 && proj.stride(1) == 1 &&
                    proj.size(1) == 2 * Hk * DK + 2 * Hv * DV + 2 * Hv && proj.size(0) >= slots.numel(),
                "gdn_decode_fused: proj rows are [q | k | v | z | b | a], one per sequence");
    TORCH_CHECK(conv_w.scalar_type() == at::kFloat && conv_w.is_contiguous() && conv_state.scalar_type() == at::kFloat &&
                    state.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16 && out.is_contiguous(),
                "gdn_decode_fused dtypes");
    TORCH_CHECK(lb::gdn_decode_fused_launch(proj.data_ptr(), proj.stride(0), conv_w.data_ptr<float>(),
                                            conv_state.data_ptr<float>(), int(conv_w.size(1)), A.data_ptr<float>(),
                                            dt_bias.data_ptr<float>(), norm_w.data_ptr<float>(), float(eps), int(act),
                                            state.data_ptr<float>(), slots.data_ptr<int>(), int(slots.numel()), int(Hk),
                                            int(Hv), int(DK), int(DV), tiled_heads ? 1 : 0, float(scale), float(l2_eps),
                                            out.data_ptr(), cur_stream()) == 0,
                "gdn_decode_fused: needs square heads of 64 or 128, conv width 4, at most 4 value heads per key head");
  });
  m.def("gdn_chunk_scratch_bytes", [](int64_t n_blocks, int64_t Hv) {
    return int64_t(lb::gdn_chunk_scratch_bytes(int(n_blocks), int(Hv)));
  });
  m.def("gdn_chunk", [](const Tensor& qkv, const Tensor& g, const Tensor& beta, Tensor& state, const Tensor& blk_t0,
                        const Tensor& blk_n, const Tensor& seq_blk0, const Tensor& seq_nchunk, const Tensor& seq_t0,
                        const Tensor& seq_len, const Tensor& slots, int64_t Hk, int64_t Hv, int64_t DK, int64_t DV,
                        bool tiled_heads, double scale, double l2_eps, Tensor& out, bool write_state, Tensor& scratch,
                        Tensor& status) {
    c10::cuda::CUDAGuard guard(qkv.device());
    TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1 &&
                    g.scalar_type() == at::kFloat && g.is_contiguous() && beta.scalar_type() == at::kFloat &&
                    beta.is_contiguous() && state.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16 &&
                    out.is_contiguous(), "gdn_chunk dtypes / layout");
    const int n_blocks = int(blk_t0.numel()), n_seqs = int(slots.numel());
    TORCH_CHECK(size_t(scratch.numel()) * scratch.element_size() >= lb::gdn_chunk_scratch_bytes(n_blocks, int(Hv)),
                "gdn_chunk: scratch too small");
    TORCH_CHECK(lb::gdn_chunk_launch(qkv.data_ptr(), qkv.stride(0), qkv.size(0), g.data_ptr<float>(),
                                     beta.data_ptr<float>(), state.data_ptr<float>(), blk_t0.data_ptr<int>(),
                                     blk_n.data_ptr<int>(), n_blocks, seq_blk0.data_ptr<int>(),
                                     seq_nchunk.data_ptr<int>(), seq_t0.data_ptr<int>(), seq_len.data_ptr<int>(),
                                     slots.data_ptr<int>(), n_seqs, int(Hk), int(Hv), int(DK), int(DV),
                                     tiled_heads ? 1 : 0, float(scale), float(l2_eps), out.data_ptr(),
                                     write_state ? 1 : 0, scratch.data_ptr(), reinterpret_cast<int*>(status.data_ptr()),
                                     cur_stream()) == 0,
                "gdn_chunk: needs heads of 128 x 128 and 16-byte aligned rows");
  });
  m.def("gdn_gates", [](const Tensor& a, const Tensor& b, const Tensor& A, const Tensor& dt_bias, Tensor& g,
                        Tensor& beta) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(lb::gdn_gates_launch(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), A.data_ptr<float>(),
                                     dt_bias.data_ptr<float>(), int(a.size(1)), a.size(0), g.data_ptr<float>(),
                                     beta.data_ptr<float>(), cur_stream()) == 0, "gdn_gates failed");
  });
  m.def("gated_rmsnorm", [](const Tensor& o, const Tensor& z, const Tensor& w, double eps, int64_t Hv, int64_t DV,
                            int64_t act, Tensor& out) {
    c10::cuda::CUDAGuard guard(o.device());
    const long T = o.numel() / (Hv * DV);
    TORCH_CHECK(lb::gated_rmsnorm_launch(o.data_ptr(), z.data_ptr(), z.stride(0), w.data_ptr<float>(), float(eps),
                                         int(DV), int(Hv), T, int(act), out.data_ptr(), cur_stream()) == 0,
                "gated_rmsnorm failed");
  });
}

void bind_comm(pybind11::module_& m) {
  m.def("wait_flag", [](const Tensor& flag, int64_t want, int64_t budget_ns, Tensor& status) {
    c10::cuda::CUDAGuard guard(flag.device());
    TORCH_CHECK(lb::wait_flag_launch(reinterpret_cast<const uint32_t*>(flag.data_ptr()), uint32_t(want),
                                     uint64_t(budget_ns), reinterpret_cast<int*>(status.data_ptr()),
                                     cur_stream()) == 0, "wait_flag failed");
  });
  m.def("comm_barrier", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                           int64_t slot_base, int64_t seq, int64_t budget_ns, Tensor& status) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::barrier_launch(p, int(slot_base), uint32_t(seq), uint64_t(budget_ns),
                                   reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0, "barrier failed");
  });
  m.def("all_reduce_fused", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                               int64_t buf_off, int64_t slot_base, Tensor& seq, Tensor& done_ctr, int64_t T, int64_t H,
                               const OptT& residual, Tensor& sum_out, const OptT& norm_w, double eps, double w_offset,
                               const OptT& norm_out, int64_t budget_ns, Tensor& status, const OptT& q_codes,
                               const OptT& q_sf, const OptT& q_gscale, int64_t ll_off, int64_t ll_rows,
                               const OptT& cmb_y, const OptT& cmb_ids, int64_t cmb_e_lo, int64_t cmb_e_hi,
                               const OptT& cmb_shared) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    lb::Nv4RowsOut q{};
    if (q_codes.has_value()) {
      TORCH_CHECK(q_sf.has_value() && q_gscale.has_value() && q_codes->dim() == 2 && q_codes->stride(1) == 1 &&
                      q_codes->size(0) >= T && q_codes->size(1) * 2 == H && q_sf->is_contiguous() &&
                      size_t(q_sf->numel()) >= lb::nv4_sf_bytes(T, H) && q_gscale->numel() >= T,
                  "all_reduce_fused: encoded rows need codes [T, H / 2], scale atoms and one scale per row");
      q.codes = reinterpret_cast<uint8_t*>(q_codes->data_ptr()); q.ld = q_codes->stride(0);
      q.sf = reinterpret_cast<uint8_t*>(q_sf->data_ptr()); q.row_gscale = q_gscale->data_ptr<float>();
      q.k4 = lb::nv4_sf_k4(H);
    }
    lb::CombineSrc cs{};
    if (cmb_y.has_value()) {
      TORCH_CHECK(ll_rows > 0 && cmb_ids.has_value() && cmb_ids->dim() == 2 && cmb_ids->is_contiguous() &&
                      cmb_ids->size(0) >= T && cmb_y->scalar_type() == at::kBFloat16 && cmb_y->stride(1) == 1 &&
                      cmb_y->size(0) >= T * cmb_ids->size(1) && cmb_y->size(1) == H,
                  "all_reduce_fused: the combine source needs pair rows [T * k, H] and ids [T, k] (decode sizes)");
      cs.y = cmb_y->data_ptr(); cs.ldy = cmb_y->stride(0); cs.ids = cmb_ids->data_ptr<int>();
      cs.k = int(cmb_ids->size(1)); cs.e_lo = int(cmb_e_lo); cs.e_hi = int(cmb_e_hi);
      if (cmb_shared.has_value()) {
        TORCH_CHECK(cmb_shared->scalar_type() == at::kBFloat16 && cmb_shared->stride(1) == 1 && cmb_shared->size(0) >= T,
                    "all_reduce_fused: shared rows [T, H] bf16");
        cs.shared = cmb_shared->data_ptr(); cs.lds = cmb_shared->stride(0);
      }
    }
    if (ll_rows > 0) {
      // pushed flag-carrying lines: one NVLink crossing
      TORCH_CHECK(lb::all_reduce_ll_launch(
                      p, buf_off, ll_off, int(ll_rows), reinterpret_cast<uint32_t*>(seq.data_ptr()),
                      reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(T), int(H),
                      residual.has_value() ? residual->data_ptr() : nullptr,
                      residual.has_value() ? residual->stride(0) : 0, sum_out.data_ptr(), sum_out.stride(0),
                      optp<float>(norm_w), float(eps), float(w_offset),
                      norm_out.has_value() ? norm_out->data_ptr() : nullptr,
                      norm_out.has_value() ? norm_out->stride(0) : 0, uint64_t(budget_ns),
                      reinterpret_cast<int*>(status.data_ptr()), cur_stream(), q, cs) == 0,
                  "all_reduce (pushed lines) failed");
      return;
    }
    TORCH_CHECK(lb::all_reduce_fused_launch(
                    p, buf_off, int(slot_base), reinterpret_cast<uint32_t*>(seq.data_ptr()),
                    reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(T), int(H),
                    residual.has_value() ? residual->data_ptr() : nullptr,
                    residual.has_value() ? residual->stride(0) : 0, sum_out.data_ptr(), sum_out.stride(0),
                    optp<float>(norm_w), float(eps), float(w_offset),
                    norm_out.has_value() ? norm_out->data_ptr() : nullptr,
                    norm_out.has_value() ? norm_out->stride(0) : 0, uint64_t(budget_ns),
                    reinterpret_cast<int*>(status.data_ptr()), cur_stream(), q) == 0,
                "all_reduce_fused failed");
  });
  m.def("argmax_exchange", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank, int64_t ax_off,
                              int64_t ax_rows, Tensor& seq, Tensor& done_ctr, const Tensor& val, const Tensor& idx,
                              int64_t vocab_offset, Tensor& picks, int64_t budget_ns, Tensor& status) {
    TORCH_CHECK(val.scalar_type() == at::kFloat && idx.scalar_type() == at::kInt && picks.scalar_type() == at::kInt &&
                    val.is_contiguous() && idx.is_contiguous() && picks.is_contiguous() && idx.numel() >= val.numel() &&
                    picks.numel() >= val.numel(), "argmax_exchange: (float value, int index) per row -> int picks");
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::argmax_exchange_launch(p, ax_off, int(ax_rows), reinterpret_cast<uint32_t*>(seq.data_ptr()),
                                           reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(val.numel()),
                                           val.data_ptr<float>(), idx.data_ptr<int>(), int(vocab_offset),
                                           picks.data_ptr<int>(), uint64_t(budget_ns),
                                           reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0,
                "argmax_exchange: too many rows for the exchange area");
  });
  m.def("reduce_scatter_fused", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                                   int64_t buf_off, int64_t out_off, int64_t slot_base, Tensor& seq, Tensor& done_ctr,
                                   int64_t row0, int64_t n_rows, int64_t H, const OptT& residual, int64_t budget_ns,
                                   Tensor& status, int64_t mc_ptr) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::reduce_scatter_launch(p, buf_off, out_off, int(slot_base),
                                          reinterpret_cast<uint32_t*>(seq.data_ptr()),
                                          reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(row0), int(n_rows),
                                          int(H), residual.has_value() ? residual->data_ptr() : nullptr,
                                          residual.has_value() ? residual->stride(0) : 0, uint64_t(budget_ns),
                                          reinterpret_cast<int*>(status.data_ptr()), cur_stream(),
                                          reinterpret_cast<void*>(mc_ptr)) == 0,
                "reduce_scatter_fused failed");
  });
  m.def("all_gather_fused", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                               int64_t src_off, int64_t slot_base, Tensor& seq, Tensor& done_ctr, int64_t T, int64_t H,
                               Tensor& out, int64_t budget_ns, Tensor& status, bool local_only) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::all_gather_launch(p, src_off, int(slot_base), reinterpret_cast<uint32_t*>(seq.data_ptr()),
                                      reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(T), int(H),
                                      out.data_ptr(), out.stride(0), uint64_t(budget_ns),
                                      reinterpret_cast<int*>(status.data_ptr()), cur_stream(), local_only ? 1 : 0) == 0,
                "all_gather_fused failed");
  });
}

namespace {
lb::EpPeers make_ep(const std::vector<int64_t>& buffers, const std::vector<int64_t>& signals, int64_t rank) {
  TORCH_CHECK(buffers.size() == signals.size() && buffers.size() <= EP_MAX_RANKS, "bad EP peer table");
  lb::EpPeers p{};
  p.world = int(buffers.size());
  p.rank = int(rank);
  for (size_t i = 0; i < buffers.size(); ++i) {
    p.buffer[i] = reinterpret_cast<void*>(buffers[i]);
    p.signal[i] = reinterpret_cast<void*>(signals[i]);
  }
  return p;
}
}  // namespace

void bind_ep(pybind11::module_& m) {
  m.def("ep_publish_counts", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                                const Tensor& counts, int64_t counts_off, Tensor& seq, Tensor& dest_base,
                                Tensor& recv_counts, Tensor& meta, int64_t cap, int64_t budget_ns, Tensor& status) {
    c10::cuda::CUDAGuard guard(counts.device());
    auto p = make_ep(buffers, signals, rank);
    TORCH_CHECK(lb::ep_publish_counts_launch(p, counts.data_ptr<int>(), int(counts.numel()), counts_off,
                                             reinterpret_cast<const uint32_t*>(seq.data_ptr()),
                                             dest_base.data_ptr<int>(), recv_counts.data_ptr<int>(),
                                             meta.data_ptr<int>(), int(cap), uint64_t(budget_ns),
                                             reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0,
                "ep_publish_counts: experts must divide by the ranks and be <= 512");
  });
  m.def("ep_push", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank, const Tensor& x,
                      const Tensor& sorted_token, const Tensor& sorted_pair, const Tensor& sorted_w,
                      const Tensor& offsets, const Tensor& dest_base, int64_t E, int64_t cap, int64_t rx_off,
                      int64_t rsrc_off, int64_t rw_off, Tensor& seq, Tensor& done_ctr) {
    c10::cuda::CUDAGuard guard(x.device());
    auto p = make_ep(buffers, signals, rank);
    TORCH_CHECK(lb::ep_push_launch(p, x.data_ptr(), x.stride(0), int(x.size(1)), sorted_token.data_ptr<int>(),
                                   sorted_pair.data_ptr<int>(), sorted_w.data_ptr<float>(), offsets.data_ptr<int>(),
                                   dest_base.data_ptr<int>(), int(E), int(cap), rx_off, rsrc_off, rw_off,
                                   reinterpret_cast<const uint32_t*>(seq.data_ptr()),
                                   reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(sorted_token.numel()),
                                   cur_stream()) == 0, "ep_push failed");
  });
  m.def("ep_sync", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank, int64_t slot_base,
                      bool signal_first, Tensor& seq, bool bump, int64_t budget_ns, Tensor& status) {
    c10::cuda::CUDAGuard guard(seq.device());
    auto p = make_ep(buffers, signals, rank);
    TORCH_CHECK(lb::ep_sync_launch(p, int(slot_base), signal_first ? 1 : 0,
                                   reinterpret_cast<uint32_t*>(seq.data_ptr()), bump ? 1 : 0, uint64_t(budget_ns),
                                   reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0, "ep_sync failed");
  });
  m.def("moe_tiles", [](const Tensor& counts, int64_t bn, Tensor& offsets, Tensor& tile_group, Tensor& tile_tok0,
                        Tensor& tile_ntok, Tensor& meta) {
    c10::cuda::CUDAGuard guard(counts.device());
    TORCH_CHECK(lb::moe_tiles_launch(counts.data_ptr<int>(), int(counts.numel()), int(bn), offsets.data_ptr<int>(),
                                     tile_group.data_ptr<int>(), tile_tok0.data_ptr<int>(), tile_ntok.data_ptr<int>(),
                                     int(tile_group.numel()), meta.data_ptr<int>(), cur_stream()) == 0,
                "moe_tiles failed");
  });
}

void bind_quant(pybind11::module_& m) {
  m.def("nvfp4_dequant", [](const Tensor& codes, const Tensor& scales, const Tensor& global_scale, Tensor& out) {
    c10::cuda::CUDAGuard guard(codes.device());
    const long rows = codes.size(0), K = codes.size(1) * 2;
    TORCH_CHECK(lb::nvfp4_dequant_launch(reinterpret_cast<const uint8_t*>(codes.data_ptr()),
                                         reinterpret_cast<const uint8_t*>(scales.data_ptr()),
                                         global_scale.data_ptr<float>(), rows, K, out.data_ptr(), cur_stream()) == 0,
                "nvfp4_dequant: K must be a multiple of 16");
  });
  m.def("nvfp4_quant", [](const Tensor& x, const Tensor& global_scale, Tensor& codes, Tensor& scales) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(lb::nvfp4_quant_launch(x.data_ptr(), x.stride(0), global_scale.data_ptr<float>(), x.size(0), x.size(1),
                                       reinterpret_cast<uint8_t*>(codes.data_ptr()),
                                       reinterpret_cast<uint8_t*>(scales.data_ptr()), cur_stream()) == 0,
                "nvfp4_quant: K must be a multiple of 16");
  });
  m.def("fp8_block_dequant", [](const Tensor& w, const Tensor& scale, int64_t br, int64_t bk, Tensor& out) {
    c10::cuda::CUDAGuard guard(w.device());
    TORCH_CHECK(lb::fp8_block_dequant_launch(reinterpret_cast<const uint8_t*>(w.data_ptr()), scale.data_ptr<float>(),
                                             w.size(0), w.size(1), int(br), int(bk), out.data_ptr(),
                                             cur_stream()) == 0, "fp8_block_dequant failed");
  });
  m.def("fp8_block_quant", [](const Tensor& x, int64_t br, int64_t bk, Tensor& out, Tensor& scale) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(lb::fp8_block_quant_launch(x.data_ptr(), x.stride(0), x.size(0), x.size(1), int(br), int(bk),
                                           reinterpret_cast<uint8_t*>(out.data_ptr()), scale.data_ptr<float>(),
                                           cur_stream()) == 0, "fp8_block_quant failed");
  });
  m.def("fp8_act_quant", [](const Tensor& x, Tensor& out, Tensor& scale) {
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && out.is_contiguous() &&
                    out.element_size() == 1 && out.numel() == x.numel() && scale.scalar_type() == at::kFloat &&
                    scale.is_contiguous() && scale.numel() == x.size(0) * (x.size(1) / 128),
                "fp8_act_quant: x bf16 [T, K], out bytes [T, K], scale f32 [T, K / 128]");
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(lb::fp8_act_quant_launch(x.data_ptr(), x.stride(0), x.size(0), x.size(1),
                                         reinterpret_cast<uint8_t*>(out.data_ptr()), scale.data_ptr<float>(),
                                         cur_stream()) == 0, "fp8_act_quant: K must be a multiple of 128, rows 8-byte aligned");
  });
  // ---- native NVFP4 (W4A4): scale atoms, activation quantiser, GEMM
  m.def("nv4_sf_bytes", [](int64_t rows, int64_t K) { return int64_t(lb::nv4_sf_bytes(rows, K)); });
  m.def("nv4_pack_scales", [](const Tensor& scales, Tensor& atoms) {
    TORCH_CHECK(scales.dim() == 2 && scales.is_contiguous() && scales.element_size() == 1 && atoms.is_contiguous() &&
                    atoms.element_size() == 1, "nv4_pack_scales: scales [rows, K / 16] bytes");
    const long rows = scales.size(0), K = scales.size(1) * 16;
    TORCH_CHECK(size_t(atoms.numel()) >= lb::nv4_sf_bytes(rows, K), "nv4_pack_scales: atom buffer too small");
    c10::cuda::CUDAGuard guard(scales.device());
    TORCH_CHECK(lb::nv4_pack_scales_launch(reinterpret_cast<const uint8_t*>(scales.data_ptr()), rows, K,
                                           reinterpret_cast<uint8_t*>(atoms.data_ptr()), cur_stream()) == 0,
                "nv4_pack_scales failed");
  });
  m.def("nv4_unpack_scales", [](const Tensor& atoms, Tensor& scales) {
    TORCH_CHECK(scales.dim() == 2 && scales.is_contiguous() && scales.element_size() == 1 && atoms.is_contiguous(),
                "nv4_unpack_scales: scales [rows, K / 16] bytes");
    const long rows = scales.size(0), K = scales.size(1) * 16;
    TORCH_CHECK(size_t(atoms.numel()) >= lb::nv4_sf_bytes(rows, K), "nv4_unpack_scales: atom buffer too small");
    c10::cuda::CUDAGuard guard(scales.device());
    TORCH_CHECK(lb::nv4_unpack_scales_launch(reinterpret_cast<const uint8_t*>(atoms.data_ptr()), rows, K,
                                             reinterpret_cast<uint8_t*>(scales.data_ptr()), cur_stream()) == 0,
                "nv4_unpack_scales failed");
  });
  m.def("nv4_act_quant", [](const Tensor& x, const OptT& residual, const OptT& sum_out, const OptT& norm_w, double eps,
                            double w_offset, const OptT& normed_out, const OptT& gscale_static, Tensor& codes,
                            Tensor& sf_atoms, const OptT& row_gscale) {
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "nv4_act_quant: x bf16 [T, K]");
    const long rows = x.size(0), K = x.size(1);
    TORCH_CHECK(codes.element_size() == 1 && codes.dim() == 2 && codes.stride(1) == 1 && codes.size(0) >= rows &&
                    codes.size(1) * 2 == K, "nv4_act_quant: codes [T, K / 2] bytes");
    TORCH_CHECK(sf_atoms.is_contiguous() && size_t(sf_atoms.numel()) >= lb::nv4_sf_bytes(rows, K),
                "nv4_act_quant: scale atom buffer too small");
    TORCH_CHECK(gscale_static.has_value() || (row_gscale.has_value() && row_gscale->numel() >= rows),
                "nv4_act_quant: a static scale or a row-scale output is needed");
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(lb::nv4_act_quant_launch(x.data_ptr(), x.stride(0), residual.has_value() ? residual->data_ptr() : nullptr,
                                         residual.has_value() ? residual->stride(0) : 0,
                                         sum_out.has_value() ? sum_out->data_ptr() : nullptr,
                                         sum_out.has_value() ? sum_out->stride(0) : 0, optp<float>(norm_w), float(eps),
                                         float(w_offset), normed_out.has_value() ? normed_out->data_ptr() : nullptr,
                                         normed_out.has_value() ? normed_out->stride(0) : 0, rows, K,
                                         optp<float>(gscale_static), reinterpret_cast<uint8_t*>(codes.data_ptr()),
                                         codes.stride(0), reinterpret_cast<uint8_t*>(sf_atoms.data_ptr()),
                                         optpm<float>(row_gscale), cur_stream()) == 0,
                "nv4_act_quant: K must be a multiple of 16 and at most 8192, rows 16-byte aligned");
  });
  m.def("expert_cache_prepare", [](const Tensor& ids, Tensor& slot_of, Tensor& expert_in, Tensor& heat, double decay,
                                   const Tensor& host_gu, const Tensor& host_dn, Tensor& slot_gu, Tensor& slot_dn,
                                   Tensor& ids_slot, Tensor& miss_list, Tensor& ctl, Tensor& stats, Tensor& status) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kInt && ids.is_contiguous() && ids_slot.is_contiguous() &&
                    ids_slot.numel() >= ids.numel() && slot_of.scalar_type() == at::kInt &&
                    expert_in.scalar_type() == at::kInt && heat.scalar_type() == at::kFloat,
                "expert_cache_prepare: int32 routing and tables, float heat");
    TORCH_CHECK(host_gu.is_pinned() && host_dn.is_pinned() && host_gu.is_contiguous() && host_dn.is_contiguous() &&
                    slot_gu.is_contiguous() && slot_dn.is_contiguous() && host_gu.size(0) == slot_of.numel() &&
                    slot_gu.size(0) == expert_in.numel() && miss_list.numel() >= 2 * expert_in.numel() &&
                    ctl.numel() >= 3 && stats.numel() >= 4 && stats.element_size() == 8,
                "expert_cache_prepare: pinned host experts [E, ...], device slots [n_slots, ...]");
    const long gu_bytes = host_gu[0].numel() * host_gu.element_size(), dn_bytes = host_dn[0].numel() * host_dn.element_size();
    c10::cuda::CUDAGuard guard(ids.device());
    TORCH_CHECK(lb::expert_cache_prepare_launch(
                    ids.data_ptr<int>(), int(ids.numel()), int(slot_of.numel()), int(expert_in.numel()),
                    slot_of.data_ptr<int>(), expert_in.data_ptr<int>(), heat.data_ptr<float>(), float(decay),
                    host_gu.data_ptr(), host_dn.data_ptr(), slot_gu.data_ptr(), slot_dn.data_ptr(), gu_bytes, dn_bytes,
                    ids_slot.data_ptr<int>(), miss_list.data_ptr<int>(),
                    reinterpret_cast<unsigned int*>(ctl.data_ptr()), reinterpret_cast<unsigned long long*>(stats.data_ptr()),
                    reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0,
                "expert_cache_prepare: at most 2048 experts, expert bytes a multiple of 16");
  });
  m.def("mamba2_scan", [](const Tensor& xbc, const Tensor& dt_raw, const Tensor& z, const Tensor& A, const Tensor& D,
                          const Tensor& dt_bias, Tensor& state, const Tensor& cu_seq, const Tensor& slots, int64_t nh,
                          int64_t hd, int64_t ng, int64_t ds, Tensor& y, bool write_state) {
    TORCH_CHECK(xbc.scalar_type() == at::kBFloat16 && dt_raw.scalar_type() == at::kBFloat16 &&
                    z.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16 && xbc.stride(1) == 1 &&
                    dt_raw.stride(1) == 1 && z.stride(1) == 1 && y.stride(1) == 1 && state.is_contiguous() &&
                    state.scalar_type() == at::kFloat && xbc.size(1) == nh * hd + 2 * ng * ds,
                "mamba2_scan: bf16 rows [T, di + 2 * ng * ds], fp32 state [slots, nh, hd, ds]");
    c10::cuda::CUDAGuard guard(xbc.device());
    TORCH_CHECK(lb::mamba2_scan_launch(xbc.data_ptr(), xbc.stride(0), dt_raw.data_ptr(), dt_raw.stride(0), z.data_ptr(),
                                       z.stride(0), A.data_ptr<float>(), D.data_ptr<float>(), dt_bias.data_ptr<float>(),
                                       state.data_ptr<float>(), cu_seq.data_ptr<int>(), slots.data_ptr<int>(),
                                       int(slots.numel()), int(nh), int(hd), int(ng), int(ds), y.data_ptr(), y.stride(0),
                                       write_state ? 1 : 0, cur_stream()) == 0,
                "mamba2_scan: unsupported head shape");
  });
  m.def("nv4_gather_rows", [](const Tensor& codes, const Tensor& sf, const OptT& gscale, const Tensor& rows,
                              const OptT& n_rows, Tensor& dst_codes, Tensor& dst_sf, const OptT& dst_gscale) {
    TORCH_CHECK(codes.dim() == 2 && dst_codes.dim() == 2 && codes.stride(1) == 1 && dst_codes.stride(1) == 1 &&
                    codes.size(1) == dst_codes.size(1) && rows.scalar_type() == at::kInt && rows.is_contiguous() &&
                    dst_codes.size(0) >= rows.numel(), "nv4_gather_rows: codes [T, K / 2] -> [rows, K / 2]");
    const long K = codes.size(1) * 2;
    TORCH_CHECK(size_t(dst_sf.numel()) >= lb::nv4_sf_bytes(rows.numel(), K) && sf.is_contiguous() && dst_sf.is_contiguous(),
                "nv4_gather_rows: scale atom buffer too small");
    TORCH_CHECK(gscale.has_value() == dst_gscale.has_value() &&
                    (!dst_gscale.has_value() || dst_gscale->numel() >= rows.numel()), "nv4_gather_rows: row scales");
    c10::cuda::CUDAGuard guard(codes.device());
    TORCH_CHECK(lb::nv4_gather_rows_launch(reinterpret_cast<const uint8_t*>(codes.data_ptr()), codes.stride(0),
                                           reinterpret_cast<const uint8_t*>(sf.data_ptr()), optp<float>(gscale), K,
                                           rows.data_ptr<int>(), optp<int>(n_rows), rows.numel(),
                                           reinterpret_cast<uint8_t*>(dst_codes.data_ptr()), dst_codes.stride(0),
                                           reinterpret_cast<uint8_t*>(dst_sf.data_ptr()), optpm<float>(dst_gscale),
                                           cur_stream()) == 0, "nv4_gather_rows: K % 64, 16-byte aligned rows");
  });
  m.def("wgemm_nv4", [](const Tensor& w, const Tensor& w_sf, const OptT& w_gscale, const Tensor& x, const Tensor& x_sf,
                        const OptT& x_gscale, int64_t x_gs_stride, const OptT& out, const OptT& residual,
                        const OptT& tok_scale, const OptT& out_rows, int64_t n_feat, bool dual, int64_t dual_offset,
                        int64_t act, int64_t bn, Tensor& status, const OptT& tile_group, const OptT& tile_tok0,
                        const OptT& tile_ntok, const OptT& meta, int64_t max_tiles, int64_t rows_per_group, int64_t n_tok,
                        const OptT& tile_out0, const OptT& q_codes, const OptT& q_sf, const OptT& q_gscale) {
    TORCH_CHECK(w.is_cuda() && w.dim() == 2 && x.dim() == 2 && w.element_size() == 1 && x.element_size() == 1 &&
                    w.stride(1) == 1 && x.stride(1) == 1 && w.size(1) == x.size(1),
                "wgemm_nv4: w [rows, K / 2] and x [tokens, K / 2] are packed e2m1 bytes with the same K");
    const long K = x.size(1) * 2;
    TORCH_CHECK(w_sf.is_contiguous() && size_t(w_sf.numel()) >= lb::nv4_sf_bytes(w.size(0), K) && x_sf.is_contiguous() &&
                    size_t(x_sf.numel()) >= lb::nv4_sf_bytes(x.size(0), K), "wgemm_nv4: scale atom buffers too small");
    c10::cuda::CUDAGuard guard(w.device());
    lb::Nv4Host h{};
    h.w = reinterpret_cast<const uint8_t*>(w.data_ptr()); h.w_rows = w.size(0); h.ldw = w.stride(0);
    h.w_sf = reinterpret_cast<const uint8_t*>(w_sf.data_ptr()); h.w_gscale = optp<float>(w_gscale);
    h.x = reinterpret_cast<const uint8_t*>(x.data_ptr()); h.x_rows = x.size(0); h.ldx = x.stride(0);
    h.x_sf = reinterpret_cast<const uint8_t*>(x_sf.data_ptr());
    h.x_gscale = optp<float>(x_gscale); h.x_gs_stride = int(x_gs_stride);
    if (out.has_value()) {
      TORCH_CHECK(out->scalar_type() == at::kBFloat16 && out->dim() == 2 && out->stride(1) == 1 && out->size(1) >= n_feat,
                  "wgemm_nv4: out must be bf16 [rows, >= n_feat]");
      h.out = out->data_ptr(); h.ldo = out->stride(0);
    }
    if (residual.has_value()) {
      TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->stride(1) == 1, "wgemm_nv4: residual bf16");
      h.residual = reinterpret_cast<const __nv_bfloat16*>(residual->data_ptr()); h.ldr = residual->stride(0);
    }
    h.tok_scale = optp<float>(tok_scale); h.out_rows = optp<int>(out_rows);
    if (q_codes.has_value()) {
      TORCH_CHECK(q_sf.has_value() && q_gscale.has_value() && q_codes->dim() == 2 && q_codes->stride(1) == 1 &&
                      q_codes->size(1) * 2 >= n_feat && q_sf->is_contiguous() &&
                      size_t(q_sf->numel()) >= lb::nv4_sf_bytes(q_codes->size(0), n_feat),
                  "wgemm_nv4: quantised output needs codes [rows, n_feat / 2], scale atoms and a tensor scale");
      h.q_codes = reinterpret_cast<uint8_t*>(q_codes->data_ptr()); h.q_ld = q_codes->stride(0);
      h.q_sf = reinterpret_cast<uint8_t*>(q_sf->data_ptr()); h.q_gscale = q_gscale->data_ptr<float>();
    }
    h.K = int(K); h.n_feat = int(n_feat); h.n_tok = int(n_tok); h.bn = int(bn); h.dual = dual; h.act = int(act);
    h.tile_group = optp<int>(tile_group); h.tile_tok0 = optp<int>(tile_tok0); h.tile_ntok = optp<int>(tile_ntok);
    h.n_tiles_dev = optp<int>(meta); h.tile_out0 = optp<int>(tile_out0); h.n_tok_tiles_max = int(max_tiles);
    h.rows_per_group = int(rows_per_group); h.dual_offset = int(dual_offset);
    h.status = reinterpret_cast<int*>(status.data_ptr());
    TORCH_CHECK(lb::wgemm_nv4_launch(h, cur_stream()) == 0, lb::wgemm_nv4_last_error());
  });
  m.def("gguf_dequant", [](const Tensor& raw, int64_t ggml_type, Tensor& out) {
    TORCH_CHECK(raw.scalar_type() == at::kByte && raw.is_contiguous() && out.scalar_type() == at::kBFloat16 &&
                    out.is_contiguous(), "gguf_dequant: raw uint8 -> bf16");
    c10::cuda::CUDAGuard guard(raw.device());
    TORCH_CHECK(lb::gguf_dequant_launch(raw.data_ptr(), int(ggml_type), out.numel(), out.data_ptr(), cur_stream()) == 0,
                "gguf_dequant: unsupported tensor type or size");
  });
  m.def("randn_bf16", [](Tensor& out, double stdv, int64_t seed) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(lb::randn_bf16_launch(out.data_ptr(), out.numel(), float(stdv), uint64_t(seed), cur_stream()) == 0,
                "randn_bf16 failed");
  });
}
