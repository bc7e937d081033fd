// Python bindings for the Gated DeltaNet, communication and block-scaled format kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.h"
#include "ep.h"
#include "gdn.h"
#include "quant.h"

namespace {
using torch::Tensor;
using OptT = c10::optional<Tensor>;
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
template <typename T>
const T* optp(const OptT& t) {
  return t.has_value() ? reinterpret_cast<const T*>(t->data_ptr()) : nullptr;
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
                          const Tensor& slots, Tensor& out, bool write_state) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kFloat, "conv1d_silu dtypes");
    TORCH_CHECK(lb::conv1d_silu_launch(x.data_ptr(), x.stride(0), w.data_ptr<float>(), optp<float>(bias),
                                       conv_state.data_ptr<float>(), cu_seq.data_ptr<int>(), slots.data_ptr<int>(),
                                       int(slots.numel()), int(x.size(1)), int(w.size(1)), out.data_ptr(),
                                       out.stride(0), write_state ? 1 : 0, cur_stream()) == 0,
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
                               const OptT& norm_out, int64_t budget_ns, Tensor& status) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::all_reduce_fused_launch(
                    p, buf_off, int(slot_base), reinterpret_cast<uint32_t*>(seq.data_ptr()),
                    reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(T), int(H),
                    residual.has_value() ? residual->data_ptr() : nullptr,
                    residual.has_value() ? residual->stride(0) : 0, sum_out.data_ptr(), sum_out.stride(0),
                    optp<float>(norm_w), float(eps), float(w_offset),
                    norm_out.has_value() ? norm_out->data_ptr() : nullptr,
                    norm_out.has_value() ? norm_out->stride(0) : 0, uint64_t(budget_ns),
                    reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0,
                "all_reduce_fused failed");
  });
  m.def("reduce_scatter_fused", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                                   int64_t buf_off, int64_t out_off, int64_t slot_base, Tensor& seq, Tensor& done_ctr,
                                   int64_t row0, int64_t n_rows, int64_t H, const OptT& residual, int64_t budget_ns,
                                   Tensor& status) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::reduce_scatter_launch(p, buf_off, out_off, int(slot_base),
                                          reinterpret_cast<uint32_t*>(seq.data_ptr()),
                                          reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(row0), int(n_rows),
                                          int(H), residual.has_value() ? residual->data_ptr() : nullptr,
                                          residual.has_value() ? residual->stride(0) : 0, uint64_t(budget_ns),
                                          reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0,
                "reduce_scatter_fused failed");
  });
  m.def("all_gather_fused", [](std::vector<int64_t> buffers, std::vector<int64_t> signals, int64_t rank,
                               int64_t src_off, int64_t slot_base, Tensor& seq, Tensor& done_ctr, int64_t T, int64_t H,
                               Tensor& out, int64_t budget_ns, Tensor& status) {
    c10::cuda::CUDAGuard guard(status.device());
    auto p = make_peers(buffers, signals, rank);
    TORCH_CHECK(lb::all_gather_launch(p, src_off, int(slot_base), reinterpret_cast<uint32_t*>(seq.data_ptr()),
                                      reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(T), int(H),
                                      out.data_ptr(), out.stride(0), uint64_t(budget_ns),
                                      reinterpret_cast<int*>(status.data_ptr()), cur_stream()) == 0,
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
