// Python bindings (module legion_b200._C): thin checks + pointer extraction around the launchers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.h"
#include "gdn.h"
#include "gemm_sm100.h"
#include "kernels.h"
namespace lb {
bool pdl_enabled();
void set_pdl(bool on);
}  // namespace lb
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

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK(t.stride(-1) == 1, name, " must be contiguous in its last dimension");
}

// out[token, feature] = W x (+ epilogue). w: [rows, K]; x: [tokens, K]; out: [out_rows, >= n_feat].
void wgemm(const Tensor& w, const Tensor& x, Tensor& out, const OptT& residual, const OptT& tok_scale,
           const OptT& out_rows, int64_t n_feat, bool dual, int64_t dual_offset, int64_t bn, int64_t split_k,
           const OptT& ws, const OptT& counters, Tensor& status, const OptT& tile_group, const OptT& tile_tok0,
           const OptT& tile_ntok, const OptT& meta, int64_t max_tiles, int64_t rows_per_group, int64_t n_tok,
           std::vector<int64_t> out_peer, const OptT& tile_out0, const OptT& w_scales, const OptT& w_gscale,
           int64_t x_group_col, int64_t k_override) {
  const bool fp4 = w_scales.has_value();     // w = NVFP4 codes [rows, K/2] uint8, w_scales = e4m3 bytes [rows, K/16]
  if (fp4) {
    TORCH_CHECK(w.scalar_type() == at::kByte && w_scales->is_contiguous() && w_scales->element_size() == 1 &&
                    w.stride(1) == 1, "wgemm: NVFP4 weights are uint8 codes with 1-byte block scales");
    TORCH_CHECK(w_scales->size(0) == w.size(0) && w_scales->size(1) * 8 == w.size(1), "wgemm: NVFP4 scale shape");
  } else {
    check_bf16(w, "w");
  }
  check_bf16(x, "x");
  TORCH_CHECK(w.dim() == 2 && x.dim() == 2 && out.dim() == 2, "wgemm expects 2-D tensors");
  TORCH_CHECK(k_override > 0 || w.size(1) * (fp4 ? 2 : 1) == x.size(1), "wgemm: K mismatch");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat, "wgemm: out must be bf16/f32");
  TORCH_CHECK(out.stride(1) == 1 && out.size(1) >= n_feat, "wgemm: bad out");
  c10::cuda::CUDAGuard guard(w.device());
  lb::WgemmHost h{};
  h.w = w.data_ptr(); h.w_rows = w.size(0); h.ldw = w.stride(0);
  h.x = x.data_ptr(); h.x_rows = x.size(0); h.ldx = x.stride(0);
  h.out = out.data_ptr(); h.ldo = out.stride(0); h.out_f32 = out.scalar_type() == at::kFloat;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    h.residual = reinterpret_cast<const __nv_bfloat16*>(residual->data_ptr());
    h.ldr = residual->stride(0);
  }
  h.tok_scale = optp<float>(tok_scale);
  h.out_rows = optp<int>(out_rows);
  h.K = int(x.size(1)); h.n_feat = int(n_feat); h.n_tok = int(n_tok);
  if (k_override > 0) {          // per-group slices of a wider activation tensor: K is the weight's width
    TORCH_CHECK(!fp4 && w.size(1) == k_override && x_group_col > 0, "wgemm: per-group columns need K == w.size(1)");
    h.K = int(k_override);
    h.x_cols = x.size(1);
    h.x_group_col = int(x_group_col);
  }
  h.w_scales = fp4 ? w_scales->data_ptr() : nullptr;
  h.w_gscale = optp<float>(w_gscale);
  h.bn = int(bn); h.dual = dual;
  h.tile_group = optp<int>(tile_group); h.tile_tok0 = optp<int>(tile_tok0); h.tile_ntok = optp<int>(tile_ntok);
  h.n_tiles_dev = optp<int>(meta);
  h.tile_out0 = optp<int>(tile_out0);
  h.n_tok_tiles_max = int(max_tiles);
  h.rows_per_group = int(rows_per_group); h.dual_offset = int(dual_offset);
  h.split_k = int(split_k);
  h.ws = optpm<float>(ws);
  h.counters = optpm<int>(counters);
  if (h.split_k > 1) {
    TORCH_CHECK(ws.has_value() && counters.has_value(), "wgemm: split-K needs ws and counters");
    const int n_tok_tiles = h.tile_group ? h.n_tok_tiles_max : (h.n_tok + h.bn - 1) / h.bn;
    const int feat_tiles = (h.n_feat + 127) / 128;
    TORCH_CHECK(size_t(ws->numel()) >= lb::wgemm_workspace_floats(h.bn, dual, n_tok_tiles, feat_tiles, h.split_k),
                "wgemm: split-K workspace too small");
    TORCH_CHECK(counters->numel() >= int64_t(n_tok_tiles) * feat_tiles, "wgemm: too few split-K counters");
  }
  h.status = reinterpret_cast<int*>(status.data_ptr());
  TORCH_CHECK(out_peer.size() <= 8, "wgemm: at most 8 peer outputs");
  h.n_out_peer = int(out_peer.size());
  for (size_t i = 0; i < out_peer.size(); ++i) h.out_peer[i] = reinterpret_cast<void*>(out_peer[i]);
  TORCH_CHECK(lb::wgemm_launch(h, cur_stream()) == 0, lb::wgemm_last_error());
}

// Block-scaled FP8: w [rows, K] and x [tokens, K] hold e4m3 bytes; w_bscale [rows / 128, K / 128] and x_bscale
// [tokens, K / 128] are fp32. Same tile / grouping / epilogue options as wgemm; out is bf16.
void wgemm_fp8_q(const Tensor& w, const Tensor& w_bscale, const Tensor& x, const Tensor& x_bscale, Tensor& out,
                 const OptT& residual, const OptT& tok_scale, const OptT& out_rows, int64_t n_feat, bool dual,
                 int64_t dual_offset, int64_t bn, int64_t split_k, const OptT& ws, const OptT& counters, Tensor& status,
                 const OptT& tile_group, const OptT& tile_tok0, const OptT& tile_ntok, const OptT& meta, int64_t max_tiles,
                 int64_t rows_per_group, int64_t n_tok, const OptT& tile_out0, const OptT& q_out, const OptT& q_scale) {
  TORCH_CHECK(w.is_cuda() && x.is_cuda() && w.element_size() == 1 && x.element_size() == 1 && w.dim() == 2 &&
                  x.dim() == 2 && w.stride(1) == 1 && x.stride(1) == 1 && w.size(1) == x.size(1),
              "wgemm_fp8: w [rows, K] and x [tokens, K] must be 1-byte e4m3 tensors with the same K");
  const int64_t K = x.size(1);
  TORCH_CHECK(w_bscale.scalar_type() == at::kFloat && w_bscale.is_contiguous() &&
                  w_bscale.numel() == ((w.size(0) + 127) / 128) * (K / 128), "wgemm_fp8: weight block scales");
  TORCH_CHECK(x_bscale.scalar_type() == at::kFloat && x_bscale.is_contiguous() && x_bscale.numel() == x.size(0) * (K / 128),
              "wgemm_fp8: activation group scales");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.stride(1) == 1 && out.size(1) >= n_feat,
              "wgemm_fp8: out must be bf16 [rows, >= n_feat]");
  c10::cuda::CUDAGuard guard(w.device());
  lb::WgemmHost h{};
  h.w = w.data_ptr(); h.w_rows = w.size(0); h.ldw = w.stride(0);
  h.x = x.data_ptr(); h.x_rows = x.size(0); h.ldx = x.stride(0);
  h.w_bscale = w_bscale.data_ptr<float>(); h.x_bscale = x_bscale.data_ptr<float>();
  h.out = out.data_ptr(); h.ldo = out.stride(0); h.out_f32 = false;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    h.residual = reinterpret_cast<const __nv_bfloat16*>(residual->data_ptr());
    h.ldr = residual->stride(0);
  }
  h.tok_scale = optp<float>(tok_scale);
  h.out_rows = optp<int>(out_rows);
  h.K = int(K); h.n_feat = int(n_feat); h.n_tok = int(n_tok);
  h.bn = int(bn); h.dual = dual;
  h.tile_group = optp<int>(tile_group); h.tile_tok0 = optp<int>(tile_tok0); h.tile_ntok = optp<int>(tile_ntok);
  h.n_tiles_dev = optp<int>(meta);
  h.tile_out0 = optp<int>(tile_out0);
  h.n_tok_tiles_max = int(max_tiles);
  h.rows_per_group = int(rows_per_group); h.dual_offset = int(dual_offset);
  h.split_k = int(split_k);
  h.ws = optpm<float>(ws);
  h.counters = optpm<int>(counters);
  if (h.split_k > 1) {
    TORCH_CHECK(ws.has_value() && counters.has_value(), "wgemm_fp8: split-K needs ws and counters");
    const int n_tok_tiles = h.tile_group ? h.n_tok_tiles_max : (h.n_tok + h.bn - 1) / h.bn;
    const int feat_tiles = (h.n_feat + 127) / 128;
    TORCH_CHECK(size_t(ws->numel()) >= lb::wgemm_workspace_floats(h.bn, dual, n_tok_tiles, feat_tiles, h.split_k),
                "wgemm_fp8: split-K workspace too small");
    TORCH_CHECK(counters->numel() >= int64_t(n_tok_tiles) * feat_tiles, "wgemm_fp8: too few split-K counters");
  }
  h.status = reinterpret_cast<int*>(status.data_ptr());
  if (q_out.has_value()) {
    // the gate/up form leaves its activated rows e4m3-encoded for the down projection; `out` is not written
    TORCH_CHECK(q_scale.has_value() && q_out->is_cuda() && q_out->element_size() == 1 && q_out->is_contiguous() &&
                    q_out->dim() == 2 && q_out->size(1) == n_feat && q_out->size(0) >= out.size(0) &&
                    q_scale->scalar_type() == at::kFloat && q_scale->is_contiguous() &&
                    q_scale->numel() >= q_out->size(0) * (n_feat / 128),
                "wgemm_fp8: encoded output [rows, n_feat] bytes with float scales [rows, n_feat / 128]");
    h.q8_out = reinterpret_cast<uint8_t*>(q_out->data_ptr());
    h.q8_scale = q_scale->data_ptr<float>();
  }
  TORCH_CHECK(lb::wgemm_launch(h, cur_stream()) == 0, lb::wgemm_last_error());
}

void wgemm_fp8(const Tensor& w, const Tensor& w_bscale, const Tensor& x, const Tensor& x_bscale, Tensor& out,
               const OptT& residual, const OptT& tok_scale, const OptT& out_rows, int64_t n_feat, bool dual,
               int64_t dual_offset, int64_t bn, int64_t split_k, const OptT& ws, const OptT& counters, Tensor& status,
               const OptT& tile_group, const OptT& tile_tok0, const OptT& tile_ntok, const OptT& meta, int64_t max_tiles,
               int64_t rows_per_group, int64_t n_tok, const OptT& tile_out0) {
  wgemm_fp8_q(w, w_bscale, x, x_bscale, out, residual, tok_scale, out_rows, n_feat, dual, dual_offset, bn, split_k, ws,
              counters, status, tile_group, tile_tok0, tile_ntok, meta, max_tiles, rows_per_group, n_tok, tile_out0,
              c10::nullopt, c10::nullopt);
}

// Dense GEMM whose kernel tail all-reduces the output over the ranks' symmetric buffers (+ residual, + RMSNorm).
// `slot` must be this rank's partial slot inside its symmetric buffer (byte offset buf_off).
void wgemm_allreduce(const Tensor& w, const Tensor& x, Tensor& slot, int64_t bn, int64_t split_k, const OptT& ws,
                     const OptT& counters, Tensor& status, std::vector<int64_t> buffers, std::vector<int64_t> signals,
                     int64_t rank, int64_t buf_off, int64_t slot_base, Tensor& seq, Tensor& ctrs, const OptT& residual,
                     Tensor& sum_out, const OptT& norm_w, double eps, double w_offset, const OptT& norm_out,
                     int64_t budget_ns, Tensor& comm_status) {
  check_bf16(w, "w");
  check_bf16(x, "x");
  check_bf16(slot, "slot");
  TORCH_CHECK(w.dim() == 2 && x.dim() == 2 && slot.dim() == 2 && w.size(1) == x.size(1), "wgemm_allreduce: shapes");
  TORCH_CHECK(slot.is_contiguous() && slot.size(0) == x.size(0) && slot.size(1) == w.size(0),
              "wgemm_allreduce: the slot must be a contiguous [tokens, features] view");
  TORCH_CHECK(buffers.size() == signals.size() && buffers.size() <= LB_MAX_RANKS && ctrs.numel() >= 2,
              "wgemm_allreduce: bad peer table");
  TORCH_CHECK(norm_w.has_value() == norm_out.has_value(), "wgemm_allreduce: norm weight and output go together");
  c10::cuda::CUDAGuard guard(w.device());
  lb::WgemmHost h{};
  h.w = w.data_ptr(); h.w_rows = w.size(0); h.ldw = w.stride(0);
  h.x = x.data_ptr(); h.x_rows = x.size(0); h.ldx = x.stride(0);
  h.out = slot.data_ptr(); h.ldo = slot.stride(0); h.out_f32 = false;
  h.K = int(w.size(1)); h.n_feat = int(w.size(0)); h.n_tok = int(x.size(0));
  h.bn = int(bn); h.dual = false;
  h.split_k = int(split_k);
  h.ws = optpm<float>(ws);
  h.counters = optpm<int>(counters);
  h.status = reinterpret_cast<int*>(status.data_ptr());
  auto& c = h.comm;
  c.enabled = 1;
  c.peers.world = int(buffers.size());
  c.peers.rank = int(rank);
  for (size_t i = 0; i < buffers.size(); ++i) {
    c.peers.buffer[i] = reinterpret_cast<void*>(buffers[i]);
    c.peers.signal[i] = reinterpret_cast<void*>(signals[i]);
  }
  c.buf_off = buf_off; c.slot_base = int(slot_base);
  c.seq_ptr = reinterpret_cast<uint32_t*>(seq.data_ptr());
  c.ctrs = reinterpret_cast<unsigned int*>(ctrs.data_ptr());
  c.T = int(x.size(0)); c.H = int(w.size(0));
  c.residual = residual.has_value() ? reinterpret_cast<const __nv_bfloat16*>(residual->data_ptr()) : nullptr;
  c.ldr = residual.has_value() ? residual->stride(0) : 0;
  c.sum_out = reinterpret_cast<__nv_bfloat16*>(sum_out.data_ptr()); c.lds = sum_out.stride(0);
  c.norm_w = optp<float>(norm_w); c.eps = float(eps); c.w_offset = float(w_offset);
  c.norm_out = norm_out.has_value() ? reinterpret_cast<__nv_bfloat16*>(norm_out->data_ptr()) : nullptr;
  c.ldn = norm_out.has_value() ? norm_out->stride(0) : 0;
  c.budget_ns = static_cast<unsigned long long>(budget_ns);
  c.status = reinterpret_cast<int*>(comm_status.data_ptr());
  TORCH_CHECK(lb::wgemm_launch(h, cur_stream()) == 0, lb::wgemm_last_error());
}

// Dense GEMM whose kernel head all-gathers the activation rows from the ranks' symmetric buffers into x_full.
void wgemm_allgather(const Tensor& w, Tensor& x_full, Tensor& out, const OptT& residual, int64_t bn, int64_t split_k,
                     const OptT& ws, const OptT& counters, Tensor& status, std::vector<int64_t> buffers,
                     std::vector<int64_t> signals, int64_t rank, int64_t src_off, int64_t slot_base, Tensor& seq,
                     Tensor& ctrs, int64_t rows_per_rank, int64_t budget_ns, Tensor& comm_status) {
  check_bf16(w, "w");
  check_bf16(x_full, "x_full");
  TORCH_CHECK(w.dim() == 2 && x_full.dim() == 2 && out.dim() == 2 && w.size(1) == x_full.size(1) &&
                  x_full.is_contiguous(), "wgemm_allgather: shapes");
  TORCH_CHECK(out.size(0) == x_full.size(0) && out.size(1) >= w.size(0) && out.stride(1) == 1, "wgemm_allgather: out");
  TORCH_CHECK(buffers.size() == signals.size() && buffers.size() <= LB_MAX_RANKS && ctrs.numel() >= 2 &&
                  x_full.size(1) % 8 == 0, "wgemm_allgather: bad peer table");
  c10::cuda::CUDAGuard guard(w.device());
  lb::WgemmHost h{};
  h.w = w.data_ptr(); h.w_rows = w.size(0); h.ldw = w.stride(0);
  h.x = x_full.data_ptr(); h.x_rows = x_full.size(0); h.ldx = x_full.stride(0);
  h.out = out.data_ptr(); h.ldo = out.stride(0); h.out_f32 = out.scalar_type() == at::kFloat;
  if (residual.has_value()) {
    h.residual = reinterpret_cast<const __nv_bfloat16*>(residual->data_ptr());
    h.ldr = residual->stride(0);
  }
  h.K = int(w.size(1)); h.n_feat = int(w.size(0)); h.n_tok = int(x_full.size(0));
  h.bn = int(bn); h.dual = false;
  h.split_k = int(split_k);
  h.ws = optpm<float>(ws);
  h.counters = optpm<int>(counters);
  h.status = reinterpret_cast<int*>(status.data_ptr());
  auto& c = h.head;
  c.enabled = 1;
  c.peers.world = int(buffers.size());
  c.peers.rank = int(rank);
  for (size_t i = 0; i < buffers.size(); ++i) {
    c.peers.buffer[i] = reinterpret_cast<void*>(buffers[i]);
    c.peers.signal[i] = reinterpret_cast<void*>(signals[i]);
  }
  c.src_off = src_off; c.slot_base = int(slot_base);
  c.seq_ptr = reinterpret_cast<uint32_t*>(seq.data_ptr());
  c.ctrs = reinterpret_cast<unsigned int*>(ctrs.data_ptr());
  c.T = int(x_full.size(0)); c.K = int(x_full.size(1)); c.rows_per_rank = int(rows_per_rank);
  c.x_local = reinterpret_cast<__nv_bfloat16*>(x_full.data_ptr());
  c.budget_ns = static_cast<unsigned long long>(budget_ns);
  c.status = reinterpret_cast<int*>(comm_status.data_ptr());
  TORCH_CHECK(lb::wgemm_launch(h, cur_stream()) == 0, lb::wgemm_last_error());
}

void rmsnorm(const Tensor& x, const OptT& res_in, const OptT& res_out, const Tensor& w, Tensor& y, double eps,
             double w_offset) {
  check_bf16(x, "x");
  TORCH_CHECK(w.scalar_type() == at::kFloat, "rmsnorm weight must be float32");
  c10::cuda::CUDAGuard guard(x.device());
  const int H = int(x.size(-1));
  const int rows = int(x.numel() / H);
  auto ld = [&](const Tensor& t) { return t.dim() >= 2 ? t.stride(-2) : long(H); };
  TORCH_CHECK(lb::rmsnorm_launch(x.data_ptr(), ld(x), res_in.has_value() ? res_in->data_ptr() : nullptr,
                                 res_in.has_value() ? ld(*res_in) : 0,
                                 res_out.has_value() ? res_out->data_ptr() : nullptr,
                                 res_out.has_value() ? ld(*res_out) : 0, w.data_ptr<float>(), y.data_ptr(), ld(y),
                                 rows, H, float(eps), float(w_offset), cur_stream()) == 0,
              "rmsnorm launch failed (hidden size must be a multiple of 8)");
}

void qk_norm_rope_append(const Tensor& qkv, int64_t q_head_stride, int64_t k_off, int64_t v_off, const OptT& qw,
                         const OptT& kw, double eps, double w_offset, const Tensor& cos_sin, int64_t rot,
                         const Tensor& positions, const Tensor& slots, Tensor& q_out, Tensor& k_cache,
                         Tensor& v_cache, int64_t Hq, int64_t Hkv, int64_t D) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(positions.scalar_type() == at::kInt && slots.scalar_type() == at::kLong, "positions i32, slots i64");
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = int(qkv.size(0));
  const long cell_stride = k_cache.stride(-3);  // [.., page, Hkv, D] -> elements between cells
  TORCH_CHECK(lb::qk_norm_rope_append_launch(qkv.data_ptr(), qkv.stride(0), int(q_head_stride), int(k_off), int(v_off),
                                             optp<float>(qw), optp<float>(kw), float(eps), float(w_offset),
                                             cos_sin.data_ptr<float>(), int(rot), positions.data_ptr<int>(),
                                             reinterpret_cast<const long*>(slots.data_ptr()), q_out.data_ptr(),
                                             k_cache.data_ptr(), v_cache.data_ptr(), cell_stride, T, int(Hq), int(Hkv),
                                             int(D), cur_stream()) == 0,
              "qk_norm_rope_append: unsupported head dim / rotary dim");
}

void sigmoid_gate(const Tensor& attn, const Tensor& qkv, int64_t q_head_stride, int64_t D, int64_t Hq, Tensor& out) {
  c10::cuda::CUDAGuard guard(attn.device());
  const long T = attn.numel() / (Hq * D);
  TORCH_CHECK(lb::sigmoid_gate_launch(attn.data_ptr(), qkv.data_ptr(), qkv.stride(0), int(q_head_stride), int(D),
                                      int(Hq), out.data_ptr(), T, cur_stream()) == 0, "sigmoid_gate failed");
}

void glu(const Tensor& x, Tensor& out, int64_t F, int64_t act) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(lb::glu_launch(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), int(F), x.size(0), int(act),
                             cur_stream()) == 0, "glu failed");
}

void embed(const Tensor& ids, const Tensor& table, Tensor& out) {
  check_bf16(table, "table");
  TORCH_CHECK(ids.scalar_type() == at::kInt, "ids must be int32");
  c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(lb::embed_launch(ids.data_ptr<int>(), table.data_ptr(), table.stride(0), out.data_ptr(), out.stride(0),
                               int(ids.numel()), int(table.size(1)), int(table.size(0)), cur_stream()) == 0,
              "embed failed");
}

void paged_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_table,
                  const Tensor& ctx_lens, double scale, int64_t window, int64_t n_splits, Tensor& o_part,
                  Tensor& ml_part, Tensor& out, bool use_tc, Tensor& status, Tensor& counters) {
  check_bf16(q, "q");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = int(q.size(0)), Hq = int(q.size(1)), D = int(q.size(2));
  const int page = int(k_cache.size(-3)), Hkv = int(k_cache.size(-2));
  const int64_t parts = n_splits * (use_tc ? 2 : 1);   // the tensor-core kernel writes two partials per split
  TORCH_CHECK(o_part.numel() >= int64_t(B) * Hq * parts * D && ml_part.numel() >= int64_t(B) * Hq * parts * 2,
              "paged_decode: partial buffers too small");
  if (use_tc && k_cache.is_contiguous() && v_cache.is_contiguous() && q.is_contiguous() && out.is_contiguous()) {
    const long n_cells = k_cache.numel() / (long(Hkv) * D);
    const int rc = lb::paged_decode_tc_launch(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), n_cells,
                                              long(Hkv) * D, block_table.data_ptr<int>(), int(block_table.size(1)),
                                              page, ctx_lens.data_ptr<int>(), float(scale), int(window), B, Hq, Hkv,
                                              D, int(n_splits), o_part.data_ptr<float>(), ml_part.data_ptr<float>(),
                                              out.data_ptr(), counters.data_ptr<int>(), int(counters.numel()),
                                              reinterpret_cast<int*>(status.data_ptr()), cur_stream());
    TORCH_CHECK(rc <= 0, lb::paged_decode_tc_last_error());
    if (rc == 0) return;
  }
  const int rc = lb::paged_decode_launch(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(-3),
                                         block_table.data_ptr<int>(), int(block_table.size(1)), page,
                                         ctx_lens.data_ptr<int>(), float(scale), int(window), B, Hq, Hkv, D,
                                         int(n_splits), o_part.data_ptr<float>(), ml_part.data_ptr<float>(),
                                         out.data_ptr(), cur_stream());
  TORCH_CHECK(rc == 0, "paged_decode: unsupported shape or launch failure (", rc, ")");
}

void prefill_attn(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                  const Tensor& ctx_lens, const Tensor& block_table, int64_t max_q_len, double scale, int64_t window,
                  bool causal, Tensor& out, Tensor& status) {
  check_bf16(q, "q");
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous(), "prefill_attn: q/out must be contiguous [T, Hq, D]");
  c10::cuda::CUDAGuard guard(q.device());
  const long T = q.size(0);
  const int Hq = int(q.size(1)), D = int(q.size(2));
  const int page = int(k_cache.size(-3)), Hkv = int(k_cache.size(-2));
  const long n_cells = k_cache.numel() / (long(Hkv) * D);
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous(), "prefill_attn: caches must be contiguous");
  const int rc = lb::prefill_attn_launch(q.data_ptr(), T, k_cache.data_ptr(), v_cache.data_ptr(), n_cells,
                                         long(Hkv) * D, cu_q.data_ptr<int>(), ctx_lens.data_ptr<int>(),
                                         block_table.data_ptr<int>(), int(block_table.size(1)), page,
                                         int(ctx_lens.numel()), int(max_q_len), Hq, Hkv, D, float(scale), int(window),
                                         causal ? 1 : 0, out.data_ptr(), reinterpret_cast<int*>(status.data_ptr()),
                                         cur_stream());
  TORCH_CHECK(rc == 0, lb::prefill_attn_last_error());
}

void mla_attn(const Tensor& q_abs, const Tensor& cache, const Tensor& cu_q, const Tensor& ctx_lens,
              const Tensor& block_table, int64_t page, int64_t max_q_len, double scale, int64_t n_splits,
              const OptT& o_part, const OptT& ml_part, Tensor& out, Tensor& status) {
  check_bf16(q_abs, "q_abs");
  check_bf16(cache, "cache");
  TORCH_CHECK(q_abs.dim() == 3 && q_abs.size(2) == 576 && q_abs.is_contiguous(), "mla_attn: q_abs must be [T, heads, 576]");
  TORCH_CHECK(cache.size(-1) == 576 && cache.is_contiguous(), "mla_attn: cache rows must be [.., 576]");
  TORCH_CHECK(out.is_contiguous() && out.size(-1) == 512 && out.numel() == q_abs.size(0) * q_abs.size(1) * 512,
              "mla_attn: out must be [T, heads, 512]");
  const long T = q_abs.size(0);
  const int nh = int(q_abs.size(1));
  if (n_splits > 1) {
    TORCH_CHECK(o_part.has_value() && ml_part.has_value() && o_part->numel() >= T * nh * n_splits * 512 &&
                    ml_part->numel() >= T * nh * n_splits * 2, "mla_attn: partial workspaces too small");
  }
  c10::cuda::CUDAGuard guard(q_abs.device());
  const int rc = lb::mla_attn_launch(q_abs.data_ptr(), T, cache.data_ptr(), cache.numel() / 576, 576,
                                     cu_q.data_ptr<int>(), ctx_lens.data_ptr<int>(), block_table.data_ptr<int>(),
                                     int(block_table.size(1)), int(page), int(ctx_lens.numel()), int(max_q_len), nh,
                                     float(scale), int(n_splits), optpm<float>(o_part), optpm<float>(ml_part),
                                     out.data_ptr(), reinterpret_cast<int*>(status.data_ptr()), cur_stream());
  TORCH_CHECK(rc == 0, lb::mla_attn_last_error());
}

void mla_prep(const Tensor& kva, const Tensor& norm_w, double eps, double w_offset, const Tensor& q, int64_t q_pe_off,
              const Tensor& cos_sin, const Tensor& positions, const Tensor& slots, Tensor& cache, Tensor& q_abs) {
  check_bf16(kva, "kva");
  check_bf16(q, "q");
  check_bf16(cache, "cache");
  TORCH_CHECK(kva.dim() == 2 && kva.size(1) == 576 && kva.stride(1) == 1, "mla_prep: kva must be [T, 576]");
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q_pe_off + 64 <= q.size(2), "mla_prep: q must be [T, heads, dn + 64]");
  TORCH_CHECK(norm_w.scalar_type() == at::kFloat && norm_w.numel() == 512, "mla_prep: norm weight float32[512]");
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.size(-1) == 64 && cos_sin.is_contiguous(),
              "mla_prep: cos_sin must be float32 [positions, 64]");
  TORCH_CHECK(positions.scalar_type() == at::kInt && slots.scalar_type() == at::kLong, "positions i32, slots i64");
  TORCH_CHECK(cache.is_contiguous() && cache.size(-1) == 576, "mla_prep: cache rows must be [.., 576]");
  TORCH_CHECK(q_abs.is_contiguous() && q_abs.size(0) == q.size(0) && q_abs.size(1) == q.size(1) && q_abs.size(2) == 576,
              "mla_prep: q_abs must be [T, heads, 576]");
  c10::cuda::CUDAGuard guard(kva.device());
  TORCH_CHECK(lb::mla_prep_launch(kva.data_ptr(), kva.stride(0), norm_w.data_ptr<float>(), float(eps), float(w_offset),
                                  q.data_ptr(), q.stride(0), int(q.stride(1)), int(q_pe_off), int(q.size(1)),
                                  cos_sin.data_ptr<float>(), positions.data_ptr<int>(), slots.data_ptr<long>(),
                                  cache.data_ptr(), 576, q_abs.data_ptr(), int(kva.size(0)), cur_stream()) == 0,
              "mla_prep launch failed");
}

void router_topk(const Tensor& logits, const OptT& bias, int64_t k, int64_t mode, bool renorm, double route_scale,
                 int64_t n_group, int64_t topk_group, Tensor& ids, Tensor& wts) {
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.stride(1) == 1, "router logits must be float32");
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(lb::router_topk_launch(logits.data_ptr<float>(), logits.stride(0), optp<float>(bias),
                                     int(logits.size(1)), int(k), int(mode), renorm ? 1 : 0, float(route_scale),
                                     int(n_group), int(topk_group), ids.data_ptr<int>(), wts.data_ptr<float>(),
                                     int(logits.size(0)), cur_stream()) == 0,
              "router_topk: unsupported (experts <= 512, k <= 32, groups <= 32)");
}

void moe_route_small(const Tensor& x, const OptT& norm_w, double eps, double w_offset, const OptT& x_normed,
                     const Tensor& w, const OptT& bias, int64_t k, int64_t mode, bool renorm, double route_scale,
                     int64_t n_group, int64_t topk_group, Tensor& logits, Tensor& ids, Tensor& wts, int64_t bn,
                     Tensor& tile_group, Tensor& slot_base, Tensor& tile_ntok, Tensor& meta, Tensor& out_rows,
                     Tensor& tok_scale, Tensor& done_ctr, int64_t e_lo, int64_t n_local, const OptT& sh_gate_w,
                     const OptT& sh_logit, bool shared_slot, Tensor& status, Tensor& active) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  const int64_t T = x.size(0), E = w.size(0);
  if (sh_gate_w.has_value()) {
    check_bf16(*sh_gate_w, "sh_gate_w");
    TORCH_CHECK(sh_gate_w->numel() == x.size(1) && sh_gate_w->is_contiguous() && sh_logit.has_value() &&
                    sh_logit->scalar_type() == at::kFloat && sh_logit->numel() >= 4 * 64 && shared_slot,
                "moe_route_small: the shared gate is one row of the hidden width with a float [4 * 64] scratch");
  }
  TORCH_CHECK(x.size(1) == w.size(1) && x.stride(1) == 1 && w.stride(1) == 1, "moe_route_small: shape mismatch");
  TORCH_CHECK(norm_w.has_value() == x_normed.has_value(), "moe_route_small: norm weight and output go together");
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.numel() >= 4 * 64 * 512,
              "moe_route_small: the logit scratch holds four planes of 64 x 512 floats (one per column split)");
  TORCH_CHECK(done_ctr.numel() >= 2 && done_ctr.element_size() == 4, "moe_route_small: two int32 counters");
  TORCH_CHECK(active.scalar_type() == at::kInt && active.numel() >= n_local, "moe_route_small: active flags [n_local]");
  const int64_t max_slots = std::min<int64_t>(E, n_local) + (shared_slot ? 1 : 0);
  TORCH_CHECK(tile_group.numel() >= max_slots && slot_base.numel() >= max_slots && tile_ntok.numel() >= max_slots &&
                  meta.numel() >= 2 && out_rows.numel() >= max_slots * bn && tok_scale.numel() >= max_slots * bn,
              "moe_route_small: tables too small");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(lb::moe_route_small_launch(
                  x.data_ptr(), x.stride(0), optp<float>(norm_w), float(eps), float(w_offset),
                  x_normed.has_value() ? x_normed->data_ptr() : nullptr,
                  x_normed.has_value() ? x_normed->stride(0) : 0, w.data_ptr(), w.stride(0), int(x.size(1)),
                  logits.data_ptr<float>(), optp<float>(bias), int(E), int(k), int(mode), renorm ? 1 : 0,
                  float(route_scale), int(n_group), int(topk_group), ids.data_ptr<int>(), wts.data_ptr<float>(),
                  int(T), int(bn), tile_group.data_ptr<int>(), slot_base.data_ptr<int>(), tile_ntok.data_ptr<int>(),
                  meta.data_ptr<int>(), out_rows.data_ptr<int>(), tok_scale.data_ptr<float>(),
                  reinterpret_cast<unsigned int*>(done_ctr.data_ptr()), int(e_lo), int(n_local),
                  sh_gate_w.has_value() ? sh_gate_w->data_ptr() : nullptr, optpm<float>(sh_logit), shared_slot ? 1 : 0,
                  reinterpret_cast<int*>(status.data_ptr()), active.data_ptr<int>(), cur_stream()) == 0,
              "moe_route_small: unsupported (tokens <= 64 and <= bn, pairs <= 1024, experts <= 512, k <= 32)");
}

void moe_plan(const Tensor& ids, const Tensor& wts, int64_t e_lo, int64_t n_local, int64_t bn, Tensor& counts,
              Tensor& offsets, Tensor& sorted_token, Tensor& sorted_pair, Tensor& sorted_w, Tensor& tile_group,
              Tensor& tile_tok0, Tensor& tile_ntok, Tensor& meta) {
  c10::cuda::CUDAGuard guard(ids.device());
  TORCH_CHECK(lb::moe_plan_launch(ids.data_ptr<int>(), wts.data_ptr<float>(), int(ids.size(0)), int(ids.size(1)),
                                  int(e_lo), int(n_local), int(bn), counts.data_ptr<int>(), offsets.data_ptr<int>(),
                                  sorted_token.data_ptr<int>(), sorted_pair.data_ptr<int>(),
                                  sorted_w.data_ptr<float>(), tile_group.data_ptr<int>(), tile_tok0.data_ptr<int>(),
                                  tile_ntok.data_ptr<int>(), int(tile_group.numel()), meta.data_ptr<int>(),
                                  cur_stream()) == 0,
              "moe_plan failed");
}

void moe_plan_aligned(const Tensor& ids, const Tensor& wts, int64_t e_lo, int64_t n_local, int64_t bn, int64_t align,
                      Tensor& counts2, Tensor& offsets, Tensor& sorted_token, Tensor& sorted_pair, Tensor& sorted_w,
                      Tensor& tile_group, Tensor& tile_tok0, Tensor& tile_ntok, Tensor& meta) {
  c10::cuda::CUDAGuard guard(ids.device());
  TORCH_CHECK(counts2.numel() >= 2 * n_local && offsets.numel() > n_local && sorted_pair.numel() >= sorted_token.numel() &&
                  sorted_w.numel() >= sorted_token.numel(), "moe_plan_aligned: buffers too small");
  TORCH_CHECK(lb::moe_plan_aligned_launch(ids.data_ptr<int>(), wts.data_ptr<float>(), int(ids.size(0)), int(ids.size(1)),
                                          int(e_lo), int(n_local), int(bn), int(align), counts2.data_ptr<int>(),
                                          offsets.data_ptr<int>(), sorted_token.data_ptr<int>(), sorted_token.numel(),
                                          sorted_pair.data_ptr<int>(), sorted_w.data_ptr<float>(),
                                          tile_group.data_ptr<int>(), tile_tok0.data_ptr<int>(), tile_ntok.data_ptr<int>(),
                                          int(tile_group.numel()), meta.data_ptr<int>(), cur_stream()) == 0,
              "moe_plan_aligned: at most 512 local experts; sorted rows must cover pairs + experts * (align - 1)");
}

void moe_plan_gather(const Tensor& ids, const Tensor& wts, int64_t e_lo, int64_t n_local, int64_t bn, Tensor& counts,
                     Tensor& offsets, Tensor& sorted_token, Tensor& sorted_pair, Tensor& sorted_w, Tensor& tile_group,
                     Tensor& tile_tok0, Tensor& tile_ntok, Tensor& meta, const Tensor& x, Tensor& x_sorted) {
  check_bf16(x, "x");
  check_bf16(x_sorted, "x_sorted");
  c10::cuda::CUDAGuard guard(ids.device());
  TORCH_CHECK(x_sorted.size(0) >= ids.numel() && x_sorted.size(1) == x.size(1), "moe_plan_gather: x_sorted too small");
  TORCH_CHECK(lb::moe_plan_gather_small_launch(
                  ids.data_ptr<int>(), wts.data_ptr<float>(), int(ids.size(0)), int(ids.size(1)), int(e_lo),
                  int(n_local), int(bn), counts.data_ptr<int>(), offsets.data_ptr<int>(),
                  sorted_token.data_ptr<int>(), sorted_pair.data_ptr<int>(), sorted_w.data_ptr<float>(),
                  tile_group.data_ptr<int>(), tile_tok0.data_ptr<int>(), tile_ntok.data_ptr<int>(),
                  int(tile_group.numel()), meta.data_ptr<int>(), x.data_ptr(), x.stride(0), x_sorted.data_ptr(),
                  x_sorted.stride(0), int(x.size(1)), cur_stream()) == 0,
              "moe_plan_gather: at most 1024 pairs and 512 local experts");
}

void gather_rows(const Tensor& src, const Tensor& rows, const Tensor& n_rows, Tensor& dst) {
  check_bf16(src, "src");
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(lb::gather_rows_launch(src.data_ptr(), src.stride(0), rows.data_ptr<int>(), n_rows.data_ptr<int>(),
                                     dst.data_ptr(), dst.stride(0), int(src.size(1)), int(dst.size(0)),
                                     cur_stream()) == 0, "gather_rows failed");
}

void moe_combine(const Tensor& y, const Tensor& ids, int64_t e_lo, int64_t e_hi, const OptT& shared,
                 const OptT& shared_gate, const OptT& residual, Tensor& out, const OptT& norm_w, double eps,
                 double w_offset, const OptT& norm_out) {
  check_bf16(y, "y");
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(norm_w.has_value() == norm_out.has_value(), "moe_combine: norm weight and output go together");
  TORCH_CHECK(lb::moe_combine_launch(y.data_ptr(), y.stride(0), ids.data_ptr<int>(), int(ids.size(1)), int(e_lo),
                                     int(e_hi), shared.has_value() ? shared->data_ptr() : nullptr,
                                     shared.has_value() ? shared->stride(0) : 0, optp<float>(shared_gate),
                                     residual.has_value() ? residual->data_ptr() : nullptr,
                                     residual.has_value() ? residual->stride(0) : 0, out.data_ptr(), out.stride(0),
                                     int(out.size(0)), int(out.size(1)), optp<float>(norm_w), float(eps),
                                     float(w_offset), norm_out.has_value() ? norm_out->data_ptr() : nullptr,
                                     norm_out.has_value() ? norm_out->stride(0) : 0, cur_stream()) == 0,
              "moe_combine failed (hidden % 8 == 0, k <= 32)");
}

void argmax(const Tensor& logits, Tensor& pv, Tensor& pi, Tensor& out, const OptT& out_val) {
  c10::cuda::CUDAGuard guard(logits.device());
  const int rows = int(logits.size(0)), V = int(logits.size(1));
  const int nblk = int(pv.numel() / rows);
  TORCH_CHECK(nblk >= 1, "argmax: partial buffer too small");
  TORCH_CHECK(lb::argmax_launch(logits.data_ptr(), logits.scalar_type() == at::kFloat, logits.stride(0), rows, V,
                                pv.data_ptr<float>(), pi.data_ptr<int>(), nblk, out.data_ptr<int>(),
                                optpm<float>(out_val), cur_stream()) == 0, "argmax failed");
}

void sample(const Tensor& logits, const Tensor& temperature, const OptT& top_k, const OptT& top_p, const OptT& min_p,
            const Tensor& seeds, const OptT& steps, Tensor& scratch, Tensor& out) {
  TORCH_CHECK(logits.scalar_type() == at::kFloat, "sample: logits must be float32");
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(scratch.numel() >= logits.size(0) * logits.size(1), "sample: scratch too small");
  TORCH_CHECK(lb::sample_launch(logits.data_ptr<float>(), logits.stride(0), int(logits.size(0)), int(logits.size(1)),
                                temperature.data_ptr<float>(), optp<int>(top_k), optp<float>(top_p),
                                optp<float>(min_p), reinterpret_cast<const unsigned long long*>(seeds.data_ptr()),
                                optp<int>(steps), scratch.data_ptr<float>(), out.data_ptr<int>(), cur_stream()) == 0,
              "sample failed");
}

void penalties_mask(Tensor& logits, const OptT& counts, const OptT& seen, const OptT& presence, const OptT& frequency,
                    const OptT& repetition, const OptT& mask) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(lb::penalties_mask_launch(logits.data_ptr<float>(), logits.stride(0), int(logits.size(0)),
                                        int(logits.size(1)), optp<int>(counts), optp<unsigned char>(seen),
                                        optp<float>(presence), optp<float>(frequency), optp<float>(repetition),
                                        optp<unsigned int>(mask), mask.has_value() ? int(mask->size(1)) : 0,
                                        cur_stream()) == 0, "penalties_mask failed");
}

}  // namespace

void bind_gdn(pybind11::module_& m);
void bind_comm(pybind11::module_& m);
void bind_quant(pybind11::module_& m);
void bind_ep(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("wgemm", &wgemm, pybind11::arg("w"), pybind11::arg("x"), pybind11::arg("out"), pybind11::arg("residual"),
        pybind11::arg("tok_scale"), pybind11::arg("out_rows"), pybind11::arg("n_feat"), pybind11::arg("dual"),
        pybind11::arg("dual_offset"), pybind11::arg("bn"), pybind11::arg("split_k"), pybind11::arg("ws"),
        pybind11::arg("counters"), pybind11::arg("status"), pybind11::arg("tile_group"), pybind11::arg("tile_tok0"),
        pybind11::arg("tile_ntok"), pybind11::arg("meta"), pybind11::arg("max_tiles"), pybind11::arg("rows_per_group"),
        pybind11::arg("n_tok"), pybind11::arg("out_peer"), pybind11::arg("tile_out0") = pybind11::none(),
        pybind11::arg("w_scales") = pybind11::none(), pybind11::arg("w_gscale") = pybind11::none(),
        pybind11::arg("x_group_col") = 0, pybind11::arg("k_override") = 0);
  m.def("wgemm_fp8", &wgemm_fp8);
  m.def("wgemm_fp8_q", &wgemm_fp8_q);
  m.def("wgemm_allreduce", &wgemm_allreduce);
  m.def("wgemm_allgather", &wgemm_allgather);
  m.def("rmsnorm", &rmsnorm);
  m.def("qk_norm_rope_append", &qk_norm_rope_append);
  m.def("sigmoid_gate", &sigmoid_gate);
  m.def("glu", &glu);
  m.def("embed", &embed);
  m.def("paged_decode", &paged_decode);
  m.def("prefill_attn", &prefill_attn);
  m.def("mla_attn", &mla_attn);
  m.def("mla_prep", &mla_prep);
  m.def("router_topk", &router_topk);
  m.def("moe_route_small", &moe_route_small);
  m.def("moe_plan", &moe_plan);
  m.def("moe_plan_gather", &moe_plan_gather);
  m.def("moe_plan_aligned", &moe_plan_aligned);
  m.def("gather_rows", &gather_rows);
  m.def("moe_combine", &moe_combine);
  m.def("argmax", &argmax);
  m.def("sample", &sample);
  m.def("penalties_mask", &penalties_mask);
  m.def("wgemm_workspace_floats", [](int64_t bn, bool dual, int64_t n_tok_tiles, int64_t feat_tiles, int64_t split_k) {
    return int64_t(lb::wgemm_workspace_floats(int(bn), dual, int(n_tok_tiles), int(feat_tiles), int(split_k)));
  });
  m.def("token_logprobs", [](const Tensor& logits, const Tensor& chosen, int64_t n_top, Tensor& chosen_lp,
                             Tensor& top_ids, Tensor& top_lp) {
    TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.stride(1) == 1, "token_logprobs: float32 logits");
    c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(lb::token_logprobs_launch(logits.data_ptr<float>(), logits.stride(0), int(logits.size(0)),
                                          int(logits.size(1)), chosen.data_ptr<int>(), int(n_top),
                                          chosen_lp.data_ptr<float>(), top_ids.data_ptr<int>(),
                                          top_lp.data_ptr<float>(), cur_stream()) == 0,
                "token_logprobs: at most 20 alternatives");
  });
  m.def("spec_accept", [](const Tensor& target, const Tensor& cu, const Tensor& draft, const Tensor& n_draft,
                          Tensor& accepted, Tensor& bonus, Tensor& any_rejected) {
    c10::cuda::CUDAGuard guard(target.device());
    TORCH_CHECK(draft.dim() == 2 && draft.is_contiguous(), "spec_accept: draft [B, k]");
    TORCH_CHECK(lb::spec_accept_launch(target.data_ptr<int>(), cu.data_ptr<int>(), draft.data_ptr<int>(),
                                       int(draft.size(1)), n_draft.data_ptr<int>(), int(draft.size(0)),
                                       accepted.data_ptr<int>(), bonus.data_ptr<int>(), any_rejected.data_ptr<int>(),
                                       cur_stream()) == 0, "spec_accept failed");
  });
  m.def("set_pdl", [](bool on) { lb::set_pdl(on); });
  m.def("pdl_enabled", []() { return lb::pdl_enabled(); });
  bind_gdn(m);
  bind_comm(m);
  bind_quant(m);
  bind_ep(m);
}
