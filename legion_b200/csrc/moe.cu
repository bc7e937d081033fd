// MoE routing: top-k selection, the expert-major routing plan that drives the grouped GEMM, row
// gather into expert order, and the weighted combine back to token order.
//
// The plan is deterministic: pairs of one expert keep their (token, choice) order, so the grouped
// GEMM and the combine give the same bits run to run.
//
// Counterparts in the reference: src/cuda/fused.cu (router_topk, router_weights, moe_combine,
// shexp_gate), src/cuda/moe_gemm.cu (prep, plan, scatter, reduce).
#include "common.cuh"
#include "ep.h"
#include "kernels.h"

namespace lb {

// One warp per token. mode 0: softmax over all experts -> top-k -> renormalise (optional).
// mode 1: sigmoid scores, selection by score + bias, optional group-limited routing (n_group groups,
// keep topk_group groups ranked by the sum of their two best biased scores), weights = unbiased
// scores of the chosen experts, renormalised and multiplied by route_scale.
template <int MAXE>
__device__ __forceinline__ void router_topk_row(const float* logits, long ldl, const float* __restrict__ bias, int E,
                                                int k, int mode, int renorm, float route_scale, int n_group,
                                                int topk_group, int* __restrict__ ids, float* __restrict__ wts,
                                                int t, int* sm_ids = nullptr, float* sm_wts = nullptr) {
  constexpr int PER = MAXE / 32;
  const int lane = threadIdx.x & 31;
  float sc[PER], sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    sc[j] = (e < E) ? __ldcg(logits + t * ldl + e) : -INFINITY;   // L2 read: the row may come from other CTAs
    mx = fmaxf(mx, sc[j]);
  }
  float inv_sum = 1.f;
  if (mode == 0) {
    // selection by the logits themselves (softmax is monotonic); the partition sum is needed only when the chosen
    // weights are not renormalised
#pragma unroll
    for (int j = 0; j < PER; ++j) sel[j] = sc[j];
    if (!renorm) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) sum += (lane + 32 * j < E) ? __expf(sc[j] - mx) : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      inv_sum = 1.f / sum;
    }
  } else {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        sc[j] = 1.f / (1.f + __expf(-sc[j]));
        sel[j] = sc[j] + (bias ? bias[e] : 0.f);
      } else {
        sc[j] = 0.f;
        sel[j] = -INFINITY;
      }
    }
    if (n_group > 1 && topk_group < n_group) {
      // group score = sum of the two best biased scores in the group; groups are contiguous ranges.
      const int gs = E / n_group;
      float keep_thresh_rank[1];
      (void)keep_thresh_rank;
      // every lane computes all group scores through shared shuffles: loop groups (n_group <= 32)
      float my_gscore = -INFINITY;  // lane g holds the score of group g
      for (int g = 0; g < n_group; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int e = lane + 32 * j;
          if (e < E && e / gs == g) {
            const float v = sel[j];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
          }
        }
        // merge (b1, b2) across lanes
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float o1 = __shfl_xor_sync(0xffffffffu, b1, o);
          const float o2 = __shfl_xor_sync(0xffffffffu, b2, o);
          const float n1 = fmaxf(b1, o1);
          const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
          b1 = n1; b2 = n2;
        }
        if (lane == g) my_gscore = b1 + (b2 == -INFINITY ? 0.f : b2);
      }
      // rank of each group = number of groups with a better score (ties: lower index wins)
      int rank = 0;
      for (int g = 0; g < n_group; ++g) {
        const float og = __shfl_sync(0xffffffffu, my_gscore, g);
        if (lane < n_group && (og > my_gscore || (og == my_gscore && g < lane))) ++rank;
      }
      const unsigned keep_mask = __ballot_sync(0xffffffffu, lane < n_group && rank < topk_group);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        if (e < E && !((keep_mask >> (e / gs)) & 1u)) sel[j] = -INFINITY;
      }
    }
  }
  // Selection: every lane sorts its PER candidates once (bitonic network on packed keys: order-preserving bits of
  // the biased score above, inverted expert index below, so the larger key is the better score and, on equal
  // scores, the lower index), then each of the k rounds is two warp-wide integer maxima over the lanes' heads and
  // a pop on the winning lane: a short dependent chain per round instead of PER compares and ten shuffles.
  unsigned long long key[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    const uint32_t u = __float_as_uint(sel[j]);
    const uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    key[j] = (e < E) ? ((static_cast<unsigned long long>(ord) << 32) | (0xFFFFFFFFu - uint32_t(e))) : 0ull;
  }
#pragma unroll
  for (int k2 = 2; k2 <= PER; k2 <<= 1) {
#pragma unroll
    for (int j2 = k2 >> 1; j2 > 0; j2 >>= 1) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int l = i ^ j2;
        if (l > i) {
          const bool desc = (i & k2) == 0;          // this block ends up descending
          const unsigned long long a = key[i], b = key[l];
          const bool sw = desc ? (a < b) : (a > b);
          key[i] = sw ? b : a;
          key[l] = sw ? a : b;
        }
      }
    }
  }
  int my_id = 0;
  for (int i = 0; i < k; ++i) {
    const uint32_t hi = uint32_t(key[0] >> 32), lo = uint32_t(key[0]);
    const uint32_t ghi = __reduce_max_sync(0xffffffffu, hi);
    const uint32_t glo = __reduce_max_sync(0xffffffffu, hi == ghi ? lo : 0u);
    const int be = int(0xFFFFFFFFu - glo);
    if (lane == (be & 31)) {
#pragma unroll
      for (int j = 0; j + 1 < PER; ++j) key[j] = key[j + 1];
      key[PER - 1] = 0ull;
    }
    if (lane == i) my_id = be;
  }
  // weights of the chosen experts from their logits (lane i < k holds choice i)
  float w = 0.f;
  if (lane < k) {
    const float l = __ldcg(logits + t * ldl + my_id);
    if (mode == 0) w = renorm ? l : __expf(l - mx) * inv_sum;
    else w = 1.f / (1.f + __expf(-l));
  }
  if (mode == 0 && renorm) {
    // softmax followed by renormalisation over the chosen experts = softmax over the chosen logits alone
    const float l0 = __shfl_sync(0xffffffffu, w, 0);      // choice 0 has the largest logit
    w = lane < k ? __expf(w - l0) : 0.f;
  }
  float wsum = w;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
  if (lane < k) {
    if (renorm) w = w / fmaxf(wsum, 6.1e-5f);
    ids[t * k + lane] = my_id;
    wts[t * k + lane] = w * route_scale;
    if (sm_ids) {     // copy for a caller that goes on working on the selection in shared memory
      sm_ids[t * k + lane] = my_id;
      sm_wts[t * k + lane] = w * route_scale;
    }
  }
}

template <int MAXE>
__global__ void __launch_bounds__(128) router_topk_kernel(const float* __restrict__ logits, long ldl,
                                                          const float* __restrict__ bias, int E, int k, int mode,
                                                          int renorm, float route_scale, int n_group, int topk_group,
                                                          int* __restrict__ ids, float* __restrict__ wts, int T) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  router_topk_row<MAXE>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group, topk_group, ids, wts, t);
}

// Decode-sized MoE front end in ONE launch (T <= 64 tokens, T * k <= 1024 pairs):
//   (optional) RMSNorm of the residual stream -> router logits -> top-k -> dense routing tables.
// A CTA owns `epc` consecutive router rows (the shared expert's gate row counts as row E). Per pass of up to 16
// tokens it stages the token rows in shared memory once (normalising them on the way when norm_w is given: warp i
// takes token i; the CTA numbered t mod grid also writes row t of x_normed), then every warp streams one weight
// row from HBM and accumulates its share of the pass's tokens against the staged rows. Staging per CTA instead of
// re-reading the tokens per expert keeps the L2 traffic on the few hot token lines at grid x T rows; with one CTA
// per expert (512 of them) those lines were the bottleneck. The last CTA to finish selects the top-k of every
// token and builds the DENSE routing: every active expert becomes one token tile that covers ALL T tokens (the
// GEMMs are weight-bandwidth bound, so the extra columns are free), which removes the gather: the gate/up GEMM
// reads the activations in place and writes rows slot * bn + t, the down GEMM drops the rows whose out_rows entry
// is -1.
//   tile_group[slot] = expert, slot_base[slot] = slot * bn, tile_ntok[slot] = T, meta = {n_active, n_active * bn}
//   out_rows[slot * bn + t] = pair index t * k + c (or -1), tok_scale[slot * bn + t] = routing weight
constexpr int ROUTE_LSTR = 64 * 512;          // floats between the logit planes of two K splits
constexpr int ROUTE_MAX_KSPLIT = 4;

template <int MAXE>
__global__ void __launch_bounds__(512) moe_route_small_kernel(
    const __nv_bfloat16* __restrict__ x, long ldx, const float* __restrict__ norm_w, float eps, float w_offset,
    __nv_bfloat16* __restrict__ x_normed, long ldn, const __nv_bfloat16* __restrict__ w, long ldw, int H,
    float* logits, const float* __restrict__ bias, int E, int k, int mode, int renorm, float route_scale, int n_group,
    int topk_group, int* ids, float* wts, int T, int bn, int* __restrict__ tile_group, int* __restrict__ slot_base,
    int* __restrict__ tile_ntok, int* __restrict__ meta, int* __restrict__ out_rows, float* __restrict__ tok_scale,
    unsigned int* done_ctr, int e_lo, int n_local, const __nv_bfloat16* __restrict__ sh_gate_w, float* sh_logit,
    int shared_slot, int epc, int tpp, int ksplit, int* status, int* __restrict__ active) {
  extern __shared__ uint4 xs_rows[];          // [tpp][H / 8 / ksplit] this CTA's columns of the pass's token rows
  __shared__ int s_last;
  __shared__ float s_logit[512];
  __shared__ float s_red[16];
  __shared__ unsigned long long s_cand[16 * 32];
  __shared__ int s_wsum[17];
  __shared__ int s_chosen[512];
  __shared__ float s_sel[512];
  __shared__ unsigned s_keep;
  griddep_wait();
  griddep_launch();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nv = H / 8;

  // K split: CTA (rg, ks) owns router rows rg * epc .. and columns ks * H / ksplit .. of them; the partial logits of
  // the splits land in separate planes (LSTR floats apart) and are added in a fixed order by whoever reads them
  const int rg = blockIdx.x / ksplit, ks = blockIdx.x % ksplit, n_rg = gridDim.x / ksplit;
  const int nvs = nv / ksplit, v_lo = ks * nvs;
  const int wpe = 16 / epc;                   // warps per router row
  const int tpw = tpp / wpe;                  // tokens of a pass per warp
  const int e = rg * epc + warp / wpe;
  const int tq = warp % wpe;
  const bool is_gate = e >= E;                // row E: the sigmoid gate of the shared expert
  const bool row_ok = e < E + (sh_gate_w ? 1 : 0);
  const uint4* w4 = reinterpret_cast<const uint4*>(is_gate ? sh_gate_w : w + long(e) * ldw) + v_lo;
  float* lg_out = logits + long(ks) * ROUTE_LSTR;
  for (int base = 0; base < T; base += tpp) {
    if (warp < tpp && base + warp < T) {
      const int t = base + warp;
      const uint4* xr = reinterpret_cast<const uint4*>(x + long(t) * ldx);
      uint4* dst = xs_rows + warp * nvs;
      float ssq = 0.f;
      // with a norm the whole row is read for its sum of squares; only this CTA's columns are kept
      const int r_lo = norm_w ? 0 : v_lo, r_hi = norm_w ? nv : v_lo + nvs;
      for (int v0 = r_lo + lane; v0 < r_hi; v0 += 256) {       // eight loads in flight per lane
        uint4 u[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (v0 + 32 * i < r_hi) u[i] = xr[v0 + 32 * i];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int v = v0 + 32 * i;
          if (v < r_hi) {
            if (v >= v_lo && v < v_lo + nvs) dst[v - v_lo] = u[i];
            if (norm_w) {
              const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const float2 f = __bfloat1622float2(xp[c]);
                ssq += f.x * f.x + f.y * f.y;
              }
            }
          }
        }
      }
      if (norm_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        const float inv = rsqrtf(ssq / float(H) + eps);
        const bool writer = (t % n_rg) == rg;
        __syncwarp();
        for (int v = lane; v < nvs; v += 32) {
          uint4 u = dst[v];
          __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&u);
          const float4 n0 = reinterpret_cast<const float4*>(norm_w)[2 * (v_lo + v)];
          const float4 n1 = reinterpret_cast<const float4*>(norm_w)[2 * (v_lo + v) + 1];
          const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(xp[i]);
            xp[i] = __floats2bfloat162_rn(f.x * inv * (nw[2 * i] + w_offset), f.y * inv * (nw[2 * i + 1] + w_offset));
          }
          dst[v] = u;
          if (writer) reinterpret_cast<uint4*>(x_normed + long(t) * ldn)[v_lo + v] = u;
        }
      }
    }
    __syncthreads();
    if (row_ok) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int v0 = lane; v0 < nvs; v0 += 256) {       // eight weight vectors in flight per lane
        uint4 wu[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (v0 + 32 * i < nvs) wu[i] = w4[v0 + 32 * i];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int v = v0 + 32 * i;
          if (v < nvs) {
            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wu[i]);
            float2 wf[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) wf[c] = __bfloat1622float2(wp[c]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int tok = tq * tpw + j;
              if (j < tpw && base + tok < T) {
                const uint4 xu = xs_rows[tok * nvs + v];
                const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xu);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const float2 xf = __bfloat1622float2(xp[c]);
                  acc[j] = fmaf(wf[c].x, xf.x, acc[j]);
                  acc[j] = fmaf(wf[c].y, xf.y, acc[j]);
                }
              }
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int tok = tq * tpw + j;
        if (j < tpw && base + tok < T) {
          float a = acc[j];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
          if (lane == 0) {
            if (is_gate) sh_logit[ks * 64 + base + tok] = a;
            else lg_out[long(base + tok) * E + e] = a;
          }
        }
      }
    }
    if (lane == 0) __threadfence();   // the writer publishes; the counter is raised after the CTA's barrier
    __syncthreads();
  }
  // ---- every CTA has written its logits: count it in. The CTAs that own tokens (token t belongs to CTA t mod grid)
  // wait for the whole grid (bounded; the grid is far smaller than the number of SMs, so all CTAs are resident),
  // then each selects the top-k of its tokens with all sixteen warps, so the selections of a step run on up to T
  // SMs at once instead of one after the other on the last one.
  const int n_tok_ctas = T < int(gridDim.x) ? T : int(gridDim.x);
  if (tid == 0) {
    __threadfence();
    atomicAdd(&done_ctr[0], 1u);
    s_last = 1;
    if (int(blockIdx.x) < n_tok_ctas) {
      uint64_t t_start = 0;                  // the clock is read only once the wait has lasted a while
      uint32_t spins = 0;
      while (*reinterpret_cast<volatile unsigned int*>(&done_ctr[0]) < gridDim.x) {
        if ((++spins & 0xff) == 0) {
          const uint64_t now = globaltimer_ns();
          if (t_start == 0) t_start = now;
          else if (now - t_start > 2000000000ull) {
            atomicCAS(status, 0, ST_TIMEOUT_FLAG);
            break;
          }
        }
      }
    }
  }
  if (int(blockIdx.x) >= n_tok_ctas) return;
  __syncthreads();
  __threadfence();
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    // thread e holds expert e: score, packed key (score bits above, inverted index below)
    const int e = tid;
    float l = -INFINITY;
    if (e < E) {
      l = __ldcg(logits + long(t) * E + e);
      for (int sp = 1; sp < ksplit; ++sp) l += __ldcg(logits + long(sp) * ROUTE_LSTR + long(t) * E + e);
    }
    float selv = l;
    if (mode == 1) selv = 1.f / (1.f + __expf(-l)) + (bias && e < E ? bias[e] : 0.f);
    s_logit[e] = l;
    if (mode == 1 && n_group > 1 && topk_group < n_group) {
      // group-limited routing: lane g of warp 0 scores group g (the sum of its two best biased scores), the groups
      // are ranked (ties: lower index first) and the experts of the groups that are not kept drop out
      const int gs = E / n_group;
      s_sel[e] = selv;
      __syncthreads();
      if (warp == 0) {
        float gscore = -INFINITY;
        if (lane < n_group) {
          float b1 = -INFINITY, b2 = -INFINITY;
          for (int i = 0; i < gs; ++i) {
            const float v = s_sel[lane * gs + i];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
          }
          gscore = b1 + (b2 == -INFINITY ? 0.f : b2);
        }
        int rank = 0;
        for (int g = 0; g < n_group; ++g) {
          const float og = __shfl_sync(0xffffffffu, gscore, g);
          if (lane < n_group && (og > gscore || (og == gscore && g < lane))) ++rank;
        }
        const unsigned keep = __ballot_sync(0xffffffffu, lane < n_group && rank < topk_group);
        if (lane == 0) s_keep = keep;
      }
      __syncthreads();
      if (e < E && !((s_keep >> (e / gs)) & 1u)) selv = -INFINITY;
    }
    float mxv = 0.f, inv_sum = 1.f;
    if (mode == 0 && !renorm) {
      // softmax weights without renormalisation need the partition sum over all experts
      float m = l;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (lane == 0) s_red[warp] = m;
      __syncthreads();
      mxv = s_red[0];
      for (int i = 1; i < 16; ++i) mxv = fmaxf(mxv, s_red[i]);
      __syncthreads();
      float sm = e < E ? __expf(l - mxv) : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
      if (lane == 0) s_red[warp] = sm;
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < 16; ++i) tot += s_red[i];
      inv_sum = 1.f / tot;
    }
    const uint32_t u = __float_as_uint(selv);
    const uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    uint32_t khi = e < E ? ord : 0u, klo = e < E ? 0xFFFFFFFFu - uint32_t(e) : 0u;
    // the warp's own best k, in order (lane i keeps choice i)
    uint32_t mhi = 0u, mlo = 0u;
    for (int i = 0; i < k; ++i) {
      const uint32_t ghi = __reduce_max_sync(0xffffffffu, khi);
      const uint32_t glo = __reduce_max_sync(0xffffffffu, khi == ghi ? klo : 0u);
      if (khi == ghi && klo == glo) { khi = 0u; klo = 0u; }
      if (lane == i) { mhi = ghi; mlo = glo; }
    }
    s_cand[warp * 32 + lane] = (static_cast<unsigned long long>(mhi) << 32) | mlo;
    __syncthreads();
    if (warp == 0) {
      // merge of the sixteen sorted lists: lane l < 16 walks list l
      int ptr = 0;
      unsigned long long head = lane < 16 ? s_cand[lane * 32] : 0ull;
      int my_id = 0;
      for (int i = 0; i < k; ++i) {
        const uint32_t hi = uint32_t(head >> 32), lo = uint32_t(head);
        const uint32_t ghi = __reduce_max_sync(0xffffffffu, hi);
        const uint32_t glo = __reduce_max_sync(0xffffffffu, hi == ghi ? lo : 0u);
        if (hi == ghi && lo == glo && lane < 16) {
          ++ptr;
          head = ptr < k ? s_cand[lane * 32 + ptr] : 0ull;
        }
        if (lane == i) my_id = int(0xFFFFFFFFu - glo);
      }
      float w = 0.f;
      if (lane < k) {
        const float lg = s_logit[my_id];
        if (mode == 0) w = renorm ? lg : __expf(lg - mxv) * inv_sum;
        else w = 1.f / (1.f + __expf(-lg));
      }
      if (mode == 0 && renorm) {
        const float l0 = __shfl_sync(0xffffffffu, w, 0);
        w = lane < k ? __expf(w - l0) : 0.f;
      }
      float wsum = w;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
      if (lane < k) {
        if (renorm) w = w / fmaxf(wsum, 6.1e-5f);
        ids[t * k + lane] = my_id;
        wts[t * k + lane] = w * route_scale;
      }
    }
    __syncthreads();
  }
  // ---- dense routing tables, indexed by local expert: rows e * bn + t of the intermediate belong to expert e and
  // token t. Each token CTA writes its token's column of out_rows / tok_scale (pair index t * k + c where the
  // token chose the expert, -1 elsewhere) and marks the experts it chose as active.
  const int P = T * k;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    s_chosen[tid] = -1;
    __syncthreads();
    if (tid < k) {
      const int e = ids[t * k + tid];                   // written by this CTA above
      s_chosen[e] = t * k + tid;
      s_logit[e] = wts[t * k + tid];
    }
    __syncthreads();
    const int local = tid - e_lo;
    if (tid < E && local >= 0 && local < n_local) {
      const int pr = s_chosen[tid];
      out_rows[local * bn + t] = pr;
      if (pr >= 0) {
        tok_scale[local * bn + t] = s_logit[tid];
        active[local] = 1;
      }
    }
    if (shared_slot && tid == 0) {
      // the shared expert (stacked behind this rank's routed experts as group n_local) is used by every token:
      // its output rows are the pairs P .. P + T - 1, weighted by the sigmoid of its gate (or 1)
      out_rows[n_local * bn + t] = P + t;
      float gl = 0.f;
      if (sh_gate_w)
        for (int sp = 0; sp < ksplit; ++sp) gl += __ldcg(&sh_logit[sp * 64 + t]);
      tok_scale[n_local * bn + t] = sh_gate_w ? 1.f / (1.f + __expf(-gl)) : 1.f;
    }
    __syncthreads();
  }
  // ---- the last token CTA to finish compacts the active experts into the tile list
  if (tid == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(&done_ctr[1], 1u);
    s_last = (old == unsigned(n_tok_ctas) - 1u);
    if (s_last) {
      done_ctr[0] = 0;
      done_ctr[1] = 0;
    }
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int act = tid < n_local ? __ldcg(active + tid) : 0;
  if (tid < n_local) active[tid] = 0;                   // ready for the next step
  const unsigned bal = __ballot_sync(0xffffffffu, act != 0);
  if (lane == 0) s_wsum[warp] = __popc(bal);
  __syncthreads();
  int before = 0, n_active = 0;
  for (int i = 0; i < 16; ++i) {
    if (i < warp) before += s_wsum[i];
    n_active += s_wsum[i];
  }
  if (act) {
    const int slot = before + __popc(bal & ((1u << lane) - 1));
    tile_group[slot] = tid;
    slot_base[slot] = tid * bn;
    tile_ntok[slot] = T;
  }
  if (tid == 0) {
    if (shared_slot) {
      tile_group[n_active] = n_local;
      slot_base[n_active] = n_local * bn;
      tile_ntok[n_active] = T;
    }
    const int n_slots = n_active + (shared_slot ? 1 : 0);
    meta[0] = n_slots;
    meta[1] = n_slots * bn;
  }
}

int moe_route_small_launch(const void* x, long ldx, const float* norm_w, float eps, float w_offset, void* x_normed,
                           long ldn, const void* w, long ldw, int H, float* logits, const float* bias, int E, int k,
                           int mode, int renorm, float route_scale, int n_group, int topk_group, int* ids, float* wts,
                           int T, int bn, int* tile_group, int* slot_base, int* tile_ntok, int* meta, int* out_rows,
                           float* tok_scale, unsigned int* done_ctr, int e_lo, int n_local, const void* sh_gate_w,
                           float* sh_logit, int shared_slot, int* status, int* active, cudaStream_t s) {
  if (T <= 0) return 0;
  if (k > 32 || E > 512 || n_group > 32 || H % 8 || T > 64 || T * k > 1024 || T > bn) return 1;
  if (sh_gate_w && (!sh_logit || !shared_slot)) return 1;
  auto sg = static_cast<const __nv_bfloat16*>(sh_gate_w);
  auto xb = static_cast<const __nv_bfloat16*>(x);
  auto xn = static_cast<__nv_bfloat16*>(x_normed);
  auto wb = static_cast<const __nv_bfloat16*>(w);
  const int epc = E >= 256 ? 8 : 4;                              // router rows per CTA
  // wide models: the columns are split over CTAs too, so that the weight stream and the staging of the token rows
  // spread over four times as many SMs (the logit and gate buffers hold ROUTE_MAX_KSPLIT planes)
  const int ksplit = (H >= 4096 && (H / 8) % ROUTE_MAX_KSPLIT == 0) ? ROUTE_MAX_KSPLIT : 1;
  const int Hs = H / ksplit;
  const int tpp = size_t(16) * Hs * 2 <= 192 * 1024 ? 16 : 8;    // tokens staged per pass
  if (size_t(tpp) * Hs * 2 > 200 * 1024) return 1;
  const int smem = tpp * Hs * 2;
  const int grid = ((E + (sh_gate_w ? 1 : 0) + epc - 1) / epc) * ksplit;
#define LB_ROUTE(MAXE)                                                                                              \
  {                                                                                                                 \
    static int smem_set = 0;                                                                                        \
    if (smem > smem_set) {                                                                                          \
      if (cudaFuncSetAttribute(moe_route_small_kernel<MAXE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=  \
          cudaSuccess)                                                                                              \
        return 1;                                                                                                   \
      smem_set = smem;                                                                                              \
    }                                                                                                               \
    launch_pdl(moe_route_small_kernel<MAXE>, dim3(grid), dim3(512), smem, s, xb, ldx, norm_w, eps, w_offset, xn,   \
               ldn, wb, ldw, H, logits, bias, E, k, mode, renorm, route_scale, n_group, topk_group, ids, wts, T,    \
               bn, tile_group, slot_base, tile_ntok, meta, out_rows, tok_scale, done_ctr, e_lo, n_local, sg,        \
               sh_logit, shared_slot, epc, tpp, ksplit, status, active);                                                    \
  }
  if (E <= 128) LB_ROUTE(128)
  else if (E <= 256) LB_ROUTE(256)
  else LB_ROUTE(512)
#undef LB_ROUTE
  return cudaGetLastError() != cudaSuccess;
}

int router_topk_launch(const float* logits, long ldl, const float* bias, int E, int k, int mode, int renorm,
                       float route_scale, int n_group, int topk_group, int* ids, float* wts, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  if (k > 32 || E > 512 || n_group > 32) return 1;
  const int blocks = (T * 32 + 127) / 128;
  if (E <= 128)
    router_topk_kernel<128><<<blocks, 128, 0, s>>>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group,
                                                   topk_group, ids, wts, T);
  else if (E <= 256)
    router_topk_kernel<256><<<blocks, 128, 0, s>>>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group,
                                                   topk_group, ids, wts, T);
  else
    router_topk_kernel<512><<<blocks, 128, 0, s>>>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group,
                                                   topk_group, ids, wts, T);
  return cudaGetLastError() != cudaSuccess;
}

// ---------------------------------------------------------------------------------------------
// routing plan
// ---------------------------------------------------------------------------------------------
// pass 1: one CTA per local expert counts its pairs.
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ ids, int n_pairs, int e_lo,
                                                        int* __restrict__ counts) {
  const int e = e_lo + blockIdx.x;
  int c = 0;
  for (int p = threadIdx.x; p < n_pairs; p += 256) c += (ids[p] == e);
  __shared__ int red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 8; ++i) t += red[i];
    counts[blockIdx.x] = t;
  }
}
// pass 2: one CTA scans the counts: row offsets per expert and the token-tile list (tile = up to bn
// consecutive sorted rows of one expert). meta = {n_tiles, n_rows}.
__global__ void __launch_bounds__(512) moe_scan_kernel(const int* __restrict__ counts, int n_local, int bn,
                                                       int* __restrict__ offsets, int* __restrict__ tile_group,
                                                       int* __restrict__ tile_tok0, int* __restrict__ tile_ntok,
                                                       int max_tiles, int* __restrict__ meta) {
  __shared__ int s_cnt[512], s_off[513], s_toff[513];
  const int e = threadIdx.x;
  s_cnt[e] = (e < n_local) ? counts[e] : 0;
  __syncthreads();
  if (e == 0) {
    int o = 0, to = 0;
    for (int i = 0; i < n_local; ++i) {
      s_off[i] = o;
      s_toff[i] = to;
      o += s_cnt[i];
      to += (s_cnt[i] + bn - 1) / bn;
    }
    s_off[n_local] = o;
    s_toff[n_local] = to;
    meta[0] = to < max_tiles ? to : max_tiles;
    meta[1] = o;
  }
  __syncthreads();
  if (e < n_local) {
    offsets[e] = s_off[e];
    const int nt = (s_cnt[e] + bn - 1) / bn;
    for (int i = 0; i < nt; ++i) {
      const int ti = s_toff[e] + i;
      if (ti < max_tiles) {
        tile_group[ti] = e;
        tile_tok0[ti] = s_off[e] + i * bn;
        tile_ntok[ti] = min(bn, s_cnt[e] - i * bn);
      }
    }
  }
  if (e == 0) offsets[n_local] = s_off[n_local];
}
// pass 3: one CTA per local expert writes its pairs, in pair order, at its offset.
__global__ void __launch_bounds__(256) moe_fill_kernel(const int* __restrict__ ids, const float* __restrict__ wts,
                                                       int n_pairs, int k, int e_lo, const int* __restrict__ offsets,
                                                       int* __restrict__ sorted_token, int* __restrict__ sorted_pair,
                                                       float* __restrict__ sorted_w) {
  const int e = e_lo + blockIdx.x;
  const int base0 = offsets[blockIdx.x];
  __shared__ int warp_tot[8];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int p0 = 0; p0 < n_pairs; p0 += 256) {
    const int p = p0 + threadIdx.x;
    const bool hit = p < n_pairs && ids[p] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(bal & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(bal);
    __syncthreads();
    int wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
    const int base = running;
    if (hit) {
      const int dst = base0 + base + wbase + before;
      sorted_token[dst] = p / k;
      sorted_pair[dst] = p;
      sorted_w[dst] = wts[p];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int w = 0; w < 8; ++w) t += warp_tot[w];
      running = base + t;
    }
    __syncthreads();
  }
}

int moe_plan_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn, int* counts,
                    int* offsets, int* sorted_token, int* sorted_pair, float* sorted_w, int* tile_group,
                    int* tile_tok0, int* tile_ntok, int max_tiles, int* meta, cudaStream_t s) {
  if (n_local <= 0 || n_local > 512) return 1;
  const int n_pairs = n_tokens * k;
  moe_count_kernel<<<n_local, 256, 0, s>>>(ids, n_pairs, e_lo, counts);
  moe_scan_kernel<<<1, 512, 0, s>>>(counts, n_local, bn, offsets, tile_group, tile_tok0, tile_ntok, max_tiles, meta);
  moe_fill_kernel<<<n_local, 256, 0, s>>>(ids, wts, n_pairs, k, e_lo, offsets, sorted_token, sorted_pair, sorted_w);
  return cudaGetLastError() != cudaSuccess;
}

// Prompt-sized steps: histogram, scan and scatter with atomics instead of one pass over all pairs per expert. The
// rows of an expert are contiguous and start on a multiple of `align` rows (the block-scaled 4-bit GEMM needs its
// token tiles on scale-atom boundaries); rows between two segments have sorted_token = -1. The order of the rows
// inside a segment is whatever the atomics give: every row's result lands in its own pair row, so nothing
// downstream depends on it.
__global__ void __launch_bounds__(256) moe_hist_kernel(const int* __restrict__ ids, int n_pairs, int e_lo, int n_local,
                                                       int* __restrict__ counts) {
  __shared__ int h[512];
  for (int i = threadIdx.x; i < n_local; i += 256) h[i] = 0;
  __syncthreads();
  for (int p = blockIdx.x * 256 + threadIdx.x; p < n_pairs; p += gridDim.x * 256) {
    const int e = ids[p] - e_lo;
    if (unsigned(e) < unsigned(n_local)) atomicAdd(&h[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_local; i += 256)
    if (h[i]) atomicAdd(&counts[i], h[i]);
}
__global__ void __launch_bounds__(512) moe_scan_aligned_kernel(const int* __restrict__ counts, int n_local, int bn,
                                                               int align, int* __restrict__ offsets,
                                                               int* __restrict__ tile_group, int* __restrict__ tile_tok0,
                                                               int* __restrict__ tile_ntok, int max_tiles,
                                                               int* __restrict__ meta) {
  __shared__ int w_rows[16], w_tiles[16];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  const int c = e < n_local ? counts[e] : 0;
  const int rows = (c + align - 1) / align * align;
  const int nt = (c + bn - 1) / bn;
  int ir = rows, it = nt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, ir, d), b = __shfl_up_sync(0xffffffffu, it, d);
    if (lane >= d) { ir += a; it += b; }
  }
  if (lane == 31) { w_rows[warp] = ir; w_tiles[warp] = it; }
  __syncthreads();
  int br = 0, bt = 0;
  for (int w = 0; w < warp; ++w) { br += w_rows[w]; bt += w_tiles[w]; }
  const int off = br + ir - rows, toff = bt + it - nt;
  if (e < n_local) {
    offsets[e] = off;
    for (int i = 0; i < nt; ++i) {
      const int ti = toff + i;
      if (ti < max_tiles) {
        tile_group[ti] = e;
        tile_tok0[ti] = off + i * bn;
        tile_ntok[ti] = min(bn, c - i * bn);
      }
    }
  }
  if (e == 511) {
    offsets[n_local] = br + ir;
    meta[0] = min(bt + it, max_tiles);
    meta[1] = br + ir;
  }
}
__global__ void __launch_bounds__(256) moe_scatter_kernel(const int* __restrict__ ids, const float* __restrict__ wts,
                                                          int n_pairs, int k, int e_lo, int n_local,
                                                          const int* __restrict__ offsets, int* __restrict__ cursor,
                                                          int* __restrict__ sorted_token, int* __restrict__ sorted_pair,
                                                          float* __restrict__ sorted_w) {
  const int p = blockIdx.x * 256 + threadIdx.x;
  if (p >= n_pairs) return;
  const int e = ids[p] - e_lo;
  if (unsigned(e) >= unsigned(n_local)) return;
  const int dst = offsets[e] + atomicAdd(&cursor[e], 1);
  sorted_token[dst] = p / k;
  sorted_pair[dst] = p;
  sorted_w[dst] = wts[p];
}

int moe_plan_aligned_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn, int align,
                            int* counts2, int* offsets, int* sorted_token, long sorted_rows, int* sorted_pair,
                            float* sorted_w, int* tile_group, int* tile_tok0, int* tile_ntok, int max_tiles, int* meta,
                            cudaStream_t s) {
  if (n_local <= 0 || n_local > 512 || align <= 0 || bn <= 0) return 1;
  const int n_pairs = n_tokens * k;
  if (sorted_rows < long(n_pairs) + long(n_local) * (align - 1)) return 1;
  cudaMemsetAsync(counts2, 0, sizeof(int) * 2 * n_local, s);
  cudaMemsetAsync(sorted_token, 0xff, sizeof(int) * sorted_rows, s);
  if (n_pairs > 0) {
    const int hgrid = min(296, (n_pairs + 255) / 256);
    moe_hist_kernel<<<hgrid, 256, 0, s>>>(ids, n_pairs, e_lo, n_local, counts2);
  }
  moe_scan_aligned_kernel<<<1, 512, 0, s>>>(counts2, n_local, bn, align, offsets, tile_group, tile_tok0, tile_ntok,
                                            max_tiles, meta);
  if (n_pairs > 0)
    moe_scatter_kernel<<<(n_pairs + 255) / 256, 256, 0, s>>>(ids, wts, n_pairs, k, e_lo, n_local, offsets,
                                                             counts2 + n_local, sorted_token, sorted_pair, sorted_w);
  return cudaGetLastError() != cudaSuccess;
}

// Decode-sized steps (at most 1024 pairs): the whole plan AND the row gather in ONE launch. Every CTA rebuilds
// the plan in shared memory (a few hundred comparisons per thread - cheaper than three more launches and their
// dependencies), CTA 0 publishes it, and all CTAs then copy their share of the rows into expert order. The
// result is bit-identical to the count / scan / fill / gather sequence.
__global__ void __launch_bounds__(512) moe_plan_gather_small_kernel(
    const int* __restrict__ ids, const float* __restrict__ wts, int n_pairs, int k, int e_lo, int n_local, int bn,
    int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ sorted_token,
    int* __restrict__ sorted_pair, float* __restrict__ sorted_w, int* __restrict__ tile_group,
    int* __restrict__ tile_tok0, int* __restrict__ tile_ntok, int max_tiles, int* __restrict__ meta,
    const __nv_bfloat16* __restrict__ x, long ldx, __nv_bfloat16* __restrict__ x_sorted, long ldxs, int H) {
  __shared__ int s_ids[1024], s_tok[1024], s_cnt[512], s_off[513], s_toff[513];
  const int tid = threadIdx.x;
  const bool pub = blockIdx.x == 0;
  const int bn_shift = 31 - __clz(bn);   // bn is a power of two
  for (int p = tid; p < n_pairs; p += 512) s_ids[p] = ids[p];
  __syncthreads();
  const int e = e_lo + tid;
  int c = 0;
  if (tid < n_local)
    for (int p = 0; p < n_pairs; ++p) c += (s_ids[p] == e);
  s_cnt[tid] = c;
  __syncthreads();
  // exclusive scans of the counts and of the tile counts: warp 0, 16 experts per lane + shuffle scan
  if (tid < 32) {
    int o = 0, to = 0;
    const int e0 = tid * 16;
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const int cc = (e0 + i < n_local) ? s_cnt[e0 + i] : 0;
      o += cc;
      to += (cc + bn - 1) >> bn_shift;
    }
    int io = o, ito = to;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, io, d), b = __shfl_up_sync(0xffffffffu, ito, d);
      if (tid >= d) { io += a; ito += b; }
    }
    int xo = io - o, xto = ito - to;     // exclusive prefixes of this lane's 16 experts
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      if (e0 + i <= n_local) { s_off[e0 + i] = xo; s_toff[e0 + i] = xto; }
      const int cc = (e0 + i < n_local) ? s_cnt[e0 + i] : 0;
      xo += cc;
      xto += (cc + bn - 1) >> bn_shift;
    }
    if (tid == 31) { s_off[n_local] = io; s_toff[n_local] = ito; }
    if (pub && tid == 31) {
      meta[0] = ito < max_tiles ? ito : max_tiles;
      meta[1] = io;
      offsets[n_local] = io;
    }
  }
  __syncthreads();
  if (tid < n_local) {
    int pos = s_off[tid];
    if (c > 0) {
      for (int p = 0; p < n_pairs; ++p) {
        if (s_ids[p] == e) {
          const int t = p / k;
          s_tok[pos] = t;
          if (pub) {
            sorted_token[pos] = t;
            sorted_pair[pos] = p;
            sorted_w[pos] = wts[p];
          }
          ++pos;
        }
      }
    }
    if (pub) {
      counts[tid] = c;
      offsets[tid] = s_off[tid];
      const int nt = (c + bn - 1) >> bn_shift;
      for (int i = 0; i < nt; ++i) {
        const int ti = s_toff[tid] + i;
        if (ti < max_tiles) {
          tile_group[ti] = tid;
          tile_tok0[ti] = s_off[tid] + i * bn;
          tile_ntok[ti] = min(bn, c - i * bn);
        }
      }
    }
  }
  __syncthreads();
  const int n_rows = s_off[n_local];
  for (int i = blockIdx.x; i < n_rows; i += gridDim.x) {
    const uint4* s4 = reinterpret_cast<const uint4*>(x + long(s_tok[i]) * ldx);
    uint4* d4 = reinterpret_cast<uint4*>(x_sorted + long(i) * ldxs);
    for (int j = tid; j < H / 8; j += 512) d4[j] = s4[j];
  }
}

int moe_plan_gather_small_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn,
                                 int* counts, int* offsets, int* sorted_token, int* sorted_pair, float* sorted_w,
                                 int* tile_group, int* tile_tok0, int* tile_ntok, int max_tiles, int* meta,
                                 const void* x, long ldx, void* x_sorted, long ldxs, int H, cudaStream_t s) {
  const int n_pairs = n_tokens * k;
  if (n_local <= 0 || n_local > 512 || n_pairs > 1024 || n_pairs <= 0 || H % 8 || (bn & (bn - 1))) return 1;
  moe_plan_gather_small_kernel<<<n_pairs, 512, 0, s>>>(
      ids, wts, n_pairs, k, e_lo, n_local, bn, counts, offsets, sorted_token, sorted_pair, sorted_w, tile_group,
      tile_tok0, tile_ntok, max_tiles, meta, static_cast<const __nv_bfloat16*>(x), ldx,
      static_cast<__nv_bfloat16*>(x_sorted), ldxs, H);
  return cudaGetLastError() != cudaSuccess;
}

int moe_tiles_launch(const int* counts, int n_local, int bn, int* offsets, int* tile_group, int* tile_tok0,
                     int* tile_ntok, int max_tiles, int* meta, cudaStream_t s) {
  if (n_local <= 0 || n_local > 512) return 1;
  moe_scan_kernel<<<1, 512, 0, s>>>(counts, n_local, bn, offsets, tile_group, tile_tok0, tile_ntok, max_tiles, meta);
  return cudaGetLastError() != cudaSuccess;
}

// dst[i, :] = src[rows[i], :] for i < *n_rows (device scalar); 16-byte vectors.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long lds, const int* __restrict__ rows,
                                   const int* __restrict__ n_rows, __nv_bfloat16* __restrict__ dst, long ldd, int H) {
  const int n = *n_rows;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int r = rows[i];
    if (r < 0) continue;                      // a padding row between two aligned segments
    const uint4* s4 = reinterpret_cast<const uint4*>(src + long(r) * lds);
    uint4* d4 = reinterpret_cast<uint4*>(dst + long(i) * ldd);
    for (int j = threadIdx.x; j < H / 8; j += blockDim.x) d4[j] = s4[j];
  }
}

int gather_rows_launch(const void* src, long lds, const int* rows, const int* n_rows, void* dst, long ldd, int H,
                       int max_rows, cudaStream_t s) {
  if (max_rows <= 0) return 0;
  if (H % 8) return 1;
  const int grid = max_rows < 4096 ? max_rows : 4096;
  gather_rows_kernel<<<grid, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(src), lds, rows, n_rows,
                                          static_cast<__nv_bfloat16*>(dst), ldd, H);
  return cudaGetLastError() != cudaSuccess;
}

// out[t, :] = (residual[t, :]) + sum_j y[t*k + j, :] (rows whose expert is outside [e_lo, e_hi) are skipped)
//             + shared[t, :] * (shared_gate ? sigmoid(shared_gate[t]) : 1)
// and, when norm_out is given, norm_out[t, :] = rmsnorm(out[t, :]) * (norm_w + w_offset): the next layer's input
// norm rides on the combine instead of a launch of its own. One CTA per token; the k row loads of a vector are
// issued together (the expert ids sit in shared memory) and summed in choice order, so the result is deterministic.
__global__ void __launch_bounds__(256) moe_combine_kernel(
    const __nv_bfloat16* __restrict__ y, long ldy, const int* __restrict__ ids, int k, int e_lo, int e_hi,
    const __nv_bfloat16* __restrict__ shared, long lds, const float* __restrict__ shared_gate,
    const __nv_bfloat16* __restrict__ residual, long ldr, __nv_bfloat16* __restrict__ out, long ldo, int H,
    const float* __restrict__ norm_w, float eps, float w_offset, __nv_bfloat16* __restrict__ norm_out, long ldn) {
  __shared__ int s_on[32];
  __shared__ float red[8];
  griddep_wait();
  griddep_launch();
  const long t = blockIdx.x;
  if (threadIdx.x < k) {
    const int e = ids[t * k + threadIdx.x];
    s_on[threadIdx.x] = (e >= e_lo && e < e_hi);
  }
  __syncthreads();
  float sg = 1.f;
  if (shared && shared_gate) sg = 1.f / (1.f + __expf(-shared_gate[t]));
  float ss = 0.f;
  for (int v = threadIdx.x; v < H / 8; v += 256) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int c0 = 0; c0 < k; c0 += 4) {
      uint4 u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        u[i] = make_uint4(0u, 0u, 0u, 0u);
        if (c0 + i < k && s_on[c0 + i]) u[i] = reinterpret_cast<const uint4*>(y + (t * k + c0 + i) * ldy)[v];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(u2[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    if (shared) {
      const uint4 u = reinterpret_cast<const uint4*>(shared + t * lds)[v];
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(u2[j]);
        acc[2 * j] += f.x * sg;
        acc[2 * j + 1] += f.y * sg;
      }
    }
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual + t * ldr)[v];
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(u2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      const float2 f = __bfloat1622float2(o2[j]);
      ss += f.x * f.x + f.y * f.y;
    }
    reinterpret_cast<uint4*>(out + t * ldo)[v] = o;
  }
  if (!norm_out) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / float(H) + eps);
  for (int v = threadIdx.x; v < H / 8; v += 256) {
    uint4 u = reinterpret_cast<const uint4*>(out + t * ldo)[v];   // written by this thread above
    __nv_bfloat162* u2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(u2[j]);
      u2[j] = __floats2bfloat162_rn(f.x * inv * (norm_w[v * 8 + 2 * j] + w_offset),
                                    f.y * inv * (norm_w[v * 8 + 2 * j + 1] + w_offset));
    }
    reinterpret_cast<uint4*>(norm_out + t * ldn)[v] = u;
  }
}

int moe_combine_launch(const void* y, long ldy, const int* ids, int k, int e_lo, int e_hi, const void* shared, long lds,
                       const float* shared_gate, const void* residual, long ldr, void* out, long ldo, int T, int H,
                       const float* norm_w, float eps, float w_offset, void* norm_out, long ldn, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || k > 32) return 1;
  return launch_pdl(moe_combine_kernel, dim3(T), dim3(256), 0, s, static_cast<const __nv_bfloat16*>(y), ldy, ids, k,
                    e_lo, e_hi, static_cast<const __nv_bfloat16*>(shared), lds, shared_gate,
                    static_cast<const __nv_bfloat16*>(residual), ldr, static_cast<__nv_bfloat16*>(out), ldo, H, norm_w,
                    eps, w_offset, static_cast<__nv_bfloat16*>(norm_out), ldn) != cudaSuccess;
}

}  // namespace lb
