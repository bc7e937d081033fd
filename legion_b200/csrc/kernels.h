// C++ launch interface of the non-GEMM kernels. Pointers are device pointers; every function
// returns 0 on success and enqueues on the given stream without synchronising.
#pragma once
#include <cuda_runtime.h>

namespace lb {

int rmsnorm_launch(const void* x, long ldx, const void* res_in, long ldri, void* res_out, long ldro, const float* w,
                   void* y, long ldy, int rows, int H, float eps, float w_offset, cudaStream_t s);

int qk_norm_rope_append_launch(const void* qkv, long ld_qkv, int q_head_stride, int k_off, int v_off, const float* qw,
                               const float* kw, float eps, float w_offset, const float* cos_sin, int rot,
                               const int* positions, const long* slots, void* q_out, void* k_cache, void* v_cache,
                               long cache_cell_stride, int T, int Hq, int Hkv, int D, cudaStream_t s);

int sigmoid_gate_launch(const void* attn, const void* qkv, long ld_qkv, int q_head_stride, int D, int Hq, void* out,
                        long T, cudaStream_t s);

int glu_launch(const void* x, long ldx, void* out, long ldo, int F, long T, int act, cudaStream_t s);

int embed_launch(const int* ids, const void* table, long ldt, void* out, long ldo, int T, int H, int vocab,
                 cudaStream_t s);

int paged_decode_launch(const void* q, const void* k_cache, const void* v_cache, long cell_stride,
                        const int* block_table, int table_width, int page, const int* ctx_lens, float scale, int window,
                        int B, int Hq, int Hkv, int D, int n_splits, float* o_part, float* ml_part, void* out,
                        cudaStream_t s);

int attn_combine_launch(const float* o_part, const float* ml_part, int n_splits, int rows, int D, void* out,
                        cudaStream_t s);

int paged_decode_tc_launch(const void* q, const void* k_cache, const void* v_cache, long n_cells, long cell_stride,
                           const int* block_table, int table_width, int page, const int* ctx_lens, float scale,
                           int window, int B, int Hq, int Hkv, int D, int n_splits, float* o_part, float* ml_part,
                           void* out, int* group_ctr, int n_group_ctr, int* status, cudaStream_t s);
const char* paged_decode_tc_last_error();

int prefill_attn_launch(const void* q, long T, const void* k_cache, const void* v_cache, long n_cells,
                        long cell_stride, const int* cu_q, const int* ctx_lens, const int* block_table,
                        int table_width, int page, int n_seqs, int max_q_len, int Hq, int Hkv, int D, float scale,
                        int window, int causal, void* out, int* status, cudaStream_t s);
const char* prefill_attn_last_error();

// Latent attention (absorbed form) over the paged latent cache: attn_mla_sm100.cu
int mla_attn_launch(const void* q_abs, long T, const void* cache, long n_cells, long cell_stride, const int* cu_q,
                    const int* ctx_lens, const int* block_table, int table_width, int page, int n_seqs,
                    int max_q_len, int nh, float scale, int n_splits, float* o_part, float* ml_part, void* out,
                    int* status, cudaStream_t s);
const char* mla_attn_last_error();
int mla_prep_launch(const void* kva, long ld_kva, const float* norm_w, float eps, float w_offset, const void* q,
                    long ld_q_tok, int q_head_stride, int q_pe_off, int nh, const float* cos_sin,
                    const int* positions, const long* slots, void* cache, long cell_stride, void* q_abs, int T,
                    cudaStream_t s);

int router_topk_launch(const float* logits, long ldl, const float* bias, int E, int k, int mode, int renorm,
                       float route_scale, int n_group, int topk_group, int* ids, float* wts, int T, cudaStream_t s);

int moe_route_small_launch(const void* x, long ldx, const float* norm_w, float eps, float w_offset, void* x_normed,
                           long ldn, const void* w, long ldw, int H, float* logits, const float* bias, int E, int k,
                           int mode, int renorm, float route_scale, int n_group, int topk_group, int* ids, float* wts,
                           int T, int bn, int* tile_group, int* slot_base, int* tile_ntok, int* meta, int* out_rows,
                           float* tok_scale, unsigned int* done_ctr, int e_lo, int n_local, const void* sh_gate_w, float* sh_logit,
                           int shared_slot, int* status, int* active, cudaStream_t s);
int moe_plan_gather_small_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn,
                                 int* counts, int* offsets, int* sorted_token, int* sorted_pair, float* sorted_w,
                                 int* tile_group, int* tile_tok0, int* tile_ntok, int max_tiles, int* meta,
                                 const void* x, long ldx, void* x_sorted, long ldxs, int H, cudaStream_t s);
int moe_plan_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn, int* counts,
                    int* offsets, int* sorted_token, int* sorted_pair, float* sorted_w, int* tile_group,
                    int* tile_tok0, int* tile_ntok, int max_tiles, int* meta, cudaStream_t s);
// Prompt-sized steps: histogram / scan / scatter with atomics; segments start on multiples of `align` rows, padding
// rows carry sorted_token = -1, the order inside a segment is unspecified. counts2: 2 * n_local ints of scratch.
int moe_plan_aligned_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn, int align,
                            int* counts2, int* offsets, int* sorted_token, long sorted_rows, int* sorted_pair,
                            float* sorted_w, int* tile_group, int* tile_tok0, int* tile_ntok, int max_tiles, int* meta,
                            cudaStream_t s);

int gather_rows_launch(const void* src, long lds, const int* rows, const int* n_rows, void* dst, long ldd, int H,
                       int max_rows, cudaStream_t s);

// Mamba-2 state-space recurrence + silu(z) gate (mamba2.cu). 256 % hd == 0, hd a power of two, ds divisible by
// 256 / hd with at most 32 columns per thread; returns 1 for other shapes.
int mamba2_scan_launch(const void* xbc, long ldx, const void* dt_raw, long lddt, const void* z, long ldz, const float* A,
                       const float* D, const float* dt_bias, float* state, const int* cu_seq, const int* slots,
                       int n_seqs, int nh, int hd, int ng, int ds, void* y, long ldy, int write_state, cudaStream_t s);

// Device-side expert cache step (residency.cu): marks the routed experts, loads the missing ones from mapped host
// memory into the coldest slots and rewrites the routing in slot numbers, all in one launch. ctl: 3 zeroed words,
// stats: {hits, misses, bytes, steps}, miss_list: 2 * n_slots ints of scratch.
int expert_cache_prepare_launch(const int* ids, int n_pairs, int E, int n_slots, int* slot_of, int* expert_in, float* heat,
                                float decay, const void* host_gu, const void* host_dn, void* slot_gu, void* slot_dn,
                                long gu_bytes, long dn_bytes, int* ids_slot, int* miss_list, unsigned int* ctl,
                                unsigned long long* stats, int* status, cudaStream_t s);

int moe_combine_launch(const void* y, long ldy, const int* ids, int k, int e_lo, int e_hi, const void* shared, long lds,
                       const float* shared_gate, const void* residual, long ldr, void* out, long ldo, int T, int H,
                       const float* norm_w, float eps, float w_offset, void* norm_out, long ldn, cudaStream_t s);

int argmax_launch(const void* logits, bool is_f32, long ld, int rows, int V, float* pv, int* pi, int nblk, int* out,
                  float* out_val, cudaStream_t s);

int sample_launch(const float* logits, long ld, int rows, int V, const float* temperature, const int* top_k,
                  const float* top_p, const float* min_p, const unsigned long long* seeds, const int* steps,
                  float* scratch, int* out, cudaStream_t s);

int penalties_mask_launch(float* logits, long ld, int rows, int V, const int* counts, const unsigned char* seen,
                          const float* presence, const float* frequency, const float* repetition,
                          const unsigned int* mask, int mask_words, cudaStream_t s);

int token_logprobs_launch(const float* logits, long ld, int rows, int V, const int* chosen, int n_top,
                          float* chosen_lp, int* top_ids, float* top_lp, cudaStream_t s);
int spec_accept_launch(const int* target, const int* cu, const int* draft, int max_draft, const int* n_draft, int B,
                       int* accepted, int* bonus, int* any_rejected, cudaStream_t s);

}  // namespace lb
