// C entry points of the sm_100a kernels. Every launcher takes raw device pointers and a stream,
// returns 0 on success and 1 on a host-side failure (tw_last_error() has the message). None of
// them allocates device memory or synchronises.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* tw_last_error();

// ---- GEMM (gemm_tcgen05.cu) ----
int tw_gemm_bf16(const void* A, long long lda, const void* B, long long ldb, long long rows_b, void* C,
                 long long ldc, const void* bias, const float* row_scale, int M, int N, int K, int swiglu,
                 int up_row_offset, const int* tile_expert, const int* num_m_tiles_dev, int n_per_expert,
                 int max_ctas, int plan_hint, uint32_t* status, cudaStream_t stream);
int tw_gemm_bf16_grouped256(const void* A, long long lda, const void* B, long long ldb, long long rows_b, void* C,
                            long long ldc, const float* row_scale, int M, int N, int K, int swiglu, int up_row_offset,
                            const int* tile_expert, const int* num_m_tiles_dev, int n_per_expert, int max_ctas,
                            uint32_t* status, cudaStream_t stream);
int tw_gemm_set_tile_override(int bn);
int tw_gemm_set_kernel_override(int kind);

// ---- norms (norm.cu) ----
int tw_rmsnorm(const void* x, void* out, const void* w, int T, int H, long long ldx, long long ldo, float eps,
               int max_ctas, cudaStream_t stream);
int tw_rmsnorm_copy(void* x, void* residual_out, const void* w, int T, int H, long long ldx, long long ldr,
                    float eps, int max_ctas, cudaStream_t stream);
int tw_add_rmsnorm(void* x, void* residual, const void* w, int T, int H, long long ldx, long long ldr,
                   float eps, int max_ctas, cudaStream_t stream);

// ---- element-wise (elementwise.cu) ----
int tw_rope_kv_write(void* qkv, long long ld, const int* positions, const int* slots, const float* cos_sin,
                     void* k_cache, void* v_cache, int T, int hq, int hkv, int D, int write_k_back,
                     cudaStream_t stream);
int tw_rope_kv_write_qknorm(void* qkv, long long ld, const int* positions, const int* slots, const float* cos_sin,
                            void* k_cache, void* v_cache, int T, int hq, int hkv, int D, int write_k_back,
                            const void* q_norm_w, const void* k_norm_w, float eps, cudaStream_t stream);
int tw_swiglu(const void* x, long long ldx, void* out, long long ldo, int T, int d, cudaStream_t stream);
int tw_embedding(const int* ids, const void* table, void* out, long long ldo, int T, int H, int vocab_start,
                 int vocab_end, cudaStream_t stream);
int tw_argmax(const float* logits, long long ld, int* out, int rows, int V, cudaStream_t stream);

// ---- sampling (sampling.cu) ----
// params: `rows` records of 32 bytes {float temperature (<= 0: greedy), int top_k (<= 0: off), float top_p,
// float min_p, uint64 seed, uint64 pad}; out: sampled token id per row.
int tw_sample(const float* logits, long long ld, int rows, int V, const void* params, int* out, cudaStream_t stream);

// ---- fp8 (e4m3) path (gemm_tcgen05.cu, quant_fp8.cu) ----
int tw_gemm_fp8(const void* A, long long lda, const void* B, long long ldb, long long rows_b, void* C,
                long long ldc, const void* bias, const float* row_scale, const float* col_scale, int M, int N,
                int K, int swiglu, int up_row_offset, const int* tile_expert, const int* num_m_tiles_dev,
                int n_per_expert, int max_ctas, int plan_hint, uint32_t* status, cudaStream_t stream);
int tw_gemm_int8(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, const void* bias,
                 const float* row_scale, const float* col_scale, int M, int N, int K, int swiglu, int max_ctas,
                 int plan_hint, uint32_t* status, cudaStream_t stream);
int tw_quant_fp8(const void* x, long long ldx, void* out, long long ldo, float* scales, int T, int H, int dynamic,
                 int max_ctas, cudaStream_t stream);
int tw_rmsnorm_quant_fp8(const void* x, void* residual, const void* w, void* out, long long ldo, float* scales,
                         int T, int H, long long ldx, long long ldr, float eps, int dynamic, int max_ctas,
                         cudaStream_t stream);

// ---- activations, KV page copy / swap, partial-attention merge (misc_ops.cu) ----
// kind: 0 silu*mul, 1 gelu*mul, 2 gelu_tanh*mul, 3 mul*silu, 4 fatrelu*mul (param = threshold),
//       5 gelu_new, 6 gelu_fast, 7 gelu_quick, 8 gelu, 9 silu (kinds >= 5 are unary: x is [T, d])
int tw_activation(const void* x, long long ldx, void* out, long long ldo, int T, int d, int kind, float param,
                  cudaStream_t stream);
int tw_copy_pages(void* cache, long long page_bytes, const long long* pairs_dev, int n_pairs, cudaStream_t stream);
int tw_swap_pages(const void* src, void* dst, long long page_bytes, const long long* pairs_host, int n_pairs,
                  cudaStream_t stream);
int tw_merge_attn_states(void* out, float* out_lse, const void* a_out, const float* a_lse, const void* b_out,
                         const float* b_lse, int T, int H, int D, cudaStream_t stream);

// ---- int8 quantisation (quant_fp8.cu) and cache utilities (cache_ops.cu) ----
int tw_quant_int8(const void* x, long long ldx, void* out, long long ldo, float* scales, int T, int H, int dynamic,
                  int max_ctas, cudaStream_t stream);
int tw_rmsnorm_quant_int8(const void* x, void* residual, const void* w, void* out, long long ldo, float* scales,
                          int T, int H, long long ldx, long long ldr, float eps, int dynamic, int max_ctas,
                          cudaStream_t stream);
int tw_gather_cache(const void* cache, void* dst, const int* block_table, const int* cu_seq, int batch,
                    int max_blocks, int page, int row_elems, cudaStream_t stream);
int tw_convert_fp8(const void* src, void* dst, long long n, float scale, int to_fp8, cudaStream_t stream);
int tw_permute_cols(const void* in, void* out, const int* perm, int rows, int cols, long long ld_in,
                    long long ld_out, cudaStream_t stream);

// ---- attention (attn_prefill.cu, attn_decode.cu) ----
int tw_attn_prefill(const void* q, long long ldq, int T, const void* k_cache, const void* v_cache,
                    int num_blocks, int page, void* out, long long ldo, const int* cu_q, const int* kv_lens,
                    const int* block_table, int max_blocks, const int* tile_seq, const int* tile_q0,
                    int num_tiles, int hq, int hkv, int D, float scale, int max_ctas, int window, float softcap,
                    uint32_t* status, cudaStream_t stream);
int tw_attn_set_variant(int variant);
int tw_attn_set_ring(int slots);
int tw_attn_decode(const void* q, long long ldq, const void* k_cache, const void* v_cache, int page, void* out,
                   long long ldo, const int* tok_row, const int* tok_seq, const int* tok_kvlen, int n_tok,
                   const int* block_table, int max_blocks, int hq, int hkv, int D, float scale, int splits,
                   float* part_o, float* part_ml, int window, float softcap, cudaStream_t stream);

int tw_attn_decode_merge(const float* part_o, const float* part_ml, const int* tok_row, int n_tok, int hq, int D,
                         int splits, void* out, long long ldo, cudaStream_t stream);
// tensor-core variant for grouped-query models with head size 128 (attn_decode_tc.cu)
int tw_attn_decode_tc(const void* q, long long ldq, const void* k_cache, const void* v_cache, int num_blocks,
                      int page, void* out, long long ldo, const int* tok_row, const int* tok_seq,
                      const int* tok_kvlen, int n_tok, const int* block_table, int max_blocks, int hq, int hkv,
                      int D, float scale, int splits, float* part_o, float* part_ml, uint32_t* status,
                      cudaStream_t stream);
int tw_attn_decode_tc_persistent(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                                 int num_blocks, int page, void* out, long long ldo, const int* tok_row,
                                 const int* tok_seq, const int* tok_kvlen, int n_tok, const int* block_table,
                                 int max_blocks, int hq, int hkv, int D, float scale, int splits, float* part_o,
                                 float* part_ml, int max_ctas, uint32_t* status, cudaStream_t stream);

// ---- mixture of experts (moe.cu) ----
int tw_moe_router(const void* x, long long ldx, const void* wg, float* topk_w, int* topk_ids, float* logits_out,
                  int T, int H, int E, int topk, int renormalize, cudaStream_t stream);
int tw_moe_align(const int* topk_ids, int n_pairs, int E, int tile_rows, int* expert_offsets,
                 int* expert_cursor, int* tile_expert, int max_tiles, int* meta, cudaStream_t stream);
int tw_moe_scatter(const void* x, long long ldx, const int* topk_ids, const float* topk_w,
                   const int* expert_offsets, int* expert_cursor, void* a_sorted, float* row_scale,
                   int* sorted_pos, int n_pairs, int topk, int H, int E, cudaStream_t stream);
int tw_moe_combine(const void* y, const int* sorted_pos, void* out, long long ldo, int T, int topk, int H,
                   cudaStream_t stream);

// ---- in-kernel collectives (comm_fused.cu) ----
// mc_base: multicast address of the symmetric buffer or NULL (peer transport). peer_bases /
// signal_pads: device arrays of `world` pointers. mode: 0 fused RS+add+norm+AG, 1 without the
// all-gather, 2 three-phase "simple fusion".
int tw_fused_rs_norm_ag(void* mc_base, void* const* peer_bases, uint32_t* const* signal_pads, int rank,
                        int world, int channel_base, unsigned long long budget_ns, uint32_t* status,
                        long long off_bytes, void* residual, long long ldr, const void* weight, int T, int H,
                        float eps, int max_ctas, int mode, int rows_in_flight, cudaStream_t stream);
// op: 0 all-reduce, 1 reduce-scatter, 2 all-gather.
int tw_collective(void* mc_base, void* const* peer_bases, uint32_t* const* signal_pads, int rank, int world,
                  int channel_base, unsigned long long budget_ns, uint32_t* status, long long off_bytes,
                  long long n_bytes, int op, int max_ctas, cudaStream_t stream);
int tw_oneshot_allreduce(void* const* peer_bases, uint32_t* const* signal_pads, int rank, int world,
                         int channel_base, unsigned long long budget_ns, uint32_t* status, long long off_bytes,
                         long long n_bytes, void* out, int max_ctas, cudaStream_t stream);
int tw_wait_probe(uint32_t* flag, unsigned long long budget_ns, uint32_t* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
