// Shared definitions of the prefill attention kernels (attn_prefill.cu, attn_prefill_split.cu).
#pragma once

#include "tw_common.cuh"

namespace tw {

constexpr int ATT_BM = 128;      // query rows per CTA
constexpr int ATT_BN = 128;      // keys per tile
constexpr int ATT_SOFTMAX_THREADS = 256;
constexpr int ATT_THREADS = 64 + ATT_SOFTMAX_THREADS;
constexpr int ATT_HALF_BYTES = 128 * 128;  // a [128 rows x 64 bf16] swizzled half tile

// 2^x in one MUFU instruction (ex2.approx with flush-to-zero; exp2f() without fast-math wraps the same
// instruction in range fix-ups that cost four more issue slots per element). Inputs here are <= 8 or -inf.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnParams {
  __nv_bfloat16* out;
  long long ldo;
  const int* cu_q;         // [B+1] first query row of each sequence
  const int* kv_lens;      // [B] keys visible to the last query of the sequence
  const int* block_table;  // [B, max_blocks]
  const int* tile_seq;     // [num_tiles] sequence of each query tile
  const int* tile_q0;      // [num_tiles] first query (within the sequence) of the tile
  int max_blocks;
  int page;                // tokens per cache page
  int hq, hkv;
  int ring;                // head-pair kernel: K/V tile slots in use
  float scale_log2;        // softmax scale * log2(e)
  int window;              // sliding window: a query at position p sees keys (p - window, p]; 0 = unlimited
  float softcap;           // logits soft cap: s -> cap * tanh(s / cap) on the scaled scores; 0 = off
  float scale;             // softmax scale (needed with the soft cap)
  uint32_t* status;
};

// Kernel of attn_prefill_split.cu: persistent CTAs, one query head per work item, the item's key range
// split between the two softmax groups. max_ctas bounds the grid (0 = every SM).
int launch_prefill_split(int D, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                         const AttnParams& p, int num_tiles, int max_ctas, cudaStream_t stream);

}  // namespace tw
