// Single-query ("decode") attention over the paged KV cache, split along the keys.
//
// Used for requests that contribute one (or a few) query tokens to a step; long query runs go to
// the tensor-core prefill kernel. The op is bandwidth-bound (every key and value row is read once
// for all query heads that share the KV head), so it is plain SIMT: replaces the paged-attention
// v1/v2 kernels and the decode path of the FlashAttention call in the reference
// (csrc/attention/attention_kernels.cuh:84-110,502-600, vllm/v1/attention/backends/flash_attn.py:713-733).
//
// Grid (token, kv head, split). A warp takes 32 keys at a time:
//   scores : lane k owns key k -> dot products with the G query heads of the group (q in shared
//            memory as fp32, broadcast reads)
//   values : lane d owns D/32 output columns -> for each of the 32 keys the probability is
//            shuffled from its owner lane and the value row is read coalesced
// Warps merge through shared memory; splits merge in a second kernel.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int DEC_GMAX = 8;
constexpr int DEC_WARPS = 4;

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ tok_row,
                   const int* __restrict__ tok_seq, const int* __restrict__ tok_kvlen,
                   const int* __restrict__ block_table, int max_blocks, int page, int hq, int hkv,
                   float scale_log2, int splits, __nv_bfloat16* __restrict__ out, long long ldo,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int window, float softcap_log2) {
  // window: the query (at position kv_len - 1) sees the last `window` keys only (0: all of them).
  // softcap_log2: soft cap of the scores times log2(e) (0: off); scores here are already in the log2 domain.
  constexpr int EPL = D / 32;  // output elements per lane
  const int G = hq / hkv;
  const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = tok_row[tok];
  const int seq = tok_seq[tok];
  const int kv_len = tok_kvlen[tok];
  const int* table = block_table + static_cast<long long>(seq) * max_blocks;

  __shared__ float q_s[DEC_GMAX][D];
  __shared__ float red_o[DEC_WARPS][DEC_GMAX][D];
  __shared__ float red_m[DEC_WARPS][DEC_GMAX];
  __shared__ float red_l[DEC_WARPS][DEC_GMAX];

  for (int i = threadIdx.x; i < DEC_GMAX * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    q_s[g][d] = (g < G) ? __bfloat162float(q[row * ldq + (kvh * G + g) * D + d]) * scale_log2 : 0.f;
  }
  __syncthreads();

  // keys of this split, in whole 32-key chunks (under a sliding window the chunks before it are skipped)
  const int key_lo = window > 0 ? max(0, kv_len - window) : 0;
  const int chunk_lo = key_lo / 32;
  const int chunks_total = (kv_len + 31) / 32;
  const int chunks_per_split = (chunks_total - chunk_lo + splits - 1) / splits;
  const int chunk_begin = chunk_lo + split * chunks_per_split;
  const int chunk_end = min(chunks_total, chunk_begin + chunks_per_split);
  const float cap_inv = softcap_log2 > 0.f ? 1.f / softcap_log2 : 0.f;

  float m[DEC_GMAX], l[DEC_GMAX], o[DEC_GMAX][EPL];
#pragma unroll
  for (int g = 0; g < DEC_GMAX; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[g][e] = 0.f;
  }

  for (int ch = chunk_begin + warp; ch < chunk_end; ch += DEC_WARPS) {
    const int key = ch * 32 + lane;
    const bool valid = key < kv_len && key >= key_lo;
    long long row_off = 0;  // element offset of this lane's key row inside the caches
    if (valid) {
      const int blk = table[key / page];
      row_off = ((static_cast<long long>(blk) * page + key % page) * hkv + kvh) * D;
    }
    float s[DEC_GMAX];
#pragma unroll
    for (int g = 0; g < DEC_GMAX; ++g) s[g] = 0.f;
    if (valid) {
      const uint4* kr = reinterpret_cast<const uint4*>(k_cache + row_off);
#pragma unroll 8
      for (int v = 0; v < D / 8; ++v) {
        const uint4 kv = kr[v];
        const uint32_t* ku = reinterpret_cast<const uint32_t*>(&kv);
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(ku[j]);
          kf[2 * j] = f.x;
          kf[2 * j + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < DEC_GMAX; ++g) {
#pragma unroll
          for (int j = 0; j < 8; ++j) s[g] += q_s[g][v * 8 + j] * kf[j];
        }
      }
    }
    // online softmax over this chunk (per query head)
    float pr[DEC_GMAX];
#pragma unroll
    for (int g = 0; g < DEC_GMAX; ++g) {
      float sv = s[g];
      if (softcap_log2 > 0.f) sv = softcap_log2 * tanhf(sv * cap_inv);
      sv = valid ? sv : -INFINITY;
      const float mc = warp_max(sv);
      const float mn = fmaxf(m[g], mc);
      const float alpha = exp2f(m[g] - mn);  // 0 on the first chunk (m = -inf)
      m[g] = mn;
      pr[g] = valid ? exp2f(sv - mn) : 0.f;
      l[g] = l[g] * alpha + pr[g];  // per-lane partial sum; reduced at the end
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[g][e] *= alpha;
    }
    // values: eight value rows are requested before the first is used, so that a warp keeps 2 KB of
    // loads in flight instead of one 256-byte row (one dependent load per key left the kernel at a
    // seventh of the memory bandwidth)
    const int n_keys = min(32, kv_len - ch * 32);
    auto accumulate = [&](uint2 vv, int kk) {
      float vf[EPL];
      const float2 a = unpack_bf16x2(vv.x);
      vf[0] = a.x;
      vf[1] = a.y;
      if (EPL == 4) {
        const float2 b = unpack_bf16x2(vv.y);
        vf[2] = b.x;
        vf[3] = b.y;
      }
#pragma unroll
      for (int g = 0; g < DEC_GMAX; ++g) {
        const float pg = __shfl_sync(0xffffffffu, pr[g], kk);
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[g][e] += pg * vf[e];
      }
    };
    auto load_row = [&](int kk) {
      const long long off = __shfl_sync(0xffffffffu, row_off, kk);
      uint2 vv = make_uint2(0u, 0u);
      if (EPL == 4) vv = *reinterpret_cast<const uint2*>(v_cache + off + lane * 4);
      else vv.x = *reinterpret_cast<const uint32_t*>(v_cache + off + lane * 2);
      return vv;
    };
    int kk = 0;
    for (; kk + 8 <= n_keys; kk += 8) {
      uint2 vv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) vv[u] = load_row(kk + u);
#pragma unroll
      for (int u = 0; u < 8; ++u) accumulate(vv[u], kk + u);
    }
    for (; kk < n_keys; ++kk) accumulate(load_row(kk), kk);
  }

  // merge the warps of the CTA
#pragma unroll
  for (int g = 0; g < DEC_GMAX; ++g) {
    l[g] = warp_sum(l[g]);
    if (lane == 0) {
      red_m[warp][g] = m[g];
      red_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) red_o[warp][g][lane * EPL + e] = o[g][e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w][g]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float a = (red_m[w][g] == -INFINITY) ? 0.f : exp2f(red_m[w][g] - mm);
      acc += red_o[w][g][d] * a;
      ll += red_l[w][g] * a;
    }
    const int h = kvh * G + g;
    if (splits == 1) {
      out[row * ldo + h * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      const long long pidx = (static_cast<long long>(tok) * hq + h) * splits + split;
      part_o[pidx * D + d] = acc;
      if (d == 0) {
        part_ml[pidx * 2] = mm;
        part_ml[pidx * 2 + 1] = ll;
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(D)
attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         const int* __restrict__ tok_row, int hq, int splits,
                         __nv_bfloat16* __restrict__ out, long long ldo) {
  const int tok = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const long long base = (static_cast<long long>(tok) * hq + h) * splits;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float acc = 0.f, ll = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    acc += part_o[(base + s) * D + d] * a;
    ll += part_ml[(base + s) * 2 + 1] * a;
  }
  out[tok_row[tok] * ldo + h * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
}

}  // namespace tw

using namespace tw;

// Reduction of split-KV partial results (also used by the tensor-core decode kernel).
extern "C" int tw_attn_decode_merge(const float* part_o, const float* part_ml, const int* tok_row, int n_tok,
                                    int hq, int D, int splits, void* out, long long ldo, cudaStream_t stream) {
  if (n_tok <= 0 || splits <= 1) return 0;
  auto ob = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 128)
    attn_decode_merge_kernel<128><<<dim3(n_tok, hq), 128, 0, stream>>>(part_o, part_ml, tok_row, hq, splits, ob, ldo);
  else if (D == 64)
    attn_decode_merge_kernel<64><<<dim3(n_tok, hq), 64, 0, stream>>>(part_o, part_ml, tok_row, hq, splits, ob, ldo);
  else {
    set_last_error("attn_decode_merge: head_dim must be 64 or 128 (got %d)", D);
    return 1;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_decode_merge launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

// part_o: [n_tok, hq, splits, D] fp32, part_ml: [n_tok, hq, splits, 2] fp32 (used when splits > 1).
extern "C" int tw_attn_decode(const void* q, long long ldq, const void* k_cache, const void* v_cache, int page,
                              void* out, long long ldo, const int* tok_row, const int* tok_seq,
                              const int* tok_kvlen, int n_tok, const int* block_table, int max_blocks,
                              int hq, int hkv, int D, float scale, int splits, float* part_o,
                              float* part_ml, int window, float softcap, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  const float softcap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  if ((D != 128 && D != 64) || hkv <= 0 || hq <= 0 || hq % hkv != 0 || hq / hkv > DEC_GMAX) {
    set_last_error("attn_decode: unsupported shape (D=%d, hq=%d, hkv=%d)", D, hq, hkv);
    return 1;
  }
  if (splits < 1) splits = 1;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) {
    set_last_error("attn_decode: split-KV needs the partial-result workspace");
    return 1;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_tok, hkv, splits);
  auto qb = reinterpret_cast<const __nv_bfloat16*>(q);
  auto kb = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  auto vb = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  auto ob = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 128) {
    attn_decode_kernel<128><<<grid, DEC_WARPS * 32, 0, stream>>>(qb, ldq, kb, vb, tok_row, tok_seq, tok_kvlen,
                                                                 block_table, max_blocks, page, hq, hkv,
                                                                 scale_log2, splits, ob, ldo, part_o, part_ml, window, softcap_log2);
    if (splits > 1)
      attn_decode_merge_kernel<128><<<dim3(n_tok, hq), 128, 0, stream>>>(part_o, part_ml, tok_row, hq, splits,
                                                                         ob, ldo);
  } else {
    attn_decode_kernel<64><<<grid, DEC_WARPS * 32, 0, stream>>>(qb, ldq, kb, vb, tok_row, tok_seq, tok_kvlen,
                                                                block_table, max_blocks, page, hq, hkv,
                                                                scale_log2, splits, ob, ldo, part_o, part_ml, window, softcap_log2);
    if (splits > 1)
      attn_decode_merge_kernel<64><<<dim3(n_tok, hq), 64, 0, stream>>>(part_o, part_ml, tok_row, hq, splits,
                                                                       ob, ldo);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_decode launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (see tw_noalloc.h): the split-KV partial results go to a fixed array in
// the library's device data segment instead of a caller-provided workspace.
#include <mutex>

#include "tw_noalloc.h"

namespace tw {

constexpr size_t NOALLOC_SCRATCH_FLOATS = TW_NOALLOC_SCRATCH_BYTES / sizeof(float);
constexpr int NOALLOC_MAX_DEVICES = 64;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_decode_scratch[NOALLOC_SCRATCH_FLOATS];

static float* g_scratch_addr[NOALLOC_MAX_DEVICES] = {nullptr};
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device; looked up once per device.
static int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    set_last_error("attn_decode_noalloc: cannot identify the current device (%s)", cudaGetErrorString(e));
    return 1;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error("attn_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                     cudaGetErrorString(e));
      return 1;
    }
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace tw

extern "C" int tw_attn_decode_noalloc(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                                      int page, void* out, long long ldo, const int* tok_row,
                                      const int* tok_seq, const int* tok_kvlen, int n_tok,
                                      const int* block_table, int max_blocks, int hq, int hkv, int D,
                                      float scale, int splits, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  const int window = 0;               // full causal attention, no soft cap
  const float softcap_log2 = 0.f;
  if ((D != 128 && D != 64) || hkv <= 0 || hq <= 0 || hq % hkv != 0 || hq / hkv > DEC_GMAX) {
    set_last_error("attn_decode_noalloc: unsupported shape (D=%d, hq=%d, hkv=%d)", D, hq, hkv);
    return 1;
  }
  if (splits < 1) splits = 1;
  const unsigned long long partials = static_cast<unsigned long long>(n_tok) * hq * splits;
  const unsigned long long need = partials * (static_cast<unsigned long long>(D) + 2ull);
  if (need > NOALLOC_SCRATCH_FLOATS) {
    set_last_error("attn_decode_noalloc: %llu tokens x heads x splits need %llu bytes of scratch, the built-in "
                   "array holds %u; lower `splits` or the batch, or use tw_attn_decode with your own workspace",
                   partials, need * 4ull, TW_NOALLOC_SCRATCH_BYTES);
    return 1;
  }
  float* scratch = nullptr;
  if (noalloc_scratch(&scratch) != 0) return 1;
  float* part_o = scratch;
  float* part_ml = scratch + partials * D;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_tok, hkv, splits);
  auto qb = reinterpret_cast<const __nv_bfloat16*>(q);
  auto kb = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  auto vb = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  auto ob = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 128) {
    attn_decode_kernel<128><<<grid, DEC_WARPS * 32, 0, stream>>>(qb, ldq, kb, vb, tok_row, tok_seq, tok_kvlen,
                                                                 block_table, max_blocks, page, hq, hkv,
                                                                 scale_log2, splits, ob, ldo, part_o, part_ml, window, softcap_log2);
    if (splits > 1)
      attn_decode_merge_kernel<128><<<dim3(n_tok, hq), 128, 0, stream>>>(part_o, part_ml, tok_row, hq, splits,
                                                                         ob, ldo);
  } else {
    attn_decode_kernel<64><<<grid, DEC_WARPS * 32, 0, stream>>>(qb, ldq, kb, vb, tok_row, tok_seq, tok_kvlen,
                                                                block_table, max_blocks, page, hq, hkv,
                                                                scale_log2, splits, ob, ldo, part_o, part_ml, window, softcap_log2);
    if (splits > 1)
      attn_decode_merge_kernel<64><<<dim3(n_tok, hq), 64, 0, stream>>>(part_o, part_ml, tok_row, hq, splits,
                                                                       ob, ldo);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_decode_noalloc launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
