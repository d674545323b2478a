// Token sampling from fp32 logits in ONE launch for the whole batch: temperature, top-k, top-p, min-p
// and the random draw, one CTA per row, no sort and no host round trip.
//
// The reference samples with a full sort of every row plus softmax / cumsum / scatter passes and one
// generator call per seeded request (vllm/v1/sample/ops/topk_topp_sampler.py:170-262,
// vllm/v1/sample/sampler.py:17-270). Here the support is described by ONE threshold on the scaled
// logit: the k-th largest value comes from a 4-pass radix select on the float bits (counts), the
// top-p boundary from a 4-pass radix select weighted by exp(x - max) (the smallest value whose
// ascending cumulative mass exceeds 1 - top_p, the reference's rule), min-p is max + log(min_p).
// The draw is the Gumbel / exponential race argmax(x_i + g_i) over the kept set, with g_i from a
// counter-based generator keyed by (row seed, token index), so a seeded request repeats exactly.
// The row (0.5 MB for a 128 K vocabulary) is re-read from L2 in every pass.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int SAMPLE_THREADS = 1024;

struct SampleRowParams {   // one per row, 32 bytes
  float temperature;       // <= 0: greedy
  int top_k;               // <= 0 or >= V: disabled
  float top_p;             // >= 1: disabled
  float min_p;             // <= 0: disabled
  unsigned long long seed;
  unsigned long long pad;
};

__device__ __forceinline__ uint32_t sortable_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float gumbel_noise(unsigned long long seed, int i) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * static_cast<unsigned long long>(i + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  const float u = (static_cast<float>(z >> 40) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1)
  return -__logf(-__logf(u));
}

__device__ __forceinline__ float block_max_f(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float x = scratch[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const SampleRowParams* __restrict__ params,
              int* __restrict__ out) {
  __shared__ float scratch[32];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ int hist_i[256];
  __shared__ float hist_f[256];
  __shared__ uint32_t s_prefix;
  __shared__ float s_remaining;
  __shared__ int s_k;

  const int row = blockIdx.x;
  const float* x = logits + row * ld;
  const SampleRowParams p = params[row];
  const bool greedy = !(p.temperature > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / p.temperature;

  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) m = fmaxf(m, x[i] * inv_t);
  m = block_max_f(m, scratch);

  uint32_t tau = 0u;                       // keep keys >= tau
  if (!greedy && p.top_k > 0 && p.top_k < V) {
    if (threadIdx.x == 0) {
      s_prefix = 0u;
      s_k = p.top_k;
    }
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = threadIdx.x; b < 256; b += SAMPLE_THREADS) hist_i[b] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = (shift == 24) ? 0u : (0xffffffffu << (shift + 8));
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
        const uint32_t key = sortable_key(x[i] * inv_t);
        if ((key & mask) == prefix) atomicAdd(&hist_i[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int k = s_k, b = 255;
        for (; b > 0; --b) {
          if (hist_i[b] >= k) break;
          k -= hist_i[b];
        }
        s_k = k;
        s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      }
      __syncthreads();
    }
    tau = s_prefix;
  }
  if (!greedy && p.top_p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
      const float xi = x[i] * inv_t;
      if (sortable_key(xi) >= tau) z += __expf(xi - m);
    }
    float zz[1] = {z};
    block_sum<1>(zz, scratch);
    if (threadIdx.x == 0) {
      s_prefix = 0u;
      s_remaining = (1.f - p.top_p) * zz[0];
    }
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = threadIdx.x; b < 256; b += SAMPLE_THREADS) hist_f[b] = 0.f;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = (shift == 24) ? 0u : (0xffffffffu << (shift + 8));
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
        const float xi = x[i] * inv_t;
        const uint32_t key = sortable_key(xi);
        if (key >= tau && (key & mask) == prefix) atomicAdd(&hist_f[(key >> shift) & 255u], __expf(xi - m));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        float rem = s_remaining;
        int b = 0, last = 0;
        for (; b < 256; ++b) {
          if (hist_f[b] > 0.f) last = b;
          if (hist_f[b] > rem) break;       // ascending cumulative mass crosses 1 - top_p inside this bin
          rem -= hist_f[b];
        }
        if (b == 256) {                     // rounding left nothing to cross: the highest occupied bin
          b = last;
          rem = 0.f;
        }
        s_remaining = rem;
        s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      }
      __syncthreads();
    }
    tau = max(tau, s_prefix);
  }
  // min-p comes last, as in the reference: p_i >= min_p * p_max  <=>  x_i >= max + log(min_p)
  if (!greedy && p.min_p > 0.f) tau = max(tau, sortable_key(m + __logf(p.min_p)));

  // the draw: argmax of x_i + gumbel_i over the kept set (plain argmax when greedy), lowest index on ties
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float xi = x[i] * inv_t;
    if (sortable_key(xi) < tau) continue;
    const float v = greedy ? xi : xi + gumbel_noise(p.seed, i);
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane];
    best_i = s_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) out[row] = (best_i == 0x7fffffff) ? 0 : best_i;
  }
}

}  // namespace tw

using namespace tw;

// params: `rows` records of 32 bytes {float temperature, int top_k, float top_p, float min_p, u64 seed, u64 pad}.
extern "C" int tw_sample(const float* logits, long long ld, int rows, int V, const void* params, int* out,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) {
    set_last_error("sample: empty vocabulary");
    return 1;
  }
  sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, reinterpret_cast<const SampleRowParams*>(params),
                                                     out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("sample launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
