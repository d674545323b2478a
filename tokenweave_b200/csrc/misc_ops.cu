// Small memory-bound kernels off the bf16 Llama/Qwen2/Mixtral hot path: gated and plain activations
// other than SwiGLU, KV-cache page copy / swap, and the merge of two partial attention results.
//
// Reference counterparts: csrc/activation_kernels.cu:20-222 (gelu_and_mul, gelu_tanh_and_mul,
// mul_and_silu, fatrelu_and_mul, gelu_new, gelu_fast, gelu_quick), csrc/cache_kernels.cu:24-130
// (swap_blocks, copy_blocks), csrc/attention/merge_attn_states.cu:16-178.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

enum ActKind : int {
  ACT_SILU_MUL = 0,       // silu(x[:d]) * x[d:]
  ACT_GELU_MUL = 1,       // gelu(x[:d]) * x[d:], erf form
  ACT_GELU_TANH_MUL = 2,  // gelu(x[:d]) * x[d:], tanh form
  ACT_MUL_SILU = 3,       // x[:d] * silu(x[d:])
  ACT_FATRELU_MUL = 4,    // (x[:d] > threshold ? x[:d] : 0) * x[d:]
  ACT_GELU_NEW = 5,       // unary from here on
  ACT_GELU_FAST = 6,
  ACT_GELU_QUICK = 7,
  ACT_GELU = 8,
  ACT_SILU = 9,
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float inner = 0.79788456080286536f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(inner));
}

template <int KIND>
__device__ __forceinline__ float act_apply(float a, float b, float param) {
  if constexpr (KIND == ACT_SILU_MUL) return silu_f(a) * b;
  if constexpr (KIND == ACT_GELU_MUL) return gelu_erf_f(a) * b;
  if constexpr (KIND == ACT_GELU_TANH_MUL) return gelu_tanh_f(a) * b;
  if constexpr (KIND == ACT_MUL_SILU) return a * silu_f(b);
  if constexpr (KIND == ACT_FATRELU_MUL) return (a > param ? a : 0.f) * b;
  if constexpr (KIND == ACT_GELU_NEW) return gelu_tanh_f(a);
  if constexpr (KIND == ACT_GELU_FAST)
    return 0.5f * a * (1.f + tanhf(a * 0.79788456f * (1.f + 0.044715f * a * a)));
  if constexpr (KIND == ACT_GELU_QUICK) return a / (1.f + __expf(-1.702f * a));
  if constexpr (KIND == ACT_GELU) return gelu_erf_f(a);
  if constexpr (KIND == ACT_SILU) return silu_f(a);
  return a;
}

// Gated kinds read x[t, j] and x[t, d + j]; unary kinds read x[t, j] only. 8 bf16 per thread and step.
template <int KIND>
__global__ void __launch_bounds__(256)
activation_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ out,
                  long long ldo, int T, int d, float param) {
  constexpr bool GATED = KIND <= ACT_FATRELU_MUL;
  const int nvec = d >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < static_cast<long long>(T) * nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / nvec);
    const int v = static_cast<int>(i - static_cast<long long>(t) * nvec);
    const uint4 g = *reinterpret_cast<const uint4*>(x + t * ldx + v * 8);
    uint4 u = g;
    if constexpr (GATED) u = *reinterpret_cast<const uint4*>(x + t * ldx + d + v * 8);
    const uint32_t* gu = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* uu = reinterpret_cast<const uint32_t*>(&u);
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gu[j]);
      const float2 b = unpack_bf16x2(uu[j]);
      ou[j] = pack_bf16x2(act_apply<KIND>(a.x, b.x, param), act_apply<KIND>(a.y, b.y, param));
    }
    *reinterpret_cast<uint4*>(out + t * ldo + v * 8) = o;
  }
}

// One CTA row per (pair, chunk): copies page `src` onto page `dst` of the same cache allocation.
__global__ void __launch_bounds__(256)
copy_pages_kernel(uint4* __restrict__ cache, long long page_vecs, const long long* __restrict__ pairs,
                  int n_pairs) {
  const int p = blockIdx.x;
  if (p >= n_pairs) return;
  const uint4* src = cache + pairs[2 * p] * page_vecs;
  uint4* dst = cache + pairs[2 * p + 1] * page_vecs;
  for (long long i = blockIdx.y * static_cast<long long>(blockDim.x) + threadIdx.x; i < page_vecs;
       i += static_cast<long long>(gridDim.y) * blockDim.x)
    dst[i] = src[i];
}

// out = softmax-weighted merge of two partial attention outputs over disjoint key sets.
// Outputs [T, H, D] bf16, log-sum-exps [H, T] fp32 (natural log). One warp per (token, head).
__global__ void __launch_bounds__(256)
merge_attn_states_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                         const __nv_bfloat16* __restrict__ a_out, const float* __restrict__ a_lse,
                         const __nv_bfloat16* __restrict__ b_out, const float* __restrict__ b_lse, int T,
                         int H, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T * H) return;
  const int t = warp / H, h = warp - t * H;
  float la = a_lse[static_cast<long long>(h) * T + t];
  float lb = b_lse[static_cast<long long>(h) * T + t];
  // an empty partial result carries lse = -inf (or +inf from some producers): give it weight zero
  if (isinf(la)) la = -INFINITY;
  if (isinf(lb)) lb = -INFINITY;
  const float m = fmaxf(la, lb);
  float wa = 0.f, wb = 0.f, lse = -INFINITY;
  if (m > -INFINITY) {
    const float ea = __expf(la - m), eb = __expf(lb - m);
    const float inv = 1.f / (ea + eb);
    wa = ea * inv;
    wb = eb * inv;
    lse = m + __logf(ea + eb);
  }
  const long long base = (static_cast<long long>(t) * H + h) * D;
  for (int v = lane; v < (D >> 3); v += 32) {
    const uint4 xa = *reinterpret_cast<const uint4*>(a_out + base + v * 8);
    const uint4 xb = *reinterpret_cast<const uint4*>(b_out + base + v * 8);
    const uint32_t* au = reinterpret_cast<const uint32_t*>(&xa);
    const uint32_t* bu = reinterpret_cast<const uint32_t*>(&xb);
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(au[j]);
      const float2 b = unpack_bf16x2(bu[j]);
      ou[j] = pack_bf16x2(a.x * wa + b.x * wb, a.y * wa + b.y * wb);
    }
    *reinterpret_cast<uint4*>(out + base + v * 8) = o;
  }
  if (out_lse != nullptr && lane == 0) out_lse[static_cast<long long>(h) * T + t] = lse;
}

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s launch failed: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

template <int KIND>
static void launch_activation(const void* x, long long ldx, void* out, long long ldo, int T, int d, float param,
                              cudaStream_t stream) {
  const long long work = static_cast<long long>(T) * (d / 8);
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  activation_kernel<KIND><<<static_cast<int>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<__nv_bfloat16*>(out), ldo, T, d, param);
}

}  // namespace tw

using namespace tw;

extern "C" int tw_activation(const void* x, long long ldx, void* out, long long ldo, int T, int d, int kind,
                             float param, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) {
    set_last_error("activation: width and strides must be multiples of 8");
    return 1;
  }
  switch (kind) {
    case ACT_SILU_MUL: launch_activation<ACT_SILU_MUL>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_GELU_MUL: launch_activation<ACT_GELU_MUL>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_GELU_TANH_MUL: launch_activation<ACT_GELU_TANH_MUL>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_MUL_SILU: launch_activation<ACT_MUL_SILU>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_FATRELU_MUL: launch_activation<ACT_FATRELU_MUL>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_GELU_NEW: launch_activation<ACT_GELU_NEW>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_GELU_FAST: launch_activation<ACT_GELU_FAST>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_GELU_QUICK: launch_activation<ACT_GELU_QUICK>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_GELU: launch_activation<ACT_GELU>(x, ldx, out, ldo, T, d, param, stream); break;
    case ACT_SILU: launch_activation<ACT_SILU>(x, ldx, out, ldo, T, d, param, stream); break;
    default:
      set_last_error("activation: unknown kind %d", kind);
      return 1;
  }
  return check_launch("activation");
}

// pairs: device array of n_pairs (src page, dst page) int64 couples; page_bytes a multiple of 16.
extern "C" int tw_copy_pages(void* cache, long long page_bytes, const long long* pairs_dev, int n_pairs,
                             cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (page_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(cache) & 15) != 0) {
    set_last_error("copy_pages: cache must be 16-byte aligned with pages a multiple of 16 bytes");
    return 1;
  }
  const long long vecs = page_bytes / 16;
  int chunks = static_cast<int>((vecs + 256 * 8 - 1) / (256 * 8));
  if (chunks < 1) chunks = 1;
  if (chunks > 64) chunks = 64;
  copy_pages_kernel<<<dim3(n_pairs, chunks), 256, 0, stream>>>(reinterpret_cast<uint4*>(cache), vecs, pairs_dev,
                                                               n_pairs);
  return check_launch("copy_pages");
}

// Copies page pairs between two allocations (device<->pinned host or device<->device), one
// asynchronous copy per run of consecutive pages. pairs_host: n_pairs (src, dst) int64 couples.
extern "C" int tw_swap_pages(const void* src, void* dst, long long page_bytes, const long long* pairs_host,
                             int n_pairs, cudaStream_t stream) {
  int i = 0;
  while (i < n_pairs) {
    int run = 1;
    while (i + run < n_pairs && pairs_host[2 * (i + run)] == pairs_host[2 * i] + run &&
           pairs_host[2 * (i + run) + 1] == pairs_host[2 * i + 1] + run)
      ++run;
    const char* s = reinterpret_cast<const char*>(src) + pairs_host[2 * i] * page_bytes;
    char* d = reinterpret_cast<char*>(dst) + pairs_host[2 * i + 1] * page_bytes;
    cudaError_t e = cudaMemcpyAsync(d, s, static_cast<size_t>(run) * page_bytes, cudaMemcpyDefault, stream);
    if (e != cudaSuccess) {
      set_last_error("swap_pages: copy failed: %s", cudaGetErrorString(e));
      return 1;
    }
    i += run;
  }
  return 0;
}

extern "C" int tw_merge_attn_states(void* out, float* out_lse, const void* a_out, const float* a_lse,
                                    const void* b_out, const float* b_lse, int T, int H, int D,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 8 != 0) {
    set_last_error("merge_attn_states: head size must be a multiple of 8");
    return 1;
  }
  const long long warps = static_cast<long long>(T) * H;
  const int blocks = static_cast<int>((warps + 7) / 8);
  merge_attn_states_kernel<<<blocks, 256, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16*>(out), out_lse, reinterpret_cast<const __nv_bfloat16*>(a_out), a_lse,
      reinterpret_cast<const __nv_bfloat16*>(b_out), b_lse, T, H, D);
  return check_launch("merge_attn_states");
}
