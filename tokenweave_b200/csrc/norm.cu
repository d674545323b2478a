// RMSNorm family (single GPU). bf16 tensors, fp32 statistics.
//
//   tw_rmsnorm          out = rmsnorm(x) * w
//   tw_rmsnorm_copy     residual_out = x ; x = rmsnorm(x) * w           (layer-0 helper)
//   tw_add_rmsnorm      x += residual ; residual = x ; x = rmsnorm(x) * w  (in place)
//
// Numerics follow the reference kernels (csrc/layernorm_kernels.cu:87-113,
// csrc/tokenweave_fused_kernels.cu:37-72): the residual add is a packed bf16 add, the sum of
// squares runs in fp32 over the bf16-rounded sums, the normalised value is rounded to bf16 and
// only then multiplied by the bf16 weight.
//
// Unlike the reference (one CTA per token, the row re-read from global memory for the second
// pass) a CTA here keeps its rows in registers between the two passes and walks a persistent
// grid, so the tensor is read once and written once; `max_ctas` bounds the SMs it occupies.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

// One row per CTA iteration; each thread owns VPT 16-byte vectors of the row.
template <int VPT, int MODE>  // MODE 0: norm to out, 1: copy+norm in place, 2: add+norm in place
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(__nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ res,
               __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ w, int T, int H,
               long long ldx, long long ldr, long long ldo, float eps) {
  __shared__ float scratch[32];
  const int nvec = H >> 3;
  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    wv[i] = (v < nvec) ? reinterpret_cast<const uint4*>(w)[v] : make_uint4(0, 0, 0, 0);
  }
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    uint4* xr = reinterpret_cast<uint4*>(x + t * ldx);
    uint4 xv[VPT];
    float ss[1] = {0.f};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      xv[i] = (v < nvec) ? xr[v] : make_uint4(0, 0, 0, 0);
    }
    if (MODE == 2) {
      uint4* rr = reinterpret_cast<uint4*>(res + t * ldr);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
          uint4 r = rr[v];
          xv[i].x = add_bf16x2(xv[i].x, r.x);
          xv[i].y = add_bf16x2(xv[i].y, r.y);
          xv[i].z = add_bf16x2(xv[i].z, r.z);
          xv[i].w = add_bf16x2(xv[i].w, r.w);
          rr[v] = xv[i];
        }
      }
    } else if (MODE == 1) {
      uint4* rr = reinterpret_cast<uint4*>(res + t * ldr);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) rr[v] = xv[i];
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&xv[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(u[j]);
        ss[0] += f.x * f.x + f.y * f.y;
      }
    }
    block_sum<1>(ss, scratch);
    const float inv = rsqrtf(ss[0] / static_cast<float>(H) + eps);
    uint4* orow = (MODE == 0) ? reinterpret_cast<uint4*>(out + t * ldo) : xr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        uint4 o;
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&xv[i]);
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv[i]);
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(u[j]);
          ou[j] = mul_bf16x2(pack_bf16x2(f.x * inv, f.y * inv), wu[j]);
        }
        orow[v] = o;
      }
    }
  }
}

template <int MODE>
static int launch_norm(void* x, void* res, void* out, const void* w, int T, int H, long long ldx,
                       long long ldr, long long ldo, float eps, int max_ctas, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldr % 8 != 0 || ldo % 8 != 0) {
    set_last_error("rmsnorm: hidden size and row strides must be multiples of 8 (H=%d)", H);
    return 1;
  }
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  int vpt = 1;
  while (threads > 1024 || (vpt < 8 && threads > 512 && nvec > 1024)) {
    vpt *= 2;
    threads = (((nvec + vpt - 1) / vpt + 31) / 32) * 32;
  }
  if (vpt > 8) {
    set_last_error("rmsnorm: hidden size %d too large", H);
    return 1;
  }
  int grid = T;
  const int cap = (max_ctas > 0) ? max_ctas : device_sm_count() * (threads <= 512 ? 4 : 2);
  if (grid > cap) grid = cap;
  auto xb = reinterpret_cast<__nv_bfloat16*>(x);
  auto rb = reinterpret_cast<__nv_bfloat16*>(res);
  auto ob = reinterpret_cast<__nv_bfloat16*>(out);
  auto wb = reinterpret_cast<const __nv_bfloat16*>(w);
#define TW_NORM_CASE(V)                                                                         \
  case V:                                                                                       \
    rmsnorm_kernel<V, MODE><<<grid, threads, 0, stream>>>(xb, rb, ob, wb, T, H, ldx, ldr, ldo, eps); \
    break;
  switch (vpt) {
    TW_NORM_CASE(1)
    TW_NORM_CASE(2)
    TW_NORM_CASE(4)
    TW_NORM_CASE(8)
  }
#undef TW_NORM_CASE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("rmsnorm launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

extern "C" int tw_rmsnorm(const void* x, void* out, const void* w, int T, int H, long long ldx,
                          long long ldo, float eps, int max_ctas, cudaStream_t stream) {
  return tw::launch_norm<0>(const_cast<void*>(x), nullptr, out, w, T, H, ldx, 8, ldo, eps, max_ctas,
                            stream);
}
extern "C" int tw_rmsnorm_copy(void* x, void* residual_out, const void* w, int T, int H, long long ldx,
                               long long ldr, float eps, int max_ctas, cudaStream_t stream) {
  return tw::launch_norm<1>(x, residual_out, nullptr, w, T, H, ldx, ldr, 8, eps, max_ctas, stream);
}
extern "C" int tw_add_rmsnorm(void* x, void* residual, const void* w, int T, int H, long long ldx,
                              long long ldr, float eps, int max_ctas, cudaStream_t stream) {
  return tw::launch_norm<2>(x, residual, nullptr, w, T, H, ldx, ldr, 8, eps, max_ctas, stream);
}
