// fp8 (e4m3) activation quantisation for the fp8 GEMM path: plain per-token / per-tensor quantisation
// and RMSNorm (optionally with the residual add) fused with dynamic per-token quantisation.
//
// Reference counterparts: csrc/quantization/fp8/common.cu (static and dynamic per-token scaled fp8
// quant), csrc/layernorm_quant_kernels.cu:21-160 (RMSNorm + static fp8 quant),
// csrc/quantization/fused_kernels/fused_layernorm_dynamic_per_token_quant.cu (RMSNorm + dynamic
// per-token quant). As in the bf16 norms of this library a CTA keeps its row in registers between
// the passes, so the activation is read once and the fp8 row written once.
#include <cuda_fp8.h>

#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr float FP8_E4M3_MAX = 448.f;

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float x = (lane < nwarps) ? scratch[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

__device__ __forceinline__ uint16_t to_e4m3x2(float a, float b) {
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}

// Two int8 values per call: round to nearest even, saturate to [-128, 127] (float_to_int8_rn of the
// reference, csrc/quantization/compressed_tensors/int8_quant_kernels.cu:13-28).
__device__ __forceinline__ uint16_t to_int8x2(float a, float b) {
  const int ia = max(-128, min(127, __float2int_rn(a)));
  const int ib = max(-128, min(127, __float2int_rn(b)));
  return static_cast<uint16_t>((ia & 0xff) | ((ib & 0xff) << 8));
}

// INT8: the output is symmetric int8 (row maximum maps to 127) instead of e4m3 (row maximum maps to 448).
// MODE 0: quantise x. MODE 1: y = rmsnorm(x) * w, quantise y. MODE 2: x += residual, residual = x,
// y = rmsnorm(x) * w, quantise y. DYNAMIC: scale[t] = max|y[t, :]| / 448 is computed and written;
// otherwise every row uses scales[0]. Each thread owns VPT vectors of 8 elements.
template <int VPT, int MODE, bool DYNAMIC, bool INT8>
__global__ void __launch_bounds__(1024)
quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ res,
                 const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ out, float* __restrict__ scales,
                 int T, int H, long long ldx, long long ldr, long long ldo, float eps) {
  __shared__ float scratch[32];
  const int nvec = H >> 3;
  uint4 wv[VPT];
  if (MODE != 0) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      wv[i] = (v < nvec) ? reinterpret_cast<const uint4*>(w)[v] : make_uint4(0, 0, 0, 0);
    }
  }
  const float static_scale = DYNAMIC ? 1.f : scales[0];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + t * ldx);
    uint4 xv[VPT];
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
          const uint4 r = rr[v];
          xv[i].x = add_bf16x2(xv[i].x, r.x);
          xv[i].y = add_bf16x2(xv[i].y, r.y);
          xv[i].z = add_bf16x2(xv[i].z, r.z);
          xv[i].w = add_bf16x2(xv[i].w, r.w);
          rr[v] = xv[i];
        }
      }
    }
    float inv = 1.f;
    if (MODE != 0) {
      float ss[1] = {0.f};
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&xv[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          ss[0] += f.x * f.x + f.y * f.y;
        }
      }
      block_sum<1>(ss, scratch);
      inv = rsqrtf(ss[0] / static_cast<float>(H) + eps);
    }
    // y = the value to quantise, kept as packed bf16 in place of x (the normalised value is rounded to
    // bf16 before the weight and after it, as in the bf16 norms, so nothing is lost by packing)
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      uint32_t* u = reinterpret_cast<uint32_t*>(&xv[i]);
      const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(u[j]);
        if (MODE != 0) {
          const float2 g = unpack_bf16x2(wu[j]);
          f.x = __bfloat162float(__float2bfloat16_rn(f.x * inv)) * g.x;
          f.y = __bfloat162float(__float2bfloat16_rn(f.y * inv)) * g.y;
          u[j] = pack_bf16x2(f.x, f.y);
          f = unpack_bf16x2(u[j]);
        }
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    float scale = static_scale;
    if (DYNAMIC) {
      amax = block_max(amax, scratch);
      scale = fmaxf(amax / (INT8 ? 127.f : FP8_E4M3_MAX), 1e-10f);
      if (threadIdx.x == 0) scales[t] = scale;
    }
    // one IEEE reciprocal per row, then a multiply per element (the reference's is_scale_inverted form,
    // csrc/quantization/fp8/common.cuh); the PyTorch oracle computes x * (1 / scale) the same way, which
    // matters because 0.6 % of bf16 inputs sit exactly on e4m3 rounding ties
    const float rscale = __frcp_rn(scale);
    uint2* orow = reinterpret_cast<uint2*>(out + t * ldo);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&xv[i]);
        const float2 a = unpack_bf16x2(u[0]), b = unpack_bf16x2(u[1]);
        const float2 c = unpack_bf16x2(u[2]), d = unpack_bf16x2(u[3]);
        uint2 o;
        if (INT8) {
          o.x = to_int8x2(a.x * rscale, a.y * rscale) | (static_cast<uint32_t>(to_int8x2(b.x * rscale, b.y * rscale)) << 16);
          o.y = to_int8x2(c.x * rscale, c.y * rscale) | (static_cast<uint32_t>(to_int8x2(d.x * rscale, d.y * rscale)) << 16);
        } else {
          o.x = to_e4m3x2(a.x * rscale, a.y * rscale) | (static_cast<uint32_t>(to_e4m3x2(b.x * rscale, b.y * rscale)) << 16);
          o.y = to_e4m3x2(c.x * rscale, c.y * rscale) | (static_cast<uint32_t>(to_e4m3x2(d.x * rscale, d.y * rscale)) << 16);
        }
        orow[v] = o;
      }
    }
  }
}

template <int MODE, bool DYNAMIC, bool INT8 = false>
static int launch_quant(const void* x, void* res, const void* w, void* out, float* scales, int T, int H,
                        long long ldx, long long ldr, long long ldo, float eps, int max_ctas, cudaStream_t stream) {
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  int vpt = 1;
  while (threads > 512) {       // keep two CTAs per SM resident for rows up to 8192 wide
    vpt *= 2;
    threads = (((nvec + vpt - 1) / vpt + 31) / 32) * 32;
  }
  if (vpt > 8) {
    set_last_error("quant_fp8: rows wider than 32768 elements are not supported (got %d)", H);
    return 1;
  }
  int grid = T;
  int cap = device_sm_count() * 4;
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto rb = reinterpret_cast<__nv_bfloat16*>(res);
  auto wb = reinterpret_cast<const __nv_bfloat16*>(w);
  auto ob = reinterpret_cast<uint8_t*>(out);
#define TW_QUANT_CASE(V)                                                                              \
  case V:                                                                                             \
    quant_fp8_kernel<V, MODE, DYNAMIC, INT8><<<grid, threads, 0, stream>>>(xb, rb, wb, ob, scales, T, H, ldx, \
                                                                           ldr, ldo, eps);                  \
    break;
  switch (vpt) {
    TW_QUANT_CASE(1)
    TW_QUANT_CASE(2)
    TW_QUANT_CASE(4)
    TW_QUANT_CASE(8)
  }
#undef TW_QUANT_CASE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("quant_fp8 launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

// out[t, :] = e4m3(x[t, :] / scale); dynamic != 0: scale[t] = max|x[t, :]| / 448 is written to scales[t],
// otherwise scales[0] is read and used for every row.
extern "C" int tw_quant_fp8(const void* x, long long ldx, void* out, long long ldo, float* scales, int T, int H,
                            int dynamic, int max_ctas, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) {
    set_last_error("quant_fp8: width and strides must be multiples of 8");
    return 1;
  }
  return dynamic ? launch_quant<0, true>(x, nullptr, nullptr, out, scales, T, H, ldx, 0, ldo, 0.f, max_ctas, stream)
                 : launch_quant<0, false>(x, nullptr, nullptr, out, scales, T, H, ldx, 0, ldo, 0.f, max_ctas, stream);
}

// residual == null: out = e4m3(rmsnorm(x) * w / scale). Otherwise x + residual is written to residual
// first and normalised. x itself is not modified.
extern "C" int tw_rmsnorm_quant_fp8(const void* x, void* residual, const void* w, void* out, long long ldo,
                                    float* scales, int T, int H, long long ldx, long long ldr, float eps,
                                    int dynamic, int max_ctas, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0 || (residual != nullptr && ldr % 8 != 0)) {
    set_last_error("rmsnorm_quant_fp8: width and strides must be multiples of 8");
    return 1;
  }
  if (residual != nullptr)
    return dynamic ? launch_quant<2, true>(x, residual, w, out, scales, T, H, ldx, ldr, ldo, eps, max_ctas, stream)
                   : launch_quant<2, false>(x, residual, w, out, scales, T, H, ldx, ldr, ldo, eps, max_ctas, stream);
  return dynamic ? launch_quant<1, true>(x, nullptr, w, out, scales, T, H, ldx, 0, ldo, eps, max_ctas, stream)
                 : launch_quant<1, false>(x, nullptr, w, out, scales, T, H, ldx, 0, ldo, eps, max_ctas, stream);
}

// Symmetric int8: out[t, :] = clamp(round(x[t, :] / scale), -128, 127); dynamic != 0: scale[t] = max|x[t, :]| / 127
// is written to scales[t], otherwise scales[0] is used for every row (the reference's static_scaled_int8_quant /
// dynamic_scaled_int8_quant, csrc/quantization/compressed_tensors/int8_quant_kernels.cu).
extern "C" int tw_quant_int8(const void* x, long long ldx, void* out, long long ldo, float* scales, int T, int H,
                             int dynamic, int max_ctas, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) {
    set_last_error("quant_int8: width and strides must be multiples of 8");
    return 1;
  }
  return dynamic ? launch_quant<0, true, true>(x, nullptr, nullptr, out, scales, T, H, ldx, 0, ldo, 0.f, max_ctas, stream)
                 : launch_quant<0, false, true>(x, nullptr, nullptr, out, scales, T, H, ldx, 0, ldo, 0.f, max_ctas, stream);
}

// (add +) RMSNorm fused with int8 quantisation; arguments as tw_rmsnorm_quant_fp8 (the reference's
// rms_norm_dynamic_per_token_quant with an int8 output, csrc/quantization/fused_kernels/).
extern "C" int tw_rmsnorm_quant_int8(const void* x, void* residual, const void* w, void* out, long long ldo,
                                     float* scales, int T, int H, long long ldx, long long ldr, float eps,
                                     int dynamic, int max_ctas, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0 || (residual != nullptr && ldr % 8 != 0)) {
    set_last_error("rmsnorm_quant_int8: width and strides must be multiples of 8");
    return 1;
  }
  if (residual != nullptr)
    return dynamic ? launch_quant<2, true, true>(x, residual, w, out, scales, T, H, ldx, ldr, ldo, eps, max_ctas, stream)
                   : launch_quant<2, false, true>(x, residual, w, out, scales, T, H, ldx, ldr, ldo, eps, max_ctas, stream);
  return dynamic ? launch_quant<1, true, true>(x, nullptr, w, out, scales, T, H, ldx, 0, ldo, eps, max_ctas, stream)
                 : launch_quant<1, false, true>(x, nullptr, w, out, scales, T, H, ldx, 0, ldo, eps, max_ctas, stream);
}
