// Mixture-of-experts routing kernels (Mixtral: 8 experts, top-2, softmax then renormalise).
//
//   tw_moe_router      gate GEMV (x . Wg^T, fp32) + softmax + top-k + renormalise, one kernel.
//                      Reference: replicated gate linear, then csrc/moe/topk_softmax_kernels.cu
//                      and the renormalisation in fused_moe.py:831-844.
//   tw_moe_align       counting sort of (token, k) pairs by expert with every expert's segment
//                      padded to the GEMM's 128-row tile; emits the expert of each row tile, the
//                      number of tiles, the sorted position of every pair.
//                      Reference: csrc/moe/moe_align_sum_kernels.cu:24-112.
//   tw_moe_scatter     copies token rows into expert-sorted order (the A operand of the grouped
//                      GEMM) and the routing weight of each sorted row.
//   tw_moe_combine     out[t] = sum_k y_sorted[pos[t,k]] (weights were applied by the second
//                      grouped GEMM's epilogue). Reference: moe_sum_kernel,
//                      moe_align_sum_kernels.cu:277-293.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int MOE_MAX_EXPERTS = 64;
constexpr int MOE_MAX_TOPK = 8;

__device__ __forceinline__ float2 moe_ffma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

// TPW tokens per warp, persistent CTAs. The gate weight [E, H] lives in shared memory; a warp reads (and converts)
// every 16 bytes of it once for its TPW tokens, and the multiply-adds are the packed two-wide fp32 form of sm_100:
// this is about one instruction per multiply-add where one token per warp with scalar FMAs took 2.1.
template <int E, int TPW>
__global__ void __launch_bounds__(512)       // 16 warps per SM: 128 registers each for the TPW x E accumulators
moe_router_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                  const __nv_bfloat16* __restrict__ wg, float* __restrict__ topk_w,
                  int* __restrict__ topk_ids, float* __restrict__ logits_out, int T, int H, int topk,
                  int renormalize) {
  extern __shared__ uint8_t smem_raw[];
  uint4* wsm = reinterpret_cast<uint4*>(smem_raw);
  const int nvec = H >> 3;
  for (int i = threadIdx.x; i < E * nvec; i += blockDim.x)
    wsm[i] = reinterpret_cast<const uint4*>(wg)[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int tb = (blockIdx.x * wpb + warp) * TPW; tb < T; tb += gridDim.x * wpb * TPW) {
    float2 acc[TPW][E];            // .x: even elements of the row, .y: odd ones
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) acc[i][e] = make_float2(0.f, 0.f);
    const uint4* xr[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i)          // tokens past the end re-read the last row; their results are dropped
      xr[i] = reinterpret_cast<const uint4*>(x + static_cast<long long>(min(tb + i, T - 1)) * ldx);
    // the row pieces of the NEXT step are requested before this step's arithmetic: with 16 warps per SM the loads
    // of one step alone would leave the memory system idle while the warps multiply
    uint4 xv[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) xv[i] = lane < nvec ? xr[i][lane] : make_uint4(0u, 0u, 0u, 0u);
    for (int v = lane; v < nvec; v += 32) {
      float2 xf[TPW][4];
#pragma unroll
      for (int i = 0; i < TPW; ++i) {
        const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) xf[i][j] = unpack_bf16x2(xu[j]);
      }
      if (v + 32 < nvec) {
#pragma unroll
        for (int i = 0; i < TPW; ++i) xv[i] = xr[i][v + 32];
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const uint4 wv = wsm[e * nvec + v];
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wf = unpack_bf16x2(wu[j]);
#pragma unroll
          for (int i = 0; i < TPW; ++i) acc[i][e] = moe_ffma2(xf[i][j], wf, acc[i][e]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      float logit[E];
#pragma unroll
      for (int e = 0; e < E; ++e) logit[e] = warp_sum(acc[i][e].x + acc[i][e].y);
      const int t = tb + i;
      if (lane == i && t < T) {             // one lane per token: the TPW tails run side by side
        float mx = logit[0];
#pragma unroll
        for (int e = 1; e < E; ++e) mx = fmaxf(mx, logit[e]);
        float p[E];
        float den = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          p[e] = __expf(logit[e] - mx);
          den += p[e];
        }
        if (logits_out != nullptr) {
#pragma unroll
          for (int e = 0; e < E; ++e) logits_out[static_cast<long long>(t) * E + e] = logit[e];
        }
        float wsum = 0.f;
        float sel_w[MOE_MAX_TOPK];
        int sel_i[MOE_MAX_TOPK];
        for (int k = 0; k < topk; ++k) {
          int bi = 0;
          float bv = -1.f;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            if (p[e] > bv) { bv = p[e]; bi = e; }
          }
          sel_w[k] = bv / den;
          sel_i[k] = bi;
          wsum += sel_w[k];
#pragma unroll
          for (int e = 0; e < E; ++e)
            if (e == bi) p[e] = -2.f;
        }
        for (int k = 0; k < topk; ++k) {
          topk_w[static_cast<long long>(t) * topk + k] = renormalize ? sel_w[k] / wsum : sel_w[k];
          topk_ids[static_cast<long long>(t) * topk + k] = sel_i[k];
        }
      }
    }
  }
}

// Single CTA: histogram -> padded exclusive scan -> per-tile expert ids.
// meta[0] = number of 128-row tiles, meta[1] = padded row count.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_ids, int n_pairs, int E, int tile_rows,
                 int* __restrict__ expert_offsets, int* __restrict__ expert_cursor,
                 int* __restrict__ tile_expert, int max_tiles, int* __restrict__ meta) {
  __shared__ int counts[MOE_MAX_EXPERTS];
  __shared__ int offsets[MOE_MAX_EXPERTS + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = off;
      off += (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
    }
    offsets[E] = off;
    meta[0] = off / tile_rows;
    meta[1] = off;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    expert_offsets[e] = offsets[e];
    if (e < E) expert_cursor[e] = 0;
  }
  const int tiles = offsets[E] / tile_rows;
  for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
    int ex = 0;
    if (m < tiles) {
      const int row = m * tile_rows;
      while (ex + 1 < E && offsets[ex + 1] <= row) ++ex;
    }
    tile_expert[m] = ex;
  }
}

// One CTA per (token, k) pair: claim a sorted row and copy the token's hidden row there.
__global__ void __launch_bounds__(256)
moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ topk_ids,
                   const float* __restrict__ topk_w, const int* __restrict__ expert_offsets,
                   int* __restrict__ expert_cursor, __nv_bfloat16* __restrict__ a_sorted,
                   float* __restrict__ row_scale, int* __restrict__ sorted_pos, int n_pairs, int topk,
                   int H, int E) {
  __shared__ int s_pos;
  const int nvec = H >> 3;
  for (int pair = blockIdx.x; pair < n_pairs; pair += gridDim.x) {
    if (threadIdx.x == 0) {
      const int e = topk_ids[pair];
      int pos = -1;
      if (e >= 0 && e < E) pos = expert_offsets[e] + atomicAdd(&expert_cursor[e], 1);
      s_pos = pos;
      sorted_pos[pair] = pos;
      if (pos >= 0) row_scale[pos] = topk_w[pair];
    }
    __syncthreads();
    const int pos = s_pos;
    if (pos >= 0) {
      const uint4* src = reinterpret_cast<const uint4*>(x + (pair / topk) * ldx);
      uint4* dst = reinterpret_cast<uint4*>(a_sorted + static_cast<long long>(pos) * H);
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = src[v];
    }
    __syncthreads();
  }
}

// out[t] = sum_k y[pos[t,k]] in fp32, rounded once.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ sorted_pos,
                   __nv_bfloat16* __restrict__ out, long long ldo, int T, int topk, int H) {
  const int nvec = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < topk; ++k) {
        const int pos = sorted_pos[t * topk + k];
        if (pos < 0) continue;
        const uint4 yv = reinterpret_cast<const uint4*>(y + static_cast<long long>(pos) * H)[v];
        const uint32_t* yu = reinterpret_cast<const uint32_t*>(&yv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(yu[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) ou[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
      reinterpret_cast<uint4*>(out + t * ldo)[v] = o;
    }
  }
}

static int moe_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s launch failed: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

extern "C" int tw_moe_router(const void* x, long long ldx, const void* wg, float* topk_w, int* topk_ids,
                             float* logits_out, int T, int H, int E, int topk, int renormalize,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || topk < 1 || topk > MOE_MAX_TOPK || topk > E) {
    set_last_error("moe_router: unsupported shape (H=%d, E=%d, topk=%d)", H, E, topk);
    return 1;
  }
  const size_t smem = static_cast<size_t>(E) * H * 2;
  if (smem > 200 * 1024) {
    set_last_error("moe_router: gate weight (%zu bytes) does not fit in shared memory", smem);
    return 1;
  }
  const int cap = device_sm_count();
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wb = reinterpret_cast<const __nv_bfloat16*>(wg);
  // tokens per warp: at most 64 accumulator registers per thread, room left for the prefetched row pieces
#define TW_ROUTER_CASE(NE, TPW)                                                                     \
  case NE: {                                                                                        \
    auto kern = moe_router_kernel<NE, TPW>;                                                         \
    int grid = (T + 16 * TPW - 1) / (16 * TPW);                                                     \
    if (grid > cap) grid = cap;                                                                     \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    kern<<<grid, 512, smem, stream>>>(xb, ldx, wb, topk_w, topk_ids, logits_out, T, H, topk,         \
                                      renormalize);                                                 \
    break;                                                                                          \
  }
  switch (E) {
    TW_ROUTER_CASE(4, 4)
    TW_ROUTER_CASE(8, 2)
    TW_ROUTER_CASE(16, 1)
    TW_ROUTER_CASE(32, 1)
    default:
      set_last_error("moe_router: number of experts %d not in {4, 8, 16, 32}", E);
      return 1;
  }
#undef TW_ROUTER_CASE
  return moe_check("moe_router");
}

extern "C" int tw_moe_align(const int* topk_ids, int n_pairs, int E, int tile_rows, int* expert_offsets,
                            int* expert_cursor, int* tile_expert, int max_tiles, int* meta,
                            cudaStream_t stream) {
  if (E > MOE_MAX_EXPERTS) {
    set_last_error("moe_align: at most %d experts", MOE_MAX_EXPERTS);
    return 1;
  }
  moe_align_kernel<<<1, 1024, 0, stream>>>(topk_ids, n_pairs, E, tile_rows, expert_offsets, expert_cursor,
                                           tile_expert, max_tiles, meta);
  return moe_check("moe_align");
}

extern "C" int tw_moe_scatter(const void* x, long long ldx, const int* topk_ids, const float* topk_w,
                              const int* expert_offsets, int* expert_cursor, void* a_sorted,
                              float* row_scale, int* sorted_pos, int n_pairs, int topk, int H, int E,
                              cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  int grid = n_pairs;
  const int cap = device_sm_count() * 8;
  if (grid > cap) grid = cap;
  moe_scatter_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, topk_ids,
                                               topk_w, expert_offsets, expert_cursor,
                                               reinterpret_cast<__nv_bfloat16*>(a_sorted), row_scale,
                                               sorted_pos, n_pairs, topk, H, E);
  return moe_check("moe_scatter");
}

extern "C" int tw_moe_combine(const void* y, const int* sorted_pos, void* out, long long ldo, int T,
                              int topk, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  int grid = T;
  const int cap = device_sm_count() * 8;
  if (grid > cap) grid = cap;
  moe_combine_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y), sorted_pos,
                                               reinterpret_cast<__nv_bfloat16*>(out), ldo, T, topk, H);
  return moe_check("moe_combine");
}
