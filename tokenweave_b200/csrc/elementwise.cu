// Memory-bound single-GPU kernels: RoPE fused with the paged KV-cache write, SwiGLU,
// embedding gather with out-of-shard masking, and greedy argmax.
//
// Reference counterparts: csrc/pos_encoding_kernels.cu:36-92 (NeoX rotary),
// csrc/cache_kernels.cu:264-305 (reshape_and_cache_flash), csrc/activation_kernels.cu:20-86
// (silu_and_mul), vllm/model_executor/layers/vocab_parallel_embedding.py:429-451 (masked
// embedding). The reference runs RoPE and the cache write as two kernels over the same q/k/v
// rows; here one kernel rotates q in place and writes rotated k and v straight into the
// cache, so k and v are read once and never written back to the activation buffer.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

__device__ __forceinline__ void rotate8(const uint4& x, const uint4& y, const float* cosp,
                                        const float* sinp, uint4& xo, uint4& yo) {
  const uint32_t* xu = reinterpret_cast<const uint32_t*>(&x);
  const uint32_t* yu = reinterpret_cast<const uint32_t*>(&y);
  uint32_t* xo_u = reinterpret_cast<uint32_t*>(&xo);
  uint32_t* yo_u = reinterpret_cast<uint32_t*>(&yo);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = unpack_bf16x2(xu[j]);
    const float2 b = unpack_bf16x2(yu[j]);
    const float c0 = cosp[2 * j], c1 = cosp[2 * j + 1];
    const float s0 = sinp[2 * j], s1 = sinp[2 * j + 1];
    xo_u[j] = pack_bf16x2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
    yo_u[j] = pack_bf16x2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
  }
}

// qkv: [T, (hq + 2*hkv) * D] (row stride ld). cos_sin: [max_pos, D] fp32, cos in the first
// D/2 columns, sin in the last D/2. Caches: [num_slots, hkv, D]; slot < 0 skips the write.
// Rows >= num_actual are left untouched (padding rows of a split).
// QKNORM: q and k heads are RMS-normalised over D (weights q_norm_w / k_norm_w, [D]) before the rotation,
// the per-head norm of the Qwen3 layout. The D/16 threads that share a head are neighbouring lanes of one
// warp (the item index is head-major and D/16 is a power of two that divides the block size), so the sum
// of squares is a shuffle reduction inside that lane group.
template <bool QKNORM>
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, const int* __restrict__ positions,
                     const int* __restrict__ slots, const float* __restrict__ cos_sin,
                     __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                     int hq, int hkv, int D, int write_k_back,
                     const __nv_bfloat16* __restrict__ q_norm_w, const __nv_bfloat16* __restrict__ k_norm_w,
                     float eps) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = (slots != nullptr) ? slots[t] : -1;
  const int half = D >> 1;
  const int vec_per_half = half >> 3;  // 16-byte vectors per half head
  __nv_bfloat16* row = qkv + t * ld;
  const float* cs = cos_sin + static_cast<long long>(pos) * D;
  const int rot_items = (hq + hkv) * vec_per_half;
  const int v_items = hkv * (D >> 3);
  for (int it = threadIdx.x; it < rot_items + v_items; it += blockDim.x) {
    if (it < rot_items) {
      const int head = it / vec_per_half;
      const int v = it - head * vec_per_half;
      __nv_bfloat16* h = row + head * D;
      uint4 x = *reinterpret_cast<const uint4*>(h + v * 8);
      uint4 y = *reinterpret_cast<const uint4*>(h + half + v * 8);
      if constexpr (QKNORM) {
        uint32_t* xu = reinterpret_cast<uint32_t*>(&x);
        uint32_t* yu = reinterpret_cast<uint32_t*>(&y);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(xu[j]);
          const float2 b = unpack_bf16x2(yu[j]);
          ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
        }
        const int lane = threadIdx.x & 31;
        const uint32_t group = (vec_per_half >= 32) ? 0xffffffffu
                                                    : (((1u << vec_per_half) - 1u) << (lane & ~(vec_per_half - 1)));
        for (int o = vec_per_half >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(group, ss, o);
        const float r = rsqrtf(ss / static_cast<float>(D) + eps);
        const __nv_bfloat16* w = (head < hq) ? q_norm_w : k_norm_w;
        const uint4 wx = *reinterpret_cast<const uint4*>(w + v * 8);
        const uint4 wy = *reinterpret_cast<const uint4*>(w + half + v * 8);
        const uint32_t* wxu = reinterpret_cast<const uint32_t*>(&wx);
        const uint32_t* wyu = reinterpret_cast<const uint32_t*>(&wy);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(xu[j]), wa = unpack_bf16x2(wxu[j]);
          const float2 b = unpack_bf16x2(yu[j]), wb = unpack_bf16x2(wyu[j]);
          xu[j] = pack_bf16x2(a.x * r * wa.x, a.y * r * wa.y);
          yu[j] = pack_bf16x2(b.x * r * wb.x, b.y * r * wb.y);
        }
      }
      uint4 xo, yo;
      rotate8(x, y, cs + v * 8, cs + half + v * 8, xo, yo);
      if (head < hq) {
        *reinterpret_cast<uint4*>(h + v * 8) = xo;
        *reinterpret_cast<uint4*>(h + half + v * 8) = yo;
      } else {
        if (write_k_back) {
          *reinterpret_cast<uint4*>(h + v * 8) = xo;
          *reinterpret_cast<uint4*>(h + half + v * 8) = yo;
        }
        if (slot >= 0) {
          __nv_bfloat16* kc = k_cache + (static_cast<long long>(slot) * hkv + (head - hq)) * D;
          *reinterpret_cast<uint4*>(kc + v * 8) = xo;
          *reinterpret_cast<uint4*>(kc + half + v * 8) = yo;
        }
      }
    } else if (slot >= 0) {
      const int i = it - rot_items;
      const uint4 val = *reinterpret_cast<const uint4*>(row + (hq + hkv) * D + i * 8);
      *reinterpret_cast<uint4*>(v_cache + static_cast<long long>(slot) * hkv * D + i * 8) = val;
    }
  }
}

// out[t, j] = silu(x[t, j]) * x[t, d + j]
__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ out,
              long long ldo, int T, int d) {
  const int nvec = d >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < static_cast<long long>(T) * nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / nvec);
    const int v = static_cast<int>(i - static_cast<long long>(t) * nvec);
    const uint4 g = *reinterpret_cast<const uint4*>(x + t * ldx + v * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(x + t * ldx + d + v * 8);
    const uint32_t* gu = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* uu = reinterpret_cast<const uint32_t*>(&u);
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gu[j]);
      const float2 b = unpack_bf16x2(uu[j]);
      ou[j] = pack_bf16x2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(out + t * ldo + v * 8) = o;
  }
}

// out[t, :] = table[ids[t] - vocab_start, :] if vocab_start <= ids[t] < vocab_end else 0
__global__ void __launch_bounds__(256)
embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                 __nv_bfloat16* __restrict__ out, long long ldo, int T, int H, int vocab_start,
                 int vocab_end) {
  const int nvec = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const int id = ids[t];
    const bool ok = id >= vocab_start && id < vocab_end;
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<long long>(id - vocab_start) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + t * ldo);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = ok ? src[v] : make_uint4(0, 0, 0, 0);
  }
}

// Row-wise argmax over fp32 logits; ties resolve to the lowest index (torch.argmax semantics).
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, long long ld, int* __restrict__ out, int V) {
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const float* row = logits + blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = (lane < nw) ? sval[lane] : -INFINITY;
    bi = (lane < nw) ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s launch failed: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

extern "C" int tw_rope_kv_write(void* qkv, long long ld, const int* positions, const int* slots,
                                const float* cos_sin, void* k_cache, void* v_cache, int T, int hq,
                                int hkv, int D, int write_k_back, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 16 != 0 || ld % 8 != 0) {
    set_last_error("rope_kv_write: head_dim must be a multiple of 16 and the row stride of 8");
    return 1;
  }
  rope_kv_write_kernel<false><<<T, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(qkv), ld, positions, slots,
                                                      cos_sin, reinterpret_cast<__nv_bfloat16*>(k_cache),
                                                      reinterpret_cast<__nv_bfloat16*>(v_cache), hq, hkv, D,
                                                      write_k_back, nullptr, nullptr, 0.f);
  return check_launch("rope_kv_write");
}

// The same with q and k heads RMS-normalised over head_dim before the rotation (Qwen3).
extern "C" int tw_rope_kv_write_qknorm(void* qkv, long long ld, const int* positions, const int* slots,
                                       const float* cos_sin, void* k_cache, void* v_cache, int T, int hq,
                                       int hkv, int D, int write_k_back, const void* q_norm_w,
                                       const void* k_norm_w, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int vph = D >> 4;
  if (D % 16 != 0 || ld % 8 != 0 || vph < 1 || vph > 32 || (vph & (vph - 1)) != 0 || !q_norm_w || !k_norm_w) {
    set_last_error("rope_kv_write_qknorm: head_dim must be 16 * a power of two (<= 512), row stride a multiple of 8");
    return 1;
  }
  rope_kv_write_kernel<true><<<T, 256, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16*>(qkv), ld, positions, slots, cos_sin, reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), hq, hkv, D, write_k_back,
      reinterpret_cast<const __nv_bfloat16*>(q_norm_w), reinterpret_cast<const __nv_bfloat16*>(k_norm_w), eps);
  return check_launch("rope_kv_write_qknorm");
}

extern "C" int tw_swiglu(const void* x, long long ldx, void* out, long long ldo, int T, int d,
                         cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) {
    set_last_error("swiglu: width and strides must be multiples of 8");
    return 1;
  }
  const long long work = static_cast<long long>(T) * (d / 8);
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  swiglu_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<__nv_bfloat16*>(out), ldo, T, d);
  return check_launch("swiglu");
}

extern "C" int tw_embedding(const int* ids, const void* table, void* out, long long ldo, int T, int H,
                            int vocab_start, int vocab_end, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldo % 8 != 0) {
    set_last_error("embedding: hidden size and stride must be multiples of 8");
    return 1;
  }
  int grid = T;
  const int cap = device_sm_count() * 8;
  if (grid > cap) grid = cap;
  embedding_kernel<<<grid, 256, 0, stream>>>(ids, reinterpret_cast<const __nv_bfloat16*>(table),
                                             reinterpret_cast<__nv_bfloat16*>(out), ldo, T, H, vocab_start,
                                             vocab_end);
  return check_launch("embedding");
}

extern "C" int tw_argmax(const float* logits, long long ld, int* out, int rows, int V, cudaStream_t stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, 1024, 0, stream>>>(logits, ld, out, V);
  return check_launch("argmax");
}
