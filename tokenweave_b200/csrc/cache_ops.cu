// KV-cache utilities and a column permutation: small memory-bound helpers next to the page copy / swap
// kernels of misc_ops.cu.
//
//   tw_gather_cache   the pages of each sequence, in block-table order, copied into one contiguous
//                     [tokens, kv_heads * D] buffer (csrc/cache_kernels.cu `gather_cache`: the input of
//                     kernels that want contiguous K / V, and of KV export)
//   tw_convert_fp8    a bf16 cache (or any bf16 tensor) to e4m3 with one scale, and back
//                     (csrc/cache_kernels.cu:264-305 `convert_fp8`: fp8 KV-cache storage)
//   tw_permute_cols   out[:, j] = in[:, perm[j]] for 16-bit elements (csrc/permute_cols.cu: activation
//                     reordering in front of act-order quantised weights)
#include <cuda_fp8.h>

#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

// grid (blocks of the longest sequence, sequences); each CTA copies the valid rows of one page
__global__ void __launch_bounds__(256)
gather_cache_kernel(const uint4* __restrict__ cache, uint4* __restrict__ dst, const int* __restrict__ block_table,
                    const int* __restrict__ cu_seq, int max_blocks, int page, int row_vec) {
  const int b = blockIdx.y, blk = blockIdx.x;
  const int seq_len = cu_seq[b + 1] - cu_seq[b];
  const int first = blk * page;
  if (first >= seq_len) return;
  const int rows = min(page, seq_len - first);
  const long long src0 = static_cast<long long>(block_table[static_cast<long long>(b) * max_blocks + blk]) * page * row_vec;
  const long long dst0 = (static_cast<long long>(cu_seq[b]) + first) * row_vec;
  const long long n = static_cast<long long>(rows) * row_vec;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) dst[dst0 + i] = cache[src0 + i];
}

template <bool TO_FP8>
__global__ void __launch_bounds__(256)
convert_fp8_kernel(const void* __restrict__ src, void* __restrict__ dst, long long n_vec, float scale) {
  // TO_FP8: 8 bf16 -> 8 e4m3 (x / scale); else 8 e4m3 -> 8 bf16 (x * scale)
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const float inv = 1.f / scale;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec; i += stride) {
    if (TO_FP8) {
      const uint4 v = reinterpret_cast<const uint4*>(src)[i];
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
      uint32_t o[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float2 a = unpack_bf16x2(u[2 * j]), b = unpack_bf16x2(u[2 * j + 1]);
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
        o[j] = lo | (hi << 16);
      }
      reinterpret_cast<uint2*>(dst)[i] = make_uint2(o[0], o[1]);
    } else {
      const uint2 v = reinterpret_cast<const uint2*>(src)[i];
      const uint32_t in[2] = {v.x, v.y};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((in[j] >> (16 * h)) & 0xffffu),
                                                           __NV_E4M3);
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r));
          o[2 * j + h] = pack_bf16x2(f.x * scale, f.y * scale);
        }
      }
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

__global__ void __launch_bounds__(256)
permute_cols_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, const int* __restrict__ perm, int rows,
                    int cols, long long ld_in, long long ld_out) {
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint16_t* src = in + r * ld_in;
    uint16_t* dst = out + r * ld_out;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = src[perm[c]];
  }
}

static int cache_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s launch failed: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

// cache: [num_blocks, page, row_elems] bf16 (row_elems = kv_heads * D, a multiple of 8); dst: [tokens, row_elems];
// cu_seq: [batch + 1] first destination row of each sequence (device); block_table: [batch, max_blocks].
extern "C" int tw_gather_cache(const void* cache, void* dst, const int* block_table, const int* cu_seq, int batch,
                               int max_blocks, int page, int row_elems, cudaStream_t stream) {
  if (batch <= 0 || max_blocks <= 0) return 0;
  if (row_elems % 8 != 0) {
    set_last_error("gather_cache: a cache row must be a multiple of 8 elements (got %d)", row_elems);
    return 1;
  }
  gather_cache_kernel<<<dim3(max_blocks, batch), 256, 0, stream>>>(
      reinterpret_cast<const uint4*>(cache), reinterpret_cast<uint4*>(dst), block_table, cu_seq, max_blocks, page,
      row_elems / 8);
  return cache_check("gather_cache");
}

// to_fp8 != 0: dst (e4m3) = src (bf16) / scale; else dst (bf16) = src (e4m3) * scale. n a multiple of 8.
extern "C" int tw_convert_fp8(const void* src, void* dst, long long n, float scale, int to_fp8, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || !(scale > 0.f)) {
    set_last_error("convert_fp8: element count must be a multiple of 8 and the scale positive");
    return 1;
  }
  const long long n_vec = n / 8;
  long long grid = (n_vec + 255) / 256;
  const long long cap = static_cast<long long>(device_sm_count()) * 8;
  if (grid > cap) grid = cap;
  if (to_fp8) convert_fp8_kernel<true><<<static_cast<int>(grid), 256, 0, stream>>>(src, dst, n_vec, scale);
  else convert_fp8_kernel<false><<<static_cast<int>(grid), 256, 0, stream>>>(src, dst, n_vec, scale);
  return cache_check("convert_fp8");
}

extern "C" int tw_permute_cols(const void* in, void* out, const int* perm, int rows, int cols, long long ld_in,
                               long long ld_out, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  int grid = rows;
  const int cap = device_sm_count() * 8;
  if (grid > cap) grid = cap;
  permute_cols_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint16_t*>(in), reinterpret_cast<uint16_t*>(out),
                                                perm, rows, cols, ld_in, ld_out);
  return cache_check("permute_cols");
}
