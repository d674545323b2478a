// bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T  (nn.Linear layout, fp32 accumulate).
//
// Replaces the cuBLAS calls of the reference's linear layers
// (vllm/model_executor/layers/linear.py:196-230) and, in grouped mode, its Triton fused-MoE
// GEMM (vllm/model_executor/layers/fused_moe/fused_moe.py:255-463).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: A tile 128x64 and B tile BNx64 per pipeline stage
//               (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1      MMA issuer: tcgen05.mma kind::f16, M=128, N=BN, K=16, operands from shared
//               memory descriptors, accumulators in TMEM (two buffers, so the epilogue of
//               tile i overlaps the main loop of tile i+1)
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 32 columns -> registers -> bf16 -> global
// The tile width BN is a run-time value (a multiple of 32 up to 256; the instruction descriptor and
// the pipeline depth are computed from it), chosen per problem by a wave-quantisation cost model:
// skinny tensor-parallel shapes such as N = 1280 waste a third of the machine with 256-wide tiles.
// Epilogues: plain, +bias[n], *row_scale[m], and SwiGLU (the B tile holds BN/2 "gate" rows and
// BN/2 "up" rows; the stored value is silu(gate)*up, BN/2 output columns per tile).
// Grouped mode: each 128-row tile of A belongs to one expert (tile_expert[m_tile]); the B rows
// are offset by expert * n_per_expert; the number of valid tiles is read from device memory.
//
// Every mbarrier wait is bounded; on a timeout the CTA reports TW_ERR_MBAR_TIMEOUT, waits for
// its copies in flight, frees its TMEM and returns.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 16;
constexpr int GEMM_MAX_STAGES = 8;
constexpr int GEMM_A_BYTES = GEMM_BM * GEMM_BK * 2;
constexpr int GEMM_SMEM_BUDGET = 200 * 1024;   // pipeline stages; barriers and slack come on top
constexpr int GEMM_TMEM_COLS = 512;

struct GemmParams {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const float* row_scale;
  const float* col_scale;   // fp8 only: per-output-channel weight scale (may be null)
  int M, N, K;
  int num_m_tiles, num_n_tiles;
  const int* tile_expert;
  const int* num_m_tiles_dev;
  int n_per_expert;
  int up_row_offset;
  int bn;        // accumulator columns per tile
  int stages;    // pipeline depth
  int kb_per_stage;  // 64-wide k-blocks per stage: 2 halves the barrier round trips per FLOP
  uint32_t* status;
};

__host__ __device__ inline int gemm_stage_bytes(int bn) { return GEMM_A_BYTES + bn * GEMM_BK * 2; }

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_tile, int& n_tile) {
  const int group_span = GEMM_GROUP_M * num_n;
  const int group = t / group_span;
  const int first_m = group * GEMM_GROUP_M;
  const int rows = min(num_m - first_m, GEMM_GROUP_M);
  const int in_group = t - group * group_span;
  m_tile = first_m + in_group % rows;
  n_tile = in_group / rows;
}

// FP8: operands are e4m3 bytes, a k-block is 128 elements (the same 128 bytes per row), the MMA is
// kind::f8f6f4 (K = 32 per instruction) and the epilogue applies acc * row_scale[m] * col_scale[n] + bias[n].
template <bool SWIGLU, bool FP8>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  const int BN = p.bn;
  const int STAGES = p.stages;
  const int KBPS = p.kb_per_stage;                  // 64-wide k-blocks per pipeline stage (1 or 2)
  const int b_bytes = BN * GEMM_BK * 2;
  const int stage_bytes = KBPS * gemm_stage_bytes(BN);
  const int OUT_COLS = SWIGLU ? BN / 2 : BN;
  constexpr int BK_ELEMS = FP8 ? 2 * GEMM_BK : GEMM_BK;
  const uint32_t IDESC = FP8 ? make_idesc_e4m3(GEMM_BM, BN) : make_idesc_bf16(GEMM_BM, BN, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * stage_bytes);
  uint64_t* empty_bar = full_bar + GEMM_MAX_STAGES;
  uint64_t* acc_full = empty_bar + GEMM_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, GEMM_TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  int num_m = p.num_m_tiles;
  if (p.num_m_tiles_dev != nullptr) num_m = min(num_m, *p.num_m_tiles_dev);
  const int num_n = p.num_n_tiles;
  const int total_tiles = num_m * num_n;
  const int num_kb = ((p.K + BK_ELEMS - 1) / BK_ELEMS + KBPS - 1) / KBPS;   // pipeline iterations per tile

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        int m_tile, n_tile;
        tile_coords(t, num_m, num_n, m_tile, n_tile);
        const int m0 = m_tile * GEMM_BM;
        int b_row0 = n_tile * OUT_COLS;
        if (p.tile_expert != nullptr) b_row0 += p.tile_expert[m_tile] * p.n_per_expert;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_error(p.status, TW_ERR_MBAR_TIMEOUT);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + stage * stage_bytes;
          uint8_t* sb = sa + KBPS * GEMM_A_BYTES;
          mbar_expect_tx(&full_bar[stage], stage_bytes);
          for (int s = 0; s < KBPS; ++s) {
            // a k-block past the end of K reads zeros (out-of-bounds fill) and adds nothing
            const int kx = (kb * KBPS + s) * BK_ELEMS;
            tma_load_2d(sa + s * GEMM_A_BYTES, &tmA, &full_bar[stage], kx, m0);
            if (SWIGLU) {
              tma_load_2d(sb + s * b_bytes, &tmB, &full_bar[stage], kx, b_row0);
              tma_load_2d(sb + s * b_bytes + (BN / 2) * GEMM_BK * 2, &tmB, &full_bar[stage], kx,
                          b_row0 + p.up_row_offset);
            } else {
              tma_load_2d(sb + s * b_bytes, &tmB, &full_bar[stage], kx, b_row0);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report_error(p.status, TW_ERR_MBAR_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * 256;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint32_t sb = sa + KBPS * GEMM_A_BYTES;
          for (int s = 0; s < KBPS; ++s) {
            const uint64_t a_desc = make_smem_desc_sw128(sa + s * GEMM_A_BYTES, 16, 1024);
            const uint64_t b_desc = make_smem_desc_sw128(sb + s * b_bytes, 16, 1024);
#pragma unroll
            for (int k = 0; k < GEMM_BK / 16; ++k) {
              // 16 bf16 = 32 bytes further along K: +2 in the descriptor's 16-byte address units
              if (FP8)
                umma_ss_f8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | s | k) != 0 ? 1u : 0u);
              else
                umma_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | s | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) {
          report_error(p.status, TW_ERR_MBAR_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        umma_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      int m_tile, n_tile;
      tile_coords(t, num_m, num_n, m_tile, n_tile);
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = m_tile * GEMM_BM + q * 32 + lane;
      const int n0 = n_tile * OUT_COLS;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 256;
      const float rs = (p.row_scale != nullptr && row < p.M) ? p.row_scale[row] : 1.f;
      __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + n0;
#pragma unroll 1
      for (int c = 0; c < OUT_COLS / 32; ++c) {
        uint32_t v[32];
        uint32_t packed[16];
        tmem_ld_32x32(taddr + c * 32, v);
        if (SWIGLU) {
          uint32_t u[32];
          tmem_ld_32x32(taddr + BN / 2 + c * 32, u);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float g0 = __uint_as_float(v[2 * j]), g1 = __uint_as_float(v[2 * j + 1]);
            float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
            if (FP8) {
              // gate and up rows of the weight carry their own channel scales; the token scale (rs)
              // de-quantises both, so it goes in before the non-linearity
              const int n = min(n0 + c * 32 + 2 * j, p.N - 2);
              g0 *= rs;
              g1 *= rs;
              if (p.col_scale != nullptr) {
                g0 *= p.col_scale[n];
                g1 *= p.col_scale[n + 1];
                u0 *= p.col_scale[p.up_row_offset + n];
                u1 *= p.col_scale[p.up_row_offset + n + 1];
              }
              packed[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0 * rs, g1 / (1.f + __expf(-g1)) * u1 * rs);
              continue;
            }
            float s0 = g0 / (1.f + __expf(-g0)) * u0;
            float s1 = g1 / (1.f + __expf(-g1)) * u1;
            packed[j] = pack_bf16x2(s0 * rs, s1 * rs);
          }
        } else {
          tmem_wait_ld();
          if (FP8) {
            const int nc = n0 + c * 32;
            if (nc + 32 <= p.N && (p.N & 7) == 0) {
              // whole chunk in range: channel scales and bias come in as 16-byte vectors (the same
              // addresses for every thread of the warp, one transaction each)
              if (p.col_scale != nullptr) {
                const float4* cs4 = reinterpret_cast<const float4*>(p.col_scale + nc);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 s = __ldg(cs4 + j);
                  v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) * (rs * s.x));
                  v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) * (rs * s.y));
                  v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) * (rs * s.z));
                  v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) * (rs * s.w));
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * rs);
              }
              if (p.bias != nullptr) {
                const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + nc);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 b = __ldg(b4 + j);
                  const uint32_t* bu = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16x2(bu[e]);
                    v[8 * j + 2 * e] = __float_as_uint(__uint_as_float(v[8 * j + 2 * e]) + f.x);
                    v[8 * j + 2 * e + 1] = __float_as_uint(__uint_as_float(v[8 * j + 2 * e + 1]) + f.y);
                  }
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int n = nc + j;
                const float cs = (p.col_scale != nullptr && n < p.N) ? p.col_scale[n] : 1.f;
                const float b = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
                v[j] = __float_as_uint(__uint_as_float(v[j]) * rs * cs + b);
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          } else if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = n0 + c * 32 + j;
              const float b = (n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
              v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
            }
          }
          if (!FP8) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]) * rs, __uint_as_float(v[2 * j + 1]) * rs);
          }
        }
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = n0 + c * 32 + j * 8;
            if (n + 8 <= p.N) {
              *reinterpret_cast<uint4*>(crow + c * 32 + j * 8) =
                  make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
            } else if (n < p.N) {
              uint16_t* c16 = reinterpret_cast<uint16_t*>(crow + c * 32 + j * 8);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const uint32_t w = packed[4 * j + (e >> 1)];
                if (n + e < p.N) c16[e] = (e & 1) ? static_cast<uint16_t>(w >> 16) : static_cast<uint16_t>(w & 0xffffu);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------- tear-down ----------------
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before shared memory is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, GEMM_TMEM_COLS);
  }
}

template <bool SWIGLU, bool FP8>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  const int smem = p.stages * p.kb_per_stage * gemm_stage_bytes(p.bn) + 256 + 1024;
  auto kern = gemm_bf16_kernel<SWIGLU, FP8>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_last_error("cudaFuncSetAttribute(smem) failed: %s", cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("gemm launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

// Kernel and tile-width choice. Cost of a candidate = waves * per-tile time. Per-k-block tile times
// (arbitrary units, fitted to sweeps on B200 at K = 8192): a single-CTA tile costs 136 up to BN = 128
// and grows linearly to 208 at BN = 256 (below 128 columns the main loop is bound by the fixed
// issue/barrier cost per k-block, not by the tensor pipe); a CTA-pair tile (256 rows) costs 155 up to
// BN = 128 and 198 at BN = 256. A fixed number of k-block equivalents per tile covers prologue,
// pipeline refill and the non-overlapped part of the epilogue.
static int g_bn_override = 0;
static int g_kernel_override = 0;   // 0 auto, 1 single-CTA tiles, 2 CTA pairs

struct GemmPlan {
  bool pair;
  int bn;
};

static double tile_cost_single(int bn) { return bn <= 128 ? 136.0 : 136.0 + (bn - 128) * 0.5625; }
static double tile_cost_pair(int bn) { return bn <= 128 ? 155.0 : 155.0 + (bn - 128) * 0.336; }

static GemmPlan choose_plan(int M, int N, int K, int sms, bool swiglu, bool grouped) {
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
  const double kb_eff = num_kb + 6.0;
  GemmPlan best{false, 256};
  double best_cost = 1e30;
  const int step1 = swiglu ? 64 : 32;
  if (g_kernel_override != 2 || grouped) {
    const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
    for (int bn = 256; bn >= 64; bn -= step1) {
      if (g_bn_override > 0 && bn != g_bn_override) continue;
      const int out_cols = swiglu ? bn / 2 : bn;
      const long long tiles = static_cast<long long>(num_m) * ((N + out_cols - 1) / out_cols);
      const long long waves = (tiles + sms - 1) / sms;
      const double cost = waves * tile_cost_single(bn) * kb_eff;
      if (cost < best_cost * 0.999) {
        best_cost = cost;
        best = GemmPlan{false, bn};
      }
    }
  }
  const int pairs = sms / 2;
  if (!grouped && g_kernel_override != 1 && pairs >= 1 && (M >= 2048 || g_kernel_override == 2)) {
    const int num_m2 = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
    for (int bn = 256; bn >= 64; bn -= 64) {
      if (g_bn_override > 0 && bn != g_bn_override) continue;
      const int out_cols = swiglu ? bn / 2 : bn;
      const long long tiles = static_cast<long long>(num_m2) * ((N + out_cols - 1) / out_cols);
      const long long waves = (tiles + pairs - 1) / pairs;
      const double cost = waves * tile_cost_pair(bn) * kb_eff * 1.02;   // ties go to the simpler kernel
      if (cost < best_cost * 0.999) {
        best_cost = cost;
        best = GemmPlan{true, bn};
      }
    }
    // Wide tiles (one accumulator, two MMAs per k-step): worth it when they bring a skinny N down to ONE wave
    // where the narrower tiles need two or more (the tile cost per column keeps falling with the width, but
    // with one accumulator the epilogue of a tile no longer hides behind the next tile's main loop).
    if (!swiglu) {
      for (int bn = 320; bn <= 512; bn += 64) {
        if (g_bn_override > 0 && bn != g_bn_override) continue;
        const long long tiles = static_cast<long long>(num_m2) * ((N + bn - 1) / bn);
        if (tiles > pairs && g_bn_override != bn) continue;
        const long long waves = (tiles + pairs - 1) / pairs;
        const double cost = waves * (tile_cost_pair(bn) * kb_eff + 0.1 * bn) * 1.02;
        if (cost < best_cost * 0.999) {
          best_cost = cost;
          best = GemmPlan{true, bn};
        }
      }
    }
  }
  return best;
}

}  // namespace tw

using namespace tw;

// Forces the tile width (0 restores the cost model). For tuning runs and tests.
extern "C" int tw_gemm_set_tile_override(int bn) {
  g_bn_override = bn;
  return 0;
}
// Forces the kernel: 0 cost model, 1 single-CTA tiles, 2 CTA pairs.
extern "C" int tw_gemm_set_kernel_override(int kind) {
  g_kernel_override = kind;
  return 0;
}

extern "C" int tw_gemm_pair(int fp8, const void* A, long long lda, const void* B, long long ldb, long long rows_b,
                            void* C, long long ldc, const void* bias, const float* row_scale, const float* col_scale,
                            int M, int N, int K, int swiglu, int up_row_offset, int bn, int max_ctas,
                            const int* tile_expert, const int* num_m_tiles_dev, int n_per_expert, uint32_t* status,
                            cudaStream_t stream);

// Shared launcher body. A is [M,K] with row stride lda, B is [rows_b, K] with row stride ldb
// (rows_b = N, 2*N for SwiGLU, or experts * n_per_expert); strides count elements (2 bytes, or 1 for fp8).
static int gemm_dispatch(bool fp8, const void* A, long long lda, const void* B, long long ldb, long long rows_b,
                         void* C, long long ldc, const void* bias, const float* row_scale, const float* col_scale,
                         int M, int N, int K, int swiglu, int up_row_offset, const int* tile_expert,
                         const int* num_m_tiles_dev, int n_per_expert, int max_ctas, int plan_hint,
                         uint32_t* status, cudaStream_t stream, int group_tile_rows = 128) {
  // group_tile_rows: rows per entry of tile_expert (grouped mode). 256: the caller padded every expert to 256
  // rows, so the CTA-pair kernel can take the groups; 128: single-CTA tiles.
  // plan_hint: 0 = cost model; otherwise kernel * 1000 + tile width (kernel 1 = single-CTA tiles,
  // 2 = CTA pairs), as produced by the tuning table.
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int in_align = fp8 ? 16 : 8;   // 16 bytes of operand elements
  if ((K % in_align) != 0 || (lda % in_align) != 0 || (ldb % in_align) != 0 || (ldc % 8) != 0) {
    set_last_error("tw_gemm: K, lda, ldb must be multiples of %d and ldc of 8 (got %d, %lld, %lld, %lld)", in_align,
                   K, lda, ldb, ldc);
    return 1;
  }
  const int esz = fp8 ? 1 : 2;
  const int bk_elems = fp8 ? 2 * GEMM_BK : GEMM_BK;
  int sms = device_sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
  if (tile_expert != nullptr && group_tile_rows == 256 && sms >= 2)
    return tw_gemm_pair(fp8, A, lda, B, ldb, rows_b, C, ldc, bias, row_scale, col_scale, M, N, K, swiglu,
                        up_row_offset, 256, sms, tile_expert, num_m_tiles_dev, n_per_expert, status, stream);
  // the cost model sees k-blocks: an fp8 problem has K / 128 of them
  GemmPlan plan = choose_plan(M, N, fp8 ? K / 2 : K, sms, swiglu != 0, tile_expert != nullptr);
  if (plan_hint > 0) {
    const int kind = plan_hint / 1000, bn = plan_hint % 1000;
    const bool pair_ok = kind == 2 && tile_expert == nullptr && sms >= 2 && bn % 64 == 0 &&
                         (bn <= 256 || (bn <= 512 && !swiglu));
    const bool single_ok = kind == 1 && bn % (swiglu ? 64 : 32) == 0 && bn <= 256;
    if (bn >= 64 && (pair_ok || single_ok)) plan = GemmPlan{pair_ok, bn};
  }
  if (plan.pair)
    return tw_gemm_pair(fp8, A, lda, B, ldb, rows_b, C, ldc, bias, row_scale, col_scale, M, N, K, swiglu, up_row_offset,
                        plan.bn, sms, nullptr, nullptr, 0, status, stream);
  const int BN = plan.bn;
  const int out_cols = swiglu ? BN / 2 : BN;
  const int num_n = (N + out_cols - 1) / out_cols;
  // Two k-blocks per stage when at least three such stages fit (216 KB of pipeline at most), else one.
  int kbps = 1;
  int stages = GEMM_SMEM_BUDGET / gemm_stage_bytes(BN);
  if (K >= 4 * bk_elems && (216 * 1024) / (2 * gemm_stage_bytes(BN)) >= 3) {
    kbps = 2;
    stages = (216 * 1024) / (2 * gemm_stage_bytes(BN));
  }
  if (stages > GEMM_MAX_STAGES) stages = GEMM_MAX_STAGES;

  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)lda * esz};
    uint32_t box[2] = {(uint32_t)bk_elems, GEMM_BM};
    if (!(fp8 ? make_tensor_map_u8(&tmA, A, 2, dims, strides, box) : make_tensor_map_bf16(&tmA, A, 2, dims, strides, box)))
      return 1;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows_b};
    uint64_t strides[1] = {(uint64_t)ldb * esz};
    uint32_t box[2] = {(uint32_t)bk_elems, (uint32_t)(swiglu ? BN / 2 : BN)};
    if (!(fp8 ? make_tensor_map_u8(&tmB, B, 2, dims, strides, box) : make_tensor_map_bf16(&tmB, B, 2, dims, strides, box)))
      return 1;
  }
  GemmParams p;
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.row_scale = row_scale;
  p.col_scale = col_scale;
  p.M = M;
  p.N = N;
  p.K = K;
  p.num_m_tiles = num_m;
  p.num_n_tiles = num_n;
  p.tile_expert = tile_expert;
  p.num_m_tiles_dev = num_m_tiles_dev;
  p.n_per_expert = n_per_expert;
  p.up_row_offset = up_row_offset;
  p.bn = BN;
  p.stages = stages;
  p.kb_per_stage = kbps;
  p.status = status;
  int grid = num_m * num_n;
  if (grid > sms) grid = sms;
  if (fp8)
    return swiglu ? launch_gemm<true, true>(tmA, tmB, p, grid, stream)
                  : launch_gemm<false, true>(tmA, tmB, p, grid, stream);
  return swiglu ? launch_gemm<true, false>(tmA, tmB, p, grid, stream)
                : launch_gemm<false, false>(tmA, tmB, p, grid, stream);
}

extern "C" int tw_gemm_bf16(const void* A, long long lda, const void* B, long long ldb, long long rows_b,
                            void* C, long long ldc, const void* bias, const float* row_scale, int M,
                            int N, int K, int swiglu, int up_row_offset, const int* tile_expert,
                            const int* num_m_tiles_dev, int n_per_expert, int max_ctas, int plan_hint,
                            uint32_t* status, cudaStream_t stream) {
  return gemm_dispatch(false, A, lda, B, ldb, rows_b, C, ldc, bias, row_scale, nullptr, M, N, K, swiglu,
                       up_row_offset, tile_expert, num_m_tiles_dev, n_per_expert, max_ctas, plan_hint, status,
                       stream);
}

// Grouped GEMM over experts padded to 256 rows each: tile_expert has one entry per 256-row tile and the groups
// run on CTA pairs (cta_group::2, M = 256 per tile).
extern "C" int tw_gemm_bf16_grouped256(const void* A, long long lda, const void* B, long long ldb, long long rows_b,
                                       void* C, long long ldc, const float* row_scale, int M, int N, int K, int swiglu,
                                       int up_row_offset, const int* tile_expert, const int* num_m_tiles_dev,
                                       int n_per_expert, int max_ctas, uint32_t* status, cudaStream_t stream) {
  if (tile_expert == nullptr) {
    set_last_error("tw_gemm_bf16_grouped256: needs the tile -> expert map");
    return 1;
  }
  return gemm_dispatch(false, A, lda, B, ldb, rows_b, C, ldc, nullptr, row_scale, nullptr, M, N, K, swiglu,
                       up_row_offset, tile_expert, num_m_tiles_dev, n_per_expert, max_ctas, 0, status, stream, 256);
}

// e4m3 x e4m3 -> bf16: C = (A * B^T) * row_scale[m] * col_scale[n] + bias[n] (scales fp32, either may be
// null). The counterpart of the reference's CUTLASS sm100 fp8 scaled-mm
// (csrc/quantization/cutlass_w8a8/c3x/scaled_mm_sm100_fp8.cu) with per-token / per-channel scales.
extern "C" int tw_gemm_fp8(const void* A, long long lda, const void* B, long long ldb, long long rows_b, void* C,
                           long long ldc, const void* bias, const float* row_scale, const float* col_scale, int M,
                           int N, int K, int swiglu, int up_row_offset, const int* tile_expert,
                           const int* num_m_tiles_dev, int n_per_expert, int max_ctas, int plan_hint,
                           uint32_t* status, cudaStream_t stream) {
  return gemm_dispatch(true, A, lda, B, ldb, rows_b, C, ldc, bias, row_scale, col_scale, M, N, K, swiglu,
                       up_row_offset, tile_expert, num_m_tiles_dev, n_per_expert, max_ctas, plan_hint, status,
                       stream);
}

// int8 x int8 -> bf16 with 32-bit integer accumulation: C = (A * B^T) * row_scale[m] * col_scale[n] + bias[n]
// (symmetric quantisation; scales fp32, either may be null). Runs on CTA pairs (tcgen05 kind::i8). The counterpart
// of the reference's CUTLASS int8 scaled-mm (csrc/quantization/cutlass_w8a8/scaled_mm_entry.cu, symmetric case).
// With `swiglu` B is [gate; up] (2 N rows, the up rows `N` further down) and C = silu(gate part) * (up part).
extern "C" int tw_gemm_int8(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc,
                            const void* bias, const float* row_scale, const float* col_scale, int M, int N, int K,
                            int swiglu, int max_ctas, int plan_hint, uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int sms = device_sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int bn = 0;
  if (plan_hint / 1000 == 2) bn = plan_hint % 1000;
  if (bn > 256 && swiglu) bn = 256;
  if (bn == 0) {
    const GemmPlan plan = choose_plan(M, N, K / 2, sms, swiglu != 0, false);
    bn = plan.pair ? plan.bn : (N > 128 || swiglu ? 256 : 128);
  }
  return tw_gemm_pair(2, A, lda, B, ldb, swiglu ? 2LL * N : N, C, ldc, bias, row_scale, col_scale, M, N, K, swiglu,
                      swiglu ? N : 0, bn, sms, nullptr, nullptr, 0, status, stream);
}
