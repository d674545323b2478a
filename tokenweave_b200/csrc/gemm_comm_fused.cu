// GEMM fused with its neighbouring collective, ONE kernel each, over NVSwitch multicast / peer memory:
//
//   tw_gemm_rs_norm     row-parallel GEMM (o_proj, down_proj) -> reduce-scatter -> residual add ->
//                       RMSNorm. GEMM CTAs write partial-sum tiles into the local copy of the symmetric
//                       buffer and, per finished tile, bump a counter on the rank that owns those
//                       rows; that rank's communication CTAs (same kernel, other CTAs) wait for the
//                       counter of a row block, pull the block summed over all ranks
//                       (multimem.ld_reduce, or peer loads), add the residual, normalise and store
//                       the normalised rows in the local copy. The reduction of a row block starts as
//                       soon as every rank has produced it, tile by tile, while the tensor cores are
//                       still busy with later tiles.
//   tw_ag_gemm          all-gather -> column-parallel GEMM (qkv_proj, gate_up_proj with SwiGLU).
//                       Communication CTAs broadcast this rank's normalised shard to every rank
//                       (multimem.st, or peer stores) and then publish a per-shard epoch flag; GEMM CTAs
//                       start with the tiles of their own shard (already local) and wait, per row
//                       tile, for the flag of the shard it comes from. No kernel-wide barrier anywhere.
//
// Reference counterparts: RowParallelLinear in-place GEMM + fused_rs_ln_cta + multimem_ag_cta run as
// separate kernels with stream order between them (vllm/model_executor/layers/linear.py:1290-1334,
// csrc/tokenweave_artifact_kernels.cu:129-204,379-426); nothing in the reference overlaps a GEMM with
// its own collective.
//
// Synchronisation is by flags in symmetric memory only: tile counters (reset by their consumer) and
// per-shard epochs (monotonic, read from device memory so a CUDA graph can replay the kernels). Every
// wait is bounded and reports TW_ERR_FLAG_TIMEOUT / TW_ERR_MBAR_TIMEOUT through the status word. The
// kernels are launched cooperatively-sized (grid <= SM count, one CTA per SM) so that GEMM CTAs and
// communication CTAs are co-resident; they never wait on each other in a cycle.
#include <string.h>

#include "comm.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int FG_BM = 128;
constexpr int FG_BK = 64;
constexpr int FG_THREADS = 512;           // GEMM role uses warps 0..5, communication role all 16
constexpr int FG_MAX_STAGES = 8;
constexpr int FG_A_BYTES = FG_BM * FG_BK * 2;
constexpr int FG_SMEM_BUDGET = 200 * 1024;
constexpr int FG_TMEM_COLS = 512;
constexpr int FG_MAX_VPT = 2;             // 16-byte vectors of a row per communication thread (H <= 8192)

struct FusedGemmParams {
  // GEMM
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  int M, N, K;
  int num_m_tiles, num_n_tiles;
  int up_row_offset;
  int bn, stages;
  int kb_per_stage;
  // collective
  uint8_t* mc_base;
  uint8_t* const* peer_bases;
  int rank, world;
  unsigned long long budget_ns;
  uint32_t* status;
  long long off_bytes;          // start of the [T_pad, H] region inside the symmetric buffer
  int rows_per_rank;            // T_pad / world
  int H;
  int comm_ctas;
  // tw_gemm_rs_norm
  uint32_t* const* tile_flags;  // [world] -> per-rank counters, one per 128-row block of that rank's shard
  __nv_bfloat16* residual;      // this rank's shard of the residual stream
  long long ldr;
  const __nv_bfloat16* weight;
  float eps;
  // tw_ag_gemm
  uint32_t* const* shard_flags; // [world] -> per-rank array of `world` epochs (entry s: shard s has arrived)
  uint32_t* epoch;              // this rank's call counter for the region (device memory)
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Waits until *p >= target (wrap-safe). One thread polls; callers broadcast the outcome.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target, unsigned long long budget_ns) {
  if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i)
      if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
    if (globaltimer_ns() - t0 > budget_ns) return false;
  }
}

__device__ __forceinline__ uint4 fg_reduce16(const FusedGemmParams& p, long long off) {
  if (p.mc_base != nullptr) return multimem_ld_reduce_bf16x8(p.mc_base + off);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int s = 0; s < p.world; ++s) {
    int peer = p.rank + 1 + s;
    if (peer >= p.world) peer -= p.world;
    const uint4 v = ld_sys_16(p.peer_bases[peer] + off);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                    pack_bf16x2(acc[6], acc[7]));
}
__device__ __forceinline__ void fg_broadcast16(const FusedGemmParams& p, long long off, const uint4& v) {
  if (p.mc_base != nullptr) {
    multimem_st_16(p.mc_base + off, v);
    return;
  }
  for (int s = 0; s < p.world; ++s) {
    int peer = p.rank + s;
    if (peer >= p.world) peer -= p.world;
    st_sys_16(p.peer_bases[peer] + off, v);
  }
}

// ---------------------------------------------------------------------------------------------
// Communication role of tw_gemm_rs_norm: for each 128-row block of this rank's shard, wait until every
// rank has produced all its tiles of the block, then RS + residual add + RMSNorm two rows at a time.
__device__ void rs_norm_role(const FusedGemmParams& p, float* scratch, int* s_ok) {
  constexpr int ROWS = 2;
  const int nvec = p.H >> 3;
  const long long row_bytes = static_cast<long long>(p.H) * 2;
  const long long shard_off = p.off_bytes + static_cast<long long>(p.rank) * p.rows_per_rank * row_bytes;
  uint8_t* local_base = p.peer_bases[p.rank];
  uint32_t* my_flags = p.tile_flags[p.rank];
  const int shard_row0 = p.rank * p.rows_per_rank;
  const int blocks = (p.rows_per_rank + FG_BM - 1) / FG_BM;
  uint4 wv[FG_MAX_VPT];
#pragma unroll
  for (int i = 0; i < FG_MAX_VPT; ++i) {
    const int v = threadIdx.x + i * FG_THREADS;
    wv[i] = (v < nvec) ? reinterpret_cast<const uint4*>(p.weight)[v] : make_uint4(0, 0, 0, 0);
  }
  for (int b = 0; b < blocks; ++b) {
    // Tiles of rows [first, last] of the global matrix feed this block; a tile covers 128 global rows, so
    // when shards are smaller than a tile the block is fed by exactly one row tile.
    const int g_first = shard_row0 + b * FG_BM;
    const int g_last = min(shard_row0 + min((b + 1) * FG_BM, p.rows_per_rank), p.M) - 1;
    uint32_t target = 0;
    if (g_last >= g_first) {
      const int tiles = g_last / FG_BM - g_first / FG_BM + 1;
      target = static_cast<uint32_t>(tiles) * p.num_n_tiles * p.world;
    }
    if (threadIdx.x == 0) {
      int ok = 1;
      if (target > 0 && !wait_flag_ge(&my_flags[b], target, p.budget_ns)) ok = 0;
      *s_ok = ok;
    }
    __syncthreads();
    if (!*s_ok) {
      if (threadIdx.x == 0) report_error(p.status, TW_ERR_FLAG_TIMEOUT);
      return;
    }
    const int rows_in_block = min(FG_BM, p.rows_per_rank - b * FG_BM);
    for (int g = blockIdx.x * ROWS; g < rows_in_block; g += p.comm_ctas * ROWS) {
      uint4 x[ROWS][FG_MAX_VPT];
      float ss[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = b * FG_BM + g + r;
#pragma unroll
        for (int i = 0; i < FG_MAX_VPT; ++i) {
          const int v = threadIdx.x + i * FG_THREADS;
          x[r][i] = make_uint4(0, 0, 0, 0);
          if (v < nvec && g + r < rows_in_block) x[r][i] = fg_reduce16(p, shard_off + row * row_bytes + v * 16);
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = b * FG_BM + g + r;
        ss[r] = 0.f;
#pragma unroll
        for (int i = 0; i < FG_MAX_VPT; ++i) {
          const int v = threadIdx.x + i * FG_THREADS;
          if (v < nvec && g + r < rows_in_block) {
            uint4* rp = reinterpret_cast<uint4*>(p.residual + row * p.ldr) + v;
            const uint4 rv = *rp;
            x[r][i].x = add_bf16x2(x[r][i].x, rv.x);
            x[r][i].y = add_bf16x2(x[r][i].y, rv.y);
            x[r][i].z = add_bf16x2(x[r][i].z, rv.z);
            x[r][i].w = add_bf16x2(x[r][i].w, rv.w);
            *rp = x[r][i];
            const uint32_t* u = reinterpret_cast<const uint32_t*>(&x[r][i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(u[j]);
              ss[r] += f.x * f.x + f.y * f.y;
            }
          }
        }
      }
      block_sum<ROWS>(ss, scratch);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int row = b * FG_BM + g + r;
        const float inv = rsqrtf(ss[r] / static_cast<float>(p.H) + p.eps);
#pragma unroll
        for (int i = 0; i < FG_MAX_VPT; ++i) {
          const int v = threadIdx.x + i * FG_THREADS;
          if (v < nvec && g + r < rows_in_block) {
            const uint32_t* u = reinterpret_cast<const uint32_t*>(&x[r][i]);
            const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv[i]);
            uint4 o;
            uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(u[j]);
              ou[j] = mul_bf16x2(pack_bf16x2(f.x * inv, f.y * inv), wu[j]);
            }
            *reinterpret_cast<uint4*>(local_base + shard_off + row * row_bytes + v * 16) = o;
          }
        }
      }
    }
    // The counter goes back to zero once every communication CTA is done with the block: the last one to
    // finish (a second counter right behind the tile counters) resets both.
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* done = &my_flags[blocks + b];
      if (atomicAdd(done, 1u) + 1u == static_cast<uint32_t>(p.comm_ctas)) {
        my_flags[b] = 0;
        *done = 0;
        __threadfence();
      }
    }
  }
}

// Communication role of tw_ag_gemm: broadcast this rank's shard rows, then publish the epoch.
__device__ void ag_role(const FusedGemmParams& p, uint32_t epoch) {
  const long long row_bytes = static_cast<long long>(p.H) * 2;
  const long long n_vec = static_cast<long long>(p.rows_per_rank) * (p.H >> 3);
  const long long shard_off = p.off_bytes + static_cast<long long>(p.rank) * p.rows_per_rank * row_bytes;
  uint8_t* local_base = p.peer_bases[p.rank];
  const long long stride = static_cast<long long>(p.comm_ctas) * FG_THREADS;
  constexpr int UNROLL = 4;
  for (long long i0 = blockIdx.x * static_cast<long long>(FG_THREADS) + threadIdx.x; i0 < n_vec; i0 += stride * UNROLL) {
    uint4 x[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < n_vec) x[u] = *reinterpret_cast<const uint4*>(local_base + shard_off + i * 16);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < n_vec) {
        if (p.mc_base != nullptr) {
          multimem_st_16(p.mc_base + shard_off + i * 16, x[u]);
        } else {
          for (int s = 1; s < p.world; ++s) {
            int peer = p.rank + s;
            if (peer >= p.world) peer -= p.world;
            st_sys_16(p.peer_bases[peer] + shard_off + i * 16, x[u]);
          }
        }
      }
    }
  }
  // Every communication CTA's stores precede the flag: each CTA fences and counts itself in; the last one
  // publishes the epoch to all ranks.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* counter = p.shard_flags[p.rank] + p.world;      // one spare word behind the epochs
    if (atomicAdd(counter, 1u) + 1u == static_cast<uint32_t>(p.comm_ctas)) {
      *counter = 0;
      __threadfence_system();
      for (int s = 0; s < p.world; ++s) st_release_sys(p.shard_flags[s] + p.rank, epoch);
    }
  }
}

// Every CTA of tw_ag_gemm read the call counter when it started; the counter moves on only after the
// last CTA of the grid is done (p.epoch[1] counts finished CTAs), so a CTA that starts late still sees
// the value its peers saw.
__device__ __forceinline__ void finish_epoch(const FusedGemmParams& p, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.epoch + 1, 1u) + 1u == gridDim.x) {
      p.epoch[1] = 0;
      __threadfence();
      p.epoch[0] = epoch;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// MODE 0: tw_gemm_rs_norm (GEMM tiles signal their owners), MODE 1: tw_ag_gemm (tiles wait for shards).
template <int MODE, bool SWIGLU>
__global__ void __launch_bounds__(FG_THREADS, 1)
fused_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const FusedGemmParams p) {
  const int BN = p.bn;
  const int STAGES = p.stages;
  const int KBPS = p.kb_per_stage;                  // 64-wide k-blocks per pipeline stage (1 or 2)
  const int b_bytes = BN * FG_BK * 2;
  const int stage_bytes = KBPS * (FG_A_BYTES + b_bytes);
  const int OUT_COLS = SWIGLU ? BN / 2 : BN;
  const uint32_t IDESC = make_idesc_bf16(FG_BM, BN, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ float scratch[2 * 32];
  __shared__ int s_ok;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t epoch = (MODE == 1) ? (*p.epoch + 1u) : 0u;

  if (static_cast<int>(blockIdx.x) < p.comm_ctas) {
    // ---------------- communication CTAs ----------------
    if (MODE == 0) rs_norm_role(p, scratch, &s_ok);
    else ag_role(p, epoch);
    if (MODE == 1) finish_epoch(p, epoch);
    return;
  }

  // ---------------- GEMM CTAs ----------------
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * stage_bytes);
  uint64_t* empty_bar = full_bar + FG_MAX_STAGES;
  uint64_t* acc_full = empty_bar + FG_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int cta = blockIdx.x - p.comm_ctas;
  const int num_ctas = gridDim.x - p.comm_ctas;

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
    tmem_alloc(tmem_slot, FG_TMEM_COLS);
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

  const int num_m = p.num_m_tiles, num_n = p.num_n_tiles;
  const int total_tiles = num_m * num_n;
  const int num_kb = ((p.K + FG_BK - 1) / FG_BK + KBPS - 1) / KBPS;   // pipeline iterations per tile
  // Row tiles in the order their inputs become available: MODE 1 starts with this rank's own shard and
  // walks the ring; MODE 0 keeps the natural order (all ranks finish row block 0 first, so rank 0's
  // communication CTAs start first, rank world-1's last).
  const int m_rot = (MODE == 1) ? ((p.rank * p.rows_per_rank) / FG_BM) % num_m : 0;
  auto tile_of = [&](int t, int& m_tile, int& n_tile) {
    // n fastest inside a row tile: a row block completes (MODE 0) / is consumed (MODE 1) as one unit
    m_tile = (t / num_n + m_rot) % num_m;
    n_tile = t % num_n;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cta; t < total_tiles && !*abort_flag; t += num_ctas) {
        int m_tile, n_tile;
        tile_of(t, m_tile, n_tile);
        const int m0 = m_tile * FG_BM;
        if (MODE == 1) {
          // rows m0 .. m0+127 come from shards s_lo .. s_hi: wait for their epochs
          const int last_row = min(m0 + FG_BM, p.M) - 1;
          const int s_lo = m0 / p.rows_per_rank, s_hi = last_row / p.rows_per_rank;
          bool ok = true;
          for (int s = s_lo; s <= s_hi && ok; ++s)
            if (s != p.rank) ok = wait_flag_ge(p.shard_flags[p.rank] + s, epoch, p.budget_ns);
          if (!ok) {
            report_error(p.status, TW_ERR_FLAG_TIMEOUT);
            *abort_flag = 1;
            break;
          }
          fence_proxy_async_all();   // rows written by other GPUs are read by the TMA unit next
        }
        const int b_row0 = n_tile * OUT_COLS;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_error(p.status, TW_ERR_MBAR_TIMEOUT);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + stage * stage_bytes;
          uint8_t* sb = sa + KBPS * FG_A_BYTES;
          mbar_expect_tx(&full_bar[stage], stage_bytes);
          for (int s = 0; s < KBPS; ++s) {
            const int kx = (kb * KBPS + s) * FG_BK;   // past the end of K: zero fill
            tma_load_2d(sa + s * FG_A_BYTES, &tmA, &full_bar[stage], kx, m0);
            if (SWIGLU) {
              tma_load_2d(sb + s * b_bytes, &tmB, &full_bar[stage], kx, b_row0);
              tma_load_2d(sb + s * b_bytes + (BN / 2) * FG_BK * 2, &tmB, &full_bar[stage], kx, b_row0 + p.up_row_offset);
            } else {
              tma_load_2d(sb + s * b_bytes, &tmB, &full_bar[stage], kx, b_row0);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = cta; t < total_tiles && !*abort_flag; t += num_ctas) {
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
          const uint32_t sb = sa + KBPS * FG_A_BYTES;
          for (int s = 0; s < KBPS; ++s) {
            const uint64_t a_desc = make_smem_desc_sw128(sa + s * FG_A_BYTES, 16, 1024);
            const uint64_t b_desc = make_smem_desc_sw128(sb + s * b_bytes, 16, 1024);
#pragma unroll
            for (int k = 0; k < FG_BK / 16; ++k)
              umma_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | s | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
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
  } else if (warp < 6) {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = cta; t < total_tiles && !*abort_flag; t += num_ctas) {
      int m_tile, n_tile;
      tile_of(t, m_tile, n_tile);
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = m_tile * FG_BM + q * 32 + lane;
      const int n0 = n_tile * OUT_COLS;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 256;
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
            packed[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
          }
        } else {
          tmem_wait_ld();
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = n0 + c * 32 + j;
              const float b = (n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
              v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
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
      if (MODE == 0) {
        // The tile is in (local) global memory once all four epilogue warps have stored their rows.
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence_system();
          const int first_row = m_tile * FG_BM;
          const int last_row = min(first_row + FG_BM, p.M) - 1;
          // every 128-row block of every owner that this tile overlaps gets one count (shards need not
          // be aligned to tiles, so a tile can feed two blocks of one owner and blocks of two owners)
          for (int o = first_row / p.rows_per_rank; o <= last_row / p.rows_per_rank; ++o) {
            const int base = o * p.rows_per_rank;
            const int lo = max(first_row, base) - base;
            const int hi = min(last_row, base + p.rows_per_rank - 1) - base;
            for (int b = lo / FG_BM; b <= hi / FG_BM; ++b) red_release_sys_add(p.tile_flags[o] + b, 1u);
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, FG_TMEM_COLS);
  }
  if (MODE == 1) finish_epoch(p, epoch);
}

static int pick_bn(int M, int N, int gemm_ctas, bool swiglu) {
  const int num_m = (M + FG_BM - 1) / FG_BM;
  double best_cost = 1e30;
  int best = 256;
  for (int bn = 256; bn >= 64; bn -= swiglu ? 64 : 32) {
    const int out_cols = swiglu ? bn / 2 : bn;
    const long long tiles = static_cast<long long>(num_m) * ((N + out_cols - 1) / out_cols);
    const long long waves = (tiles + gemm_ctas - 1) / gemm_ctas;
    const double cost = waves * (bn <= 128 ? 136.0 : 136.0 + (bn - 128) * 0.5625);
    if (cost < best_cost * 0.999) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

template <int MODE>
static int launch_fused(const void* A, long long lda, const void* B, long long ldb, long long rows_b, int swiglu,
                        FusedGemmParams& p, int max_ctas, cudaStream_t stream) {
  if ((p.K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (p.ldc % 8) != 0 || p.H % 8 != 0 ||
      p.H / 8 > FG_MAX_VPT * FG_THREADS) {
    set_last_error("fused gemm: unsupported strides or hidden size (K=%d, H=%d)", p.K, p.H);
    return 1;
  }
  int sms = device_sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (p.comm_ctas < 1 || p.comm_ctas >= sms) {
    set_last_error("fused gemm: comm_ctas=%d must be in [1, %d)", p.comm_ctas, sms);
    return 1;
  }
  const int gemm_ctas_max = sms - p.comm_ctas;
  p.bn = pick_bn(p.M, p.N, gemm_ctas_max, swiglu != 0);
  const int out_cols = swiglu ? p.bn / 2 : p.bn;
  p.num_m_tiles = (p.M + FG_BM - 1) / FG_BM;
  p.num_n_tiles = (p.N + out_cols - 1) / out_cols;
  const int one_kb = FG_A_BYTES + p.bn * FG_BK * 2;
  p.kb_per_stage = (p.K >= 256 && FG_SMEM_BUDGET / (2 * one_kb) >= 3) ? 2 : 1;
  p.stages = FG_SMEM_BUDGET / (p.kb_per_stage * one_kb);
  if (p.stages > FG_MAX_STAGES) p.stages = FG_MAX_STAGES;
  int gemm_ctas = p.num_m_tiles * p.num_n_tiles;
  if (gemm_ctas > gemm_ctas_max) gemm_ctas = gemm_ctas_max;
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.M};
    uint64_t strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {FG_BK, FG_BM};
    if (!make_tensor_map_bf16(&tmA, A, 2, dims, strides, box)) return 1;
  }
  {
    uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)rows_b};
    uint64_t strides[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {FG_BK, (uint32_t)(swiglu ? p.bn / 2 : p.bn)};
    if (!make_tensor_map_bf16(&tmB, B, 2, dims, strides, box)) return 1;
  }
  const int smem = p.stages * p.kb_per_stage * one_kb + 256 + 1024;
  void (*kern)(CUtensorMap, CUtensorMap, FusedGemmParams) =
      swiglu ? fused_gemm_kernel<MODE, true> : fused_gemm_kernel<MODE, false>;
  // the kernel also has a few hundred bytes of static shared memory, so the dynamic part cannot take
  // the whole 227 KB
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FG_SMEM_BUDGET + 4096);
  if (e != cudaSuccess) {
    set_last_error("fused gemm: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return 1;
  }
  kern<<<p.comm_ctas + gemm_ctas, FG_THREADS, smem, stream>>>(tmA, tmB, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("fused gemm launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

static void fill_comm(FusedGemmParams& p, void* mc_base, void* const* peer_bases, int rank, int world,
                      unsigned long long budget_ns, uint32_t* status, long long off_bytes, int T, int H, int comm_ctas) {
  p.mc_base = reinterpret_cast<uint8_t*>(mc_base);
  p.peer_bases = reinterpret_cast<uint8_t* const*>(peer_bases);
  p.rank = rank;
  p.world = world;
  p.budget_ns = budget_ns;
  p.status = status;
  p.off_bytes = off_bytes;
  p.rows_per_rank = T / world;
  p.H = H;
  p.comm_ctas = comm_ctas;
}

// Row-parallel GEMM + reduce-scatter + residual add + RMSNorm. `out_local` is this rank's copy of the
// [T, N] region of the symmetric buffer (row stride N) that starts `off_bytes` into the buffer: the GEMM
// writes its partial sums there; on return this rank's shard rows [rank*T/world, (rank+1)*T/world) hold
// rmsnorm(sum over ranks + residual) * weight and the residual shard (row stride ldr) is updated.
// T (padded token count) must be a multiple of world; the first M <= T rows are computed.
// tile_flags: device array of `world` pointers to each rank's 2 * ceil(T/world/128) zero-initialised words.
extern "C" int tw_gemm_rs_norm(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                               const void* bias, void* out_local, void* mc_base, void* const* peer_bases,
                               uint32_t* const* tile_flags, int rank, int world, unsigned long long budget_ns,
                               uint32_t* status, long long off_bytes, int T, void* residual, long long ldr,
                               const void* weight, float eps, int comm_ctas, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || T <= 0) return 0;
  if (T % world != 0 || M > T) {
    set_last_error("tw_gemm_rs_norm: T=%d must be a multiple of world=%d and >= M=%d", T, world, M);
    return 1;
  }
  FusedGemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = reinterpret_cast<__nv_bfloat16*>(out_local);
  p.ldc = N;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.M = M;
  p.N = N;
  p.K = K;
  fill_comm(p, mc_base, peer_bases, rank, world, budget_ns, status, off_bytes, T, N, comm_ctas);
  p.tile_flags = tile_flags;
  p.residual = reinterpret_cast<__nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.weight = reinterpret_cast<const __nv_bfloat16*>(weight);
  p.eps = eps;
  return launch_fused<0>(A, lda, B, ldb, N, 0, p, max_ctas, stream);
}

// All-gather + column-parallel GEMM. `a_local` is this rank's copy of the [T, H] region (row stride H) whose
// shard rows [rank*T/world, ...) hold this rank's normalised activations; they are broadcast to every rank
// and C[M, N] = region[:M] * B^T (+bias, or SwiGLU with B = [gate; up]) is computed as the shards arrive.
// shard_flags: device array of `world` pointers to each rank's world + 1 words (zero-initialised);
// epoch: this rank's call counter for the region (one zero-initialised word of device memory).
extern "C" int tw_ag_gemm(const void* a_local, const void* B, long long ldb, long long rows_b, void* C, long long ldc,
                          const void* bias, int M, int N, int K, int swiglu, int up_row_offset, void* mc_base,
                          void* const* peer_bases, uint32_t* const* shard_flags, uint32_t* epoch, int rank, int world,
                          unsigned long long budget_ns, uint32_t* status, long long off_bytes, int T, int comm_ctas,
                          int max_ctas, cudaStream_t stream) {
  if (M <= 0 || T <= 0) return 0;
  if (T % world != 0 || M > T) {
    set_last_error("tw_ag_gemm: T=%d must be a multiple of world=%d and >= M=%d", T, world, M);
    return 1;
  }
  FusedGemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.M = M;
  p.N = N;
  p.K = K;
  p.up_row_offset = up_row_offset;
  fill_comm(p, mc_base, peer_bases, rank, world, budget_ns, status, off_bytes, T, K, comm_ctas);
  p.shard_flags = shard_flags;
  p.epoch = epoch;
  return launch_fused<1>(a_local, K, B, ldb, rows_b, swiglu, p, max_ctas, stream);
}
