// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] = A[M,K] * B[N,K]^T, one 256 x BN output tile
// per pair of SMs.
//
// Why pairs: with one CTA per tile every SM pulls a 128x64 slice of A and a BNx64 slice of B from L2
// per k-block (48 KB at BN = 256). As a pair, each CTA loads its own 128 rows of A and only HALF of
// the B slice (32 KB per SM per k-block); the MMA unit of the leader CTA reads both halves. That cuts
// the L2 -> SM traffic per FLOP by a third and makes room for a deeper TMA pipeline (6 stages).
// No cluster-multicast copy is involved: every CTA issues ordinary tiled TMA loads into its own shared
// memory; only the completion signal goes to the leader's mbarrier (cta_group::2 form of the copy).
//
// Roles per CTA (320 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only; both CTAs'
// warp 1 take part in the paired TMEM allocation), warps 2..9 epilogue of the CTA's own 128 rows: two
// warps per 32-row slice of tensor memory (warp w reads lanes 32 (w % 4) ..), one taking the even and one
// the odd 32-column chunks of the tile, so that a tile with a short K loop (K = 1024: o_proj under 8-way
// tensor parallelism) is not held up by its own write-back.
// Barriers: full[s] lives in the leader and counts the bytes of both CTAs; empty[s] and acc_full[a]
// exist in both CTAs and are signalled by the leader's tcgen05.commit (one commit per CTA);
// acc_empty[a] lives in the leader and collects one arrival per epilogue warp of both CTAs.
// Write-back (tiles up to 256 columns): a thread owns one ROW of the accumulator, so direct stores would touch 32
// different lines per instruction, half a sector each. Instead every epilogue warp packs 32 rows x 32 columns
// of bf16 into its own 2 KB of shared memory (two buffers, the 64-byte swizzle of the tensor map: no bank
// conflicts) and one lane sends it with a TMA store, which writes whole sectors, clips the edges of C itself and
// leaves the warp free to fetch its next chunk. Wide tiles keep the direct stores (no shared memory to spare).
// FP8: operands are e4m3 bytes, a k-block is 128 elements (the same 128 bytes per row), the MMA is
// kind::f8f6f4 (K = 32 per instruction) and the epilogue applies acc * row_scale[m] * col_scale[n] + bias[n].
// INT8 (KIND 2): the same with signed 8-bit operands, kind::i8 and 32-bit integer accumulators that the epilogue
// converts to fp32 before scaling (the reference's CUTLASS int8 scaled-mm, csrc/quantization/cutlass_w8a8/).
// Wide tiles (256 < BN <= 512, plain epilogue only): one accumulator of BN columns, two MMAs of BN / 2
// columns per k-step. A skinny N (the QKV projection under 8-way tensor parallelism has N = 1280) then
// fits one wave of 256 x 320 tiles where 256-wide tiles need two waves at half occupancy. Each CTA holds
// a quarter of the tile's B rows per MMA: rows [r q, r q + q) and [2 q + r q, 2 q + r q + q) of the tile,
// q = BN / 4, r the CTA's rank, so that the columns of the two MMAs come out in order.
// Every wait is bounded (TW_ERR_MBAR_TIMEOUT); the pair leaves together through a cluster barrier.
#include <string.h>

#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int G2_BM = 128;          // rows per CTA (256 per pair)
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 320;
constexpr int G2_EPI_WARPS = 8;
constexpr int G2_GROUP_M = 8;       // pair-tiles per rasterisation group
constexpr int G2_MAX_STAGES = 8;
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;
constexpr int G2_SMEM_BUDGET = 192 * 1024;      // pipeline stages of the tiles up to 256 columns wide ...
constexpr int G2_EPI_STAGE_BYTES = G2_EPI_WARPS * 2 * 2048;   // ... plus two 32 x 32 bf16 staging buffers per epilogue warp
constexpr int G2_TMEM_COLS = 512;

struct Gemm2Params {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const float* row_scale;
  const float* col_scale;         // fp8 only: per-output-channel weight scale (may be null)
  int M, N, K;
  int num_m_tiles, num_n_tiles;   // in 256-row pair tiles
  // grouped mode (mixture of experts): pair tile m belongs to expert tile_expert[m], whose weights start
  // n_per_expert rows into B; the number of valid pair tiles is read from device memory
  const int* tile_expert;
  const int* num_m_tiles_dev;
  int n_per_expert;
  int up_row_offset;
  int bn, stages;
  int kb_per_stage;
  uint32_t* status;
};

static int g_pair_kbps = 2;   // 64-wide k-blocks per pipeline stage: 2 halves the barrier round trips per FLOP

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled TMA load into this CTA's shared memory whose completion bytes are credited to an mbarrier
// given by its cluster address (the leader's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ss_pair_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ss_pair_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Instruction descriptor for kind::i8: signed 8-bit A and B (format 1), 32-bit integer accumulator (format 2),
// both operands K-major.
__host__ __device__ constexpr uint32_t make_idesc_s8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
constexpr int KIND_BF16 = 0, KIND_E4M3 = 1, KIND_S8 = 2;
template <int KIND>
__device__ __forceinline__ void umma_pair_kind(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  if (KIND == KIND_E4M3) umma_ss_pair_f8(d_tmem, a_desc, b_desc, idesc, accumulate);
  else if (KIND == KIND_S8) umma_ss_pair_i8(d_tmem, a_desc, b_desc, idesc, accumulate);
  else umma_ss_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int t, int num_m, int num_n, int& m_tile, int& n_tile) {
  const int group_span = G2_GROUP_M * num_n;
  const int group = t / group_span;
  const int first_m = group * G2_GROUP_M;
  const int rows = min(num_m - first_m, G2_GROUP_M);
  const int in_group = t - group * group_span;
  m_tile = first_m + in_group % rows;
  n_tile = in_group / rows;
}

// WIDE is a template argument: the one thread that issues the MMAs sets the pace of the main loop, and the
// narrow kernel must not carry the wide one's extra instructions.
template <bool SWIGLU, bool WIDE, int KIND>
__global__ void __launch_bounds__(G2_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const Gemm2Params p) {
  const int BN = p.bn;
  const int HALF_N = BN / 2;                       // B rows held by each CTA
  const int STAGES = p.stages;
  const int KBPS = p.kb_per_stage;                 // 64-wide k-blocks per pipeline stage (1 or 2)
  const int b_half_bytes = HALF_N * G2_BK * 2;
  const int stage_bytes = KBPS * (G2_A_BYTES + b_half_bytes);
  const int OUT_COLS = SWIGLU ? BN / 2 : BN;
  // WIDE (BN > 256): two MMAs of BN / 2 columns per k-step, one accumulator
  const int MMA_N = WIDE ? BN / 2 : BN;
  constexpr int NUM_ACC = WIDE ? 1 : 2;
  constexpr bool FP8 = KIND != KIND_BF16;            // 8-bit operands (e4m3 or int8): scales in the epilogue
  const uint32_t IDESC = KIND == KIND_E4M3 ? make_idesc_e4m3(2 * G2_BM, MMA_N)
                         : KIND == KIND_S8 ? make_idesc_s8(2 * G2_BM, MMA_N)
                                           : make_idesc_bf16(2 * G2_BM, MMA_N, 0, 0);
  constexpr int BK_ELEMS = FP8 ? 2 * G2_BK : G2_BK;     // elements per k-block: 128 bytes of a row either way

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr bool TMA_EPI = !WIDE;                     // write-back through shared memory and TMA stores
  uint8_t* epi_stage = smem + STAGES * stage_bytes;   // 1024-byte aligned: the stage sizes are multiples of 4 KB
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + (TMA_EPI ? G2_EPI_STAGE_BYTES : 0));
  uint64_t* empty_bar = full_bar + G2_MAX_STAGES;
  uint64_t* acc_full = empty_bar + G2_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * G2_EPI_WARPS);   // the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, G2_TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (TMA_EPI) tma_prefetch_desc(&tmC);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before anyone signals across
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  int num_m = p.num_m_tiles;
  if (p.num_m_tiles_dev != nullptr) num_m = min(num_m, *p.num_m_tiles_dev);
  const int num_n = p.num_n_tiles;
  const int total_tiles = num_m * num_n;
  const int num_kb = ((p.K + BK_ELEMS - 1) / BK_ELEMS + KBPS - 1) / KBPS;   // pipeline iterations per tile
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < total_tiles && !*abort_flag; t += num_pairs) {
        int m_tile, n_tile;
        pair_tile_coords(t, num_m, num_n, m_tile, n_tile);
        const int m0 = m_tile * 2 * G2_BM + rank * G2_BM;
        const int e_row0 = p.tile_expert != nullptr ? p.tile_expert[m_tile] * p.n_per_expert : 0;
        int b_row0;
        if (SWIGLU) b_row0 = e_row0 + n_tile * OUT_COLS + (rank ? p.up_row_offset : 0);   // leader: gate rows, peer: up rows
        else b_row0 = e_row0 + n_tile * BN + rank * HALF_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_error(p.status, TW_ERR_MBAR_TIMEOUT);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + stage * stage_bytes;
          uint8_t* sb = sa + KBPS * G2_A_BYTES;
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * stage_bytes);
          for (int s = 0; s < KBPS; ++s) {
            // a k-block past the end of K reads zeros (out-of-bounds fill) and adds nothing
            const int kx = (kb * KBPS + s) * BK_ELEMS;
            tma_load_2d_pair(sa + s * G2_A_BYTES, &tmA, leader_full, kx, m0);
            if (WIDE) {
              // this CTA's quarter of the B rows of each of the two MMAs (the tensor map's box is BN / 4 rows)
              const int q = BN / 4;
              tma_load_2d_pair(sb + s * b_half_bytes, &tmB, leader_full, kx, e_row0 + n_tile * BN + rank * q);
              tma_load_2d_pair(sb + s * b_half_bytes + q * G2_BK * 2, &tmB, leader_full, kx,
                               e_row0 + n_tile * BN + 2 * q + rank * q);
            } else {
              tma_load_2d_pair(sb + s * b_half_bytes, &tmB, leader_full, kx, b_row0);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = pair; t < total_tiles && !*abort_flag; t += num_pairs) {
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
          const uint32_t sb = sa + KBPS * G2_A_BYTES;
          for (int s = 0; s < KBPS; ++s) {
            const uint64_t a_desc = make_smem_desc_sw128(sa + s * G2_A_BYTES, 16, 1024);
            const uint64_t b_desc = make_smem_desc_sw128(sb + s * b_half_bytes, 16, 1024);
#pragma unroll
            for (int k = 0; k < G2_BK / 16; ++k) {
              // 32 bytes further along K per instruction: +2 in the descriptor's 16-byte address units
              umma_pair_kind<KIND>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | s | k) != 0 ? 1u : 0u);
              if (WIDE) {
                // second half of the columns: the next BN / 4 rows of this CTA's B tile (and of the peer's)
                const uint64_t b2 = make_smem_desc_sw128(sb + s * b_half_bytes + (BN / 4) * G2_BK * 2, 16, 1024);
                umma_pair_kind<KIND>(d_tmem + MMA_N, a_desc + 2 * k, b2 + 2 * k, IDESC, (kb | s | k) != 0 ? 1u : 0u);
              }
            }
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          const uint32_t e_local = smem_u32(&empty_bar[stage]);
          umma_commit_pair(map_to_cta(e_local, 0));
          umma_commit_pair(map_to_cta(e_local, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) {
          report_error(p.status, TW_ERR_MBAR_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        const uint32_t f_local = smem_u32(&acc_full[acc]);
        umma_commit_pair(map_to_cta(f_local, 0));
        umma_commit_pair(map_to_cta(f_local, 1));
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9 of both CTAs) ----------------
    const int q = warp & 3;                  // this warp reads tensor-memory lanes 32 q .. 32 q + 31
    const int par = (warp - 2) >> 2;         // warps 2..5: even 32-column chunks, warps 6..9: odd ones
    int acc = 0;
    uint32_t acc_phase = 0;
    uint8_t* my_stage = epi_stage + (warp - 2) * 4096;
    int sbuf = 0;
    for (int t = pair; t < total_tiles && !*abort_flag; t += num_pairs) {
      int m_tile, n_tile;
      pair_tile_coords(t, num_m, num_n, m_tile, n_tile);
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = m_tile * 2 * G2_BM + rank * G2_BM + q * 32 + lane;
      const int n0 = n_tile * OUT_COLS;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 256;
      const float rs = (p.row_scale != nullptr && row < p.M) ? p.row_scale[row] : 1.f;
      __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + n0;
#pragma unroll 1
      for (int c = par; c < OUT_COLS / 32; c += 2) {
        uint32_t v[32];
        uint32_t packed[16];
        tmem_ld_32x32(taddr + c * 32, v);
        const int nc = n0 + c * 32;
        if (SWIGLU) {
          uint32_t u[32];
          tmem_ld_32x32(taddr + BN / 2 + c * 32, u);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float g0, g1, u0, u1;
            if (KIND == KIND_S8) {
              g0 = __int2float_rn(static_cast<int>(v[2 * j])), g1 = __int2float_rn(static_cast<int>(v[2 * j + 1]));
              u0 = __int2float_rn(static_cast<int>(u[2 * j])), u1 = __int2float_rn(static_cast<int>(u[2 * j + 1]));
            } else {
              g0 = __uint_as_float(v[2 * j]), g1 = __uint_as_float(v[2 * j + 1]);
              u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
            }
            if (FP8) {
              // gate and up rows of the weight carry their own channel scales; the token scale (rs)
              // de-quantises both, so it goes in before the non-linearity
              const int n = min(nc + 2 * j, p.N - 2);
              g0 *= rs;
              g1 *= rs;
              if (p.col_scale != nullptr) {
                g0 *= p.col_scale[n];
                g1 *= p.col_scale[n + 1];
                u0 *= p.col_scale[p.up_row_offset + n];
                u1 *= p.col_scale[p.up_row_offset + n + 1];
              }
            }
            packed[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0 * rs, g1 / (1.f + __expf(-g1)) * u1 * rs);
          }
        } else if (FP8) {
          tmem_wait_ld();
          if (KIND == KIND_S8) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__int2float_rn(static_cast<int>(v[j])));
          }
          if (nc + 32 <= p.N && (p.N & 7) == 0) {
            // whole chunk in range: channel scales and bias come in as 16-byte vectors (the same addresses
            // for every thread of the warp, one transaction each)
            if (p.col_scale != nullptr) {
              const float4* cs4 = reinterpret_cast<const float4*>(p.col_scale + nc);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 sc = __ldg(cs4 + j);
                v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) * (rs * sc.x));
                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) * (rs * sc.y));
                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) * (rs * sc.z));
                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) * (rs * sc.w));
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * rs);
            }
            if (p.bias != nullptr) {
              const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + nc);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 bv = __ldg(b4 + j);
                const uint32_t* bu = reinterpret_cast<const uint32_t*>(&bv);
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
              const float bb = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
              v[j] = __float_as_uint(__uint_as_float(v[j]) * rs * cs + bb);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        } else {
          tmem_wait_ld();
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = nc + j;
              const float bb = (n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
              v[j] = __float_as_uint(__uint_as_float(v[j]) + bb);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]) * rs, __uint_as_float(v[2 * j + 1]) * rs);
        }
        if (TMA_EPI) {
          uint8_t* dst = my_stage + sbuf * 2048;
          // the store sent from this buffer two chunks ago must have read it
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          // row `lane` of the 32 x 32 block: 64 bytes; its four 16-byte pieces are XOR-swizzled with bits 7..8 of the
          // row's offset (the 64-byte swizzle of the tensor map), which also spreads a quarter-warp over all banks
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(dst + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, dst, nc, m_tile * 2 * G2_BM + static_cast<int>(rank) * G2_BM + q * 32);
            tma_store_commit();
          }
          sbuf ^= 1;
        } else if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = nc + j * 8;
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
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------- tear-down ----------------
  if (TMA_EPI && warp >= 2 && lane == 0) tma_store_wait_all<0>();   // shared memory stays until the stores have left
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                 // nobody signals a barrier of, or reads TMEM paired with, an exited CTA
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, G2_TMEM_COLS);
  }
}

template <bool SWIGLU, bool WIDE, int KIND>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const Gemm2Params& p,
                       int pairs, cudaStream_t stream) {
  const int stage_bytes = p.kb_per_stage * (G2_A_BYTES + (p.bn / 2) * G2_BK * 2);
  const int smem = p.stages * stage_bytes + (WIDE ? 0 : G2_EPI_STAGE_BYTES) + 256 + 1024;
  auto kern = gemm_bf16_pair_kernel<SWIGLU, WIDE, KIND>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_last_error("gemm pair: cudaFuncSetAttribute(smem) failed: %s", cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(G2_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, p);
  if (e != cudaSuccess) {
    set_last_error("gemm pair launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

// 1 or 2 k-blocks (of 64) per pipeline stage of the CTA-pair kernel; for tuning runs.
extern "C" int tw_gemm_set_pair_kbps(int kbps) {
  g_pair_kbps = (kbps == 1) ? 1 : 2;
  return 0;
}

// Same contract as tw_gemm_bf16 / tw_gemm_fp8 (`fp8`: 0 bf16 operands, 1 e4m3, 2 signed int8; the 8-bit kinds take
// row and column scales). `bn` is the tile width (multiple of 64, <= 256, or up to 512
// without SwiGLU), `max_ctas` bounds the SMs used (rounded down to an even number). Grouped mode: tile_expert has
// one entry per 256-row tile of A (the caller pads every expert to 256 rows). Strides count elements (2 bytes, or 1
// for fp8).
extern "C" int tw_gemm_pair(int fp8, const void* A, long long lda, const void* B, long long ldb, long long rows_b,
                            void* C, long long ldc, const void* bias, const float* row_scale, const float* col_scale,
                            int M, int N, int K, int swiglu, int up_row_offset, int bn, int max_ctas,
                            const int* tile_expert, const int* num_m_tiles_dev, int n_per_expert, uint32_t* status,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int in_align = fp8 ? 16 : 8;     // 16 bytes of operand elements
  if ((K % in_align) != 0 || (lda % in_align) != 0 || (ldb % in_align) != 0 || (ldc % 8) != 0 || bn % 64 != 0 ||
      bn < 64 || bn > 512 || (bn > 256 && swiglu) || fp8 < 0 || fp8 > 2) {
    set_last_error("tw_gemm_pair: bad strides or tile width (K=%d, bn=%d)", K, bn);
    return 1;
  }
  int sms = device_sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int pairs_avail = sms / 2;
  if (pairs_avail < 1) {
    set_last_error("tw_gemm_pair: needs at least 2 SMs");
    return 1;
  }
  const int esz = fp8 ? 1 : 2;
  const int bk_elems = fp8 ? 2 * G2_BK : G2_BK;
  const int num_m = (M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int out_cols = swiglu ? bn / 2 : bn;
  const int num_n = (N + out_cols - 1) / out_cols;
  int kbps = (g_pair_kbps == 2 && K >= 4 * bk_elems) ? 2 : 1;
  // wide tiles: two k-blocks per stage only while three such stages fit (216 KB of pipeline at most)
  if (bn > 256 && (216 * 1024) / (2 * (G2_A_BYTES + (bn / 2) * G2_BK * 2)) < 3) kbps = 1;
  const int stage_bytes = kbps * (G2_A_BYTES + (bn / 2) * G2_BK * 2);
  int stages = (bn > 256 ? 216 * 1024 : G2_SMEM_BUDGET) / stage_bytes;
  if (stages > G2_MAX_STAGES) stages = G2_MAX_STAGES;

  CUtensorMap tmA, tmB, tmC;
  {
    // C as the TMA stores of the epilogue see it: 32 x 32 blocks of bf16; rows and columns past M and N are clipped
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)ldc * 2};
    uint32_t box[2] = {32, 32};
    if (!make_tensor_map_bf16_sw64(&tmC, C, 2, dims, strides, box)) return 1;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)lda * esz};
    uint32_t box[2] = {(uint32_t)bk_elems, G2_BM};
    if (!(fp8 ? make_tensor_map_u8(&tmA, A, 2, dims, strides, box) : make_tensor_map_bf16(&tmA, A, 2, dims, strides, box)))
      return 1;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows_b};
    uint64_t strides[1] = {(uint64_t)ldb * esz};
    uint32_t box[2] = {(uint32_t)bk_elems, (uint32_t)(bn > 256 ? bn / 4 : bn / 2)};   // wide tiles: two loads of a quarter each
    if (!(fp8 ? make_tensor_map_u8(&tmB, B, 2, dims, strides, box) : make_tensor_map_bf16(&tmB, B, 2, dims, strides, box)))
      return 1;
  }
  Gemm2Params p;
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
  p.up_row_offset = up_row_offset;
  p.tile_expert = tile_expert;
  p.num_m_tiles_dev = num_m_tiles_dev;
  p.n_per_expert = n_per_expert;
  p.bn = bn;
  p.stages = stages;
  p.kb_per_stage = kbps;
  p.status = status;
  int pairs = num_m * num_n;
  if (pairs > pairs_avail) pairs = pairs_avail;
  if (fp8 == 2) {
    if (bn > 256) return launch_pair<false, true, KIND_S8>(tmA, tmB, tmC, p, pairs, stream);
    return swiglu ? launch_pair<true, false, KIND_S8>(tmA, tmB, tmC, p, pairs, stream)
                  : launch_pair<false, false, KIND_S8>(tmA, tmB, tmC, p, pairs, stream);
  }
  if (fp8) {
    if (bn > 256) return launch_pair<false, true, KIND_E4M3>(tmA, tmB, tmC, p, pairs, stream);
    return swiglu ? launch_pair<true, false, KIND_E4M3>(tmA, tmB, tmC, p, pairs, stream)
                  : launch_pair<false, false, KIND_E4M3>(tmA, tmB, tmC, p, pairs, stream);
  }
  if (bn > 256) return launch_pair<false, true, KIND_BF16>(tmA, tmB, tmC, p, pairs, stream);
  return swiglu ? launch_pair<true, false, KIND_BF16>(tmA, tmB, tmC, p, pairs, stream)
                : launch_pair<false, false, KIND_BF16>(tmA, tmB, tmC, p, pairs, stream);
}

extern "C" int tw_gemm_bf16_pair(const void* A, long long lda, const void* B, long long ldb, long long rows_b,
                                 void* C, long long ldc, const void* bias, const float* row_scale, int M, int N,
                                 int K, int swiglu, int up_row_offset, int bn, int max_ctas, const int* tile_expert,
                                 const int* num_m_tiles_dev, int n_per_expert, uint32_t* status,
                                 cudaStream_t stream) {
  return tw_gemm_pair(0, A, lda, B, ldb, rows_b, C, ldc, bias, row_scale, nullptr, M, N, K, swiglu, up_row_offset, bn,
                      max_ctas, tile_expert, num_m_tiles_dev, n_per_expert, status, stream);
}
