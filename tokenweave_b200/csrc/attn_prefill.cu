// Causal variable-length attention over a paged KV cache for sm_100a (prefill and chunked
// prefill). Replaces the FlashAttention-2 varlen call the reference falls back to on Blackwell
// (vllm/v1/attention/backends/flash_attn.py:713-733, vllm/attention/utils/fa_utils.py:29-34).
//
// One CTA per (128-query tile, query head), 320 threads:
//   warp 0      TMA producer: the Q tile once, then K and V tiles of 128 keys, one
//               cp.async.bulk.tensor.4d per cache page and 64-column half, straight from the
//               paged cache [blocks, page, kv_heads, D] through the request's block table
//   warp 1      MMA issuer (tcgen05, accumulators in TMEM):
//                 S[j&1] = Q K_j^T     (M=128, N=128, K=D, both operands K-major)
//                 O     += P_j V_j      (M=128, N=D,   K=128, V is an MN-major operand)
//               S is double-buffered, so Q K_{j+1}^T runs while the softmax of tile j does.
//   warps 2..9  softmax: TWO threads per query row, each owning 64 of the tile's 128 keys. A thread
//               reads its half row of S from TMEM once (64 registers), the two halves exchange their
//               maxima through shared memory, then exponentiate (exp2, scale folded in) and write
//               bf16 P into shared memory in the swizzled K-major operand layout. O stays in TMEM
//               across tiles and is rescaled only when the running maximum grows by more than 2^8
//               (the stale maximum is a valid softmax reference; P stays below 256).
// Every wait is bounded; a timeout reports TW_ERR_MBAR_TIMEOUT and leaves by the tear-down.
#include "attn_prefill_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

template <int D>
struct AttnSmem {
  static constexpr int HALVES = D / 64;
  static constexpr int Q_BYTES = HALVES * ATT_HALF_BYTES;
  static constexpr int KV_BYTES = HALVES * ATT_HALF_BYTES;  // one K or V tile
  static constexpr int P_BYTES = 2 * ATT_HALF_BYTES;        // 128 rows x 128 keys, bf16
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int OFF_XCHG = OFF_BAR + 256;            // float [2 parities][2 halves][128 rows]
  static constexpr int TOTAL = OFF_XCHG + 2 * 2 * 128 * 4 + 1024;
};

// The two threads of a query row sit in warps w and w + 4 (same TMEM lane quarter). Each such warp pair
// meets on its own named barrier (ids 1..4, 64 threads), so the four pairs drift apart in time and their
// load / max / exp2 / store phases overlap on the SM instead of marching in lockstep.
__device__ __forceinline__ void softmax_pair_sync(int quarter) {
  asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using S = AttnSmem<D>;
  constexpr int HALVES = S::HALVES;
  constexpr int OCOLS = D / 2;     // O columns per softmax thread
  constexpr uint32_t IDESC_QK = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(ATT_BM, D, 0, 1);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0;    // two S buffers: [0,128) and [128,256)
  constexpr uint32_t COL_O = 256;  // O accumulator: D columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* p_ready = bars + 11;
  uint64_t* o_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(smem + S::OFF_XCHG);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x;
  const int tile = blockIdx.y;
  const int kvh = head / (p.hq / p.hkv);

  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int q_begin = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q_begin;
  const int kv_len = p.kv_lens[seq];
  const int rows_valid = min(ATT_BM, q_len - q0);
  // absolute position of query i of the sequence: kv_len - q_len + i
  const int pos0 = kv_len - q_len + q0;
  const int kv_end = min(kv_len, pos0 + rows_valid);  // keys [0, kv_end) are needed
  const int n_tiles = (kv_end + ATT_BN - 1) / ATT_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_ready, ATT_SOFTMAX_THREADS);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_tiles > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, S::Q_BYTES);
#pragma unroll
      for (int h = 0; h < HALVES; ++h)
        tma_load_2d(smem + S::OFF_Q + h * ATT_HALF_BYTES, &tmQ, q_full, head * D + h * 64, q_begin + q0);
      const int pages_per_tile = ATT_BN / p.page;
      const int last_page = (kv_len - 1) / p.page;
      const int* table = p.block_table + static_cast<long long>(seq) * p.max_blocks;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        // K tile
        if (!mbar_wait(&k_empty[st], ph ^ 1)) { report_error(p.status, TW_ERR_MBAR_TIMEOUT); *abort_flag = 1; break; }
        mbar_expect_tx(&k_full[st], S::KV_BYTES);
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int block = table[min(j * pages_per_tile + pg, last_page)];
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_4d(smem + S::OFF_K + st * S::KV_BYTES + h * ATT_HALF_BYTES + pg * p.page * 128, &tmK,
                        &k_full[st], h * 64, kvh, 0, block);
        }
        // V tile
        if (!mbar_wait(&v_empty[st], ph ^ 1)) { report_error(p.status, TW_ERR_MBAR_TIMEOUT); *abort_flag = 1; break; }
        mbar_expect_tx(&v_full[st], S::KV_BYTES);
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int block = table[min(j * pages_per_tile + pg, last_page)];
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_4d(smem + S::OFF_V + st * S::KV_BYTES + h * ATT_HALF_BYTES + pg * p.page * 128, &tmV,
                        &v_full[st], h * 64, kvh, 0, block);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t q_addr = smem_u32(smem + S::OFF_Q);
      const uint32_t p_addr = smem_u32(smem + S::OFF_P);
      bool ok = mbar_wait(q_full, 0);
      auto issue_qk = [&](int j) {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + S::OFF_K + st * S::KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * ATT_HALF_BYTES + (k & 3) * 32;
          umma_ss(tmem_base + COL_S + st * ATT_BN, make_smem_desc_sw128(q_addr + off, 16, 1024),
                  make_smem_desc_sw128(k_addr + off, 16, 1024), IDESC_QK, k != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        if (!mbar_wait(p_ready, j & 1)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], (j >> 1) & 1)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + S::OFF_V + st * S::KV_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          const uint32_t a_off = (k >> 2) * ATT_HALF_BYTES + (k & 3) * 32;
          umma_ss(tmem_base + COL_O, make_smem_desc_sw128(p_addr + a_off, 16, 1024),
                  make_smem_desc_sw128(v_addr + k * 16 * 128, ATT_HALF_BYTES, 1024), IDESC_PV,
                  (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else if (n_tiles > 0) {
    // ---------------- softmax + epilogue (warps 2..9, two threads per row) ----------------
    const int qr = warp & 3;                        // TMEM lane quarter of this warp
    const int kh = (warp - 2) >> 2;                 // which 64-key half of the tile this thread owns
    const int r = qr * 32 + lane;                   // row within the tile
    const int pos = pos0 + min(r, rows_valid - 1);  // padding rows copy the last valid row's mask
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qr * 32) << 16);
    uint8_t* p_half = smem + S::OFF_P + kh * ATT_HALF_BYTES + r * 128;
    float m_ref = -INFINITY;  // softmax reference (a stale running maximum), log2 domain
    float l_sum = 0.f;        // this thread's half of the row sum
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      // The trip count is the same for all 256 threads whatever happens (the named barriers below are
      // unbounded): after a failed wait the remaining waits are skipped, not the iterations.
      const int sb = j & 1;
      if (ok) ok = mbar_wait(&s_full[sb], (j >> 1) & 1);
      tc_fence_after_sync();
      const uint32_t t_s = t_lane + COL_S + sb * ATT_BN + kh * 64;
      const int k_base = j * ATT_BN + kh * 64;      // first key of this thread's half
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(t_s, s0);
      tmem_ld_32x32(t_s + 32, s1);
      tmem_wait_ld();
      // warp-uniform: lane 0 holds the smallest position of the warp
      const bool need_mask = (k_base + 63) > __shfl_sync(0xffffffffu, pos, 0);
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (k_base + i > pos) s0[i] = __float_as_uint(-INFINITY);
          if (k_base + 32 + i > pos) s1[i] = __float_as_uint(-INFINITY);
        }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
      // the two halves of a row agree on the tile's maximum
      float* xm = xchg + (j & 1) * 256;
      xm[kh * 128 + r] = mx;
      softmax_pair_sync(qr);
      mx = fmaxf(mx, xm[(kh ^ 1) * 128 + r]) * p.scale_log2;
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_ref = mx;
      } else if (mx > m_ref + 8.f) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
        rescale = true;
      }
      // probabilities of this half row, packed to bf16 in registers
      uint32_t pk[32];
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float a = fast_exp2(__uint_as_float(s0[2 * i]) * p.scale_log2 - m_ref);
        const float b = fast_exp2(__uint_as_float(s0[2 * i + 1]) * p.scale_log2 - m_ref);
        const float c = fast_exp2(__uint_as_float(s1[2 * i]) * p.scale_log2 - m_ref);
        const float d = fast_exp2(__uint_as_float(s1[2 * i + 1]) * p.scale_log2 - m_ref);
        part += (a + b) + (c + d);
        pk[i] = pack_bf16x2(a, b);
        pk[16 + i] = pack_bf16x2(c, d);
      }
      l_sum = l_sum * alpha + part;
      if (j > 0) {
        // the P buffer and O are free once P_{j-1} V_{j-1} has completed
        if (ok) ok = mbar_wait(o_done, (j - 1) & 1);
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < OCOLS / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(t_lane + COL_O + kh * OCOLS + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(t_lane + COL_O + kh * OCOLS + c * 32, v);
          }
          tmem_wait_st();
        }
      }
      // 64 keys = eight 16-byte chunks of this row in the swizzled K-major operand layout
#pragma unroll
      for (int q8 = 0; q8 < 8; ++q8) {
        const int chunk = q8 ^ (r & 7);
        *reinterpret_cast<uint4*>(p_half + chunk * 16) =
            make_uint4(pk[4 * q8], pk[4 * q8 + 1], pk[4 * q8 + 2], pk[4 * q8 + 3]);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(p_ready);     // arrive even after a failed wait so the issuer is not left hanging
    }
    if (ok) ok = mbar_wait(o_done, (n_tiles - 1) & 1);
    // row sum = the two halves' partial sums
    float* xs = xchg + (n_tiles & 1) * 256;
    xs[kh * 128 + r] = l_sum;
    softmax_pair_sync(qr);
    const float l_row = l_sum + xs[(kh ^ 1) * 128 + r];
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.f / l_row;
      __nv_bfloat16* orow = p.out + static_cast<long long>(q_begin + q0 + r) * p.ldo + head * D + kh * OCOLS;
#pragma unroll 1
      for (int c = 0; c < OCOLS / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + COL_O + kh * OCOLS + c * 32, v);
        tmem_wait_ld();
        if (r < rows_valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * q4 + 0]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = o;
          }
        }
      }
    } else {
      report_error(p.status, TW_ERR_MBAR_TIMEOUT);
      *abort_flag = 1;
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------
// Head-pair variant: one CTA serves the SAME 128-query tile of TWO query heads that share a KV head
// (grouped-query attention), so every K and V tile is fetched once for both, and the two heads' softmax
// groups can run out of phase: while group A exponentiates tile j, the tensor core works on Q_B K_j^T
// and P_B V_{j-1}. Measured on B200 (8192 to 16384 tokens): 5 to 17 % faster than one head per CTA. The
// time does not depend on the head size (64 and 128 measure the same) nor on the depth of the K/V ring:
// the softmax warps (two per scheduler) bound it, at 44 % MUFU and 44 % tensor utilisation.
//   warp 0      TMA: Q_A and Q_B once; K_0 V_0 K_1 V_1 ... through a ring of tile slots (three fit
//               beside Q and P at head size 128, six at 64)
//   warp 1      MMA: S_A, S_B (one TMEM buffer each), O_A, O_B (TMEM, 4 x 128 columns in all)
//   warps 2..5  softmax of head A, one thread per query row (the row's 128 scores are read from TMEM
//               twice, in chunks of 32 through two register buffers, the next chunk's load in flight
//               while the current one is reduced or exponentiated); warps 6..9 the same for head B
template <int D>
struct AttnPairSmem {
  static constexpr int HALVES = D / 64;
  static constexpr int Q_BYTES = HALVES * ATT_HALF_BYTES;     // one head's Q tile
  static constexpr int KV_BYTES = HALVES * ATT_HALF_BYTES;    // one K or V tile
  static constexpr int P_BYTES = 2 * ATT_HALF_BYTES;          // one head's P tile: 128 rows x 128 keys
  static constexpr int RING_MAX = (D == 64) ? 6 : 3;           // K/V tile slots that fit beside Q and P
  static constexpr int OFF_Q = 0;                              // [2 heads]
  static constexpr int OFF_P = OFF_Q + 2 * Q_BYTES;            // [2 heads]
  static constexpr int OFF_RING = OFF_P + 2 * P_BYTES;         // [RING]
  static constexpr int OFF_BAR = OFF_RING + RING_MAX * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using S = AttnPairSmem<D>;
  constexpr int HALVES = S::HALVES;
  const int RING = p.ring;          // 3 .. RING_MAX slots in use
  constexpr uint32_t IDESC_QK = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(ATT_BM, D, 0, 1);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0;     // S_A at 0, S_B at 128
  constexpr uint32_t COL_O = 256;   // O_A at 256, O_B at 384

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* ring_full = bars + 1;    // [6]
  uint64_t* ring_empty = bars + 7;   // [6]
  uint64_t* s_full = bars + 13;      // [2 heads]
  uint64_t* p_ready = bars + 15;     // [2 heads]
  uint64_t* o_done = bars + 17;      // [2 heads]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head0 = blockIdx.x * 2;          // heads head0 and head0 + 1 share a KV head
  const int tile = blockIdx.y;
  const int kvh = head0 / (p.hq / p.hkv);

  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int q_begin = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q_begin;
  const int kv_len = p.kv_lens[seq];
  const int rows_valid = min(ATT_BM, q_len - q0);
  const int pos0 = kv_len - q_len + q0;
  const int kv_end = min(kv_len, pos0 + rows_valid);
  const int n_tiles = (kv_end + ATT_BN - 1) / ATT_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < RING; ++i) {
      mbar_init(&ring_full[i], 1);
      mbar_init(&ring_empty[i], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&p_ready[g], 128);
      mbar_init(&o_done[g], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_tiles > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * S::Q_BYTES);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(smem + S::OFF_Q + g * S::Q_BYTES + h * ATT_HALF_BYTES, &tmQ, q_full,
                      (head0 + g) * D + h * 64, q_begin + q0);
      const int pages_per_tile = ATT_BN / p.page;
      const int last_page = (kv_len - 1) / p.page;
      const int* table = p.block_table + static_cast<long long>(seq) * p.max_blocks;
      // stream of tiles K_0 V_0 K_1 V_1 ...: element i lives in ring slot i % 3
      for (int i = 0; i < 2 * n_tiles; ++i) {
        const int j = i >> 1;
        const int slot = i % RING;
        const uint32_t ph = (i / RING) & 1;
        if (!mbar_wait(&ring_empty[slot], ph ^ 1)) { report_error(p.status, TW_ERR_MBAR_TIMEOUT); *abort_flag = 1; break; }
        mbar_expect_tx(&ring_full[slot], S::KV_BYTES);
        const CUtensorMap* tm = (i & 1) ? &tmV : &tmK;
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int block = table[min(j * pages_per_tile + pg, last_page)];
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_4d(smem + S::OFF_RING + slot * S::KV_BYTES + h * ATT_HALF_BYTES + pg * p.page * 128, tm,
                        &ring_full[slot], h * 64, kvh, 0, block);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      bool ok = mbar_wait(q_full, 0);
      // S_g = Q_g K_j^T; K_j is stream element 2j. `last` releases the slot (both heads have read it).
      auto issue_qk = [&](int g, int j, bool last) {
        const int i = 2 * j, slot = i % RING;
        if (!mbar_wait(&ring_full[slot], (i / RING) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t q_addr = smem_u32(smem + S::OFF_Q + g * S::Q_BYTES);
        const uint32_t k_addr = smem_u32(smem + S::OFF_RING + slot * S::KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * ATT_HALF_BYTES + (k & 3) * 32;
          umma_ss(tmem_base + COL_S + g * ATT_BN, make_smem_desc_sw128(q_addr + off, 16, 1024),
                  make_smem_desc_sw128(k_addr + off, 16, 1024), IDESC_QK, k != 0 ? 1u : 0u);
        }
        if (last) umma_commit(&ring_empty[slot]);
        umma_commit(&s_full[g]);
        return true;
      };
      // O_g += P_g V_j; V_j is stream element 2j + 1.
      auto issue_pv = [&](int g, int j, bool last) {
        const int i = 2 * j + 1, slot = i % RING;
        if (!mbar_wait(&p_ready[g], j & 1)) return false;
        if (!mbar_wait(&ring_full[slot], (i / RING) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t p_addr = smem_u32(smem + S::OFF_P + g * S::P_BYTES);
        const uint32_t v_addr = smem_u32(smem + S::OFF_RING + slot * S::KV_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          const uint32_t a_off = (k >> 2) * ATT_HALF_BYTES + (k & 3) * 32;
          umma_ss(tmem_base + COL_O + g * 128, make_smem_desc_sw128(p_addr + a_off, 16, 1024),
                  make_smem_desc_sw128(v_addr + k * 16 * 128, ATT_HALF_BYTES, 1024), IDESC_PV,
                  (j | k) != 0 ? 1u : 0u);
        }
        if (last) umma_commit(&ring_empty[slot]);
        umma_commit(&o_done[g]);
        return true;
      };
      if (ok) ok = issue_qk(0, 0, false);
      if (ok) ok = issue_qk(1, 0, true);
      for (int j = 0; ok && j < n_tiles; ++j) {
        ok = issue_pv(0, j, false);
        if (ok && j + 1 < n_tiles) ok = issue_qk(0, j + 1, false);
        if (ok) ok = issue_pv(1, j, true);
        if (ok && j + 1 < n_tiles) ok = issue_qk(1, j + 1, true);
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else if (n_tiles > 0) {
    // ---------------- softmax + epilogue: warps 2..5 head A, warps 6..9 head B ----------------
    const int g = (warp - 2) >> 2;
    const int qr = warp & 3;                        // TMEM lane quarter of this warp
    const int r = qr * 32 + lane;                   // row within the tile
    const int pos = pos0 + min(r, rows_valid - 1);  // padding rows copy the last valid row's mask
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qr * 32) << 16);
    const uint32_t t_s = t_lane + COL_S + g * ATT_BN;
    const uint32_t t_o = t_lane + COL_O + g * 128;
    uint8_t* p_row = smem + S::OFF_P + g * S::P_BYTES + r * 128;
    float m_ref = -INFINITY;
    float l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (ok) ok = mbar_wait(&s_full[g], j & 1);
      tc_fence_after_sync();
      const int k_base = j * ATT_BN;
      const bool need_mask = (k_base + ATT_BN - 1) > __shfl_sync(0xffffffffu, pos, 0);
      // The row's 128 scores travel TMEM -> registers in four chunks of 32 columns through two register
      // buffers; the load of the next chunk is in flight while the current one is reduced or
      // exponentiated, and the reductions run on four independent accumulators (no 32-long chains).
      uint32_t s0[32], s1[32];
      auto mask_chunk = [&](uint32_t (&buf)[32], int chunk) {
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (k_base + chunk * 32 + i > pos) buf[i] = __float_as_uint(-INFINITY);
        }
      };
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto max_chunk = [&](const uint32_t (&buf)[32]) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          m4[0] = fmaxf(m4[0], __uint_as_float(buf[4 * i]));
          m4[1] = fmaxf(m4[1], __uint_as_float(buf[4 * i + 1]));
          m4[2] = fmaxf(m4[2], __uint_as_float(buf[4 * i + 2]));
          m4[3] = fmaxf(m4[3], __uint_as_float(buf[4 * i + 3]));
        }
      };
      // pass 1: row maximum; chunks 2 and 3 stay in registers for pass 2
      tmem_ld_32x32(t_s, s0);
      tmem_wait_ld();
      tmem_ld_32x32(t_s + 32, s1);
      mask_chunk(s0, 0);
      max_chunk(s0);
      tmem_wait_ld();
      tmem_ld_32x32(t_s + 64, s0);
      mask_chunk(s1, 1);
      max_chunk(s1);
      tmem_wait_ld();
      tmem_ld_32x32(t_s + 96, s1);
      mask_chunk(s0, 2);
      max_chunk(s0);
      tmem_wait_ld();
      mask_chunk(s1, 3);
      max_chunk(s1);
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_ref = mx;
      } else if (mx > m_ref + 8.f) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
        rescale = true;
      }
      // pass 2: exponentials. A chunk of 32 keys becomes 16 packed bf16 pairs = four 16-byte pieces of
      // the row in the swizzled K-major P tile.
      uint32_t pk0[16], pk1[16];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      auto exp_chunk = [&](const uint32_t (&buf)[32], uint32_t (&pk)[16]) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = fast_exp2(__uint_as_float(buf[2 * i]) * p.scale_log2 - m_ref);
          const float b = fast_exp2(__uint_as_float(buf[2 * i + 1]) * p.scale_log2 - m_ref);
          sum4[i & 3] += a + b;
          pk[i] = pack_bf16x2(a, b);
        }
      };
      auto store_chunk = [&](const uint32_t (&pk)[16], int chunk) {
        uint8_t* half = p_row + (chunk >> 1) * ATT_HALF_BYTES;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int piece = ((chunk & 1) * 4 + t) ^ (r & 7);
          *reinterpret_cast<uint4*>(half + piece * 16) = make_uint4(pk[4 * t], pk[4 * t + 1], pk[4 * t + 2], pk[4 * t + 3]);
        }
      };
      exp_chunk(s0, pk0);                 // chunk 2, still in registers
      tmem_ld_32x32(t_s, s0);             // chunk 0 comes back while chunk 3 is exponentiated
      exp_chunk(s1, pk1);                 // chunk 3
      if (j > 0) {
        // P_g and O_g are free once P_g V_{j-1} has completed
        if (ok) ok = mbar_wait(&o_done[g], (j - 1) & 1);
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, rescale)) {
          tmem_wait_ld();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(t_o + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, v);
          }
          tmem_wait_st();
        }
      }
      store_chunk(pk0, 2);
      store_chunk(pk1, 3);
      tmem_wait_ld();                     // chunk 0 has arrived
      tmem_ld_32x32(t_s + 32, s1);        // chunk 1 comes back while chunk 0 is exponentiated
      mask_chunk(s0, 0);
      exp_chunk(s0, pk0);
      store_chunk(pk0, 0);
      tmem_wait_ld();
      mask_chunk(s1, 1);
      exp_chunk(s1, pk1);
      store_chunk(pk1, 1);
      l_sum = l_sum * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&p_ready[g]);   // arrive even after a failed wait so the issuer is not left waiting
    }
    if (ok) ok = mbar_wait(&o_done[g], (n_tiles - 1) & 1);
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.f / l_sum;
      __nv_bfloat16* orow = p.out + static_cast<long long>(q_begin + q0 + r) * p.ldo + (head0 + g) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_o + c * 32, v);
        tmem_wait_ld();
        if (r < rows_valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * q4 + 0]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = o;
          }
        }
      }
    } else {
      report_error(p.status, TW_ERR_MBAR_TIMEOUT);
      *abort_flag = 1;
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

constexpr int ATTN_DEFAULT_VARIANT = 0;
constexpr bool ATTN_AUTO_SPLIT = true;   // what "automatic" picks: the persistent split kernel, or the per-tile kernels
static int g_attn_variant = ATTN_DEFAULT_VARIANT;   // 0 auto, 1 one head per CTA, 2 head pairs
static int g_attn_ring = 0;                          // 0: as many K/V slots as fit

template <int D>
static int launch_prefill_pair(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                               const AttnParams& p, int num_tiles, cudaStream_t stream) {
  using S = AttnPairSmem<D>;
  auto kern = attn_prefill_pair_kernel<D>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) {
      set_last_error("attn_prefill (head pairs): cudaFuncSetAttribute(smem=%d) failed: %s", S::TOTAL,
                     cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  dim3 grid(p.hq / 2, num_tiles);
  AttnParams pp = p;
  pp.ring = (g_attn_ring >= 3 && g_attn_ring <= S::RING_MAX) ? g_attn_ring : S::RING_MAX;
  kern<<<grid, ATT_THREADS, S::TOTAL, stream>>>(tmQ, tmK, tmV, pp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_prefill (head pairs) launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

template <int D>
static int launch_prefill(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                          const AttnParams& p, int num_tiles, cudaStream_t stream) {
  using S = AttnSmem<D>;
  auto kern = attn_prefill_kernel<D>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) {
      set_last_error("attn_prefill: cudaFuncSetAttribute(smem=%d) failed: %s", S::TOTAL,
                     cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  dim3 grid(p.hq, num_tiles);
  kern<<<grid, ATT_THREADS, S::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_prefill launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace tw

using namespace tw;

// q: [T, hq*D] rows with stride ldq (may alias a packed qkv buffer). Caches:
// [num_blocks, page, hkv, D]. tile_seq/tile_q0 list the 128-query tiles (device arrays).
extern "C" int tw_attn_prefill(const void* q, long long ldq, int T, const void* k_cache, const void* v_cache,
                               int num_blocks, int page, void* out, long long ldo, const int* cu_q,
                               const int* kv_lens, const int* block_table, int max_blocks,
                               const int* tile_seq, const int* tile_q0, int num_tiles, int hq, int hkv,
                               int D, float scale, int max_ctas, int window, float softcap, uint32_t* status,
                               cudaStream_t stream) {
  if (num_tiles <= 0 || T <= 0) return 0;
  if (D != 128 && D != 64) {
    set_last_error("attn_prefill: head_dim must be 64 or 128 (got %d)", D);
    return 1;
  }
  if (page < 8 || page > 128 || (128 % page) != 0) {
    set_last_error("attn_prefill: page size must divide 128 and be >= 8 (got %d)", page);
    return 1;
  }
  if (hq % hkv != 0 || ldq % 8 != 0 || ldo % 8 != 0) {
    set_last_error("attn_prefill: bad head counts or strides");
    return 1;
  }
  CUtensorMap tmQ, tmK, tmV;
  {
    uint64_t dims[2] = {(uint64_t)hq * D, (uint64_t)T};
    uint64_t strides[1] = {(uint64_t)ldq * 2};
    uint32_t box[2] = {64, ATT_BM};
    if (!make_tensor_map_bf16(&tmQ, q, 2, dims, strides, box)) return 1;
  }
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)hkv, (uint64_t)page, (uint64_t)num_blocks};
    uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)hkv * D * 2, (uint64_t)page * hkv * D * 2};
    uint32_t box[4] = {64, 1, (uint32_t)page, 1};
    if (!make_tensor_map_bf16(&tmK, k_cache, 4, dims, strides, box)) return 1;
    if (!make_tensor_map_bf16(&tmV, v_cache, 4, dims, strides, box)) return 1;
  }
  AttnParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.cu_q = cu_q;
  p.kv_lens = kv_lens;
  p.block_table = block_table;
  p.tile_seq = tile_seq;
  p.tile_q0 = tile_q0;
  p.max_blocks = max_blocks;
  p.page = page;
  p.hq = hq;
  p.hkv = hkv;
  p.ring = 3;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window > 0 ? window : 0;
  p.softcap = softcap > 0.f ? softcap : 0.f;
  p.scale = scale;
  p.status = status;
  // Persistent kernel with the key range of an item split between the softmax groups (variant 3): the
  // only one that honours an SM budget.
  // (sliding window and soft cap exist in that kernel only)
  if (g_attn_variant == 3 || (g_attn_variant == 0 && ATTN_AUTO_SPLIT) || p.window > 0 || p.softcap > 0.f)
    return launch_prefill_split(D, tmQ, tmK, tmV, p, num_tiles, max_ctas, stream);
  // Query heads that share a KV head go two to a CTA when the group size is even.
  const bool pair = ((hq / hkv) % 2 == 0) && g_attn_variant != 1;
  if (pair)
    return D == 128 ? launch_prefill_pair<128>(tmQ, tmK, tmV, p, num_tiles, stream)
                    : launch_prefill_pair<64>(tmQ, tmK, tmV, p, num_tiles, stream);
  return D == 128 ? launch_prefill<128>(tmQ, tmK, tmV, p, num_tiles, stream)
                  : launch_prefill<64>(tmQ, tmK, tmV, p, num_tiles, stream);
}

// Kernel choice for tuning runs and tests: 0 automatic, 1 one head per CTA, 2 head pairs where legal,
// 3 persistent CTAs with the key range split between the softmax groups,
// negative: back to the library default.
extern "C" int tw_attn_set_ring(int slots) {
  g_attn_ring = slots;
  return 0;
}
extern "C" int tw_attn_set_variant(int variant) {
  g_attn_variant = variant < 0 ? ATTN_DEFAULT_VARIANT : variant;
  return 0;
}
