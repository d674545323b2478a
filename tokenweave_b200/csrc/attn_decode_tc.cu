// Single-query ("decode") attention on the tensor cores for grouped-query models, head size 128.
//
// The SIMT decode kernel (attn_decode.cu) spends its time issuing FMAs: every key costs G x D
// multiply-adds for the scores and as many for the values, and at 8 query heads per KV head that is
// what bounds it, not memory. Here the G query heads of a KV group are the N dimension of two small
// tcgen05 MMAs with the KEYS (scores) and the HEAD DIMENSION (values) as M, so that the 128-row tiles
// of the tensor core are full even though a token has only G <= 16 query rows:
//
//   S^T[128 keys, 16]  = K_j[128 keys, D]   . Q[16, D]^T        (A, B K-major; N = 16 >= G)
//   O^T[D = 128, 16]  += V_j^T[D, 128 keys] . P^T[16, 128 keys]  (A = V MN-major; B = P K-major)
//
// One CTA per (token, KV head, split), 192 threads:
//   warp 0      TMA: K and V tiles of 128 keys through a ring of 3 slots each, one 4-D box per cache
//               page and 64-column half, straight from the paged cache through the block table
//   warp 1      MMA issuer; S^T double-buffered in TMEM (2 x 16 columns), O^T in 16 more
//   warps 2..5  softmax: thread r owns KEY r of the tile (TMEM lane r of S^T: 16 scores, one per
//               head). The per-head maximum over the tile's keys is a warp reduction (one
//               redux.sync.max.f32 per head) plus a four-way exchange through shared memory; P goes to shared memory as bf16 in the
//               swizzled K-major operand layout (row = head, column = key). In the epilogue the
//               same thread owns output column d = r (TMEM lane r of O^T).
// O is rescaled lazily (only when a head's running maximum grew by more than 2^8), as in the prefill
// kernel. With splits > 1 the un-normalised O, the reference maximum and the sum go to the partial
// buffers that attn_decode_merge_kernel reduces. Every wait is bounded.
#include "tw_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int DTC_D = 128;
constexpr int DTC_BN = 128;                 // keys per tile
constexpr int DTC_NH = 16;                  // N of both MMAs (query heads, zero-padded)
constexpr int DTC_RING = 3;
constexpr int DTC_THREADS = 64 + 128;
constexpr int DTC_HALF_BYTES = 128 * 128;   // [128 rows x 64 bf16], 128-byte swizzle
constexpr int DTC_KV_BYTES = 2 * DTC_HALF_BYTES;
constexpr int DTC_Q_BYTES = 2 * DTC_NH * 128;    // [16 x 128] bf16 as two swizzled halves
constexpr int DTC_P_BYTES = 2 * DTC_NH * 128;    // [16 heads x 128 keys] bf16, two 64-key blocks
constexpr int DTC_OFF_K = 0;
constexpr int DTC_OFF_V = DTC_OFF_K + DTC_RING * DTC_KV_BYTES;
constexpr int DTC_OFF_Q = DTC_OFF_V + DTC_RING * DTC_KV_BYTES;
constexpr int DTC_OFF_P = DTC_OFF_Q + DTC_Q_BYTES;             // two buffers
constexpr int DTC_OFF_BAR = DTC_OFF_P + 2 * DTC_P_BYTES;
constexpr int DTC_OFF_XCHG = DTC_OFF_BAR + 256;               // float [2][4 warps][16]
constexpr int DTC_SMEM = DTC_OFF_XCHG + 2 * 4 * 16 * 4 + 1024;

__device__ __forceinline__ float dtc_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void dtc_softmax_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

struct DecodeTcParams {
  const __nv_bfloat16* q;
  long long ldq;
  __nv_bfloat16* out;
  long long ldo;
  const int* tok_row;
  const int* tok_seq;
  const int* tok_kvlen;
  const int* block_table;
  int max_blocks, page, hq, hkv, splits;
  float scale_log2;
  float* part_o;
  float* part_ml;
  uint32_t* status;
};

// GT: query heads per KV head as a compile-time constant (4, 8 or 16), or 0 to read it from the arguments. The
// softmax costs a few instructions per head, key and tile, all in the 128 threads that own the keys; with the
// group size known the loops over the 16 columns of S^T shrink to the heads that exist.
template <int GT>
__global__ void __launch_bounds__(DTC_THREADS, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const DecodeTcParams p) {
  constexpr uint32_t IDESC_S = make_idesc_bf16(DTC_BN, DTC_NH, 0, 0);   // A = K (K-major), B = Q (K-major)
  constexpr uint32_t IDESC_O = make_idesc_bf16(DTC_D, DTC_NH, 1, 0);    // A = V (MN-major), B = P (K-major)
  constexpr uint32_t TMEM_COLS = 64;
  constexpr uint32_t COL_S = 0;     // two S^T buffers of 16 columns
  constexpr uint32_t COL_O = 32;    // O^T: 16 columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DTC_OFF_BAR);
  uint64_t* k_full = bars + 0;    // [3]
  uint64_t* k_empty = bars + 3;   // [3]
  uint64_t* v_full = bars + 6;    // [3]
  uint64_t* v_empty = bars + 9;   // [3]
  uint64_t* s_full = bars + 12;   // [2]
  uint64_t* p_ready = bars + 14;
  uint64_t* o_done = bars + 15;
  uint64_t* q_ready = bars + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(smem + DTC_OFF_XCHG);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = GT > 0 ? GT : p.hq / p.hkv;
  const int row = p.tok_row[tok];
  const int seq = p.tok_seq[tok];
  const int kv_len = p.tok_kvlen[tok];
  const int tiles_total = (kv_len + DTC_BN - 1) / DTC_BN;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int t_begin = split * tiles_per_split;
  const int t_end = min(tiles_total, t_begin + tiles_per_split);
  const int n_tiles = max(0, t_end - t_begin);

  if (threadIdx.x == 0) {
    for (int i = 0; i < DTC_RING; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    mbar_init(q_ready, 128);
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
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int pages_per_tile = DTC_BN / p.page;
      const int last_page = (kv_len - 1) / p.page;
      const int* table = p.block_table + static_cast<long long>(seq) * p.max_blocks;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % DTC_RING;
        const uint32_t ph = (j / DTC_RING) & 1;
        const int tile = t_begin + j;
        if (!mbar_wait(&k_empty[st], ph ^ 1)) { report_error(p.status, TW_ERR_MBAR_TIMEOUT); *abort_flag = 1; break; }
        mbar_expect_tx(&k_full[st], DTC_KV_BYTES);
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int block = table[min(tile * pages_per_tile + pg, last_page)];
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_4d(smem + DTC_OFF_K + st * DTC_KV_BYTES + h * DTC_HALF_BYTES + pg * p.page * 128, &tmK,
                        &k_full[st], h * 64, kvh, 0, block);
        }
        if (!mbar_wait(&v_empty[st], ph ^ 1)) { report_error(p.status, TW_ERR_MBAR_TIMEOUT); *abort_flag = 1; break; }
        mbar_expect_tx(&v_full[st], DTC_KV_BYTES);
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int block = table[min(tile * pages_per_tile + pg, last_page)];
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_4d(smem + DTC_OFF_V + st * DTC_KV_BYTES + h * DTC_HALF_BYTES + pg * p.page * 128, &tmV,
                        &v_full[st], h * 64, kvh, 0, block);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t q_addr = smem_u32(smem + DTC_OFF_Q);
      bool ok = mbar_wait(q_ready, 0);
      auto issue_s = [&](int j) {
        const int st = j % DTC_RING;
        if (!mbar_wait(&k_full[st], (j / DTC_RING) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + DTC_OFF_K + st * DTC_KV_BYTES);
#pragma unroll
        for (int k = 0; k < DTC_D / 16; ++k) {
          // 16 elements of the head dimension per instruction: 32 bytes along the swizzled 128-byte row
          const uint32_t a_off = (k >> 2) * DTC_HALF_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * (DTC_NH * 128) + (k & 3) * 32;
          umma_ss(tmem_base + COL_S + (j & 1) * DTC_NH, make_smem_desc_sw128(k_addr + a_off, 16, 1024),
                  make_smem_desc_sw128(q_addr + b_off, 16, 1024), IDESC_S, k != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int st = j % DTC_RING;
        if (!mbar_wait(p_ready, j & 1)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], (j / DTC_RING) & 1)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + DTC_OFF_V + st * DTC_KV_BYTES);
        const uint32_t p_addr = smem_u32(smem + DTC_OFF_P + (j & 1) * DTC_P_BYTES);
#pragma unroll
        for (int k = 0; k < DTC_BN / 16; ++k) {
          // 16 keys per instruction: 16 rows of the V tile, 32 bytes along P's key axis
          const uint32_t b_off = (k >> 2) * (DTC_NH * 128) + (k & 3) * 32;
          umma_ss(tmem_base + COL_O, make_smem_desc_sw128(v_addr + k * 16 * 128, DTC_HALF_BYTES, 1024),
                  make_smem_desc_sw128(p_addr + b_off, 16, 1024), IDESC_O, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..5) ----------------
    const int qr = warp & 3;                 // TMEM lane quarter this warp may touch
    const int r = qr * 32 + lane;            // key within the tile / output column in the epilogue
    const int sw = warp - 2;                 // 0..3: slot in the exchange arrays
    const int t = threadIdx.x - 64;          // 0..127
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qr * 32) << 16);

    // Q (and the zero padding up to 16 heads) into the swizzled K-major operand layout; both P buffers zeroed
    {
      const int g = t >> 3;                  // head row 0..15, eight threads per row
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cidx = (t & 7) * 2 + u;    // 16-byte chunk of the 128-element row
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (g < G)
          v = *reinterpret_cast<const uint4*>(p.q + row * p.ldq + (static_cast<long long>(kvh) * G + g) * DTC_D + cidx * 8);
        const int half = cidx >> 3, c = cidx & 7;
        *reinterpret_cast<uint4*>(smem + DTC_OFF_Q + half * (DTC_NH * 128) + g * 128 + ((c ^ (g & 7)) * 16)) = v;
      }
      for (int i = t; i < 2 * DTC_P_BYTES / 16; i += 128)
        *reinterpret_cast<uint4*>(smem + DTC_OFF_P + i * 16) = make_uint4(0u, 0u, 0u, 0u);
      fence_proxy_async_smem();
      mbar_arrive(q_ready);
    }
    // the other threads' zeroes of P must be visible before anyone writes probabilities
    dtc_softmax_sync();

    float m_ref[DTC_NH], l_part[DTC_NH];
#pragma unroll
    for (int g = 0; g < DTC_NH; ++g) {
      m_ref[g] = -INFINITY;
      l_part[g] = 0.f;
    }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      // fixed trip count for all 128 threads (the named barrier below is unbounded): after a failed wait
      // the remaining waits are skipped, not the iterations
      const int sb = j & 1;
      if (ok) ok = mbar_wait(&s_full[sb], (j >> 1) & 1);
      tc_fence_after_sync();
      uint32_t sv[16];
      tmem_ld_32x16(t_lane + COL_S + sb * DTC_NH, sv);
      tmem_wait_ld();
      // Scores stay in the MMA's units until the exponent: max commutes with the (positive) scale, and
      // 2^(s * scale - m) is one FMA and one MUFU. Only a tile that reaches past the context masks keys.
      float s[DTC_NH], mx[DTC_NH];
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) s[g] = __uint_as_float(sv[g]);
      if ((t_begin + j + 1) * DTC_BN > kv_len) {            // the same for the whole CTA
        const bool valid = (t_begin + j) * DTC_BN + r < kv_len;
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) s[g] = valid ? s[g] : -INFINITY;
      }
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) mx[g] = (g < G) ? warp_max_redux(s[g]) : 0.f;
      float* xm = xchg + sb * 64;
      if (lane == 0) {
#pragma unroll
        for (int g4 = 0; g4 < DTC_NH; g4 += 4)
          if (g4 < G)
            *reinterpret_cast<float4*>(xm + sw * 16 + g4) = make_float4(mx[g4], mx[g4 + 1], mx[g4 + 2], mx[g4 + 3]);
      }
      dtc_softmax_sync();
      float mt_all[DTC_NH];
#pragma unroll
      for (int g4 = 0; g4 < DTC_NH; g4 += 4) {
        // the four warps' maxima of four heads: four 16-byte loads
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a, c = a, d = a;
        if (g4 < G) {
          a = *reinterpret_cast<const float4*>(xm + g4);
          b = *reinterpret_cast<const float4*>(xm + 16 + g4);
          c = *reinterpret_cast<const float4*>(xm + 32 + g4);
          d = *reinterpret_cast<const float4*>(xm + 48 + g4);
        }
        mt_all[g4] = fmaxf(fmaxf(a.x, b.x), fmaxf(c.x, d.x)) * p.scale_log2;
        mt_all[g4 + 1] = fmaxf(fmaxf(a.y, b.y), fmaxf(c.y, d.y)) * p.scale_log2;
        mt_all[g4 + 2] = fmaxf(fmaxf(a.z, b.z), fmaxf(c.z, d.z)) * p.scale_log2;
        mt_all[g4 + 3] = fmaxf(fmaxf(a.w, b.w), fmaxf(c.w, d.w)) * p.scale_log2;
      }
      // The reference maxima move only when a head's maximum grew by more than 2^8 (rare after the first tiles):
      // one combined test here, the per-head work in the branch. All 128 threads see the same maxima and decide alike.
      bool rescale = false;
      float alpha[DTC_NH];
      if (j == 0) {
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g)
          if (g < G) m_ref[g] = mt_all[g];
      } else {
        float over = -1.f;
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g)
          if (g < G) over = fmaxf(over, mt_all[g] - m_ref[g]);
        if (over > 8.f) {
          rescale = true;
#pragma unroll
          for (int g = 0; g < DTC_NH; ++g) {
            alpha[g] = 1.f;
            if (g < G && mt_all[g] > m_ref[g] + 8.f) {
              alpha[g] = dtc_exp2(m_ref[g] - mt_all[g]);
              m_ref[g] = mt_all[g];
            }
            l_part[g] *= alpha[g];
          }
        }
      }
      uint8_t* p_buf = smem + DTC_OFF_P + sb * DTC_P_BYTES + (r >> 6) * (DTC_NH * 128);
      const int kc = (r & 63) >> 3, ke = r & 7;     // 16-byte chunk and element of this key inside its 64-key block
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) {
        if (g < G) {
          const float pv = dtc_exp2(fmaf(s[g], p.scale_log2, -m_ref[g]));
          l_part[g] += pv;
          *reinterpret_cast<__nv_bfloat16*>(p_buf + g * 128 + ((kc ^ (g & 7)) * 16) + ke * 2) = __float2bfloat16(pv);
        }
      }
      // Every tile waits for the previous tile's P.V, needed or not: the parity wait only tells "the phase
      // before the current one has completed", so a thread that skipped a phase could take the completion of
      // tile j - 2 for that of tile j (late V tiles make that happen) and read O too early in the epilogue.
      if (j > 0) {
        if (ok) ok = mbar_wait(o_done, (j - 1) & 1);
        tc_fence_after_sync();
      }
      if (rescale) {
        // O^T accumulated so far refers to the old maxima: scale column g by alpha[g]
        uint32_t ov[16];
        tmem_ld_32x16(t_lane + COL_O, ov);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) ov[g] = __float_as_uint(__uint_as_float(ov[g]) * alpha[g]);
        tmem_st_32x16(t_lane + COL_O, ov);
        tmem_wait_st();
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(p_ready);       // arrive even after a failed wait so that the issuer is not left hanging
    }

    // row sums over the 128 keys-per-tile owners
    float l_tot[DTC_NH];
#pragma unroll
    for (int g = 0; g < DTC_NH; ++g) l_tot[g] = (g < G) ? warp_sum(l_part[g]) : 0.f;
    float* xs = xchg + (n_tiles & 1) * 64;
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) xs[sw * 16 + g] = l_tot[g];
    }
    dtc_softmax_sync();
#pragma unroll
    for (int g = 0; g < DTC_NH; ++g) l_tot[g] = (xs[g] + xs[16 + g]) + (xs[32 + g] + xs[48 + g]);

    if (n_tiles > 0 && ok) ok = mbar_wait(o_done, (n_tiles - 1) & 1);
    if (ok) {
      uint32_t ov[16];
      if (n_tiles > 0) {
        tc_fence_after_sync();
        tmem_ld_32x16(t_lane + COL_O, ov);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) ov[g] = 0u;
      }
      const int d = r;
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) {
        if (g < G) {
          const int h = kvh * G + g;
          const float o = __uint_as_float(ov[g]);
          if (p.splits == 1) {
            p.out[row * p.ldo + h * DTC_D + d] = __float2bfloat16(l_tot[g] > 0.f ? o / l_tot[g] : 0.f);
          } else {
            const long long pidx = (static_cast<long long>(tok) * p.hq + h) * p.splits + split;
            p.part_o[pidx * DTC_D + d] = o;
            if (d == 0) {
              p.part_ml[pidx * 2] = m_ref[g];
              p.part_ml[pidx * 2 + 1] = l_tot[g];
            }
          }
        }
      }
    } else {
      report_error(p.status, TW_ERR_MBAR_TIMEOUT);
      *abort_flag = 1;
    }
  }

  if (*abort_flag) {
    // let copies and MMAs in flight land before shared memory and TMEM are given back
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
// Persistent variant: one CTA per SM walks the list of (token, KV head, split) items. TMEM, the barriers
// and the K/V ring live across items, so the producer is already fetching the next item's tiles while the
// softmax warps finish the current one: the per-CTA start-up cost and the uneven last wave of the
// one-item-per-CTA kernel go away. Barrier phases run on a tile counter that never resets.
constexpr int DTP_OFF_K = 0;
constexpr int DTP_OFF_V = DTP_OFF_K + DTC_RING * DTC_KV_BYTES;
constexpr int DTP_OFF_Q = DTP_OFF_V + DTC_RING * DTC_KV_BYTES;
constexpr int DTP_OFF_P = DTP_OFF_Q + DTC_Q_BYTES;             // two buffers
constexpr int DTP_OFF_BAR = DTP_OFF_P + 2 * DTC_P_BYTES;
constexpr int DTP_OFF_XCHG = DTP_OFF_BAR + 256;               // float [3][4 warps][16]
constexpr int DTP_SMEM = DTP_OFF_XCHG + 3 * 4 * 16 * 4 + 1024;

struct DtpItem {
  int tok, kvh, split, row, seq, kv_len, t_begin, n_tiles;
};
__device__ __forceinline__ DtpItem dtp_item(const DecodeTcParams& p, int idx) {
  DtpItem it;
  it.split = idx % p.splits;
  const int rest = idx / p.splits;
  it.kvh = rest % p.hkv;
  it.tok = rest / p.hkv;
  it.row = p.tok_row[it.tok];
  it.seq = p.tok_seq[it.tok];
  it.kv_len = p.tok_kvlen[it.tok];
  const int tiles_total = (it.kv_len + DTC_BN - 1) / DTC_BN;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  it.t_begin = it.split * tiles_per_split;
  it.n_tiles = max(0, min(tiles_total, it.t_begin + tiles_per_split) - it.t_begin);
  return it;
}

template <int GT>
__global__ void __launch_bounds__(DTC_THREADS, 1)
attn_decode_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                                 const DecodeTcParams p, const int n_items) {
  constexpr uint32_t IDESC_S = make_idesc_bf16(DTC_BN, DTC_NH, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc_bf16(DTC_D, DTC_NH, 1, 0);
  constexpr uint32_t TMEM_COLS = 64;
  constexpr uint32_t COL_S = 0;
  constexpr uint32_t COL_O = 32;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DTP_OFF_BAR);
  uint64_t* k_full = bars + 0;    // [3]
  uint64_t* k_empty = bars + 3;   // [3]
  uint64_t* v_full = bars + 6;    // [3]
  uint64_t* v_empty = bars + 9;   // [3]
  uint64_t* s_full = bars + 12;   // [2]
  uint64_t* p_ready = bars + 14;
  uint64_t* o_done = bars + 15;
  uint64_t* q_ready = bars + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* abort_seen = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2]: the softmax group's common view
  float* xchg = reinterpret_cast<float*>(smem + DTP_OFF_XCHG);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = GT > 0 ? GT : p.hq / p.hkv;

  if (threadIdx.x == 0) {
    for (int i = 0; i < DTC_RING; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    mbar_init(q_ready, 128);
    *abort_flag = 0;
    abort_seen[0] = 0;
    abort_seen[1] = 0;
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
    // ---------------- TMA producer: tiles of all items of this CTA, back to back ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int pages_per_tile = DTC_BN / p.page;
      uint32_t jt = 0;
      bool ok = true;
      for (int idx = blockIdx.x; ok && idx < n_items; idx += gridDim.x) {
        if (*abort_flag) break;
        const DtpItem it = dtp_item(p, idx);
        const int last_page = (it.kv_len - 1) / p.page;
        const int* table = p.block_table + static_cast<long long>(it.seq) * p.max_blocks;
        for (int j = 0; ok && j < it.n_tiles; ++j, ++jt) {
          const int st = jt % DTC_RING;
          const uint32_t ph = (jt / DTC_RING) & 1;
          const int tile = it.t_begin + j;
          ok = mbar_wait(&k_empty[st], ph ^ 1);
          if (!ok) break;
          mbar_expect_tx(&k_full[st], DTC_KV_BYTES);
          for (int pg = 0; pg < pages_per_tile; ++pg) {
            const int block = table[min(tile * pages_per_tile + pg, last_page)];
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_4d(smem + DTP_OFF_K + st * DTC_KV_BYTES + h * DTC_HALF_BYTES + pg * p.page * 128, &tmK,
                          &k_full[st], h * 64, it.kvh, 0, block);
          }
          ok = mbar_wait(&v_empty[st], ph ^ 1);
          if (!ok) break;
          mbar_expect_tx(&v_full[st], DTC_KV_BYTES);
          for (int pg = 0; pg < pages_per_tile; ++pg) {
            const int block = table[min(tile * pages_per_tile + pg, last_page)];
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_4d(smem + DTP_OFF_V + st * DTC_KV_BYTES + h * DTC_HALF_BYTES + pg * p.page * 128, &tmV,
                          &v_full[st], h * 64, it.kvh, 0, block);
          }
        }
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(smem + DTP_OFF_Q);
      uint32_t jt = 0, items_done = 0;
      bool ok = true;
      auto issue_s = [&](uint32_t jtile) {
        const int st = jtile % DTC_RING;
        if (!mbar_wait(&k_full[st], (jtile / DTC_RING) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + DTP_OFF_K + st * DTC_KV_BYTES);
#pragma unroll
        for (int k = 0; k < DTC_D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * DTC_HALF_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * (DTC_NH * 128) + (k & 3) * 32;
          umma_ss(tmem_base + COL_S + (jtile & 1) * DTC_NH, make_smem_desc_sw128(k_addr + a_off, 16, 1024),
                  make_smem_desc_sw128(q_addr + b_off, 16, 1024), IDESC_S, k != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[jtile & 1]);
        return true;
      };
      for (int idx = blockIdx.x; ok && idx < n_items; idx += gridDim.x) {
        if (*abort_flag) break;
        const DtpItem it = dtp_item(p, idx);
        if (it.n_tiles == 0) continue;
        // Q of this item is in place (one buffer: the previous item's MMAs have all completed, its
        // epilogue waited for them before the softmax warps wrote the new Q)
        ok = mbar_wait(q_ready, items_done & 1);
        if (!ok) break;
        tc_fence_after_sync();
        ok = issue_s(jt);
        for (int j = 0; ok && j < it.n_tiles; ++j, ++jt) {
          if (j + 1 < it.n_tiles) {
            ok = issue_s(jt + 1);
            if (!ok) break;
          }
          const int st = jt % DTC_RING;
          if (!mbar_wait(p_ready, jt & 1)) { ok = false; break; }
          if (!mbar_wait(&v_full[st], (jt / DTC_RING) & 1)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t v_addr = smem_u32(smem + DTP_OFF_V + st * DTC_KV_BYTES);
          const uint32_t p_addr = smem_u32(smem + DTP_OFF_P + (jt & 1) * DTC_P_BYTES);
#pragma unroll
          for (int k = 0; k < DTC_BN / 16; ++k) {
            const uint32_t b_off = (k >> 2) * (DTC_NH * 128) + (k & 3) * 32;
            umma_ss(tmem_base + COL_O, make_smem_desc_sw128(v_addr + k * 16 * 128, DTC_HALF_BYTES, 1024),
                    make_smem_desc_sw128(p_addr + b_off, 16, 1024), IDESC_O, (j | k) != 0 ? 1u : 0u);
          }
          umma_commit(&v_empty[st]);
          umma_commit(o_done);
        }
        ++items_done;
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..5) ----------------
    const int qr = warp & 3;
    const int r = qr * 32 + lane;
    const int sw = warp - 2;
    const int t = threadIdx.x - 64;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qr * 32) << 16);
    for (int i = t; i < 2 * DTC_P_BYTES / 16; i += 128)
      *reinterpret_cast<uint4*>(smem + DTP_OFF_P + i * 16) = make_uint4(0u, 0u, 0u, 0u);
    uint32_t jt = 0, visit = 0;
    bool ok = true;
    for (int idx = blockIdx.x; idx < n_items; idx += gridDim.x, ++visit) {
      // One decision for all 128 threads (they meet on an unbounded named barrier inside the item): thread 0
      // publishes what it sees of the abort flag in a slot that alternates between visits, so that a slow
      // thread still reading this visit's slot is not overtaken by the next visit's value.
      if (!ok) *abort_flag = 1;
      if (t == 0) abort_seen[visit & 1] = *abort_flag;
      dtc_softmax_sync();
      if (abort_seen[visit & 1]) break;
      const DtpItem it = dtp_item(p, idx);
      if (it.n_tiles == 0) {
        // an empty split (or an empty sequence): neutral partial result
        for (int g = 0; g < G; ++g) {
          const int h = it.kvh * G + g;
          if (p.splits == 1) {
            p.out[it.row * p.ldo + h * DTC_D + r] = __float2bfloat16(0.f);
          } else {
            const long long pidx = (static_cast<long long>(it.tok) * p.hq + h) * p.splits + it.split;
            p.part_o[pidx * DTC_D + r] = 0.f;
            if (r == 0) {
              p.part_ml[pidx * 2] = -INFINITY;
              p.part_ml[pidx * 2 + 1] = 0.f;
            }
          }
        }
        continue;
      }
      {
        const int g = t >> 3;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int cidx = (t & 7) * 2 + u;
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (g < G)
            v = *reinterpret_cast<const uint4*>(p.q + it.row * p.ldq +
                                                (static_cast<long long>(it.kvh) * G + g) * DTC_D + cidx * 8);
          const int half = cidx >> 3, c = cidx & 7;
          *reinterpret_cast<uint4*>(smem + DTP_OFF_Q + half * (DTC_NH * 128) + g * 128 + ((c ^ (g & 7)) * 16)) = v;
        }
        fence_proxy_async_smem();
        mbar_arrive(q_ready);
      }
      float m_ref[DTC_NH], l_part[DTC_NH];
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) {
        m_ref[g] = -INFINITY;
        l_part[g] = 0.f;
      }
      for (int j = 0; j < it.n_tiles; ++j, ++jt) {
        const int sb = jt & 1;
        if (ok) ok = mbar_wait(&s_full[sb], (jt >> 1) & 1);
        tc_fence_after_sync();
        uint32_t sv[16];
        tmem_ld_32x16(t_lane + COL_S + sb * DTC_NH, sv);
        tmem_wait_ld();
        // Scores stay in the MMA's units until the exponent: max commutes with the (positive) scale, and
        // 2^(s * scale - m) is one FMA and one MUFU. Only a tile that reaches past the context masks keys.
        float s[DTC_NH], mx[DTC_NH];
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) s[g] = __uint_as_float(sv[g]);
        if ((it.t_begin + j + 1) * DTC_BN > it.kv_len) {            // the same for the whole CTA
          const bool valid = (it.t_begin + j) * DTC_BN + r < it.kv_len;
#pragma unroll
          for (int g = 0; g < DTC_NH; ++g) s[g] = valid ? s[g] : -INFINITY;
        }
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) mx[g] = (g < G) ? warp_max_redux(s[g]) : 0.f;
        float* xm = xchg + sb * 64;
        if (lane == 0) {
#pragma unroll
          for (int g4 = 0; g4 < DTC_NH; g4 += 4)
            if (g4 < G)
              *reinterpret_cast<float4*>(xm + sw * 16 + g4) = make_float4(mx[g4], mx[g4 + 1], mx[g4 + 2], mx[g4 + 3]);
        }
        dtc_softmax_sync();
        float mt_all[DTC_NH];
#pragma unroll
        for (int g4 = 0; g4 < DTC_NH; g4 += 4) {
          // the four warps' maxima of four heads: four 16-byte loads
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a, c = a, d = a;
          if (g4 < G) {
            a = *reinterpret_cast<const float4*>(xm + g4);
            b = *reinterpret_cast<const float4*>(xm + 16 + g4);
            c = *reinterpret_cast<const float4*>(xm + 32 + g4);
            d = *reinterpret_cast<const float4*>(xm + 48 + g4);
          }
          mt_all[g4] = fmaxf(fmaxf(a.x, b.x), fmaxf(c.x, d.x)) * p.scale_log2;
          mt_all[g4 + 1] = fmaxf(fmaxf(a.y, b.y), fmaxf(c.y, d.y)) * p.scale_log2;
          mt_all[g4 + 2] = fmaxf(fmaxf(a.z, b.z), fmaxf(c.z, d.z)) * p.scale_log2;
          mt_all[g4 + 3] = fmaxf(fmaxf(a.w, b.w), fmaxf(c.w, d.w)) * p.scale_log2;
        }
        // The reference maxima move only when a head's maximum grew by more than 2^8 (rare after the first tiles):
        // one combined test here, the per-head work in the branch. All 128 threads see the same maxima and decide alike.
        bool rescale = false;
        float alpha[DTC_NH];
        if (j == 0) {
#pragma unroll
          for (int g = 0; g < DTC_NH; ++g)
            if (g < G) m_ref[g] = mt_all[g];
        } else {
          float over = -1.f;
#pragma unroll
          for (int g = 0; g < DTC_NH; ++g)
            if (g < G) over = fmaxf(over, mt_all[g] - m_ref[g]);
          if (over > 8.f) {
            rescale = true;
#pragma unroll
            for (int g = 0; g < DTC_NH; ++g) {
              alpha[g] = 1.f;
              if (g < G && mt_all[g] > m_ref[g] + 8.f) {
                alpha[g] = dtc_exp2(m_ref[g] - mt_all[g]);
                m_ref[g] = mt_all[g];
              }
              l_part[g] *= alpha[g];
            }
          }
        }
        uint8_t* p_buf = smem + DTP_OFF_P + sb * DTC_P_BYTES + (r >> 6) * (DTC_NH * 128);
        const int kc = (r & 63) >> 3, ke = r & 7;     // 16-byte chunk and element of this key inside its 64-key block
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) {
          if (g < G) {
            const float pv = dtc_exp2(fmaf(s[g], p.scale_log2, -m_ref[g]));
            l_part[g] += pv;
            *reinterpret_cast<__nv_bfloat16*>(p_buf + g * 128 + ((kc ^ (g & 7)) * 16) + ke * 2) = __float2bfloat16(pv);
          }
        }
        if (j > 0) {        // keeps every thread's view of o_done's phase exact (see the one-item kernel)
          if (ok) ok = mbar_wait(o_done, (jt - 1) & 1);
          tc_fence_after_sync();
        }
        if (rescale) {
          uint32_t ov[16];
          tmem_ld_32x16(t_lane + COL_O, ov);
          tmem_wait_ld();
#pragma unroll
          for (int g = 0; g < DTC_NH; ++g) ov[g] = __float_as_uint(__uint_as_float(ov[g]) * alpha[g]);
          tmem_st_32x16(t_lane + COL_O, ov);
          tmem_wait_st();
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(p_ready);
      }
      float l_tot[DTC_NH];
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) l_tot[g] = (g < G) ? warp_sum(l_part[g]) : 0.f;
      float* xs = xchg + 2 * 64;
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) xs[sw * 16 + g] = l_tot[g];
      }
      dtc_softmax_sync();
#pragma unroll
      for (int g = 0; g < DTC_NH; ++g) l_tot[g] = (xs[g] + xs[16 + g]) + (xs[32 + g] + xs[48 + g]);
      if (ok) ok = mbar_wait(o_done, (jt - 1) & 1);
      tc_fence_after_sync();
      uint32_t ov[16];
      tmem_ld_32x16(t_lane + COL_O, ov);
      tmem_wait_ld();
      tc_fence_before_sync();
      if (ok) {
#pragma unroll
        for (int g = 0; g < DTC_NH; ++g) {
          if (g < G) {
            const int h = it.kvh * G + g;
            const float o = __uint_as_float(ov[g]);
            if (p.splits == 1) {
              p.out[it.row * p.ldo + h * DTC_D + r] = __float2bfloat16(l_tot[g] > 0.f ? o / l_tot[g] : 0.f);
            } else {
              const long long pidx = (static_cast<long long>(it.tok) * p.hq + h) * p.splits + it.split;
              p.part_o[pidx * DTC_D + r] = o;
              if (r == 0) {
                p.part_ml[pidx * 2] = m_ref[g];
                p.part_ml[pidx * 2 + 1] = l_tot[g];
              }
            }
          }
        }
      }
    }
    if (!ok) {
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

}  // namespace tw

using namespace tw;

// Same contract as tw_attn_decode (attn_decode.cu); head size 128, at most 16 query heads per KV head,
// page sizes that divide 128. `num_blocks` is the extent of the caches' first dimension (for the tensor maps).
// The caller runs attn_decode_merge through tw_attn_decode_merge when splits > 1.
extern "C" int tw_attn_decode_tc(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                                 int num_blocks, int page, void* out, long long ldo, const int* tok_row,
                                 const int* tok_seq, const int* tok_kvlen, int n_tok, const int* block_table,
                                 int max_blocks, int hq, int hkv, int D, float scale, int splits, float* part_o,
                                 float* part_ml, uint32_t* status, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  if (D != DTC_D || hkv <= 0 || hq % hkv != 0 || hq / hkv > DTC_NH) {
    set_last_error("attn_decode_tc: needs head_dim 128 and at most 16 query heads per KV head (D=%d, hq=%d, hkv=%d)",
                   D, hq, hkv);
    return 1;
  }
  if (page < 8 || page > 128 || (128 % page) != 0 || ldq % 8 != 0) {
    set_last_error("attn_decode_tc: page size must divide 128 and be >= 8 (got %d); q rows 16-byte aligned", page);
    return 1;
  }
  if (splits < 1) splits = 1;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) {
    set_last_error("attn_decode_tc: split-KV needs the partial-result workspace");
    return 1;
  }
  CUtensorMap tmK, tmV;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)hkv, (uint64_t)page, (uint64_t)num_blocks};
    uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)hkv * D * 2, (uint64_t)page * hkv * D * 2};
    uint32_t box[4] = {64, 1, (uint32_t)page, 1};
    if (!make_tensor_map_bf16(&tmK, k_cache, 4, dims, strides, box)) return 1;
    if (!make_tensor_map_bf16(&tmV, v_cache, 4, dims, strides, box)) return 1;
  }
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM);
    if (e != cudaSuccess) {
      set_last_error("attn_decode_tc: cudaFuncSetAttribute(smem=%d) failed: %s", DTC_SMEM, cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  DecodeTcParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.ldq = ldq;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.tok_row = tok_row;
  p.tok_seq = tok_seq;
  p.tok_kvlen = tok_kvlen;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.page = page;
  p.hq = hq;
  p.hkv = hkv;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.status = status;
  const dim3 grid(n_tok, hkv, splits);
  const int group = hq / hkv;
  if (group == 8) attn_decode_tc_kernel<8><<<grid, DTC_THREADS, DTC_SMEM, stream>>>(tmK, tmV, p);
  else if (group == 4) attn_decode_tc_kernel<4><<<grid, DTC_THREADS, DTC_SMEM, stream>>>(tmK, tmV, p);
  else attn_decode_tc_kernel<0><<<grid, DTC_THREADS, DTC_SMEM, stream>>>(tmK, tmV, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_decode_tc launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  if (splits > 1) return tw_attn_decode_merge(part_o, part_ml, tok_row, n_tok, hq, D, splits, out, ldo, stream);
  return 0;
}

// Persistent variant of tw_attn_decode_tc: `max_ctas` CTAs (0: one per SM) walk the (token, KV head, split)
// items. Same arguments otherwise.
extern "C" int tw_attn_decode_tc_persistent(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                                            int num_blocks, int page, void* out, long long ldo, const int* tok_row,
                                            const int* tok_seq, const int* tok_kvlen, int n_tok,
                                            const int* block_table, int max_blocks, int hq, int hkv, int D,
                                            float scale, int splits, float* part_o, float* part_ml, int max_ctas,
                                            uint32_t* status, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  if (D != DTC_D || hkv <= 0 || hq % hkv != 0 || hq / hkv > DTC_NH) {
    set_last_error("attn_decode_tc_persistent: needs head_dim 128 and at most 16 query heads per KV head "
                   "(D=%d, hq=%d, hkv=%d)", D, hq, hkv);
    return 1;
  }
  if (page < 8 || page > 128 || (128 % page) != 0 || ldq % 8 != 0) {
    set_last_error("attn_decode_tc_persistent: page size must divide 128 and be >= 8 (got %d); q rows 16-byte aligned",
                   page);
    return 1;
  }
  if (splits < 1) splits = 1;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) {
    set_last_error("attn_decode_tc_persistent: split-KV needs the partial-result workspace");
    return 1;
  }
  CUtensorMap tmK, tmV;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)hkv, (uint64_t)page, (uint64_t)num_blocks};
    uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)hkv * D * 2, (uint64_t)page * hkv * D * 2};
    uint32_t box[4] = {64, 1, (uint32_t)page, 1};
    if (!make_tensor_map_bf16(&tmK, k_cache, 4, dims, strides, box)) return 1;
    if (!make_tensor_map_bf16(&tmV, v_cache, 4, dims, strides, box)) return 1;
  }
  static thread_local int configured_dev = -1;
  static thread_local int sm_count = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tc_persistent_kernel<0>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, DTP_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tc_persistent_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTP_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tc_persistent_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTP_SMEM);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      set_last_error("attn_decode_tc_persistent: device set-up failed: %s", cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  DecodeTcParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.ldq = ldq;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.tok_row = tok_row;
  p.tok_seq = tok_seq;
  p.tok_kvlen = tok_kvlen;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.page = page;
  p.hq = hq;
  p.hkv = hkv;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.status = status;
  const long long items = static_cast<long long>(n_tok) * hkv * splits;
  if (items > 0x7fffffffLL) {
    set_last_error("attn_decode_tc_persistent: too many work items");
    return 1;
  }
  const int cap = max_ctas > 0 ? max_ctas : sm_count;
  const int grid = static_cast<int>(items < cap ? items : cap);
  const int group = hq / hkv, n_items = static_cast<int>(items);
  if (group == 8) attn_decode_tc_persistent_kernel<8><<<grid, DTC_THREADS, DTP_SMEM, stream>>>(tmK, tmV, p, n_items);
  else if (group == 4) attn_decode_tc_persistent_kernel<4><<<grid, DTC_THREADS, DTP_SMEM, stream>>>(tmK, tmV, p, n_items);
  else attn_decode_tc_persistent_kernel<0><<<grid, DTC_THREADS, DTP_SMEM, stream>>>(tmK, tmV, p, n_items);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_decode_tc_persistent launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  if (splits > 1) return tw_attn_decode_merge(part_o, part_ml, tok_row, n_tok, hq, D, splits, out, ldo, stream);
  return 0;
}
