// Causal variable-length prefill attention over a paged KV cache for sm_100a, persistent form.
//
// The kernels of attn_prefill.cu launch one CTA per (query tile, head or head pair); a causal batch then
// has work items whose cost grows linearly with the tile's position, and with few heads per GPU
// (tensor parallelism over 8 GPUs leaves 8 query heads) there are fewer items than SMs: the launch
// lasts as long as its heaviest item while most SMs idle. Here
//   * a work item is ONE query head of one 128-query tile, and the item's key tiles are cut in two
//     halves that the two softmax groups of the CTA process concurrently (each with its own S, P and O
//     in tensor memory and its own K/V ring), so an item costs half its key range in time and the two
//     groups keep the tensor pipe busy out of phase; the halves are merged in the epilogue
//     (log-sum-exp combine straight from tensor memory, no scratch in global memory);
//   * CTAs are persistent: the grid is min(SM budget, items) and CTA c takes items c, 2G-1-c, 2G+c, ...
//     of the list sorted by cost (heaviest first, the host sorts the tiles), which pairs heavy with light
//     items; the SM budget lets the token-split schedule keep SMs free for a concurrent collective;
//   * P never touches shared memory: the softmax threads write bf16 probabilities back into the upper
//     half of their S columns (tcgen05.st) and the P V product reads its A operand from tensor memory
//     (tcgen05.mma with a TMEM operand), which frees 64 KB for a deeper K/V ring and removes the
//     shared-memory stores and the proxy fence of every tile. A row's 128 scores are read from tensor
//     memory once (four loads in flight, one wait) and the softmax runs from registers with the packed
//     two-wide fp32 instructions and the three-input maximum of sm_100.
// Tried and dropped: softmax steps of 64 keys with S double-buffered per group (Q K^T of the next step
// then never waits for the softmax). An M = 128 MMA with N = 64 takes as long as one with N = 128, so
// the Q K^T time doubled and the kernel was 40 % slower. Also dropped: every 2nd, 3rd or 4th pair of
// exponentials as a cubic on the FMA pipe instead of ex2.approx (correct to 8e-5, but 17 to 25 % slower at
// every share: the softmax warps are bound by issue slots, and the polynomial costs six times the
// instructions of the MUFU form).
// Replaces the FlashAttention-2 varlen call the reference makes on Blackwell
// (vllm/v1/attention/backends/flash_attn.py:713-733, vllm/attention/utils/fa_utils.py:29-34).
//
// Roles (320 threads): warp 0 TMA producer (Q per item; K_t V_t of group A and of group B through two
// rings of three 128-key tiles), warp 1 MMA issuer, warps 2..5 softmax group A (one thread per query
// row), warps 6..9 group B. Every mbarrier wait is bounded; after a timeout the roles keep their trip
// counts (the named barriers of the epilogue are not bounded) but skip further waits, and the CTA
// reports TW_ERR_MBAR_TIMEOUT and leaves through its tear-down.
#include "attn_prefill_common.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

constexpr int SPL_RING = 3;   // K/V tile slots per softmax group

template <int D>
struct SplitSmem {
  static constexpr int HALVES = D / 64;
  static constexpr int Q_BYTES = HALVES * ATT_HALF_BYTES;
  static constexpr int KV_BYTES = HALVES * ATT_HALF_BYTES;      // one K or V tile of 128 keys
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_RING = OFF_Q + Q_BYTES;              // [2 groups][SPL_RING]
  static constexpr int OFF_BAR = OFF_RING + 2 * SPL_RING * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;            // barriers, then slack for the 1024-byte alignment
};

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bf16 pairs, one 32-bit column per two K elements, one
// lane per row) comes from tensor memory.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x2(uint32_t taddr, uint32_t a, uint32_t b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x2(uint32_t taddr, uint32_t& a, uint32_t& b) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(taddr) : "memory");
}

// Three-input maximum and the packed two-wide fp32 forms of sm_100: half the issue slots per score.
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  uint64_t ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One work item: a 128-query tile of one head.
struct SplitItem {
  // key tiles [j_lo, j_lo + n_tiles) are needed (j_lo > 0 only under a sliding window);
  // group A takes the first n_a of them, group B the rest
  int head, kvh, seq, q_begin, q0, rows_valid, pos0, kv_len, j_lo, n_tiles, n_a;
};

__device__ __forceinline__ SplitItem split_item(const AttnParams& p, int idx) {
  SplitItem it;
  const int tile = idx / p.hq;
  it.head = idx - tile * p.hq;
  it.kvh = it.head / (p.hq / p.hkv);
  it.seq = p.tile_seq[tile];
  it.q0 = p.tile_q0[tile];
  it.q_begin = p.cu_q[it.seq];
  const int q_len = p.cu_q[it.seq + 1] - it.q_begin;
  it.kv_len = p.kv_lens[it.seq];
  it.rows_valid = min(ATT_BM, q_len - it.q0);
  it.pos0 = it.kv_len - q_len + it.q0;                       // absolute position of the tile's first query
  const int kv_end = min(it.kv_len, it.pos0 + it.rows_valid);  // keys [0, kv_end) are needed
  // under a sliding window the tile's first query sees nothing before key pos0 - window + 1
  it.j_lo = p.window > 0 ? max(0, it.pos0 - p.window + 1) / ATT_BN : 0;
  it.n_tiles = (kv_end + ATT_BN - 1) / ATT_BN - it.j_lo;
  it.n_a = (it.n_tiles + 1) / 2;
  return it;
}

// Items of CTA `c` of `G`: round r takes the c-th item of the r-th block of G items, counted from the
// front in even rounds and from the back in odd ones (heavy items meet light ones).
__device__ __forceinline__ int split_item_index(int round, int c, int G) {
  return round * G + ((round & 1) ? (G - 1 - c) : c);
}

// The two softmax threads of a query row sit in warps w (group A) and w + 4 (group B), the same TMEM
// lane quarter; each such warp pair meets on its own named barrier (ids 1..4, 64 threads).
__device__ __forceinline__ void split_pair_sync(int quarter) {
  asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
}

// OPTS: sliding window and logits soft cap compiled in (a separate instantiation, so that the plain causal
// kernel keeps its register budget).
template <int D, bool OPTS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_prefill_split_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const AttnParams p, const int total_items) {
  using S = SplitSmem<D>;
  constexpr int HALVES = S::HALVES;
  constexpr int R = SPL_RING;
  constexpr uint32_t IDESC_QK = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(ATT_BM, D, 0, 1);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0;     // S_A at 0, S_B at 128; P_g lives in columns [64, 128) of S_g
  constexpr uint32_t COL_P = 64;
  constexpr uint32_t COL_O = 256;   // O_A at 256, O_B at 384

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;
  uint64_t* ring_full = bars + 2;     // [2][R]
  uint64_t* ring_empty = bars + 8;    // [2][R]
  uint64_t* s_full = bars + 14;       // [2]
  uint64_t* p_ready = bars + 16;      // [2]
  uint64_t* o_done = bars + 18;       // [2]
  uint64_t* epi_done = bars + 20;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const int cta = blockIdx.x;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 2 * R; ++i) {
      mbar_init(&ring_full[i], 1);
      mbar_init(&ring_empty[i], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&p_ready[g], 128);
      mbar_init(&o_done[g], 1);
    }
    mbar_init(epi_done, ATT_SOFTMAX_THREADS);
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
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      uint32_t e[2] = {0u, 0u};           // ring elements loaded so far, per group
      const int pages_per_tile = ATT_BN / p.page;
      bool ok = true;
      int items_done = 0;
      for (int round = 0; ok; ++round) {
        const int idx = split_item_index(round, cta, G);
        if (idx >= total_items) break;
        const SplitItem it = split_item(p, idx);
        if (items_done > 0 && !mbar_wait(q_empty, (items_done - 1) & 1)) { ok = false; break; }
        mbar_expect_tx(q_full, S::Q_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(smem + S::OFF_Q + h * ATT_HALF_BYTES, &tmQ, q_full, it.head * D + h * 64, it.q_begin + it.q0);
        const int last_page = (it.kv_len - 1) / p.page;
        const int* table = p.block_table + static_cast<long long>(it.seq) * p.max_blocks;
        auto load_tile = [&](int g, const CUtensorMap* tm, int j) {
          const int slot = e[g] % R;
          const uint32_t ph = (e[g] / R) & 1;
          if (!mbar_wait(&ring_empty[g * R + slot], ph ^ 1)) return false;
          mbar_expect_tx(&ring_full[g * R + slot], S::KV_BYTES);
          uint8_t* dst = smem + S::OFF_RING + (g * R + slot) * S::KV_BYTES;
          for (int pg = 0; pg < pages_per_tile; ++pg) {
            const int block = table[min(j * pages_per_tile + pg, last_page)];
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
              tma_load_4d(dst + h * ATT_HALF_BYTES + pg * p.page * 128, tm, &ring_full[g * R + slot], h * 64, it.kvh, 0,
                          block);
          }
          ++e[g];
          return true;
        };
        const int n_b = it.n_tiles - it.n_a;
        for (int t = 0; t < it.n_a && ok; ++t) {
          ok = load_tile(0, &tmK, it.j_lo + t);
          if (ok && t < n_b) ok = load_tile(1, &tmK, it.j_lo + it.n_a + t);
          if (ok) ok = load_tile(0, &tmV, it.j_lo + t);
          if (ok && t < n_b) ok = load_tile(1, &tmV, it.j_lo + it.n_a + t);
        }
        ++items_done;
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t e[2] = {0u, 0u};           // ring elements consumed so far, per group
      uint32_t cnt[2] = {0u, 0u};         // key tiles whose P V has been issued, per group
      const uint32_t q_addr = smem_u32(smem + S::OFF_Q);
      bool ok = true;
      int items_done = 0;
      for (int round = 0; ok; ++round) {
        const int idx = split_item_index(round, cta, G);
        if (idx >= total_items) break;
        const SplitItem it = split_item(p, idx);
        const int n_b = it.n_tiles - it.n_a;
        if (!mbar_wait(q_full, items_done & 1)) { ok = false; break; }
        // S_g carried the (m, l) exchange of the previous item's epilogue
        if (items_done > 0 && !mbar_wait(epi_done, (items_done - 1) & 1)) { ok = false; break; }
        tc_fence_after_sync();
        int qk_issued = 0;
        auto issue_qk = [&](int g) {
          const int slot = e[g] % R;
          if (!mbar_wait(&ring_full[g * R + slot], (e[g] / R) & 1)) return false;
          tc_fence_after_sync();
          const uint32_t k_addr = smem_u32(smem + S::OFF_RING + (g * R + slot) * S::KV_BYTES);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k >> 2) * ATT_HALF_BYTES + (k & 3) * 32;
            umma_ss(tmem_base + COL_S + g * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                    make_smem_desc_sw128(k_addr + off, 16, 1024), IDESC_QK, k != 0 ? 1u : 0u);
          }
          umma_commit(&ring_empty[g * R + slot]);
          umma_commit(&s_full[g]);
          ++e[g];
          if (++qk_issued == it.n_tiles) umma_commit(q_empty);   // the Q tile may be replaced once these are done
          return true;
        };
        auto issue_pv = [&](int g, bool first) {
          if (!mbar_wait(&p_ready[g], cnt[g] & 1)) return false;
          const int slot = e[g] % R;
          if (!mbar_wait(&ring_full[g * R + slot], (e[g] / R) & 1)) return false;
          tc_fence_after_sync();
          const uint32_t v_addr = smem_u32(smem + S::OFF_RING + (g * R + slot) * S::KV_BYTES);
#pragma unroll
          for (int k = 0; k < ATT_BN / 16; ++k)
            umma_ts(tmem_base + COL_O + g * 128, tmem_base + COL_S + g * 128 + COL_P + k * 8,
                    make_smem_desc_sw128(v_addr + k * 16 * 128, ATT_HALF_BYTES, 1024), IDESC_PV,
                    (first && k == 0) ? 0u : 1u);
          umma_commit(&ring_empty[g * R + slot]);
          umma_commit(&o_done[g]);
          ++e[g];
          ++cnt[g];
          return true;
        };
        ok = issue_qk(0);
        if (ok && n_b > 0) ok = issue_qk(1);
        for (int t = 0; ok && t < it.n_a; ++t) {
          ok = issue_pv(0, t == 0);
          if (ok && t + 1 < it.n_a) ok = issue_qk(0);
          if (ok && t < n_b) ok = issue_pv(1, t == 0);
          if (ok && t + 1 < n_b) ok = issue_qk(1);
        }
        ++items_done;
      }
      if (!ok) {
        report_error(p.status, TW_ERR_MBAR_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- softmax + epilogue: warps 2..5 group A, warps 6..9 group B ----------------
    const int g = (warp - 2) >> 2;
    const int qr = warp & 3;                        // TMEM lane quarter of this warp
    const int r = qr * 32 + lane;                   // row within the tile
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qr * 32) << 16);
    const uint32_t t_s = t_lane + COL_S + g * 128;
    const uint32_t t_p = t_s + COL_P;
    uint32_t cnt = 0;                               // key tiles this group has processed
    bool ok = true;
    for (int round = 0;; ++round) {
      const int idx = split_item_index(round, cta, G);
      if (idx >= total_items) break;
      const SplitItem it = split_item(p, idx);
      const int n_b = it.n_tiles - it.n_a;
      const int n_mine = g == 0 ? it.n_a : n_b;
      const int j0 = it.j_lo + (g == 0 ? 0 : it.n_a);
      const float cap_mul = (OPTS && p.softcap > 0.f) ? p.softcap / p.scale : 0.f;
      const float cap_in = (OPTS && p.softcap > 0.f) ? p.scale / p.softcap : 0.f;
      const int pos = it.pos0 + min(r, it.rows_valid - 1);   // padding rows copy the last valid row's mask
      const int pos_w = (OPTS && p.window > 0) ? pos - p.window + 1 : 0;    // first key this row sees
      float m_ref = -INFINITY;   // softmax reference (a stale running maximum), log2 domain
      float l_sum = 0.f;
      for (int t = 0; t < n_mine; ++t) {
        if (ok) ok = mbar_wait(&s_full[g], cnt & 1);
        tc_fence_after_sync();
        const int k_base = (j0 + t) * ATT_BN;
        // warp-uniform: lane 0 holds the warp's smallest position, lane 31 its largest
        bool need_mask = (k_base + ATT_BN - 1) > __shfl_sync(0xffffffffu, pos, 0);
        if (OPTS) need_mask = need_mask || k_base < __shfl_sync(0xffffffffu, pos_w, 31);
        // The row's 128 scores come to registers in one go (four loads in flight, one wait): the latency of
        // tensor-memory loads is paid once per tile, and everything below runs from registers.
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_32x32(t_s, s0);
        tmem_ld_32x32(t_s + 32, s1);
        tmem_ld_32x32(t_s + 64, s2);
        tmem_ld_32x32(t_s + 96, s3);
        tmem_wait_ld();
        if (OPTS && p.softcap > 0.f) {
          // s -> cap * tanh(s * scale / cap), kept in units of the raw scores (the scale is applied below)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s0[i] = __float_as_uint(cap_mul * fast_tanh(__uint_as_float(s0[i]) * cap_in));
            s1[i] = __float_as_uint(cap_mul * fast_tanh(__uint_as_float(s1[i]) * cap_in));
            s2[i] = __float_as_uint(cap_mul * fast_tanh(__uint_as_float(s2[i]) * cap_in));
            s3[i] = __float_as_uint(cap_mul * fast_tanh(__uint_as_float(s3[i]) * cap_in));
          }
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (k_base + i > pos || (OPTS && k_base + i < pos_w)) s0[i] = __float_as_uint(-INFINITY);
            if (k_base + 32 + i > pos || (OPTS && k_base + 32 + i < pos_w)) s1[i] = __float_as_uint(-INFINITY);
            if (k_base + 64 + i > pos || (OPTS && k_base + 64 + i < pos_w)) s2[i] = __float_as_uint(-INFINITY);
            if (k_base + 96 + i > pos || (OPTS && k_base + 96 + i < pos_w)) s3[i] = __float_as_uint(-INFINITY);
          }
        }
        // row maximum: three-input max, one chain per chunk
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          m4[0] = max3f(m4[0], __uint_as_float(s0[2 * i]), __uint_as_float(s0[2 * i + 1]));
          m4[1] = max3f(m4[1], __uint_as_float(s1[2 * i]), __uint_as_float(s1[2 * i + 1]));
          m4[2] = max3f(m4[2], __uint_as_float(s2[2 * i]), __uint_as_float(s2[2 * i + 1]));
          m4[3] = max3f(m4[3], __uint_as_float(s3[2 * i]), __uint_as_float(s3[2 * i + 1]));
        }
        const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
        float alpha = 1.f;
        bool rescale = false;
        if (t == 0) {
          m_ref = mx;
        } else if (mx > m_ref + 8.f) {
          alpha = fast_exp2(m_ref - mx);
          m_ref = mx;
          rescale = true;
        }
        // a row of group B can have every key of its first tiles masked: its reference stays -inf and the
        // exponentials below must see a finite subtrahend
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        // exponentials, two scores per instruction where the ISA has a packed form (scale and subtract,
        // running sum, bf16 conversion); 32 keys become 16 columns of P, which overwrites S columns
        // 64..127 (every score is in registers by now)
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nm2 = make_float2(-m_use, -m_use);
        float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        uint32_t pk[16];
        auto exp_chunk = [&](const uint32_t (&buf)[32]) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = ffma2(make_float2(__uint_as_float(buf[2 * i]), __uint_as_float(buf[2 * i + 1])), sc2, nm2);
            const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            sum2[i & 1] = fadd2(sum2[i & 1], e);
            pk[i] = pack_bf16x2(e.x, e.y);
          }
        };
        exp_chunk(s0);
        tmem_st_32x16(t_p, pk);
        exp_chunk(s1);
        tmem_st_32x16(t_p + 16, pk);
        if (t > 0 && __any_sync(0xffffffffu, rescale)) {
          // O_g may be touched once P V of the previous tile has completed
          if (ok) ok = mbar_wait(&o_done[g], (cnt - 1) & 1);
          tc_fence_after_sync();
          const uint32_t t_o = t_lane + COL_O + g * 128;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(t_o + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, v);
          }
        }
        exp_chunk(s2);
        tmem_st_32x16(t_p + 32, pk);
        exp_chunk(s3);
        tmem_st_32x16(t_p + 48, pk);
        l_sum = l_sum * alpha + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&p_ready[g]);   // arrive even after a failed wait so the issuer is not left waiting
        ++cnt;
      }
      if (n_mine > 0 && ok) ok = mbar_wait(&o_done[g], (cnt - 1) & 1);
      tc_fence_after_sync();
      // ---- epilogue: merge the two halves of the key range; group g writes output columns [g D/2, (g+1) D/2) ----
      tmem_st_32x2(t_s, __float_as_uint(m_ref), __float_as_uint(l_sum));
      tmem_wait_st();
      tc_fence_before_sync();
      split_pair_sync(qr);
      tc_fence_after_sync();
      uint32_t om_u, ol_u;
      tmem_ld_32x2(t_lane + COL_S + (g ^ 1) * 128, om_u, ol_u);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(epi_done);        // S_A and S_B are free for the next item
      const float o_m = __uint_as_float(om_u), o_l = __uint_as_float(ol_u);
      const float m_all = fmaxf(m_ref, o_m);
      const float f_me = fast_exp2(m_ref - m_all), f_ot = fast_exp2(o_m - m_all);
      const float inv = 1.f / (l_sum * f_me + o_l * f_ot);
      const float f_a = (g == 0 ? f_me : f_ot) * inv, f_b = (g == 0 ? f_ot : f_me) * inv;
      __nv_bfloat16* orow =
          p.out + static_cast<long long>(it.q_begin + it.q0 + r) * p.ldo + it.head * D + g * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t a[32], b[32];
        const uint32_t col = COL_O + g * (D / 2) + c * 32;
        tmem_ld_32x32(t_lane + col, a);
        if (n_b > 0) tmem_ld_32x32(t_lane + col + 128, b);
        tmem_wait_ld();
        if (n_b > 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            a[i] = __float_as_uint(__uint_as_float(a[i]) * f_a + __uint_as_float(b[i]) * f_b);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * f_a);
        }
        if (r < it.rows_valid && ok) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(a[8 * q4 + 0]), __uint_as_float(a[8 * q4 + 1]));
            o.y = pack_bf16x2(__uint_as_float(a[8 * q4 + 2]), __uint_as_float(a[8 * q4 + 3]));
            o.z = pack_bf16x2(__uint_as_float(a[8 * q4 + 4]), __uint_as_float(a[8 * q4 + 5]));
            o.w = pack_bf16x2(__uint_as_float(a[8 * q4 + 6]), __uint_as_float(a[8 * q4 + 7]));
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = o;
          }
        }
      }
      // both groups have read O_A and O_B before either signals the first P of the next item
      tc_fence_before_sync();
      split_pair_sync(qr);
      tc_fence_after_sync();
    }
    if (!ok) {
      report_error(p.status, TW_ERR_MBAR_TIMEOUT);
      *abort_flag = 1;
    }
  }

  // ---------------- tear-down ----------------
  if (*abort_flag) {
    // give copies that may still be in flight time to land before shared memory is released
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

template <int D, bool OPTS>
static int launch_split_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p,
                          int num_tiles, int max_ctas, cudaStream_t stream) {
  using S = SplitSmem<D>;
  auto kern = attn_prefill_split_kernel<D, OPTS>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) {
      set_last_error("attn_prefill (split): cudaFuncSetAttribute(smem=%d) failed: %s", S::TOTAL, cudaGetErrorString(e));
      return 1;
    }
    configured_dev = dev;
  }
  const long long items = static_cast<long long>(num_tiles) * p.hq;
  int grid = device_sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (items < grid) grid = static_cast<int>(items);
  kern<<<grid, ATT_THREADS, S::TOTAL, stream>>>(tmQ, tmK, tmV, p, static_cast<int>(items));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("attn_prefill (split) launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

int launch_prefill_split(int D, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                         const AttnParams& p, int num_tiles, int max_ctas, cudaStream_t stream) {
  if (p.window > 0 || p.softcap > 0.f)
    return D == 128 ? launch_split_t<128, true>(tmQ, tmK, tmV, p, num_tiles, max_ctas, stream)
                    : launch_split_t<64, true>(tmQ, tmK, tmV, p, num_tiles, max_ctas, stream);
  return D == 128 ? launch_split_t<128, false>(tmQ, tmK, tmV, p, num_tiles, max_ctas, stream)
                  : launch_split_t<64, false>(tmQ, tmK, tmV, p, num_tiles, max_ctas, stream);
}

}  // namespace tw
