// In-kernel communication primitives over NVLink 5 / NVSwitch: multimem (NVLS) loads with
// in-switch reduction and broadcast stores, system-scope peer loads/stores, and a bounded
// cross-GPU CTA barrier on per-rank signal pads.
//
// The reference's device library (csrc/tokenweave_multimem_utils.cuh:67-207) spins without a
// bound and traps on failure; here every wait has a time budget and reports through the status
// word, so a missing peer costs one bounded wait and leaves the context usable.
#pragma once

#include "tw_common.cuh"

namespace tw {

// 16-byte multimem load: 8 bf16 summed over every GPU bound to the multicast object, fp32
// accumulation inside the switch, result rounded to bf16.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16-byte multimem store: the same 16 bytes land in every GPU's copy.
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_sys_16(const void* addr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_16(void* addr, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};"
               ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

enum class MemOrder { Relaxed, AcqRel };

template <MemOrder O, bool PUT>
__device__ __forceinline__ uint32_t cas_sys(uint32_t* addr, uint32_t cmp, uint32_t val) {
  uint32_t old;
  if (O == MemOrder::Relaxed) {
    asm volatile("atom.global.relaxed.sys.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  } else if (PUT) {
    asm volatile("atom.global.release.sys.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  } else {
    asm volatile("atom.global.acquire.sys.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  }
  return old;
}

// Raise the flag at `addr` (0 -> 1). Waits for a previous signal to be consumed first.
template <MemOrder O>
__device__ __forceinline__ bool put_signal(uint32_t* addr, uint64_t budget_ns) {
  if (cas_sys<O, true>(addr, 0u, 1u) == 0u) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (cas_sys<O, true>(addr, 0u, 1u) == 0u) return true;
    if (globaltimer_ns() - t0 > budget_ns) return false;
  }
}
// Consume the flag at `addr` (1 -> 0).
template <MemOrder O>
__device__ __forceinline__ bool wait_signal(uint32_t* addr, uint64_t budget_ns) {
  if (cas_sys<O, false>(addr, 1u, 0u) == 1u) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (cas_sys<O, false>(addr, 1u, 0u) == 1u) return true;
    if (globaltimer_ns() - t0 > budget_ns) return false;
  }
}

// Barrier between CTA `blockIdx.x` of every rank, one-way signals only. Thread t < world stores 1
// into rank t's flag [set][blockIdx.x * world + rank] (a plain system-scope store: nothing comes
// back over NVLink), then polls its own flag [set][.. + t] in local memory until it reads 1 and
// clears it. `seq` counts the barriers of the kernel: consecutive barriers alternate between two
// flag sets, which is what makes the plain store safe — a peer can run at most one barrier ahead
// (it cannot pass barrier k + 1 without this rank's signal for it, sent only after barrier k was
// consumed and cleared here), so its next signal lands in the other set, and the set of barrier k
// is written again only at barrier k + 2. Every kernel runs an even number of barriers, so each
// starts on set 0 and the pads are all-zero between kernels: no epoch, replayable from a CUDA
// graph. (The reference's compare-and-swap protocol, csrc/tokenweave_multimem_utils.cuh:157-207,
// pays a remote atomic round trip per signal; measured here that was about 8 us per barrier.)
// Returns false (for the whole CTA) if any wait ran out of budget.
constexpr int BARRIER_SET_WORDS = 128 * 8;   // flags of one set: up to 128 CTAs x 8 ranks

template <MemOrder O>
__device__ __forceinline__ bool barrier_all_ranks(uint32_t* const* signal_pads, int channel_base, int rank,
                                                  int world, uint64_t budget_ns, int seq) {
  int failed = 0;
  if (O == MemOrder::AcqRel) __syncthreads();  // every thread's stores precede the release
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    const int base = channel_base + (seq & 1) * BARRIER_SET_WORDS + blockIdx.x * world;
    uint32_t* remote = signal_pads[peer] + base + rank;
    uint32_t* local = signal_pads[rank] + base + peer;
    if (O == MemOrder::AcqRel)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(1u) : "memory");
    else
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(1u) : "memory");
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
      uint32_t v = 0;
      for (int i = 0; i < 64 && v == 0; ++i) {
        if (O == MemOrder::AcqRel)
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
        else
          asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
      }
      if (v != 0) break;
      if (globaltimer_ns() - t0 > budget_ns) {
        failed = 1;
        break;
      }
    }
    if (!failed) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(local), "r"(0u) : "memory");
  }
  return __syncthreads_or(failed) == 0;
}

}  // namespace tw
