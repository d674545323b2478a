// Collective kernels issued from inside CUDA kernels over NVSwitch: the fused
// reduce-scatter + residual-add + RMSNorm + all-gather that replaces each tensor-parallel
// all-reduce of a decoder layer, stand-alone all-reduce / reduce-scatter / all-gather, the
// three-phase "simple fusion" and no-all-gather ablations, and a one-shot peer all-reduce.
//
// Reference counterparts: csrc/tokenweave_fused_kernels.cu:80-155 (fused kernel),
// csrc/tokenweave_artifact_kernels.cu:129-685 (ablations and multimem collectives),
// vllm/distributed/triton_comm/triton_comm.py:115-237 (Triton collectives, replaced here),
// csrc/custom_all_reduce.cuh:296-364 (one-shot / two-shot peer all-reduce).
//
// Two transports, chosen per launch: NVLS multimem (in-switch reduction on load, broadcast on
// store) when the symmetric buffer has a multicast mapping, else plain peer loads/stores
// (each rank pulls its shard from every peer and pushes the result to every peer).
//
// Differences from the reference kernel, all aimed at keeping more bytes in flight from few CTAs
// on NVLink 5: a CTA works on ROWS token rows at once (ROWS independent 16-byte multimem loads per
// thread before the first use), the rows stay in registers between the statistics pass and the
// normalisation pass (the reference re-reads the residual from HBM), and one block reduction
// serves ROWS rows. Numerics are the reference's: bf16 packed residual add, fp32 sum of squares
// over the rounded sums, normalise in fp32, round, multiply by the bf16 weight.
#include "comm.cuh"
#include "tw_host.h"
#include "tw_kernels.h"

namespace tw {

struct CommCtx {
  uint8_t* mc_base;               // multicast VA of the symmetric buffer (nullptr: peer transport)
  uint8_t* const* peer_bases;     // [world] unicast VA of every rank's copy (device array)
  uint32_t* const* signal_pads;   // [world] signal pad of every rank (device array)
  int rank, world;
  int channel_base;               // first signal-pad slot this launch may use
  unsigned long long budget_ns;   // time budget of every cross-GPU wait
  uint32_t* status;
};

// Sum of the 16 bytes at `off` over all ranks, pulled through peer pointers, fp32 accumulation.
__device__ __forceinline__ uint4 peer_reduce_bf16x8(const CommCtx& c, long long off) {
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int s = 0; s < c.world; ++s) {
    int peer = c.rank + 1 + s;
    if (peer >= c.world) peer -= c.world;
    const uint4 v = ld_sys_16(c.peer_bases[peer] + off);
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
__device__ __forceinline__ void peer_broadcast_16(const CommCtx& c, long long off, const uint4& v) {
  for (int s = 0; s < c.world; ++s) {
    int peer = c.rank + s;
    if (peer >= c.world) peer -= c.world;
    st_sys_16(c.peer_bases[peer] + off, v);
  }
}

// ---------------------------------------------------------------------------------------------
// Fused RS + residual add + RMSNorm + AG. The [T, H] bf16 region starts `off_bytes` into the
// symmetric buffer; this rank owns rows [rank*rows_per_rank, (rank+1)*rows_per_rank). `residual`
// points at this rank's shard of the residual stream (row stride ldr). mode: 0 = product kernel,
// 1 = no all-gather (normalised rows written to the local copy only).
template <int ROWS, bool MC>
__global__ void __launch_bounds__(1024)
fused_rs_norm_ag_kernel(const CommCtx c, long long off_bytes, __nv_bfloat16* __restrict__ residual,
                        long long ldr, const __nv_bfloat16* __restrict__ weight, int rows_per_rank, int H,
                        float eps, int mode) {
  __shared__ float scratch[ROWS * 32];
  const int nvec = H >> 3;
  const int v = threadIdx.x;
  const bool active = v < nvec;
  if (!barrier_all_ranks<MemOrder::Relaxed>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 0)) {
    if (threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
    return;
  }
  const uint4 wv = active ? reinterpret_cast<const uint4*>(weight)[v] : make_uint4(0, 0, 0, 0);
  const long long row_bytes = static_cast<long long>(H) * 2;
  const long long shard_off = off_bytes + static_cast<long long>(c.rank) * rows_per_rank * row_bytes;
  uint8_t* local_base = c.peer_bases[c.rank];

  // Software pipeline: the reduce-scatter loads of row group i+1 are in flight while group i goes
  // through the residual add, the block reduction and the broadcast stores.
  auto load_group = [&](int g, uint4 (&x)[ROWS]) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      x[r] = make_uint4(0, 0, 0, 0);
      if (active && g + r < rows_per_rank) {
        const long long off = shard_off + (g + r) * row_bytes + v * 16;
        x[r] = MC ? multimem_ld_reduce_bf16x8(c.mc_base + off) : peer_reduce_bf16x8(c, off);
      }
    }
  };
  const int step = gridDim.x * ROWS;
  uint4 x[ROWS];
  int g = blockIdx.x * ROWS;
  if (g < rows_per_rank) load_group(g, x);
  for (; g < rows_per_rank; g += step) {
    uint4 xn[ROWS];
    const bool more = g + step < rows_per_rank;
    if (more) load_group(g + step, xn);
    float ss[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      ss[r] = 0.f;
      if (active && g + r < rows_per_rank) {
        uint4* rp = reinterpret_cast<uint4*>(residual + (g + r) * ldr) + v;
        const uint4 rv = *rp;
        x[r].x = add_bf16x2(x[r].x, rv.x);
        x[r].y = add_bf16x2(x[r].y, rv.y);
        x[r].z = add_bf16x2(x[r].z, rv.z);
        x[r].w = add_bf16x2(x[r].w, rv.w);
        *rp = x[r];
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&x[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          ss[r] += f.x * f.x + f.y * f.y;
        }
      }
    }
    block_sum<ROWS>(ss, scratch);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (active && g + r < rows_per_rank) {
        const float inv = rsqrtf(ss[r] / static_cast<float>(H) + eps);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&x[r]);
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
        uint4 o;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          ou[j] = mul_bf16x2(pack_bf16x2(f.x * inv, f.y * inv), wu[j]);
        }
        const long long off = shard_off + (g + r) * row_bytes + v * 16;
        if (mode == 1) {
          *reinterpret_cast<uint4*>(local_base + off) = o;
        } else if (MC) {
          multimem_st_16(c.mc_base + off, o);
        } else {
          peer_broadcast_16(c, off, o);
        }
      }
    }
    if (more) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) x[r] = xn[r];
    }
  }
  if (!barrier_all_ranks<MemOrder::AcqRel>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 1)) {
    if (threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
  }
}

// "Simple fusion" ablation: the same result as three phases with the intermediate written to the
// local copy and re-read, and a cross-GPU barrier between phases.
template <bool MC>
__global__ void __launch_bounds__(1024)
simple_fusion_kernel(const CommCtx c, long long off_bytes, __nv_bfloat16* __restrict__ residual, long long ldr,
                     const __nv_bfloat16* __restrict__ weight, int rows_per_rank, int H, float eps) {
  __shared__ float scratch[32];
  const int nvec = H >> 3;
  const int v = threadIdx.x;
  const bool active = v < nvec;
  const long long row_bytes = static_cast<long long>(H) * 2;
  const long long shard_off = off_bytes + static_cast<long long>(c.rank) * rows_per_rank * row_bytes;
  uint8_t* local_base = c.peer_bases[c.rank];
  bool ok = barrier_all_ranks<MemOrder::Relaxed>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 0);
  if (ok) {
    // phase 1: reduce-scatter into the local copy
    for (int g = blockIdx.x; g < rows_per_rank; g += gridDim.x) {
      if (active) {
        const long long off = shard_off + g * row_bytes + v * 16;
        const uint4 x = MC ? multimem_ld_reduce_bf16x8(c.mc_base + off) : peer_reduce_bf16x8(c, off);
        *reinterpret_cast<uint4*>(local_base + off) = x;
      }
    }
    ok = barrier_all_ranks<MemOrder::AcqRel>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 1);
  }
  if (ok) {
    // phase 2: residual add + RMSNorm on the local shard
    const uint4 wv = active ? reinterpret_cast<const uint4*>(weight)[v] : make_uint4(0, 0, 0, 0);
    for (int g = blockIdx.x; g < rows_per_rank; g += gridDim.x) {
      float ss[1] = {0.f};
      uint4 x = make_uint4(0, 0, 0, 0);
      const long long off = shard_off + g * row_bytes + v * 16;
      if (active) {
        x = *reinterpret_cast<const uint4*>(local_base + off);
        uint4* rp = reinterpret_cast<uint4*>(residual + g * ldr) + v;
        const uint4 rv = *rp;
        x.x = add_bf16x2(x.x, rv.x);
        x.y = add_bf16x2(x.y, rv.y);
        x.z = add_bf16x2(x.z, rv.z);
        x.w = add_bf16x2(x.w, rv.w);
        *rp = x;
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          ss[0] += f.x * f.x + f.y * f.y;
        }
      }
      block_sum<1>(ss, scratch);
      if (active) {
        const float inv = rsqrtf(ss[0] / static_cast<float>(H) + eps);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&x);
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
        uint4 o;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          ou[j] = mul_bf16x2(pack_bf16x2(f.x * inv, f.y * inv), wu[j]);
        }
        *reinterpret_cast<uint4*>(local_base + off) = o;
      }
    }
    ok = barrier_all_ranks<MemOrder::AcqRel>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 2);
  }
  if (ok) {
    // phase 3: all-gather
    for (int g = blockIdx.x; g < rows_per_rank; g += gridDim.x) {
      if (active) {
        const long long off = shard_off + g * row_bytes + v * 16;
        const uint4 o = *reinterpret_cast<const uint4*>(local_base + off);
        if (MC) multimem_st_16(c.mc_base + off, o);
        else peer_broadcast_16(c, off, o);
      }
    }
    ok = barrier_all_ranks<MemOrder::AcqRel>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 3);
  }
  if (!ok && threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// Stand-alone collectives over `n_vec` 16-byte vectors starting `off_bytes` into the buffer; rank r
// owns vectors [r*n_vec/world, (r+1)*n_vec/world). op: 0 all-reduce (in place), 1 reduce-scatter
// (own slice reduced in place in the local copy), 2 all-gather (own slice broadcast).
template <bool MC>
__global__ void __launch_bounds__(1024)
collective_kernel(const CommCtx c, long long off_bytes, long long n_vec, int op) {
  if (!barrier_all_ranks<MemOrder::Relaxed>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 0)) {
    if (threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
    return;
  }
  const long long per_rank = n_vec / c.world;
  const long long first = per_rank * c.rank;
  uint8_t* local_base = c.peer_bases[c.rank];
  constexpr int UNROLL = 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < per_rank;
       i0 += stride * UNROLL) {
    uint4 x[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < per_rank) {
        const long long off = off_bytes + (first + i) * 16;
        if (op == 2) x[u] = *reinterpret_cast<const uint4*>(local_base + off);
        else x[u] = MC ? multimem_ld_reduce_bf16x8(c.mc_base + off) : peer_reduce_bf16x8(c, off);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < per_rank) {
        const long long off = off_bytes + (first + i) * 16;
        if (op == 1) *reinterpret_cast<uint4*>(local_base + off) = x[u];
        else if (MC) multimem_st_16(c.mc_base + off, x[u]);
        else peer_broadcast_16(c, off, x[u]);
      }
    }
  }
  if (!barrier_all_ranks<MemOrder::AcqRel>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 1)) {
    if (threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
  }
}

// One-shot peer all-reduce: every rank pulls the whole message from every peer and writes the sum
// to a private output (the small-message path of a classic custom all-reduce).
__global__ void __launch_bounds__(512)
oneshot_allreduce_kernel(const CommCtx c, long long off_bytes, long long n_vec, uint4* __restrict__ out) {
  if (!barrier_all_ranks<MemOrder::Relaxed>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 0)) {
    if (threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
    return;
  }
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec; i += stride)
    out[i] = peer_reduce_bf16x8(c, off_bytes + i * 16);
  // peers may overwrite their buffers only after everyone has finished reading them
  if (!barrier_all_ranks<MemOrder::AcqRel>(c.signal_pads, c.channel_base, c.rank, c.world, c.budget_ns, 1)) {
    if (threadIdx.x == 0) report_error(c.status, TW_ERR_PEER_TIMEOUT);
  }
}

// Waits (bounded) for a flag that the caller may or may not set: the device half of the
// failure-detection path. Reports TW_ERR_PEER_TIMEOUT through `status` and returns normally.
__global__ void wait_probe_kernel(uint32_t* flag, unsigned long long budget_ns, uint32_t* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_signal<MemOrder::AcqRel>(flag, budget_ns)) report_error(status, TW_ERR_PEER_TIMEOUT);
  }
}

static int comm_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s launch failed: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

static CommCtx make_ctx(void* mc_base, void* const* peer_bases, uint32_t* const* signal_pads, int rank,
                        int world, int channel_base, unsigned long long budget_ns, uint32_t* status) {
  CommCtx c;
  c.mc_base = reinterpret_cast<uint8_t*>(mc_base);
  c.peer_bases = reinterpret_cast<uint8_t* const*>(peer_bases);
  c.signal_pads = signal_pads;
  c.rank = rank;
  c.world = world;
  c.channel_base = channel_base;
  c.budget_ns = budget_ns;
  c.status = status;
  return c;
}

}  // namespace tw

using namespace tw;

extern "C" int tw_fused_rs_norm_ag(void* mc_base, void* const* peer_bases, uint32_t* const* signal_pads,
                                   int rank, int world, int channel_base, unsigned long long budget_ns,
                                   uint32_t* status, long long off_bytes, void* residual, long long ldr,
                                   const void* weight, int T, int H, float eps, int max_ctas, int mode,
                                   int rows_in_flight, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T % world != 0 || H % 8 != 0 || H / 8 > 1024 || ldr % 8 != 0 || off_bytes % 16 != 0) {
    set_last_error("fused_rs_norm_ag: need T %% world == 0, H %% 8 == 0, H <= 8192 (T=%d, H=%d, world=%d)", T,
                   H, world);
    return 1;
  }
  const int rows_per_rank = T / world;
  const int threads = ((H / 8 + 31) / 32) * 32;
  int grid = max_ctas > 0 ? max_ctas : 16;
  int rows = rows_in_flight;
  if (rows <= 0) rows = rows_per_rank >= grid * 4 ? 4 : (rows_per_rank >= grid * 2 ? 2 : 1);
  if (grid > 128) grid = 128;     // barrier flags exist for 128 CTAs x 8 ranks
  if (grid * rows > rows_per_rank) grid = (rows_per_rank + rows - 1) / rows;
  if (grid < 1) grid = 1;
  const CommCtx c = make_ctx(mc_base, peer_bases, signal_pads, rank, world, channel_base, budget_ns, status);
  auto res = reinterpret_cast<__nv_bfloat16*>(residual);
  auto w = reinterpret_cast<const __nv_bfloat16*>(weight);
  const bool mc = mc_base != nullptr;
  if (mode == 2) {
    if (mc) simple_fusion_kernel<true><<<grid, threads, 0, stream>>>(c, off_bytes, res, ldr, w, rows_per_rank, H, eps);
    else simple_fusion_kernel<false><<<grid, threads, 0, stream>>>(c, off_bytes, res, ldr, w, rows_per_rank, H, eps);
    return comm_check("simple_fusion");
  }
#define TW_FUSED_CASE(R)                                                                                    \
  case R:                                                                                                   \
    if (mc) fused_rs_norm_ag_kernel<R, true><<<grid, threads, 0, stream>>>(c, off_bytes, res, ldr, w,       \
                                                                           rows_per_rank, H, eps, mode);    \
    else fused_rs_norm_ag_kernel<R, false><<<grid, threads, 0, stream>>>(c, off_bytes, res, ldr, w,         \
                                                                         rows_per_rank, H, eps, mode);      \
    break;
  switch (rows) {
    TW_FUSED_CASE(1)
    TW_FUSED_CASE(2)
    TW_FUSED_CASE(4)
    default:
      set_last_error("fused_rs_norm_ag: rows_in_flight must be 1, 2 or 4");
      return 1;
  }
#undef TW_FUSED_CASE
  return comm_check("fused_rs_norm_ag");
}

extern "C" int tw_collective(void* mc_base, void* const* peer_bases, uint32_t* const* signal_pads, int rank,
                             int world, int channel_base, unsigned long long budget_ns, uint32_t* status,
                             long long off_bytes, long long n_bytes, int op, int max_ctas, cudaStream_t stream) {
  if (n_bytes <= 0) return 0;
  if (n_bytes % (16ll * world) != 0 || off_bytes % 16 != 0) {
    set_last_error("collective: message of %lld bytes is not a multiple of 16*world", n_bytes);
    return 1;
  }
  const long long n_vec = n_bytes / 16;
  int grid = max_ctas > 0 ? max_ctas : 16;
  const long long per_rank = n_vec / world;
  int threads = 1024;
  if (per_rank < 1024) threads = static_cast<int>(((per_rank + 31) / 32) * 32);
  const long long need = (per_rank + threads - 1) / threads;
  if (grid > 128) grid = 128;
  if (grid > need) grid = static_cast<int>(need);
  if (grid < 1) grid = 1;
  const CommCtx c = make_ctx(mc_base, peer_bases, signal_pads, rank, world, channel_base, budget_ns, status);
  if (mc_base != nullptr) collective_kernel<true><<<grid, threads, 0, stream>>>(c, off_bytes, n_vec, op);
  else collective_kernel<false><<<grid, threads, 0, stream>>>(c, off_bytes, n_vec, op);
  return comm_check("collective");
}

extern "C" int tw_oneshot_allreduce(void* const* peer_bases, uint32_t* const* signal_pads, int rank, int world,
                                    int channel_base, unsigned long long budget_ns, uint32_t* status,
                                    long long off_bytes, long long n_bytes, void* out, int max_ctas,
                                    cudaStream_t stream) {
  if (n_bytes <= 0) return 0;
  if (n_bytes % 16 != 0 || off_bytes % 16 != 0) {
    set_last_error("oneshot_allreduce: message must be a multiple of 16 bytes");
    return 1;
  }
  const long long n_vec = n_bytes / 16;
  int grid = max_ctas > 0 ? max_ctas : 36;
  if (grid > 128) grid = 128;
  const long long need = (n_vec + 511) / 512;
  if (grid > need) grid = static_cast<int>(need);
  const CommCtx c = make_ctx(nullptr, peer_bases, signal_pads, rank, world, channel_base, budget_ns, status);
  oneshot_allreduce_kernel<<<grid, 512, 0, stream>>>(c, off_bytes, n_vec, reinterpret_cast<uint4*>(out));
  return comm_check("oneshot_allreduce");
}

extern "C" int tw_wait_probe(uint32_t* flag, unsigned long long budget_ns, uint32_t* status,
                             cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, budget_ns, status);
  return comm_check("wait_probe");
}
