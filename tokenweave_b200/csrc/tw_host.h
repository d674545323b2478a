// Host-side helpers shared by the .cu launchers: error strings and TMA tensor-map creation
// through the driver entry point (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tw {

// Last host-side error of a launcher, readable through tw_last_error() by the bindings.
void set_last_error(const char* fmt, ...);
const char* last_error();

// Encode a tiled tensor map for a bf16 tensor of `rank` dimensions (innermost first).
// `strides_bytes[i]` is the byte stride of dimension i+1 (dimension 0 is contiguous).
// Swizzle is always 128 bytes, out-of-bounds elements read as zero.
// Returns false (and sets the last error) if the driver refuses the encoding.
bool make_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box);

// The same with the 64-byte swizzle (boxes whose rows are 64 bytes: the write-back blocks of the GEMM epilogue).
bool make_tensor_map_bf16_sw64(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                               const uint64_t* strides_bytes, const uint32_t* box);

// The same for a tensor of 8-bit elements (fp8 operands).
bool make_tensor_map_u8(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box);

int device_sm_count();

}  // namespace tw
