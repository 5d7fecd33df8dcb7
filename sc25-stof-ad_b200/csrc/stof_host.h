// Host-side helpers shared by the C-ABI translation units: error text, argument checks,
// and TMA tensor-map construction through the driver entry point (resolved at run time so
// that the library links against the CUDA runtime only and still loads on a box without a GPU).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/stof_b200.h"

namespace stof {

void set_error(const char* fmt, ...);   // defined in stof_common.cu

#define STOF_REQUIRE(cond, ...)            \
    do {                                   \
        if (!(cond)) {                     \
            stof::set_error(__VA_ARGS__);  \
            return STOF_E_INVALID;         \
        }                                  \
    } while (0)

#define STOF_CUDA(call)                                                                   \
    do {                                                                                  \
        cudaError_t e__ = (call);                                                         \
        if (e__ != cudaSuccess) {                                                         \
            stof::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
            return STOF_E_CUDA;                                                           \
        }                                                                                 \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Encodes a tiled fp16 tensor map with 128-byte swizzle.  dims/box innermost first; strides in
// bytes for dims 1..rank-1.  Returns 0 on success (message set otherwise).
int make_tensor_map_f16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                        const uint32_t* box);

int sm_count();   // multiprocessors of the current device (cached per device)

}  // namespace stof
