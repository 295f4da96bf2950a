// Shared host-side plumbing of the cpmk_b200 C-ABI library: error reporting, per-device state and
// the library-owned workspace.  Device helpers used by more than one kernel file live here too.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/cpmk_b200.h"

namespace cpmk {

// ---- error reporting --------------------------------------------------------------------------
void set_error(const char *fmt, ...);

#define CPMK_CUDA_TRY(expr)                                                                     \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess) {                                                                \
            ::cpmk::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return CPMK_ECUDA;                                                                  \
        }                                                                                       \
    } while (0)

#define CPMK_REQUIRE(cond, ...)                                                                 \
    do {                                                                                        \
        if (!(cond)) {                                                                          \
            ::cpmk::set_error(__VA_ARGS__);                                                     \
            return CPMK_EINVAL;                                                                 \
        }                                                                                       \
    } while (0)

// Checks the launch that was just issued (configuration errors surface here, not at the next sync).
#define CPMK_LAUNCH_CHECK()                                                                     \
    do {                                                                                        \
        cudaError_t _e = cudaGetLastError();                                                    \
        if (_e != cudaSuccess) {                                                                \
            ::cpmk::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
            return CPMK_ECUDA;                                                                  \
        }                                                                                       \
    } while (0)

// ---- per-device state -------------------------------------------------------------------------
// Workspace layout (one per (device, stream) pair, created on first use, never freed before exit):
//   [0, 256)                     status words (uint32): word 0 = first bounded-wait failure code
//   [256, 256 + 64 KiB)          tickets (uint32 counters, zero between calls; self-cleaning)
//   [kScratchOffset, kBytes)     scratch for partial results
struct Workspace {
    static constexpr size_t kStatusBytes = 256;
    static constexpr size_t kTicketBytes = 64 * 1024;
    static constexpr size_t kScratchOffset = kStatusBytes + kTicketBytes;
    static constexpr size_t kBytes = 16u << 20;
    static constexpr size_t kScratchBytes = kBytes - kScratchOffset;

    char *base = nullptr;
    uint32_t *status() const { return reinterpret_cast<uint32_t *>(base); }
    uint32_t *tickets() const { return reinterpret_cast<uint32_t *>(base + kStatusBytes); }
    char *scratch() const { return base + kScratchOffset; }
};

struct DeviceInfo {
    int device = -1;
    int arch = 0;        // major * 10 + minor
    int sm_count = 0;
    int max_smem_optin = 0;
};

// Returns CPMK_OK and fills *info for the current device; CPMK_EARCH when it is not sm_10x.
int32_t current_device_info(DeviceInfo *info);

// The workspace of (current device, stream); allocates it on first use.
int32_t get_workspace(cudaStream_t stream, Workspace *ws);

// Element-wise GELU over `count` fp16 values (cpmk_gelu.cu); in == out is allowed.
int32_t launch_gelu(int64_t count, const void *in, void *out, cudaStream_t stream);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda): a 3-d map
// over `ptr` with extents dims[0] (contiguous) .. dims[2], byte strides of dimensions 1 and 2, a box, element type
// fp16 (esz 2) / 8-bit (esz 1) / int32 (esz 4), 128-byte swizzle or none.  Returns false when the driver refuses.
bool encode_tiled_3d(void *map_out, int esz, const void *ptr, const uint64_t dims[3], const uint64_t strides[2], const uint32_t box[3], bool swizzle128);

inline cudaStream_t as_stream(cpmk_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace cpmk
