// Helpers of the loadable kernel modules (modules/gemm_module.cu, modules/gemv_module.cu).
//
// The reference loads `gemm.fatbin` / `gemv.fatbin` with cuModuleLoadData and launches their
// `extern "C"` kernels by name with grids and blocks computed in Python (cpm_kernels/kernels/base.py:
// 20-71, kernels/gemm.py:21-125, kernels/gemv.py:18-283).  The modules built from these files export
// the same names with the same parameter lists, so they load through that loader unchanged.  Every
// kernel derives its work split from gridDim / blockDim at run time: it is correct under the launch
// shapes the reference computes (including block sizes that are not a multiple of 32) and under any
// other shape a caller prefers, as long as grid.x covers `batch`.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "../cpmk_quant_device.cuh"

namespace cpmk {
namespace mod {

__device__ __forceinline__ int block_threads() { return blockDim.x * blockDim.y * blockDim.z; }
__device__ __forceinline__ int flat_tid() { return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z); }

// Lanes of this warp that exist (the last warp of a block may be partial).
__device__ __forceinline__ int lanes_in_warp(int tid, int nthreads) {
    const int first = tid & ~31;
    return nthreads - first < 32 ? nthreads - first : 32;
}

template <typename T, typename Op>
__device__ __forceinline__ T warp_combine(T v, int tid, int nthreads, Op op) {
    const int lanes = lanes_in_warp(tid, nthreads);
    const unsigned mask = lanes == 32 ? 0xffffffffu : ((1u << lanes) - 1u);
    const int lane = tid & 31;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const T other = __shfl_xor_sync(mask, v, o);
        if ((lane ^ o) < lanes) v = op(v, other);
    }
    return v;
}

// Combines one value per thread over the whole block (any thread count up to 1024) and returns the
// result to every thread.  `buf` holds 33 values of shared memory; three barriers.
template <typename T, typename Op>
__device__ __forceinline__ T block_combine(T v, T *buf, Op op) {
    const int tid = flat_tid(), nthreads = block_threads();
    v = warp_combine(v, tid, nthreads, op);
    if ((tid & 31) == 0) buf[tid >> 5] = v;
    __syncthreads();
    if (tid == 0) {
        const int nwarps = (nthreads + 31) >> 5;
        for (int w = 1; w < nwarps; ++w) v = op(v, buf[w]);
        buf[32] = v;
    }
    __syncthreads();
    v = buf[32];
    __syncthreads();          // buf may be reused by the caller's next row
    return v;
}

struct MaxOp {
    __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};
struct SumOp {
    __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
    __device__ __forceinline__ int operator()(int a, int b) const { return a + b; }
};

__device__ __forceinline__ bool is_aligned(const void *p, unsigned bytes) { return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0; }

}  // namespace mod
}  // namespace cpmk
