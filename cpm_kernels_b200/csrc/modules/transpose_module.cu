// Loadable kernel module `transpose.fatbin` for sm_100a: the batched fp16 transpose under the name and
// parameter list that the reference's loader looks up (cpm_kernels/kernels/transpose.py:4-27;
// cuda/transpose.cu:6-22 defines its meaning: out[b, c, r] = in[b, r, c] for in (batch, n, m)).
// A drop-in for the reference's own `transpose.fatbin`.
//
// The blocks of the grid, however the caller shaped it, share all 64 x 64 tiles of all batches in a
// block-stride loop, and the threads of a block, however many, share a tile's elements: rows are read
// and written as 32-bit pairs when n and m are even and the pointers 4-byte aligned, else element by
// element.  The reference's launch (one 32 x 32 block per 32 x 32 tile) is one of the valid shapes.
#include "common.cuh"

using namespace cpmk;
using namespace cpmk::mod;

namespace {
constexpr int kEdge = 64;
constexpr int kPitch = kEdge + 2;          // halves per tile row in shared memory (33 words: odd, so columns spread over the banks)
}

extern "C" __global__ void cu_transpose(int32_t batch, int32_t n, int32_t m, const half *in, half *out) {
    __shared__ __align__(4) unsigned short tile[kEdge * kPitch];
    const int tid = flat_tid(), nthreads = block_threads();
    const int64_t nblocks = (int64_t)gridDim.x * gridDim.y * gridDim.z;
    const int64_t block = blockIdx.x + (int64_t)gridDim.x * (blockIdx.y + (int64_t)gridDim.y * blockIdx.z);
    const int32_t tiles_r = (n + kEdge - 1) / kEdge, tiles_c = (m + kEdge - 1) / kEdge;
    const int64_t per_batch = (int64_t)tiles_r * tiles_c, total = per_batch * batch;
    const int64_t plane = (int64_t)n * m;
    const bool pairs = ((n | m) & 1) == 0 && is_aligned(in, 4) && is_aligned(out, 4);
    const unsigned short *src_all = reinterpret_cast<const unsigned short *>(in);
    unsigned short *dst_all = reinterpret_cast<unsigned short *>(out);

    for (int64_t t = block; t < total; t += nblocks) {
        const int64_t b = t / per_batch;
        const int32_t rest = (int32_t)(t - b * per_batch);
        const int32_t r0 = (rest / tiles_c) * kEdge, c0 = (rest % tiles_c) * kEdge;
        const unsigned short *src = src_all + b * plane;
        unsigned short *dst = dst_all + b * plane;
        if (pairs) {
            // phase 1: word (y, x) of the tile holds in[r0 + y, c0 + 2x .. 2x + 1]
            for (int e = tid; e < kEdge * (kEdge / 2); e += nthreads) {
                const int y = e >> 5, x = e & 31;
                if (r0 + y < n && c0 + 2 * x < m)
                    *reinterpret_cast<uint32_t *>(&tile[y * kPitch + 2 * x]) =
                        __ldcs(reinterpret_cast<const uint32_t *>(src + (int64_t)(r0 + y) * m + c0 + 2 * x));
            }
            __syncthreads();
            // phase 2: output row c0 + y takes the pair (tile[2x][y], tile[2x + 1][y])
            for (int e = tid; e < kEdge * (kEdge / 2); e += nthreads) {
                const int y = e >> 5, x = e & 31;
                if (c0 + y < m && r0 + 2 * x < n) {
                    const uint32_t v = (uint32_t)tile[(2 * x) * kPitch + y] | ((uint32_t)tile[(2 * x + 1) * kPitch + y] << 16);
                    __stcs(reinterpret_cast<uint32_t *>(dst + (int64_t)(c0 + y) * n + r0 + 2 * x), v);
                }
            }
        } else {
            for (int e = tid; e < kEdge * kEdge; e += nthreads) {
                const int y = e >> 6, x = e & 63;
                if (r0 + y < n && c0 + x < m) tile[y * kPitch + x] = src[(int64_t)(r0 + y) * m + c0 + x];
            }
            __syncthreads();
            for (int e = tid; e < kEdge * kEdge; e += nthreads) {
                const int y = e >> 6, x = e & 63;
                if (c0 + y < m && r0 + x < n) dst[(int64_t)(c0 + y) * n + r0 + x] = tile[x * kPitch + y];
            }
        }
        __syncthreads();
    }
}
