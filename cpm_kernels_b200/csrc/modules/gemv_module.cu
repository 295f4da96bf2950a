// Loadable kernel module `gemv.fatbin` for sm_100a: the decode-time matrix-vector kernels under the
// names and parameter lists that the reference's loader looks up (cpm_kernels/kernels/gemv.py:6-16;
// cuda/gemv.cu:26-164 defines their meaning).  A drop-in for the reference's own `gemv.fatbin`.
//
// Work split as in gemm_module.cu: grid.x walks batches, grid.y walks output elements (or 32-column
// strips for the transposed form), the threads of a block share one dot product.  Dot products read
// the matrix with 128-bit loads where alignment allows and accumulate in fp32 (the reference adds
// fp16 pairs, cuda/gemv.cu:90-97, and its tests allow 5e-2 for it); the int8 form is exact.
#include "common.cuh"

using namespace cpmk;
using namespace cpmk::mod;

namespace {

constexpr int kStrip = 32;

// sum_i mat[i] * vec[i] over dim_in fp16 pairs, shared by the threads of the block; fp32 partial per thread.
__device__ __forceinline__ float dot_fp16_partial(const half *mat, const half *vec, int32_t dim_in) {
    const int tid = flat_tid(), t = block_threads();
    float acc = 0.f;
    if ((dim_in & 7) == 0 && is_aligned(mat, 16) && is_aligned(vec, 16)) {
        for (int i = tid; i < (dim_in >> 3); i += t) {
            const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(mat) + i);
            const uint4 b = __ldg(reinterpret_cast<const uint4 *>(vec) + i);
            const __half2 *ha = reinterpret_cast<const __half2 *>(&a);
            const __half2 *hb = reinterpret_cast<const __half2 *>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
                acc = fmaf(fa.x, fb.x, acc);
                acc = fmaf(fa.y, fb.y, acc);
            }
        }
    } else {
        for (int i = tid; i < dim_in; i += t) acc = fmaf(__half2float(mat[i]), __half2float(__ldg(vec + i)), acc);
    }
    return acc;
}

}  // namespace

// out[b] = half(max_i |vec[b,i]| / 127.0)                                          (cuda/gemv.cu:26-40)
extern "C" __global__ void cu_gemv_calc_scale(int32_t batch, int32_t n, const half *vec, half *out) {
    __shared__ float buf[33];
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x) {
        float amax = 0.f;
        for (int i = tid; i < n; i += t) amax = fmaxf(fabsf(__half2float(vec[(int64_t)b * n + i])), amax);
        amax = block_combine(amax, buf, MaxOp());
        if (tid == 0) out[b] = scale_from_amax(amax);
    }
}

// out[b,i] = (int8_t) nearbyintf((float)vec[b,i] / (float)scale[b])                (cuda/gemv.cu:43-54)
extern "C" __global__ void cu_gemv_round(int32_t batch, int32_t n, const half *vec, const half *scale, int8_t *out) {
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x) {
        const float s = __half2float(__ldg(scale + b));
        for (int64_t i = (int64_t)blockIdx.y * t + tid; i < n; i += (int64_t)gridDim.y * t)
            out[(int64_t)b * n + i] = round_reference(__half2float(vec[(int64_t)b * n + i]), s);
    }
}

// out[b,o] = half(((float)sum_i mat[o,i] * vec[b,i]) * scale_vec[b] * scale_mat[o])   (cuda/gemv.cu:57-76)
extern "C" __global__ void cu_gemv_broadcast_mat_int8(int32_t batch, int32_t dim_out, int32_t dim_in, const half *scale_mat,
                                                      const char4 *mat, const half *scale_vec, const char4 *vec, half *out) {
    __shared__ int buf[33];
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int o = blockIdx.y; o < dim_out; o += gridDim.y) {
            const int8_t *mrow = reinterpret_cast<const int8_t *>(mat) + (int64_t)o * dim_in;
            const int8_t *vrow = reinterpret_cast<const int8_t *>(vec) + (int64_t)b * dim_in;
            int acc = 0;
            if ((dim_in & 15) == 0 && is_aligned(mrow, 16) && is_aligned(vrow, 16)) {
                for (int i = tid; i < (dim_in >> 4); i += t) {
                    const int4 a = __ldcs(reinterpret_cast<const int4 *>(mrow) + i);
                    const int4 v = __ldg(reinterpret_cast<const int4 *>(vrow) + i);
                    acc = __dp4a(a.x, v.x, acc);
                    acc = __dp4a(a.y, v.y, acc);
                    acc = __dp4a(a.z, v.z, acc);
                    acc = __dp4a(a.w, v.w, acc);
                }
            } else if ((dim_in & 3) == 0 && is_aligned(mrow, 4) && is_aligned(vrow, 4)) {
                for (int i = tid; i < (dim_in >> 2); i += t)
                    acc = __dp4a(reinterpret_cast<const int *>(mrow)[i], __ldg(reinterpret_cast<const int *>(vrow) + i), acc);
            } else {
                for (int i = tid; i < dim_in; i += t) acc += (int)mrow[i] * (int)vrow[i];
            }
            acc = block_combine(acc, buf, SumOp());
            if (tid == 0) {
                const float v = __fmul_rn(__fmul_rn((float)acc, __half2float(__ldg(scale_vec + b))), __half2float(__ldg(scale_mat + o)));
                out[(int64_t)b * dim_out + o] = __float2half_rn(v);
            }
        }
}

// out[b,o] = sum_i mat[b,o,i] * vec[b,i]                                           (cuda/gemv.cu:79-106)
extern "C" __global__ void cu_gemv_fp16(int32_t batch, int32_t dim_out, int32_t dim_in, const half2 *mat, const half2 *vec, half *out) {
    __shared__ float buf[33];
    const int tid = flat_tid();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int o = blockIdx.y; o < dim_out; o += gridDim.y) {
            const half *mrow = reinterpret_cast<const half *>(mat) + ((int64_t)b * dim_out + o) * dim_in;
            const half *vrow = reinterpret_cast<const half *>(vec) + (int64_t)b * dim_in;
            const float acc = block_combine(dot_fp16_partial(mrow, vrow, dim_in), buf, SumOp());
            if (tid == 0) out[(int64_t)b * dim_out + o] = __float2half_rn(acc);
        }
}

// out[b,o] = sum_i mat[b,i,o] * vec[b,i]                                           (cuda/gemv.cu:109-135)
extern "C" __global__ void cu_gemv_fp16_transpose(int32_t batch, int32_t dim_out, int32_t dim_in, const half *mat, const half *vec, half *out) {
    __shared__ float red[32][kStrip];
    const int t = block_threads(), tid = flat_tid();
    const int ncx = t < kStrip ? t : kStrip, nry = t / ncx, cx0 = tid % ncx, ry = tid / ncx;
    const bool active = ry < nry;
    const bool vec8 = (dim_out & 7) == 0 && is_aligned(mat, 16) && (t & 3) == 0 && t >= 32;
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int col0 = blockIdx.y * kStrip; col0 < dim_out; col0 += gridDim.y * kStrip) {
            const half *base = mat + (int64_t)b * dim_in * dim_out;
            const half *v = vec + (int64_t)b * dim_in;
            if (vec8) {
                // 4 column groups of 8 columns x (threads / 4) row lanes, 128-bit loads
                const int cg = tid & 3, lane = tid >> 2, nlanes = t >> 2;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                const int col = col0 + cg * 8;
                if (col < dim_out) {
                    for (int r = lane; r < dim_in; r += nlanes) {
                        const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(base + (int64_t)r * dim_out + col));
                        const float x = __half2float(__ldg(v + r));
                        const __half2 *h = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __half22float2(h[j]);
                            acc[2 * j] = fmaf(f.x, x, acc[2 * j]);
                            acc[2 * j + 1] = fmaf(f.y, x, acc[2 * j + 1]);
                        }
                    }
                }
                const int lanes = lanes_in_warp(tid, t);
                const unsigned mask = lanes == 32 ? 0xffffffffu : ((1u << lanes) - 1u);
                const int wl = tid & 31;
#pragma unroll
                for (int o = 16; o >= 4; o >>= 1) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float other = __shfl_xor_sync(mask, acc[j], o);
                        if ((wl ^ o) < lanes) acc[j] += other;
                    }
                }
                if (wl < 4) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) red[tid >> 5][cg * 8 + j] = acc[j];
                }
                __syncthreads();
                if (tid < kStrip && col0 + tid < dim_out) {
                    const int nwarps = (t + 31) >> 5;
                    float s = red[0][tid];
                    for (int w = 1; w < nwarps; ++w) s += red[w][tid];
                    out[(int64_t)b * dim_out + col0 + tid] = __float2half_rn(s);
                }
            } else {
                for (int cx = cx0; cx < kStrip; cx += ncx) {
                    float acc = 0.f;
                    const int col = col0 + cx;
                    if (active && col < dim_out)
                        for (int r = ry; r < dim_in; r += nry) acc = fmaf(__half2float(base[(int64_t)r * dim_out + col]), __half2float(__ldg(v + r)), acc);
                    if (active) red[ry][cx] = acc;
                }
                __syncthreads();
                if (ry == 0) {
                    for (int cx = cx0; cx < kStrip; cx += ncx) {
                        if (col0 + cx >= dim_out) continue;
                        float s = red[0][cx];
                        for (int y = 1; y < nry; ++y) s += red[y][cx];
                        out[(int64_t)b * dim_out + col0 + cx] = __float2half_rn(s);
                    }
                }
            }
            __syncthreads();
        }
}

// out[b,o] = sum_i mat[o,i] * vec[b,i]: one matrix shared by every batch entry      (cuda/gemv.cu:138-164)
extern "C" __global__ void cu_gemv_broadcast_mat_fp16(int32_t batch, int32_t dim_out, int32_t dim_in, const half2 *mat, const half2 *vec, half *out) {
    __shared__ float buf[33];
    const int tid = flat_tid();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int o = blockIdx.y; o < dim_out; o += gridDim.y) {
            const half *mrow = reinterpret_cast<const half *>(mat) + (int64_t)o * dim_in;
            const half *vrow = reinterpret_cast<const half *>(vec) + (int64_t)b * dim_in;
            const float acc = block_combine(dot_fp16_partial(mrow, vrow, dim_in), buf, SumOp());
            if (tid == 0) out[(int64_t)b * dim_out + o] = __float2half_rn(acc);
        }
}
