// Loadable kernel module `gemm.fatbin` for sm_100a: the quantisation / dequantisation kernels of the
// int8 linear layer under the names and parameter lists that the reference's loader looks up
// (cpm_kernels/kernels/gemm.py:6-19 lists them; cuda/gemm.cu:6-205 defines their meaning).  A drop-in
// for the reference's own `gemm.fatbin`: same symbols, same arguments, same results bit for bit.
//
// Work split: grid.x walks batches, grid.y walks rows (row kernels) or 32-column strips (column
// kernels), the threads of a block -- however many, in whatever shape -- share one row or strip.
// The reference's launchers give one block per row / strip; smaller grids work too (every kernel
// loops), which lifts the reference's limit of 65535 rows per call for callers that clamp grid.y.
// Where pointers and the row length allow, accesses are 128-bit; rounding uses the division-free
// rule of cpmk_round_rule.h with the reference expression as the fallback.
#include "common.cuh"

using namespace cpmk;
using namespace cpmk::mod;

namespace {

constexpr int kStrip = 32;          // columns per strip of the column kernels: the launchers size grid.y = ceil(m / 32)

// Threads of a block laid over a 32-column strip: `ncx` threads across the columns, `nry` row lanes.
struct StripSplit {
    int ncx, nry, cx0, ry;
    bool active;
    __device__ StripSplit() {
        const int t = block_threads(), tid = flat_tid();
        ncx = t < kStrip ? t : kStrip;
        nry = t / ncx;
        cx0 = tid % ncx;
        ry = tid / ncx;
        active = ry < nry;
    }
};

// 8 columns x all rows of a strip per thread with 128-bit loads: 4 column groups x (threads / 4) row lanes.
// f(vector, row) folds one 128-bit load into acc[8]; partial results are combined across row lanes with `op`
// and the 32 column results are left in red[0][0..31].
template <typename Fold, typename Op>
__device__ __forceinline__ void strip_vector_pass(const __half *base, int32_t n, int32_t m, int32_t col0, float init,
                                                  float (*red)[kStrip], Fold fold, Op op) {
    const int tid = flat_tid(), t = block_threads();
    const int cg = tid & 3, lane = tid >> 2, nlanes = t >> 2;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = init;
    const int col = col0 + cg * 8;
    if (col < m) {
        for (int r = lane; r < n; r += nlanes) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(base + (int64_t)r * m + col));
            fold(v, r, acc);
        }
    }
    // row lanes of one warp that share a column group: lanes differing in bits 2..4
    const int lanes = lanes_in_warp(tid, t);
    const unsigned mask = lanes == 32 ? 0xffffffffu : ((1u << lanes) - 1u);
    const int wl = tid & 31;
#pragma unroll
    for (int o = 16; o >= 4; o >>= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_xor_sync(mask, acc[i], o);
            if ((wl ^ o) < lanes) acc[i] = op(acc[i], other);
        }
    }
    if (wl < 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) red[tid >> 5][cg * 8 + i] = acc[i];
    }
    __syncthreads();
    if (tid < kStrip) {
        const int nwarps = (t + 31) >> 5;
        float v = red[0][tid];
        for (int w = 1; w < nwarps; ++w) v = op(v, red[w][tid]);
        red[0][tid] = v;
    }
    __syncthreads();
}

// The same with 2-byte loads, for any row length, alignment and thread count.  f(row, col) gives one term.
template <typename Term, typename Op>
__device__ __forceinline__ void strip_scalar_pass(int32_t n, int32_t m, int32_t col0, float init, float (*red)[kStrip],
                                                  Term term, Op op) {
    const StripSplit sp;
    for (int cx = sp.cx0; cx < kStrip; cx += sp.ncx) {
        float acc = init;
        const int col = col0 + cx;
        if (sp.active && col < m)
            for (int r = sp.ry; r < n; r += sp.nry) acc = op(acc, term(r, col));
        if (sp.active) red[sp.ry][cx] = acc;
    }
    __syncthreads();
    if (sp.ry == 0) {
        for (int cx = sp.cx0; cx < kStrip; cx += sp.ncx) {
            float v = red[0][cx];
            for (int y = 1; y < sp.nry; ++y) v = op(v, red[y][cx]);
            red[0][cx] = v;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void unpack8(const uint4 &v, float *f) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __half22float2(h[i]);
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}

__device__ __forceinline__ uint2 pack8(const int8_t *q) {
    uint2 o;
    o.x = (uint32_t)(uint8_t)q[0] | ((uint32_t)(uint8_t)q[1] << 8) | ((uint32_t)(uint8_t)q[2] << 16) | ((uint32_t)(uint8_t)q[3] << 24);
    o.y = (uint32_t)(uint8_t)q[4] | ((uint32_t)(uint8_t)q[5] << 8) | ((uint32_t)(uint8_t)q[6] << 16) | ((uint32_t)(uint8_t)q[7] << 24);
    return o;
}

}  // namespace

// out[b,r,i] = (int8_t) nearbyintf((float)mat[b,r,i] / (float)scale[b,r])        (cuda/gemm.cu:6-18)
extern "C" __global__ void cu_gemm_round(int32_t batch, int32_t n, int32_t m, const half *mat, const half *scale, int8_t *out) {
    const int tid = flat_tid(), t = block_threads();
    const bool vec = (m & 7) == 0 && is_aligned(mat, 16) && is_aligned(out, 8);
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            const float s = __half2float(__ldg(scale + row));
            const half *src = mat + row * m;
            int8_t *dst = out + row * m;
            if (vec) {
                float r_up, r_dn;
                cpmk_round_prepare(s, &r_up, &r_dn);
                const bool scale_ok = cpmk_scale_in_domain(s);
                for (int i = tid; i < (m >> 3); i += t) {
                    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(src) + i);
                    const float amax = half2_max_to_float(absmax8(v, __float2half2_rn(0.f)));
                    const float ru = (scale_ok && cpmk_round_domain_ok(amax, r_up)) ? r_up : __int_as_float(0x7fc00000);
                    reinterpret_cast<uint2 *>(dst)[i] = round8_one_scale(v, s, ru, r_dn);
                }
            } else {
                for (int i = tid; i < m; i += t) dst[i] = round_reference(__half2float(src[i]), s);
            }
        }
}

// The same with one scale per column: scale[b,i]                                   (cuda/gemm.cu:22-33)
extern "C" __global__ void cu_gemm_round_transpose(int32_t batch, int32_t n, int32_t m, const half *mat, const half *scale, int8_t *out) {
    const int tid = flat_tid(), t = block_threads();
    const bool vec = (m & 7) == 0 && is_aligned(mat, 16) && is_aligned(scale, 16) && is_aligned(out, 8);
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            const half *src = mat + row * m;
            const half *sc = scale + (int64_t)b * m;
            int8_t *dst = out + row * m;
            if (vec) {
                for (int i = tid; i < (m >> 3); i += t) {
                    float x[8], s[8];
                    unpack8(__ldcs(reinterpret_cast<const uint4 *>(src) + i), x);
                    unpack8(__ldg(reinterpret_cast<const uint4 *>(sc) + i), s);
                    int8_t q[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) q[j] = round_reference(x[j], s[j]);
                    reinterpret_cast<uint2 *>(dst)[i] = pack8(q);
                }
            } else {
                for (int i = tid; i < m; i += t) dst[i] = round_reference(__half2float(src[i]), __half2float(__ldg(sc + i)));
            }
        }
}

// out[b,r,c] = half(((float)mat[b,r,c] * sx) * sy[c])                              (cuda/gemm.cu:37-57)
extern "C" __global__ void cu_gemm_scale(int32_t batch, int32_t n, int32_t m, const int32_t *mat, const half *scale_x, const half *scale_y,
                                         half *out, bool broad_cast_x, bool broad_cast_y) {
    const int tid = flat_tid(), t = block_threads();
    const bool vec = (m & 7) == 0 && is_aligned(mat, 16) && is_aligned(scale_y, 16) && is_aligned(out, 16);
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            const float sx = __half2float(__ldg(scale_x + (broad_cast_x ? r : row)));
            const half *sy = scale_y + (broad_cast_y ? 0 : (int64_t)b * m);
            const int32_t *src = mat + row * m;
            half *dst = out + row * m;
            if (vec) {
                for (int i = tid; i < (m >> 3); i += t) {
                    const int4 a0 = __ldcs(reinterpret_cast<const int4 *>(src) + 2 * i);
                    const int4 a1 = __ldcs(reinterpret_cast<const int4 *>(src) + 2 * i + 1);
                    const int acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    float s[8];
                    unpack8(__ldg(reinterpret_cast<const uint4 *>(sy) + i), s);
                    __align__(16) half o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(__fmul_rn(__fmul_rn((float)acc[j], sx), s[j]));
                    reinterpret_cast<uint4 *>(dst)[i] = *reinterpret_cast<const uint4 *>(o);
                }
            } else {
                for (int i = tid; i < m; i += t)
                    dst[i] = __float2half_rn(__fmul_rn(__fmul_rn((float)src[i], sx), __half2float(__ldg(sy + i))));
            }
        }
}

// out[b,r] = half(max_i |mat[b,r,i]| / 127.0)                                      (cuda/gemm.cu:60-76)
extern "C" __global__ void cu_gemm_calc_scale(int32_t batch, int32_t n, int32_t m, const half *mat, half *out) {
    __shared__ float buf[33];
    const int tid = flat_tid(), t = block_threads();
    const bool vec = (m & 7) == 0 && is_aligned(mat, 16);
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            const half *src = mat + row * m;
            float amax = 0.f;
            if (vec) {
                __half2 m2 = __float2half2_rn(0.f);
                for (int i = tid; i < (m >> 3); i += t) m2 = absmax8(__ldcs(reinterpret_cast<const uint4 *>(src) + i), m2);
                amax = half2_max_to_float(m2);
            } else {
                for (int i = tid; i < m; i += t) amax = fmaxf(fabsf(__half2float(src[i])), amax);
            }
            amax = block_combine(amax, buf, MaxOp());
            if (tid == 0) out[row] = scale_from_amax(amax);
        }
}

// out[b,c] = half(max_r |in[b,r,c]| / 127.0)                                       (cuda/gemm.cu:79-98)
extern "C" __global__ void cu_gemm_calc_scale_transpose(int32_t batch, int32_t n, int32_t m, const half *in, half *out) {
    __shared__ float red[32][kStrip];
    const int tid = flat_tid(), t = block_threads();
    const bool vec = (m & 7) == 0 && is_aligned(in, 16) && (t & 3) == 0 && t >= 32;
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int col0 = blockIdx.y * kStrip; col0 < m; col0 += gridDim.y * kStrip) {
            const half *base = in + (int64_t)b * n * m;
            if (vec) {
                strip_vector_pass(base, n, m, col0, 0.f, red,
                                  [](const uint4 &v, int, float *acc) {
                                      float x[8];
                                      unpack8(v, x);
#pragma unroll
                                      for (int i = 0; i < 8; ++i) acc[i] = fmaxf(fabsf(x[i]), acc[i]);
                                  },
                                  MaxOp());
            } else {
                strip_scalar_pass(n, m, col0, 0.f, red,
                                  [&](int r, int col) { return fabsf(__half2float(base[(int64_t)r * m + col])); }, MaxOp());
            }
            for (int c = tid; c < kStrip; c += t)
                if (col0 + c < m) out[(int64_t)b * m + col0 + c] = scale_from_amax(red[0][c]);
            __syncthreads();
        }
}

// v = mat * scale_y[c];  s = max_c |v| / 127 (kept in fp32);  scale_x[b,r] = half(s);  out = (int8_t)nearbyintf(v / s)
//                                                                                  (cuda/gemm.cu:103-134)
extern "C" __global__ void cu_gemm_backward_round_scale(int32_t batch, int32_t n, int32_t m, const half *mat, const half *scale_y,
                                                        int8_t *out, half *scale_x, bool broad_cast_y) {
    __shared__ float buf[33];
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            const half *src = mat + row * m;
            const half *sy = scale_y + (broad_cast_y ? 0 : (int64_t)b * m);
            float amax = 0.f;
            for (int i = tid; i < m; i += t) amax = fmaxf(fabsf(__fmul_rn(__half2float(src[i]), __half2float(__ldg(sy + i)))), amax);
            amax = block_combine(amax, buf, MaxOp());
            const float s = __fdiv_rn(amax, 127.0f);
            if (tid == 0) scale_x[row] = __float2half_rn(s);
            for (int i = tid; i < m; i += t)
                out[row * m + i] = (int8_t)nearbyintf(__fdiv_rn(__fmul_rn(__half2float(src[i]), __half2float(__ldg(sy + i))), s));
        }
}

// The column form: v = mat * scale_x[r];  s = max_r |v| / 127;  scale_y[b,c] = half(s);  out = (int8_t)nearbyintf(v / s)
//                                                                                  (cuda/gemm.cu:137-172)
extern "C" __global__ void cu_gemm_backward_scale_round(int32_t batch, int32_t n, int32_t m, const half *mat, const half *scale_x,
                                                        int8_t *out, half *scale_y, bool broad_cast_x) {
    __shared__ float red[32][kStrip];
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int col0 = blockIdx.y * kStrip; col0 < m; col0 += gridDim.y * kStrip) {
            const half *base = mat + (int64_t)b * n * m;
            const half *sx = scale_x + (broad_cast_x ? 0 : (int64_t)b * n);
            auto value = [&](int r, int col) { return __fmul_rn(__half2float(base[(int64_t)r * m + col]), __half2float(__ldg(sx + r))); };
            strip_scalar_pass(n, m, col0, 0.f, red, [&](int r, int col) { return fabsf(value(r, col)); }, MaxOp());
            for (int c = tid; c < kStrip; c += t)
                if (col0 + c < m) scale_y[(int64_t)b * m + col0 + c] = __float2half_rn(__fdiv_rn(red[0][c], 127.0f));
            const StripSplit sp;
            for (int cx = sp.cx0; cx < kStrip; cx += sp.ncx) {
                const int col = col0 + cx;
                if (!sp.active || col >= m) continue;
                const float s = __fdiv_rn(red[0][cx], 127.0f);
                for (int r = sp.ry; r < n; r += sp.nry)
                    out[(int64_t)b * n * m + (int64_t)r * m + col] = (int8_t)nearbyintf(__fdiv_rn(value(r, col), s));
            }
            __syncthreads();
        }
}

// out[b,r,c] = half(scale_x[b,r] * (float)mat[b,r,c])                              (cuda/gemm.cu:176-189)
extern "C" __global__ void cu_gemm_scale_x(int32_t batch, int32_t n, int32_t m, const int32_t *mat, const half *scale_x, half *out) {
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            const float sx = __half2float(__ldg(scale_x + row));
            for (int i = tid; i < m; i += t) out[row * m + i] = __float2half_rn(__fmul_rn(sx, (float)mat[row * m + i]));
        }
}

// out[b,r,c] = half((float)mat[b,r,c] * scale_y[b,c])                              (cuda/gemm.cu:192-205)
extern "C" __global__ void cu_gemm_scale_y(int32_t batch, int32_t n, int32_t m, const int32_t *mat, const half *scale_y, half *out) {
    const int tid = flat_tid(), t = block_threads();
    for (int b = blockIdx.x; b < batch; b += gridDim.x)
        for (int r = blockIdx.y; r < n; r += gridDim.y) {
            const int64_t row = (int64_t)b * n + r;
            for (int i = tid; i < m; i += t)
                out[row * m + i] = __float2half_rn(__fmul_rn((float)mat[row * m + i], __half2float(__ldg(scale_y + (int64_t)b * m + i))));
        }
}
