// Layer norm -> per-row affine -> column quantisation in one entry point, for activations in the (batch, hidden, seq)
// layout: what feeds the int8 linear that follows a layer norm in that layout.  The reference runs four kernels for it
// -- cu_layernorm_forward (cuda/layernorm.cu:6-71), cu_arith_ln_mul or cu_arith_ln_mul_add (cuda/arith.cu:97-127),
// cu_gemm_calc_scale_transpose and cu_gemm_round_transpose (cuda/gemm.cu:22-33, 79-98) -- which read or write the
// fp16 tensor seven times.  Here the normalised and the scaled tensor are never stored: three passes read the input
// (from L2 after the first, when it fits) and the last one writes the int8 codes.
//
// Same bits as that chain.  The statistics follow the reference's summation order exactly: rows in chunks of 1024, a
// chunk as 32 blocks of 32 rows, the 32 rows of a block and the 32 block sums of a chunk each combined by the
// shuffle-down tree (offsets 16, 8, 4, 2, 1), chunk sums accumulated in order; var = fma(-mean, mean, S2 / n);
// rstd = rsqrtf(var + eps); y = half((x - mean) * rstd); the affine step in fp16 arithmetic.
#include <stdlib.h>

#include "cpmk_common.cuh"
#include "cpmk_quant_device.cuh"

namespace cpmk {
namespace {

constexpr int kLnBlock = 256;
constexpr int kLnStripCols = 64;        // pass A: columns per block (128-byte row segments)
constexpr int kLnWideCols = 512;        // passes B and C: columns per block (1 KiB row segments: 64 threads x 8 columns)
constexpr int kLnRowLanes = kLnBlock / (kLnWideCols / 8);   // 4 row lanes per block
constexpr int kLnChunkRows = 1024;      // the reference's outer loop step (WARP_SZ * WARP_SZ)

// Pass A: the sums of x (if RD_MEAN) and of x * x over one chunk of 1024 rows for a strip of 64 columns.
// Warp g takes row block g of the chunk's 32 blocks of 32 rows; lane (c8, l4) takes columns 8 c8 .. 8 c8 + 7 of the
// strip and the eight rows l4, l4 + 4, ..., l4 + 28 of the block.  The shuffle-down tree over the 32 rows of a block
// -- x[l] + x[l + 16], then offsets 8, 4, 2, 1 -- has the third-level values
//   c[l4] = ((x[l4] + x[l4+16]) + (x[l4+8] + x[l4+24])) + ((x[l4+4] + x[l4+20]) + (x[l4+12] + x[l4+28])),
// which a lane forms from its own rows in two rounds of four 16-byte loads, and the block's sum
// (c[0] + c[2]) + (c[1] + c[3]) comes from two exchanges between lanes: the same additions as the reference's.
// sums layout: [quantity (0: x, 1: x*x)][batch][chunk][m] floats.
// Two blocks per SM: 1024 threads of 32 registers for the RMS form (one row block per warp), 512 threads of 64
// registers when the sums of x are needed too (two row blocks per warp, one after the other).
template <bool RD_MEAN>
struct LnSumsShape {
    static constexpr int kRowBlocksPerWarp = RD_MEAN ? 2 : 1;
    static constexpr int kThreads = 1024 / kRowBlocksPerWarp;
};
template <bool RD_MEAN>
__global__ void __launch_bounds__(LnSumsShape<RD_MEAN>::kThreads, 2) ln_chunk_sums_kernel(int32_t n, int32_t m, int32_t chunks, const __half *__restrict__ mat,
                                                                    float *__restrict__ sums) {
    __shared__ __align__(16) float block_sums[2][32][kLnStripCols];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c8 = lane & 7, l4 = lane >> 3;
    const int b = blockIdx.z, chunk = blockIdx.y, batch = gridDim.z;
    const int col = blockIdx.x * kLnStripCols + 8 * c8;
    const bool col_ok = col < m;                                   // m is a multiple of 8: a thread's columns are all in or all out
#pragma unroll 1
    for (int gi = 0; gi < LnSumsShape<RD_MEAN>::kRowBlocksPerWarp; ++gi) {
        const int g = warp * LnSumsShape<RD_MEAN>::kRowBlocksPerWarp + gi;
        const int r0 = chunk * kLnChunkRows + g * 32 + l4;
        const __half *base = mat + (int64_t)b * n * m + (int64_t)r0 * m + col;
        float c2[8], c1[8];
        // round 0: rows l4, l4+16, l4+8, l4+24 -> (x[l4] + x[l4+16]) + (x[l4+8] + x[l4+24]);  round 1: the same, 4 rows on
#pragma unroll
        for (int round = 0; round < 2; ++round) {
            const int offs[4] = {4 * round, 4 * round + 16, 4 * round + 8, 4 * round + 24};
            uint4 x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                x[k] = (col_ok && r0 + offs[k] < n) ? __ldg(reinterpret_cast<const uint4 *>(base + offs[k] * m)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) f[k] = __half22float2(reinterpret_cast<const __half2 *>(&x[k])[j]);
                const float qx = __fadd_rn(__fadd_rn(__fmul_rn(f[0].x, f[0].x), __fmul_rn(f[1].x, f[1].x)),
                                           __fadd_rn(__fmul_rn(f[2].x, f[2].x), __fmul_rn(f[3].x, f[3].x)));
                const float qy = __fadd_rn(__fadd_rn(__fmul_rn(f[0].y, f[0].y), __fmul_rn(f[1].y, f[1].y)),
                                           __fadd_rn(__fmul_rn(f[2].y, f[2].y), __fmul_rn(f[3].y, f[3].y)));
                c2[2 * j] = round == 0 ? qx : __fadd_rn(c2[2 * j], qx);
                c2[2 * j + 1] = round == 0 ? qy : __fadd_rn(c2[2 * j + 1], qy);
                if (RD_MEAN) {
                    const float px = __fadd_rn(__fadd_rn(f[0].x, f[1].x), __fadd_rn(f[2].x, f[3].x));
                    const float py = __fadd_rn(__fadd_rn(f[0].y, f[1].y), __fadd_rn(f[2].y, f[3].y));
                    c1[2 * j] = round == 0 ? px : __fadd_rn(c1[2 * j], px);
                    c1[2 * j + 1] = round == 0 ? py : __fadd_rn(c1[2 * j + 1], py);
                }
            }
        }
        // (c[0] + c[2]) + (c[1] + c[3]): lanes l4 and l4 ^ 2 first, then l4 ^ 1; float addition commutes, so every lane
        // of a column group ends with the same bits
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            c2[i] = __fadd_rn(c2[i], __shfl_xor_sync(0xffffffffu, c2[i], 16));
            c2[i] = __fadd_rn(c2[i], __shfl_xor_sync(0xffffffffu, c2[i], 8));
            if (RD_MEAN) {
                c1[i] = __fadd_rn(c1[i], __shfl_xor_sync(0xffffffffu, c1[i], 16));
                c1[i] = __fadd_rn(c1[i], __shfl_xor_sync(0xffffffffu, c1[i], 8));
            }
        }
        if (l4 == 0) {
            float4 *dst2 = reinterpret_cast<float4 *>(&block_sums[1][g][8 * c8]);
            dst2[0] = make_float4(c2[0], c2[1], c2[2], c2[3]);
            dst2[1] = make_float4(c2[4], c2[5], c2[6], c2[7]);
            if (RD_MEAN) {
                float4 *dst1 = reinterpret_cast<float4 *>(&block_sums[0][g][8 * c8]);
                dst1[0] = make_float4(c1[0], c1[1], c1[2], c1[3]);
                dst1[1] = make_float4(c1[4], c1[5], c1[6], c1[7]);
            }
        }
    }
    __syncthreads();
    // the chunk's 32 block sums of one column, same tree; threads 0..63: x * x, threads 64..127: x
    const int q = threadIdx.x >> 6, c = threadIdx.x & 63;
    if (q < 2 && (q == 0 || RD_MEAN)) {
        const int which = q == 0 ? 1 : 0;
        float w[32];
#pragma unroll
        for (int l = 0; l < 32; ++l) w[l] = block_sums[which][l][c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int l = 0; l < o; ++l) w[l] = __fadd_rn(w[l], w[l + o]);
        }
        const int gc = blockIdx.x * kLnStripCols + c;
        if (gc < m) sums[(((int64_t)which * batch + b) * chunks + chunk) * m + gc] = w[0];
    }
}

struct LnParams {
    int32_t n, m, chunks, splits, rows_per_split;
    float eps;
    const __half *mat, *alpha, *beta;
    const float *sums;
    __half *amax_partial;      // [split][batch][m]
    __half *scale;             // (batch, m)
    int8_t *out;               // (batch, n, m)
};

// Passes B (PASS 0: column maxima of |y| over a row range) and C (PASS 1: scales and codes).
// Thread (t8, rl): columns c0 + 8 t8 .. + 7 of the 512-column strip, rows rl, rl + 4, ... of the block's row range
// (whole 1 KiB row segments per block: narrow strips leave most of every DRAM page to other blocks at other times).
template <int PASS, bool RD_MEAN, bool BIAS>
__global__ void __launch_bounds__(kLnBlock, PASS == 0 ? 3 : 2) ln_quant_kernel(const LnParams p) {
    __shared__ __align__(16) __half lane_max[kLnRowLanes][kLnWideCols];
    __shared__ __align__(16) float col_const[PASS == 0 ? 2 : 5][kLnWideCols];      // 1/std, mean; pass C also: r_up, r_dn, scale
    const int t8 = threadIdx.x & (kLnWideCols / 8 - 1), rl = threadIdx.x / (kLnWideCols / 8);
    const int b = blockIdx.z, split = blockIdx.y, batch = gridDim.z;
    const int col = blockIdx.x * kLnWideCols + 8 * t8;
    const bool col_ok = col < p.m;                                 // m is a multiple of 8 on this path
    const int r_begin = split * p.rows_per_split;
    const int r_end = min(p.n, r_begin + p.rows_per_split);

    // Per-column constants are derived once per block: the four row lanes of a column group split its 8 columns,
    // two each (columns col + 2 rl, col + 2 rl + 1), and share the results through shared memory.
    const int my2 = 8 * t8 + 2 * rl;                               // first of the thread's two columns, within the strip
    // statistics: chunk sums accumulated in order, as the reference's outer loop does
    if (col_ok) {
        float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
        for (int c = 0; c < p.chunks; ++c) {
            const float2 t2 = __ldg(reinterpret_cast<const float2 *>(p.sums + (((int64_t)batch + b) * p.chunks + c) * p.m + col + 2 * rl));
            s2.x = __fadd_rn(s2.x, t2.x), s2.y = __fadd_rn(s2.y, t2.y);
            if (RD_MEAN) {
                const float2 t1 = __ldg(reinterpret_cast<const float2 *>(p.sums + ((int64_t)b * p.chunks + c) * p.m + col + 2 * rl));
                s1.x = __fadd_rn(s1.x, t1.x), s1.y = __fadd_rn(s1.y, t1.y);
            }
        }
        const float fn = (float)p.n;
        const float sum2[2] = {s2.x, s2.y}, sum1[2] = {s1.x, s1.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float var = __fdiv_rn(sum2[i], fn), mu = 0.f;
            if (RD_MEAN) {
                mu = __fdiv_rn(sum1[i], fn);
                var = __fmaf_rn(-mu, mu, var);
            }
            col_const[0][my2 + i] = rsqrtf(__fadd_rn(var, p.eps));
            if (RD_MEAN) col_const[1][my2 + i] = mu;
        }
    }
    __syncthreads();
    float mean[8], rstd[8];
    {
        const float4 a = *reinterpret_cast<const float4 *>(&col_const[0][8 * t8]), d = *reinterpret_cast<const float4 *>(&col_const[0][8 * t8 + 4]);
        rstd[0] = a.x, rstd[1] = a.y, rstd[2] = a.z, rstd[3] = a.w, rstd[4] = d.x, rstd[5] = d.y, rstd[6] = d.z, rstd[7] = d.w;
        if (RD_MEAN) {
            const float4 e = *reinterpret_cast<const float4 *>(&col_const[1][8 * t8]), f = *reinterpret_cast<const float4 *>(&col_const[1][8 * t8 + 4]);
            mean[0] = e.x, mean[1] = e.y, mean[2] = e.z, mean[3] = e.w, mean[4] = f.x, mean[5] = f.y, mean[6] = f.z, mean[7] = f.w;
        }
    }

    // y = affine(half((x - mean) * rstd)) for 8 columns of one row
    auto transform = [&](const uint4 &v, int r, __half2 (&y)[4]) {
        const __half a = __ldg(p.alpha + r);
        const __half bb = BIAS ? __ldg(p.beta + r) : __float2half(0.f);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            // one packed conversion: each half is rounded to nearest on its own, as two __float2half calls would
            const __half2 yy = RD_MEAN ? __floats2half2_rn(__fmul_rn(__fsub_rn(f.x, mean[2 * j]), rstd[2 * j]),
                                                           __fmul_rn(__fsub_rn(f.y, mean[2 * j + 1]), rstd[2 * j + 1]))
                                       : __floats2half2_rn(__fmul_rn(f.x, rstd[2 * j]), __fmul_rn(f.y, rstd[2 * j + 1]));
            const __half2 a2 = __half2half2(a);
            y[j] = BIAS ? __hfma2(yy, a2, __half2half2(bb)) : __hmul2(yy, a2);
        }
    };
    const __half *base = p.mat + (int64_t)b * p.n * p.m + col;

    if (PASS == 0) {
        __half2 m2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) m2[j] = __float2half2_rn(0.f);
        if (col_ok) {
            // four rows per iteration, loads first: one 16-byte load in flight per thread does not cover the latency
            for (int r0 = r_begin + rl; r0 < r_end; r0 += 4 * kLnRowLanes) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    v[u] = r0 + kLnRowLanes * u < r_end ? __ldg(reinterpret_cast<const uint4 *>(base + (int64_t)(r0 + kLnRowLanes * u) * p.m))
                                                        : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (r0 + kLnRowLanes * u < r_end) {
                        __half2 y[4];
                        transform(v[u], r0 + kLnRowLanes * u, y);
#pragma unroll
                        for (int j = 0; j < 4; ++j) m2[j] = __hmax2(__habs2(y[j]), m2[j]);
                    }
                }
            }
        }
        *reinterpret_cast<uint4 *>(&lane_max[rl][8 * t8]) = *reinterpret_cast<const uint4 *>(m2);
        __syncthreads();
        for (int c = threadIdx.x; c < kLnWideCols; c += kLnBlock) {
            __half mx = lane_max[0][c];
#pragma unroll
            for (int l = 1; l < kLnRowLanes; ++l) mx = __hmax(mx, lane_max[l][c]);
            const int gc = blockIdx.x * kLnWideCols + c;
            if (gc < p.m) p.amax_partial[((int64_t)split * batch + b) * p.m + gc] = mx;
        }
        return;
    }

    // PASS 1: fold the maxima of the row ranges, derive the scales and multipliers (two columns per thread), round
    if (col_ok) {
        __half2 mx = __float2half2_rn(0.f);
        const __half *part = p.amax_partial + (int64_t)b * p.m + col + 2 * rl;
        for (int sp0 = 0; sp0 < p.splits; sp0 += 8) {              // eight independent loads at a time
            unsigned v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = sp0 + u < p.splits ? __ldg(reinterpret_cast<const unsigned *>(part + (int64_t)(sp0 + u) * batch * p.m)) : 0u;
#pragma unroll
            for (int u = 0; u < 8; ++u) mx = __hmax2(*reinterpret_cast<const __half2 *>(&v[u]), mx);
        }
        const float2 a = __half22float2(mx);
        const float amax[2] = {a.x, a.y};
        __half sh[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sh[i] = scale_from_amax(amax[i]);
            const float sf = __half2float(sh[i]);
            float up, dn;
            cpmk_round_prepare(sf, &up, &dn);
            // a column outside the rule's domain gets a NaN multiplier: its elements then fail the agreement test below
            if (!(cpmk_scale_in_domain(sf) && cpmk_round_domain_ok(amax[i], up))) up = __int_as_float(0x7fc00000);
            col_const[2][my2 + i] = up;
            col_const[3][my2 + i] = dn;
            col_const[4][my2 + i] = sf;
        }
        if (split == 0) *reinterpret_cast<__half2 *>(p.scale + (int64_t)b * p.m + col + 2 * rl) = __halves2half2(sh[0], sh[1]);
    }
    __syncthreads();
    if (!col_ok) return;
    float2 ru[4], rd[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        ru[j] = *reinterpret_cast<const float2 *>(&col_const[2][8 * t8 + 2 * j]);
        rd[j] = *reinterpret_cast<const float2 *>(&col_const[3][8 * t8 + 2 * j]);
    }
    int8_t *obase = p.out + (int64_t)b * p.n * p.m + col;
    const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
    constexpr int kRowsInFlight = 4;
    for (int r0 = r_begin + rl; r0 < r_end; r0 += kRowsInFlight * kLnRowLanes) {
        uint4 vv[kRowsInFlight];
#pragma unroll
        for (int u = 0; u < kRowsInFlight; ++u)
            vv[u] = r0 + kLnRowLanes * u < r_end ? __ldg(reinterpret_cast<const uint4 *>(base + (int64_t)(r0 + kLnRowLanes * u) * p.m))
                                                 : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < kRowsInFlight; ++u) {
            const int r = r0 + kLnRowLanes * u;
            if (r >= r_end) break;
            __half2 y[4];
            transform(vv[u], r, y);
            // both roundings of every element; their disagreement is summed on the FMA pipe as squared differences
            // (zero iff all agree; NaN -- a NaN or infinite element, or the out-of-domain marker -- propagates)
            float2 dn[4];
            float2 bad = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(y[j]);
                const float2 up = __ffma2_rn(f, ru[j], magic);
                dn[j] = __ffma2_rn(f, rd[j], magic);
                const float2 d = __fadd2_rn(up, make_float2(-dn[j].x, -dn[j].y));
                bad = __ffma2_rn(d, d, bad);
            }
            uint32_t bits[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bits[2 * j] = __float_as_uint(dn[j].x);
                bits[2 * j + 1] = __float_as_uint(dn[j].y);
            }
            const float bad_sum = bad.x + bad.y;
            if (!(bad_sum == 0.f)) {
                if (bad_sum < 64.f) {
                    // finite: every disagreement is an exact tie (up = dn + 1), resolved to the even neighbour
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 up = __ffma2_rn(__half22float2(y[j]), ru[j], magic);
                        bits[2 * j] = resolve_tie(__float_as_uint(up.x), bits[2 * j]);
                        bits[2 * j + 1] = resolve_tie(__float_as_uint(up.y), bits[2 * j + 1]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(y[j]);
                        bits[2 * j] = (uint8_t)round_reference(f.x, col_const[4][8 * t8 + 2 * j]);
                        bits[2 * j + 1] = (uint8_t)round_reference(f.y, col_const[4][8 * t8 + 2 * j + 1]);
                    }
                }
            }
            uint2 q;
            q.x = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
            q.y = __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410);
            *reinterpret_cast<uint2 *>(obase + (int64_t)r * p.m) = q;
        }
    }
}

template <bool RD_MEAN, bool BIAS>
int32_t launch_ln_quant(const LnParams &p, int32_t batch, const dim3 &grid_a, const dim3 &grid_bc, float *sums, cudaStream_t stream) {
    ln_chunk_sums_kernel<RD_MEAN><<<grid_a, LnSumsShape<RD_MEAN>::kThreads, 0, stream>>>(p.n, p.m, p.chunks, p.mat, sums);
    CPMK_LAUNCH_CHECK();
    ln_quant_kernel<0, RD_MEAN, BIAS><<<grid_bc, kLnBlock, 0, stream>>>(p);
    CPMK_LAUNCH_CHECK();
    ln_quant_kernel<1, RD_MEAN, BIAS><<<grid_bc, kLnBlock, 0, stream>>>(p);
    CPMK_LAUNCH_CHECK();
    (void)batch;
    return CPMK_OK;
}

}  // namespace
}  // namespace cpmk

using namespace cpmk;

extern "C" int32_t cpmk_layernorm_quantize_cols(int32_t batch, int32_t n, int32_t m, const void *mat, float eps, int32_t rd_mean,
                                                const void *alpha, const void *beta, void *scale_out, void *q_out, cpmk_stream_t stream_) {
    cudaStream_t stream = as_stream(stream_);
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    CPMK_REQUIRE(batch >= 0 && n >= 0 && m >= 0, "negative size: batch=%d n=%d m=%d", batch, n, m);
    CPMK_REQUIRE(batch <= 65535, "batch %d exceeds 65535", batch);
    if (batch == 0 || m == 0) return CPMK_OK;
    CPMK_REQUIRE(n > 0, "layer norm over an empty axis (n = 0)");
    CPMK_REQUIRE(mat && alpha && scale_out && q_out, "null tensor pointer");
    // 128-bit accesses to rows of the input and of the statistics
    CPMK_REQUIRE(m % 8 == 0 && aligned16(mat) && aligned16(scale_out) && (reinterpret_cast<uintptr_t>(q_out) & 7u) == 0,
                 "m must be a multiple of 8 and the tensors 16-byte aligned (m = %d)", m);
    Workspace ws;
    rc = get_workspace(stream, &ws);
    if (rc) return rc;
    LnParams p;
    p.n = n;
    p.m = m;
    p.chunks = (n + kLnChunkRows - 1) / kLnChunkRows;
    p.eps = eps;
    p.mat = static_cast<const __half *>(mat);
    p.alpha = static_cast<const __half *>(alpha);
    p.beta = static_cast<const __half *>(beta);
    const int strips = (m + kLnStripCols - 1) / kLnStripCols;            // pass A
    const int wide_strips = (m + kLnWideCols - 1) / kLnWideCols;        // passes B and C
    // row ranges: about two blocks per SM, so that all of them are resident at once (three fit; a second, nearly empty
    // wave would double the time), at least 32 rows each
    int64_t splits = ((int64_t)info.sm_count * 2) / ((int64_t)wide_strips * batch);
    const int64_t by_rows = (n + 31) / 32;
    if (splits > by_rows) splits = by_rows;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
    int rps = (int)((n + splits - 1) / splits);
    rps = (rps + 31) / 32 * 32;
    p.rows_per_split = rps;
    p.splits = (n + rps - 1) / rps;
    const size_t sums_bytes = sizeof(float) * 2 * (size_t)batch * p.chunks * m;
    const size_t amax_bytes = sizeof(__half) * (size_t)p.splits * batch * m;
    CPMK_REQUIRE(sums_bytes + amax_bytes + 256 <= Workspace::kScratchBytes, "tensor too large for the fused layer norm (batch=%d n=%d m=%d)", batch, n, m);
    float *sums = reinterpret_cast<float *>(ws.scratch());
    p.sums = sums;
    p.amax_partial = reinterpret_cast<__half *>(ws.scratch() + ((sums_bytes + 255) / 256) * 256);
    p.scale = static_cast<__half *>(scale_out);
    p.out = static_cast<int8_t *>(q_out);
    const dim3 grid_a(strips, p.chunks, batch), grid_bc(wide_strips, p.splits, batch);
    CPMK_REQUIRE(p.chunks <= 65535, "n = %d is too large", n);
    if (rd_mean) return beta ? launch_ln_quant<true, true>(p, batch, grid_a, grid_bc, sums, stream) : launch_ln_quant<true, false>(p, batch, grid_a, grid_bc, sums, stream);
    return beta ? launch_ln_quant<false, true>(p, batch, grid_a, grid_bc, sums, stream) : launch_ln_quant<false, false>(p, batch, grid_a, grid_bc, sums, stream);
}
