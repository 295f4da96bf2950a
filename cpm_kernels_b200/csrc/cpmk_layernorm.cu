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

// lane 0 of x += shfl_down(x, 16), 8, 4, 2, 1 over 32 values, for two columns at once; v holds the 16 sums of the
// first level (rows l and l + 16)
__device__ __forceinline__ float2 tree_sum16(float2 (&v)[16]) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
        for (int l = 0; l < o; ++l) {
            v[l].x = __fadd_rn(v[l].x, v[l + o].x);
            v[l].y = __fadd_rn(v[l].y, v[l + o].y);
        }
    }
    return v[0];
}

// Pass A: the sums of x (if RD_MEAN) and of x * x over one chunk of 1024 rows for a strip of 64 columns.
// Thread (cp, g): column pair cp of the strip, row block g of the chunk's 32 blocks of 32 rows.
// sums layout: [quantity (0: x, 1: x*x)][batch][chunk][m] floats.
constexpr int kLnSumsBlock = 1024;      // pass A: 32 column pairs x 32 row blocks, one 32-row block per thread
template <bool RD_MEAN>
__global__ void __launch_bounds__(kLnSumsBlock) ln_chunk_sums_kernel(int32_t n, int32_t m, int32_t chunks, const __half *__restrict__ mat,
                                                                 float *__restrict__ sums) {
    __shared__ float block_sums[2][32][kLnStripCols];
    const int cp = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int b = blockIdx.z, chunk = blockIdx.y, batch = gridDim.z;
    const int col = blockIdx.x * kLnStripCols + 2 * cp;
    const bool col_ok = col < m;                                   // m is even: both columns of the pair are in or out
    const __half *base = mat + (int64_t)b * n * m + col;
    {
        const int blk = g;
        const int r0 = chunk * kLnChunkRows + blk * 32;
        __half2 h[32];
#pragma unroll
        for (int l = 0; l < 32; ++l)
            h[l] = (col_ok && r0 + l < n) ? __ldg(reinterpret_cast<const __half2 *>(base + (int64_t)(r0 + l) * m)) : __float2half2_rn(0.f);
        // the first level of the tree pairs rows l and l + 16: formed as the values are converted, 16 partial sums live
        float2 v[16];
#pragma unroll
        for (int l = 0; l < 16; ++l) {
            const float2 f = __half22float2(h[l]), g2 = __half22float2(h[l + 16]);
            v[l] = make_float2(__fadd_rn(__fmul_rn(f.x, f.x), __fmul_rn(g2.x, g2.x)), __fadd_rn(__fmul_rn(f.y, f.y), __fmul_rn(g2.y, g2.y)));
        }
        const float2 s2 = tree_sum16(v);
        block_sums[1][blk][2 * cp] = s2.x;
        block_sums[1][blk][2 * cp + 1] = s2.y;
        if (RD_MEAN) {
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                const float2 f = __half22float2(h[l]), g2 = __half22float2(h[l + 16]);
                v[l] = make_float2(__fadd_rn(f.x, g2.x), __fadd_rn(f.y, g2.y));
            }
            const float2 s1 = tree_sum16(v);
            block_sums[0][blk][2 * cp] = s1.x;
            block_sums[0][blk][2 * cp + 1] = s1.y;
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
__global__ void __launch_bounds__(kLnBlock, 3) ln_quant_kernel(const LnParams p) {
    __shared__ __align__(16) __half lane_max[kLnRowLanes][kLnWideCols];
    const int t8 = threadIdx.x & (kLnWideCols / 8 - 1), rl = threadIdx.x / (kLnWideCols / 8);
    const int b = blockIdx.z, split = blockIdx.y, batch = gridDim.z;
    const int col = blockIdx.x * kLnWideCols + 8 * t8;
    const bool col_ok = col < p.m;                                 // m is a multiple of 8 on this path
    const int r_begin = split * p.rows_per_split;
    const int r_end = min(p.n, r_begin + p.rows_per_split);

    // statistics of the thread's 8 columns: chunk sums accumulated in order, as the reference's outer loop does
    float mean[8], rstd[8];
    if (col_ok) {
        float s1[8], s2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) s1[i] = s2[i] = 0.f;
        for (int c = 0; c < p.chunks; ++c) {
            const float4 *q2 = reinterpret_cast<const float4 *>(p.sums + (((int64_t)batch + b) * p.chunks + c) * p.m + col);
            const float4 a = __ldg(q2), d = __ldg(q2 + 1);
            const float t2[8] = {a.x, a.y, a.z, a.w, d.x, d.y, d.z, d.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) s2[i] = __fadd_rn(s2[i], t2[i]);
            if (RD_MEAN) {
                const float4 *q1 = reinterpret_cast<const float4 *>(p.sums + ((int64_t)b * p.chunks + c) * p.m + col);
                const float4 e = __ldg(q1), f = __ldg(q1 + 1);
                const float t1[8] = {e.x, e.y, e.z, e.w, f.x, f.y, f.z, f.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) s1[i] = __fadd_rn(s1[i], t1[i]);
            }
        }
        const float fn = (float)p.n;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float var = __fdiv_rn(s2[i], fn);
            mean[i] = 0.f;
            if (RD_MEAN) {
                mean[i] = __fdiv_rn(s1[i], fn);
                var = __fmaf_rn(-mean[i], mean[i], var);
            }
            rstd[i] = rsqrtf(__fadd_rn(var, p.eps));
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
            __half y0, y1;
            if (RD_MEAN) {
                y0 = __float2half(__fmul_rn(__fsub_rn(f.x, mean[2 * j]), rstd[2 * j]));
                y1 = __float2half(__fmul_rn(__fsub_rn(f.y, mean[2 * j + 1]), rstd[2 * j + 1]));
            } else {
                y0 = __float2half(__fmul_rn(f.x, rstd[2 * j]));
                y1 = __float2half(__fmul_rn(f.y, rstd[2 * j + 1]));
            }
            const __half2 yy = __halves2half2(y0, y1), a2 = __half2half2(a);
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

    // PASS 1: fold the maxima of the row ranges, derive the scales, round
    if (!col_ok) return;
    __half2 m2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) m2[j] = __float2half2_rn(0.f);
    for (int sp0 = 0; sp0 < p.splits; sp0 += 8) {              // eight independent loads at a time
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            v[u] = sp0 + u < p.splits ? __ldg(reinterpret_cast<const uint4 *>(p.amax_partial + ((int64_t)(sp0 + u) * batch + b) * p.m + col))
                                      : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const __half2 *h = reinterpret_cast<const __half2 *>(&v[u]);
#pragma unroll
            for (int j = 0; j < 4; ++j) m2[j] = __hmax2(h[j], m2[j]);
        }
    }
    float s[8], r_up[8], r_dn[8];
    __align__(16) __half sh[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __half22float2(m2[j]);
        sh[2 * j] = scale_from_amax(a.x);
        sh[2 * j + 1] = scale_from_amax(a.y);
        s[2 * j] = __half2float(sh[2 * j]);
        s[2 * j + 1] = __half2float(sh[2 * j + 1]);
        cpmk_round_prepare(s[2 * j], &r_up[2 * j], &r_dn[2 * j]);
        cpmk_round_prepare(s[2 * j + 1], &r_up[2 * j + 1], &r_dn[2 * j + 1]);
        if (!(cpmk_scale_in_domain(s[2 * j]) && cpmk_round_domain_ok(a.x, r_up[2 * j]))) r_up[2 * j] = __int_as_float(0x7fc00000);
        if (!(cpmk_scale_in_domain(s[2 * j + 1]) && cpmk_round_domain_ok(a.y, r_up[2 * j + 1]))) r_up[2 * j + 1] = __int_as_float(0x7fc00000);
    }
    if (split == 0 && rl == 0) *reinterpret_cast<uint4 *>(p.scale + (int64_t)b * p.m + col) = *reinterpret_cast<const uint4 *>(sh);
    int8_t *obase = p.out + (int64_t)b * p.n * p.m + col;
    const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
    for (int r0 = r_begin + rl; r0 < r_end; r0 += 2 * kLnRowLanes) {
      uint4 vv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u)
          vv[u] = r0 + kLnRowLanes * u < r_end ? __ldg(reinterpret_cast<const uint4 *>(base + (int64_t)(r0 + kLnRowLanes * u) * p.m))
                                               : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = r0 + kLnRowLanes * u;
        if (r >= r_end) break;
        const uint4 v = vv[u];
        __half2 y[4];
        transform(v, r, y);
        uint32_t bits[8];
        bool agree = true, regular = true;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(y[j]);
            const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
            const float2 dn = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
            agree = agree && up.x == dn.x && up.y == dn.y;
            // a tie inside the domain has up = dn + 1; NaN and the out-of-domain marker fail both comparisons
            regular = regular && (up.x == dn.x || up.x - dn.x == 1.f) && (up.y == dn.y || up.y - dn.y == 1.f);
            bits[2 * j] = resolve_tie(__float_as_uint(up.x), __float_as_uint(dn.x));
            bits[2 * j + 1] = resolve_tie(__float_as_uint(up.y), __float_as_uint(dn.y));
        }
        if (!agree && !regular) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(y[j]);
                bits[2 * j] = (uint8_t)round_reference(f.x, s[2 * j]);
                bits[2 * j + 1] = (uint8_t)round_reference(f.y, s[2 * j + 1]);
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
    ln_chunk_sums_kernel<RD_MEAN><<<grid_a, kLnSumsBlock, 0, stream>>>(p.n, p.m, p.chunks, p.mat, sums);
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
