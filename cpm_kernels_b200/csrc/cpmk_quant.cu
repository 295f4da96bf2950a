// Quantisation passes of the int8 linear layer for sm_100a: absmax scale, int8 rounding, their fused
// forms, and the int32 -> fp16 dequantisation.  All of them are HBM-bound streaming kernels: 128-bit
// coalesced loads, registers as the only staging, shuffle reductions, no division per element
// (see cpmk_round_rule.h).
//
// Replaces cuda/gemm.cu:6-205 of the reference (one 1024-thread block per row, 2-byte loads, 1-byte
// stores, an fp32 division per element, grid.y = n <= 65535).
#include <cuda.h>
#include <stdlib.h>

#include <mutex>

#include "cpmk_common.cuh"
#include "cpmk_ptx.cuh"
#include "cpmk_round_rule.h"
#include "cpmk_quant_device.cuh"

namespace cpmk {
namespace {

constexpr int kBlock = 256;

// ------------------------------------------------------------------------------------------------
// Row quantisation: `group` threads share one row (group = 8..256, a power of two), each holding up
// to NV 128-bit vectors of it in registers, so the row is read from HBM exactly once.
// MODE 0: scale and codes (fused);  1: scale only;  2: codes only, scale given.
// ------------------------------------------------------------------------------------------------
// FULL: every block has all its rows and every thread all NV vectors (no bounds predicates).
// PAIR: one launch quantises two operands of the same row length (the activations and the weight of a linear layer):
// blocks from `second.first_block` on work on the second operand.  One grid instead of two saves the ramp and the tail
// of the smaller launch.
struct SecondOperand {
    int64_t rows;
    const __half *mat;
    __half *scale;
    int8_t *out;
    unsigned first_block;
};
// MULTI: the scales and codes of the FIRST operand are written to `n` destinations instead of one (this GPU's buffer
// and its peers', reached through peer-mapped addresses): a rank that holds a slice of the activations' rows quantises
// it once and the stores themselves distribute the result -- the all-gather of the codes costs no second kernel and no
// second read.  Only stores cross the link.
constexpr int kMaxQuantDst = 8;
struct MultiDst {
    int32_t n;
    int8_t *codes[kMaxQuantDst];      // element (0, 0) of these rows in each destination
    __half *scale[kMaxQuantDst];
};
template <int NV, int MODE, bool FULL, bool PAIR = false, bool MULTI = false>
__global__ void __launch_bounds__(kBlock, NV <= 4 ? 6 : 4) quant_rows_kernel(int64_t rows, int32_t m, int group, const __half *__restrict__ mat,
                                                            __half *__restrict__ scale, int8_t *__restrict__ out,
                                                            const SecondOperand second = SecondOperand(), const MultiDst multi = MultiDst()) {
    __shared__ float warp_max[kBlock / 32];
    const int tid = threadIdx.x;
    unsigned block = blockIdx.x;
    bool multi_here = MULTI;
    if (PAIR && block >= second.first_block) {
        block -= second.first_block;
        rows = second.rows;
        mat = second.mat;
        scale = second.scale;
        out = second.out;
        multi_here = false;
    }
    // group is a power of two: shifts, not divisions (a division's latency would sit in front of the first load)
    const int group_log2 = 31 - __clz(group);
    const int rows_per_block = kBlock >> group_log2;
    const int lane_in_row = tid & (group - 1);
    const int64_t row = (int64_t)block * rows_per_block + (tid >> group_log2);
    const bool row_ok = FULL || row < rows;
    const int nvec = m >> 3;
    const uint4 *src = reinterpret_cast<const uint4 *>(mat + (row_ok ? row : 0) * (int64_t)m);

    uint4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int idx = lane_in_row + j * group;
        v[j] = (FULL || (row_ok && idx < nvec)) ? __ldcs(src + idx) : make_uint4(0, 0, 0, 0);
    }
    __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
    for (int j = 0; j < NV; ++j) m2 = absmax8(v[j], m2);
    const float local_max = half2_max_to_float(m2);

    float s;
    if (MODE == 2) {
        s = row_ok ? __half2float(scale[row]) : 1.0f;
    } else {
        float amax = local_max;
        const int shuffle_span = group < 32 ? group : 32;
        for (int o = shuffle_span >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (group > 32) {
            if ((tid & 31) == 0) warp_max[tid >> 5] = amax;
            __syncthreads();
            const int first_warp = (tid >> group_log2) * (group >> 5);
            amax = warp_max[first_warp];
            for (int w = 1; w < (group >> 5); ++w) amax = fmaxf(amax, warp_max[first_warp + w]);
        }
        const __half sh = scale_from_amax(amax);
        if (row_ok && lane_in_row == 0) {
            if (MULTI && multi_here) {
#pragma unroll
                for (int d = 0; d < kMaxQuantDst; ++d)
                    if (d < multi.n) multi.scale[d][row] = sh;
            } else {
                scale[row] = sh;
            }
        }
        s = __half2float(sh);
    }
    if (MODE == 1) return;
    float r_up, r_dn;
    cpmk_round_prepare(s, &r_up, &r_dn);
    if (!(cpmk_scale_in_domain(s) && cpmk_round_domain_ok(local_max, r_up))) r_up = __int_as_float(0x7fc00000);
    if (MULTI && multi_here) {
        uint2 q[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) q[j] = round8_one_scale(v[j], s, r_up, r_dn);
        const int64_t offset = (row_ok ? row : 0) * (int64_t)m;
#pragma unroll
        for (int d = 0; d < kMaxQuantDst; ++d) {
            if (d < multi.n) {
                uint2 *dst = reinterpret_cast<uint2 *>(multi.codes[d] + offset);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int idx = lane_in_row + j * group;
                    if (FULL || (row_ok && idx < nvec)) dst[idx] = q[j];
                }
            }
        }
        return;
    }
    uint2 *dst = reinterpret_cast<uint2 *>(out + (row_ok ? row : 0) * (int64_t)m);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int idx = lane_in_row + j * group;
        if (FULL || (row_ok && idx < nvec)) dst[idx] = round8_one_scale(v[j], s, r_up, r_dn);
    }
}

// Any row length / alignment: one block per row, scalar accesses, the reference expressions.
template <int MODE>
__global__ void __launch_bounds__(kBlock) quant_rows_generic_kernel(int64_t rows, int32_t m, const __half *__restrict__ mat,
                                                                    __half *__restrict__ scale, int8_t *__restrict__ out) {
    __shared__ float warp_max[kBlock / 32];
    __shared__ float row_scale;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const __half *src = mat + row * (int64_t)m;
        float s;
        if (MODE == 2) {
            s = __half2float(scale[row]);
        } else {
            float amax = 0.f;
            for (int i = threadIdx.x; i < m; i += kBlock) amax = fmaxf(fabsf(__half2float(src[i])), amax);
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < kBlock / 32; ++w) amax = fmaxf(amax, warp_max[w]);
                const __half sh = scale_from_amax(amax);
                scale[row] = sh;
                row_scale = __half2float(sh);
            }
            __syncthreads();
            s = row_scale;
        }
        if (MODE != 1) {
            for (int i = threadIdx.x; i < m; i += kBlock) out[row * (int64_t)m + i] = round_reference(__half2float(src[i]), s);
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------
// Column quantisation (reduction over the slow axis n of a (batch, n, m) tensor).
// A block covers a strip of 64 columns (8 threads x 8 halves) and 32 rows per step; the rows are cut
// into `splits` chunks so that the grid fills the machine.  Pass 1 writes per-chunk column maxima
// to scratch; pass 2 folds them, derives the scale and rounds.  Pass 2 walks chunks and rows in the
// opposite order to pass 1 so that it meets the most recently read lines in L2 first.
// ------------------------------------------------------------------------------------------------
constexpr int kStripCols = 64;
constexpr int kStripRows = 32;

__global__ void __launch_bounds__(kBlock) colmax_partial_kernel(int32_t n, int32_t m, int32_t rows_per_split, int32_t strip0,
                                                                const __half *__restrict__ mat, __half *__restrict__ partial) {
    __shared__ __half2 red[kStripRows][kStripCols / 2 + 1];
    const int cl = threadIdx.x & 7, rl = threadIdx.x >> 3;
    const int strip = strip0 + blockIdx.x;
    const int col = strip * kStripCols + cl * 8;
    const int split = blockIdx.y, b = blockIdx.z, splits = gridDim.y;
    const int r_begin = split * rows_per_split;
    const int r_end = min(n, r_begin + rows_per_split);
    const __half *base = mat + (int64_t)b * n * m;

    __half2 m2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) m2[i] = __float2half2_rn(0.f);
    if (col < m) {
        int r = r_begin + rl;
#pragma unroll 4
        for (; r < r_end; r += kStripRows) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(base + (int64_t)r * m + col));
            const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) m2[i] = __hmax2(__habs2(h[i]), m2[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) red[rl][cl * 4 + i] = m2[i];
    __syncthreads();
    if (threadIdx.x < kStripCols / 2) {
        __half2 acc = red[0][threadIdx.x];
#pragma unroll 8
        for (int r = 1; r < kStripRows; ++r) acc = __hmax2(acc, red[r][threadIdx.x]);
        const int c = strip * kStripCols + threadIdx.x * 2;
        if (c < m) *reinterpret_cast<__half2 *>(partial + ((int64_t)split * gridDim.z + b) * m + c) = acc;
    }
    (void)splits;
}

// scale[b, c] = half(max over splits / 127)
__global__ void __launch_bounds__(kBlock) colmax_finish_kernel(int32_t batch, int32_t m, int32_t splits,
                                                               const __half *__restrict__ partial, __half *__restrict__ scale) {
    const int64_t idx = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (idx >= (int64_t)batch * m) return;
    float amax = 0.f;
    for (int s = 0; s < splits; ++s) amax = fmaxf(amax, __half2float(partial[(int64_t)s * batch * m + idx]));
    scale[idx] = scale_from_amax(amax);
}

// SRC 0: fold the partial maxima, write the scale (blocks of split 0) and round.
// SRC 1: scale given by the caller (gemm_round_transpose); validity of the rule is checked per code.
template <int SRC>
__global__ void __launch_bounds__(kBlock) quant_cols_round_kernel(int32_t n, int32_t m, int32_t rows_per_split, int32_t splits, int32_t strip0,
                                                                  const __half *__restrict__ mat, const __half *__restrict__ partial,
                                                                  __half *__restrict__ scale, int8_t *__restrict__ out) {
    const int cl = threadIdx.x & 7, rl = threadIdx.x >> 3;
    const int col = (strip0 + blockIdx.x) * kStripCols + cl * 8;
    if (col >= m) return;
    const int split = gridDim.y - 1 - blockIdx.y, b = blockIdx.z, batch = gridDim.z;
    const int r_begin = split * rows_per_split;
    const int r_end = min(n, r_begin + rows_per_split);

    float s[8], r_up[8], r_dn[8];
    if (SRC == 0) {
        __half2 m2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) m2[i] = __float2half2_rn(0.f);
        for (int sp = 0; sp < splits; ++sp) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(partial + ((int64_t)sp * batch + b) * m + col));
            const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) m2[i] = __hmax2(h[i], m2[i]);
        }
        __align__(16) __half sh[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(m2[i]);
            sh[2 * i] = scale_from_amax(a.x);
            sh[2 * i + 1] = scale_from_amax(a.y);
            s[2 * i] = __half2float(sh[2 * i]);
            s[2 * i + 1] = __half2float(sh[2 * i + 1]);
            cpmk_round_prepare(s[2 * i], &r_up[2 * i], &r_dn[2 * i]);
            cpmk_round_prepare(s[2 * i + 1], &r_up[2 * i + 1], &r_dn[2 * i + 1]);
            if (!(cpmk_scale_in_domain(s[2 * i]) && cpmk_round_domain_ok(a.x, r_up[2 * i]))) r_up[2 * i] = __int_as_float(0x7fc00000);
            if (!(cpmk_scale_in_domain(s[2 * i + 1]) && cpmk_round_domain_ok(a.y, r_up[2 * i + 1]))) r_up[2 * i + 1] = __int_as_float(0x7fc00000);
        }
        if (split == 0 && rl == 0) *reinterpret_cast<uint4 *>(scale + (int64_t)b * m + col) = *reinterpret_cast<const uint4 *>(sh);
    } else {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(scale + (int64_t)b * m + col));
        const __half *h = reinterpret_cast<const __half *>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s[i] = __half2float(h[i]);
            cpmk_round_prepare(s[i], &r_up[i], &r_dn[i]);
            if (!cpmk_scale_in_domain(s[i])) r_up[i] = __int_as_float(0x7fc00000);
        }
    }

    const __half *base = mat + (int64_t)b * n * m;
    int8_t *obase = out + (int64_t)b * n * m;
    // rows of this thread, walked downwards: r = r_last, r_last - 32, ...
    const int count = (r_end - r_begin - rl + kStripRows - 1) / kStripRows;   // rows r_begin + rl + 32 i < r_end
#pragma unroll 2
    for (int i = count - 1; i >= 0; --i) {
        const int r = r_begin + rl + i * kStripRows;
        const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(base + (int64_t)r * m + col));
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
        uint32_t bits[8];
        bool ok = true;
        uint32_t range = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
            const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
            const float2 dn = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
            ok = ok && (up.x == dn.x);
            ok = ok && (up.y == dn.y);
            bits[2 * j] = __float_as_uint(dn.x);
            bits[2 * j + 1] = __float_as_uint(dn.y);
            if (SRC == 1) {
                // a code is valid iff its pattern is 0x4B400000 + q with -128 <= q <= 127
                range |= ((bits[2 * j] + 0x80u) ^ 0x4B400000u) | ((bits[2 * j + 1] + 0x80u) ^ 0x4B400000u);
            }
        }
        if (SRC == 1) ok = ok && (range < 0x100u);
        if (!ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
                const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
                const float2 dn = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
                // a tie inside the domain: up = dn + 1 (false for NaN / the out-of-domain marker), the even neighbour;
                // anything else irregular: the reference expression
                const bool fast_x = (up.x == dn.x || up.x - dn.x == 1.f) && (SRC != 1 || range < 0x100u);
                const bool fast_y = (up.y == dn.y || up.y - dn.y == 1.f) && (SRC != 1 || range < 0x100u);
                bits[2 * j] = fast_x ? resolve_tie(__float_as_uint(up.x), __float_as_uint(dn.x)) : (uint8_t)round_reference(f.x, s[2 * j]);
                bits[2 * j + 1] = fast_y ? resolve_tie(__float_as_uint(up.y), __float_as_uint(dn.y)) : (uint8_t)round_reference(f.y, s[2 * j + 1]);
            }
        }
        uint2 q;
        q.x = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
        q.y = __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410);
        *reinterpret_cast<uint2 *>(obase + (int64_t)r * m + col) = q;
    }
}

// ------------------------------------------------------------------------------------------------
// Streaming form of the fused column quantisation for operands of a few MB and more.  Same two passes, but each
// block owns a strip of up to 2048 columns (4 KiB row segments) and a range of rows, and pulls the segments through
// a 3-stage shared-memory ring with 1-d bulk asynchronous copies (one producer thread; eight segments per stage;
// two blocks per SM), so that ~190 KiB per SM are in flight without register staging.  Each of the 256 consumer
// threads owns eight columns.  PASS 0 leaves per-range column maxima in scratch; PASS 1 folds them, derives the
// scales and rounds, walking ranges and rows in the opposite order so that it starts on what L2 still holds.
// ------------------------------------------------------------------------------------------------
constexpr int kCsCols = 2048;
constexpr int kCsRows = 8;
constexpr int kCsStages = 3;
constexpr int kCsStageBytes = kCsRows * kCsCols * 2;            // 32 KiB
constexpr int kCsRingBytes = kCsStages * kCsStageBytes;         // 96 KiB
constexpr int kCsThreads = (kCsRows + 1) * 32;                  // 8 consumer warps + 1 producer warp
constexpr uint32_t kErrColqProducer = 0x301;
constexpr uint32_t kErrColqConsumer = 0x302;

template <int PASS>
__global__ void __launch_bounds__(kCsThreads, 2) quant_cols_stream_kernel(int32_t n, int32_t m, int32_t rows_per_split, int32_t splits,
                                                                          int32_t strip_cols, const __half *__restrict__ mat, __half *__restrict__ partial,
                                                                          __half *__restrict__ scale, int8_t *__restrict__ out,
                                                                          uint32_t *status) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t bars[2 * kCsStages];
    __shared__ uint32_t abort_word;
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + kCsStages);
    const uint32_t ring_base = smem_u32(ring);
    volatile uint32_t *abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strip = blockIdx.x, b = blockIdx.z, batch = gridDim.z;
    const int split = PASS == 0 ? (int)blockIdx.y : (int)(gridDim.y - 1 - blockIdx.y);
    const int c0 = strip * strip_cols;                                  // strip_cols <= kCsCols, a multiple of 8
    const int width = (m - c0) < strip_cols ? (m - c0) : strip_cols;
    const uint32_t seg_bytes = (uint32_t)width * 2u;
    const int i0 = split * rows_per_split;
    const int i1 = min(n, i0 + rows_per_split);
    const int groups = (i1 - i0 + kCsRows - 1) / kCsRows;
    const __half *base = mat + (int64_t)b * n * m + c0;

    if (threadIdx.x == 0) {
        for (int st = 0; st < kCsStages; ++st) {
            mbar_init(full_bar + 8 * st, 1);
            mbar_init(empty_bar + 8 * st, kCsRows);
        }
        abort_word = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == kCsRows) {
        // producer warp, one lane per row segment: a single thread issuing the eight copies of a stage one after another
        // took ~2600 cycles per stage (measured), about as long as the consumers need for it
        uint32_t stage = 0, phase = 0;
        // the maxima pass asks L2 to keep what it reads, the rounding pass (which reads the same rows again, last first)
        // releases it
        const uint64_t policy = PASS == 0 ? l2_policy_evict_last() : l2_policy_evict_first();
        for (int gi = 0; gi < groups; ++gi) {
            const int g = PASS == 0 ? gi : groups - 1 - gi;
            int ok = 1;
            if (lane == 0) ok = mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kErrColqProducer) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const int row = i0 + g * kCsRows;
            const int nr = (i1 - row) < kCsRows ? (i1 - row) : kCsRows;
            if (lane == 0) mbar_expect_tx(full_bar + 8 * stage, (uint32_t)nr * seg_bytes);
            __syncwarp();
            if (lane < nr)
                bulk_load_1d_hint(ring_base + stage * kCsStageBytes + (uint32_t)lane * (kCsCols * 2), base + (int64_t)(row + lane) * m, seg_bytes,
                                  full_bar + 8 * stage, policy);
            if (++stage == kCsStages) { stage = 0; phase ^= 1u; }
        }
    } else {
        const int t = threadIdx.x;                           // 0..255: columns c0 + 8 t .. + 7
        const bool col_ok = t * 8 < width;
        const int col = c0 + t * 8;
        __half2 m2[4];
        float s[8], r_up[8], r_dn[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) m2[i] = __float2half2_rn(0.f);
        if (PASS == 1 && col_ok) {
            for (int sp = 0; sp < splits; ++sp) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(partial + ((int64_t)sp * batch + b) * m + col));
                const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) m2[i] = __hmax2(h[i], m2[i]);
            }
            __align__(16) __half sh[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __half22float2(m2[i]);
                sh[2 * i] = scale_from_amax(a.x);
                sh[2 * i + 1] = scale_from_amax(a.y);
                s[2 * i] = __half2float(sh[2 * i]);
                s[2 * i + 1] = __half2float(sh[2 * i + 1]);
                cpmk_round_prepare(s[2 * i], &r_up[2 * i], &r_dn[2 * i]);
                cpmk_round_prepare(s[2 * i + 1], &r_up[2 * i + 1], &r_dn[2 * i + 1]);
                if (!(cpmk_scale_in_domain(s[2 * i]) && cpmk_round_domain_ok(a.x, r_up[2 * i]))) r_up[2 * i] = __int_as_float(0x7fc00000);
                if (!(cpmk_scale_in_domain(s[2 * i + 1]) && cpmk_round_domain_ok(a.y, r_up[2 * i + 1]))) r_up[2 * i + 1] = __int_as_float(0x7fc00000);
            }
            if (split == 0) *reinterpret_cast<uint4 *>(scale + (int64_t)b * m + col) = *reinterpret_cast<const uint4 *>(sh);
        }
        int8_t *obase = out + (int64_t)b * n * m + col;
        uint32_t stage = 0, phase = 0;
        for (int gi = 0; gi < groups; ++gi) {
            const int g = PASS == 0 ? gi : groups - 1 - gi;
            const int row = i0 + g * kCsRows;
            const int nr = (i1 - row) < kCsRows ? (i1 - row) : kCsRows;
            if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, status, kErrColqConsumer)) break;
            if (col_ok) {
                const uint8_t *src = ring + (size_t)stage * kCsStageBytes + (size_t)t * 16;
                if (PASS == 0) {
#pragma unroll
                    for (int r = 0; r < kCsRows; ++r) {
                        if (r < nr) {
                            const uint4 w = *reinterpret_cast<const uint4 *>(src + (size_t)r * (kCsCols * 2));
                            const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
                            for (int j = 0; j < 4; ++j) m2[j] = __hmax2(__habs2(h[j]), m2[j]);
                        }
                    }
                } else {
                    // every row of the stage goes out on the division-free path with no branch in between (a branch per
                    // row makes each row wait for the previous one's dependency chain); rows with a tie, a NaN or an
                    // out-of-domain scale are redone afterwards
                    uint32_t redo = 0u, irregular = 0u;       // rows with a disagreement / of those, rows with a NaN sum
                    const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
                    const float2 minus_one = make_float2(-1.f, -1.f);
                    int8_t *orow = obase + (int64_t)row * m;
#pragma unroll
                    for (int r = 0; r < kCsRows; ++r) {
                        // (slots of rows beyond nr hold older data: computed, never stored, never counted)
                        const uint4 w = *reinterpret_cast<const uint4 *>(src + (size_t)r * (kCsCols * 2));
                        const __half2 *h = reinterpret_cast<const __half2 *>(&w);
                        float2 dn[4];
                        float2 bad = make_float2(0.f, 0.f);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __half22float2(h[j]);
                            const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
                            dn[j] = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
                            const float2 d = __ffma2_rn(dn[j], minus_one, up);
                            bad = __ffma2_rn(d, d, bad);
                        }
                        uint2 q;
                        q.x = __byte_perm(__byte_perm(__float_as_uint(dn[0].x), __float_as_uint(dn[0].y), 0x0040),
                                          __byte_perm(__float_as_uint(dn[1].x), __float_as_uint(dn[1].y), 0x0040), 0x5410);
                        q.y = __byte_perm(__byte_perm(__float_as_uint(dn[2].x), __float_as_uint(dn[2].y), 0x0040),
                                          __byte_perm(__float_as_uint(dn[3].x), __float_as_uint(dn[3].y), 0x0040), 0x5410);
                        const float bad_sum = bad.x + bad.y;
                        if (r < nr) {
                            *reinterpret_cast<uint2 *>(orow + (int64_t)r * m) = q;
                            redo |= (bad_sum == 0.f ? 0u : 1u) << r;
                            irregular |= (bad_sum < 64.f ? 0u : 1u) << r;          // NaN compares false
                        }
                    }
                    while (redo) {
                        const int r = __ffs((int)redo) - 1;
                        redo &= redo - 1u;
                        const uint4 w = *reinterpret_cast<const uint4 *>(src + (size_t)r * (kCsCols * 2));
                        const __half2 *h = reinterpret_cast<const __half2 *>(&w);
                        uint32_t bits[8];
                        if (!((irregular >> r) & 1u)) {
                            // exact ties only: the even neighbour, no division.  Columns whose scale has few
                            // significant bits tie on many rows, so this path must stay cheap.
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __half22float2(h[j]);
                                const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
                                const float2 dn = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
                                bits[2 * j] = resolve_tie(__float_as_uint(up.x), __float_as_uint(dn.x));
                                bits[2 * j + 1] = resolve_tie(__float_as_uint(up.y), __float_as_uint(dn.y));
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __half22float2(h[j]);
                                bits[2 * j] = (uint8_t)round_reference(f.x, s[2 * j]);
                                bits[2 * j + 1] = (uint8_t)round_reference(f.y, s[2 * j + 1]);
                            }
                        }
                        uint2 q;
                        q.x = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
                        q.y = __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410);
                        *reinterpret_cast<uint2 *>(orow + (int64_t)r * m) = q;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
            if (++stage == kCsStages) { stage = 0; phase ^= 1u; }
        }
        if (PASS == 0 && col_ok && !*abort_flag)
            *reinterpret_cast<uint4 *>(partial + ((int64_t)split * batch + b) * m + col) = *reinterpret_cast<const uint4 *>(m2);
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);     // let copies in flight land before the ring is released
    }
}

// ------------------------------------------------------------------------------------------------
// Resident-strip form of the fused column quantisation: the operand is read from HBM once.
// A thread-block cluster owns a strip of 64 columns; each of its CTAs loads its share of the strip's rows into shared
// memory with tiled TMA copies (128-row boxes of 16 KiB, all requested up front; the column maxima of a box are taken
// as soon as it lands), the CTAs exchange their 64 column maxima through distributed shared memory, and every CTA
// rounds its rows out of shared memory.  3 bytes per element reach HBM instead of 5, in one launch, with no scratch and
// no tickets.  Up to 768 rows (96 KiB) per CTA, two or three CTAs per SM in different phases of their work, clusters of
// 1 to 8 CTAs: operands of up to 6144 rows (taller ones stay with the two-pass kernels, which measured faster there).
// ------------------------------------------------------------------------------------------------
constexpr int kRsCols = 64;
constexpr int kRsChunkRows = 128;
constexpr int kRsChunkBytes = kRsCols * kRsChunkRows * 2;      // 16 KiB
constexpr int kRsMaxChunks = 6;
constexpr int kRsMaxCluster = 16;
constexpr uint32_t kErrColqResident = 0x303;

// The codes of eight neighbouring columns of one row, each column with its own scale (see cpmk_round_rule.h).
__device__ __forceinline__ uint2 round8_per_column(const uint4 &v, const float (&s)[8], const float (&r_up)[8], const float (&r_dn)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
    const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
    uint32_t bits[8];
    float2 bad = make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
        const float2 dn = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
        const float2 d = __fadd2_rn(up, make_float2(-dn.x, -dn.y));
        bad = __ffma2_rn(d, d, bad);
        bits[2 * j] = __float_as_uint(dn.x);
        bits[2 * j + 1] = __float_as_uint(dn.y);
    }
    const float bad_sum = bad.x + bad.y;
    if (!(bad_sum == 0.f)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            const float2 up = __ffma2_rn(f, make_float2(r_up[2 * j], r_up[2 * j + 1]), magic);
            const float2 dn = __ffma2_rn(f, make_float2(r_dn[2 * j], r_dn[2 * j + 1]), magic);
            // a tie inside the domain: up = dn + 1 (false for NaN / the out-of-domain marker), the even neighbour;
            // anything else irregular: the reference expression
            const bool fast_x = up.x == dn.x || up.x - dn.x == 1.f;
            const bool fast_y = up.y == dn.y || up.y - dn.y == 1.f;
            bits[2 * j] = fast_x ? resolve_tie(__float_as_uint(up.x), __float_as_uint(dn.x)) : (uint8_t)round_reference(f.x, s[2 * j]);
            bits[2 * j + 1] = fast_y ? resolve_tie(__float_as_uint(up.y), __float_as_uint(dn.y)) : (uint8_t)round_reference(f.y, s[2 * j + 1]);
        }
    }
    uint2 q;
    q.x = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
    q.y = __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410);
    return q;
}

__global__ void __launch_bounds__(kBlock, 2) quant_cols_resident_kernel(const __grid_constant__ CUtensorMap tmap, int32_t n, int32_t m, int32_t rows_per_cta,
                                                                        int32_t chunks, __half *__restrict__ scale, int8_t *__restrict__ out,
                                                                        uint32_t *status) {
    extern __shared__ __align__(128) uint8_t strip[];            // [rows_per_cta][64] fp16, row after row
    __shared__ __align__(8) uint64_t bars[kRsMaxChunks];
    __shared__ __half2 red[kStripRows][kRsCols / 2 + 1];
    __shared__ __align__(16) __half my_max[kRsCols];
    __shared__ float col_s[kRsCols], col_up[kRsCols], col_dn[kRsCols];
    __shared__ uint32_t abort_word;
    volatile uint32_t *abort_flag = &abort_word;
    const uint32_t rank = cluster_rank_of_cta(), cluster = cluster_num_ctas();
    const int t = threadIdx.x, cl = t & 7, rl = t >> 3;
    const int strip_idx = blockIdx.x / cluster, b = blockIdx.y;
    const int c0 = strip_idx * kRsCols;
    const int row0 = (int)rank * rows_per_cta;
    const uint32_t strip_base = smem_u32(strip), bar_base = smem_u32(bars);

    if (t == 0) {
        for (int c = 0; c < chunks; ++c) mbar_init(bar_base + 8 * c, 1);
        abort_word = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // rows beyond n (and columns beyond m) are filled with zeros by the copy and still count towards its bytes
        for (int c = 0; c < chunks; ++c) {
            mbar_expect_tx(bar_base + 8 * c, kRsChunkBytes);
            tma_load_tile_3d(strip_base + c * kRsChunkBytes, &tmap, c0, row0 + c * kRsChunkRows, b, bar_base + 8 * c);
        }
    }
    __syncthreads();

    // ---- column maxima of this CTA's rows, box by box as they land ----
    __half2 m2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) m2[i] = __float2half2_rn(0.f);
    bool alive = true;
    for (int c = 0; c < chunks; ++c) {
        if (!mbar_wait(bar_base + 8 * c, 0u, abort_flag, status, kErrColqResident)) { alive = false; break; }
#pragma unroll
        for (int i = 0; i < kRsChunkRows / kStripRows; ++i) {
            const int r = c * kRsChunkRows + rl + i * kStripRows;
            const uint4 v = *reinterpret_cast<const uint4 *>(strip + ((size_t)r * kRsCols + cl * 8) * 2);
            const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) m2[j] = __hmax2(__habs2(h[j]), m2[j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) red[rl][cl * 4 + i] = m2[i];
    __syncthreads();
    if (t < kRsCols / 2) {
        __half2 acc = red[0][t];
#pragma unroll 8
        for (int r = 1; r < kStripRows; ++r) acc = __hmax2(acc, red[r][t]);
        reinterpret_cast<__half2 *>(my_max)[t] = acc;
    }
    // ---- exchange: every CTA of the cluster reads the 64 maxima of all of them ----
    cluster_arrive_release();
    cluster_wait_acquire();
    if (t < kRsCols) {
        float amax = 0.f;
        const uint32_t mine = smem_u32(&my_max[t]);
        uint16_t peer[kRsMaxCluster];
#pragma unroll
        for (uint32_t r = 0; r < (uint32_t)kRsMaxCluster; ++r) peer[r] = r < cluster ? ld_dsmem_u16(dsmem_address(mine, r)) : (uint16_t)0;
#pragma unroll
        for (int r = 0; r < kRsMaxCluster; ++r) amax = fmaxf(amax, __half2float(__ushort_as_half(peer[r])));
        const __half sh = scale_from_amax(amax);
        const float s = __half2float(sh);
        float r_up, r_dn;
        cpmk_round_prepare(s, &r_up, &r_dn);
        if (!(cpmk_scale_in_domain(s) && cpmk_round_domain_ok(amax, r_up))) r_up = __int_as_float(0x7fc00000);
        col_s[t] = s;
        col_up[t] = r_up;
        col_dn[t] = r_dn;
        if (rank == 0 && alive && c0 + t < m) scale[(int64_t)b * m + c0 + t] = sh;
    }
    // nobody reads this CTA's maxima after this arrival; the matching wait is at the end, so that no CTA exits earlier
    cluster_arrive_release();
    __syncthreads();

    // ---- round this CTA's rows out of shared memory ----
    const int col = c0 + cl * 8;
    if (alive && !*abort_flag && col < m) {
        float s[8], r_up[8], r_dn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j] = col_s[cl * 8 + j];
            r_up[j] = col_up[cl * 8 + j];
            r_dn[j] = col_dn[cl * 8 + j];
        }
        int8_t *obase = out + (int64_t)b * n * m + col;
        const int r_end = min(rows_per_cta, n - row0);                // rows of this CTA inside the operand
#pragma unroll 4
        for (int r = rl; r < r_end; r += kStripRows) {
            const uint4 v = *reinterpret_cast<const uint4 *>(strip + ((size_t)r * kRsCols + cl * 8) * 2);
            *reinterpret_cast<uint2 *>(obase + (int64_t)(row0 + r) * m) = round8_per_column(v, s, r_up, r_dn);
        }
    }
    cluster_wait_acquire();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);          // let copies in flight land before the strip is released
    }
}

// Any shape: one thread per column, the reference expressions (m not a multiple of 8).
template <int MODE>
__global__ void __launch_bounds__(kBlock) quant_cols_generic_kernel(int32_t batch, int32_t n, int32_t m, const __half *__restrict__ mat,
                                                                    __half *__restrict__ scale, int8_t *__restrict__ out) {
    const int64_t idx = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (idx >= (int64_t)batch * m) return;
    const int b = (int)(idx / m), c = (int)(idx % m);
    const __half *base = mat + (int64_t)b * n * m + c;
    float s;
    if (MODE == 2) {
        s = __half2float(scale[idx]);
    } else {
        float amax = 0.f;
        for (int r = 0; r < n; ++r) amax = fmaxf(fabsf(__half2float(base[(int64_t)r * m])), amax);
        const __half sh = scale_from_amax(amax);
        scale[idx] = sh;
        s = __half2float(sh);
    }
    if (MODE != 1)
        for (int r = 0; r < n; ++r) out[(int64_t)b * n * m + (int64_t)r * m + c] = round_reference(__half2float(base[(int64_t)r * m]), s);
}

// ------------------------------------------------------------------------------------------------
// Dequantisation: out = half(((float)acc * sx) * sy).  MODE 0: both scales; 1: scale_x only
// (out = half(sx * (float)acc)); 2: scale_y only.
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kBlock) dequant_kernel(int64_t total_vec, int32_t n, int32_t m, const int32_t *__restrict__ mat,
                                                         const __half *__restrict__ scale_x, const __half *__restrict__ scale_y,
                                                         __half *__restrict__ out, int bx, int by) {
    const int64_t g = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (g >= total_vec) return;
    const int vec_per_row = m >> 3;
    const int64_t row = g / vec_per_row;              // b * n + r
    const int col = (int)(g - row * vec_per_row) << 3;
    const int b = (int)(row / n);
    const int r = (int)(row - (int64_t)b * n);
    float sx = 1.f;
    if (MODE != 2) sx = __half2float(__ldg(scale_x + (bx ? r : row)));
    float sy[8];
    if (MODE != 1) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(scale_y + (by ? 0 : (int64_t)b * m) + col));
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            sy[2 * i] = f.x;
            sy[2 * i + 1] = f.y;
        }
    }
    const int4 a0 = __ldcs(reinterpret_cast<const int4 *>(mat + g * 8));
    const int4 a1 = __ldcs(reinterpret_cast<const int4 *>(mat + g * 8) + 1);
    const int acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    __align__(16) __half o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v;
        if (MODE == 0) v = __fmul_rn(__fmul_rn((float)acc[i], sx), sy[i]);
        else if (MODE == 1) v = __fmul_rn(sx, (float)acc[i]);
        else v = __fmul_rn((float)acc[i], sy[i]);
        o[i] = __float2half_rn(v);
    }
    *reinterpret_cast<uint4 *>(out + g * 8) = *reinterpret_cast<const uint4 *>(o);
}

template <int MODE>
__global__ void __launch_bounds__(kBlock) dequant_generic_kernel(int64_t total, int32_t n, int32_t m, const int32_t *__restrict__ mat,
                                                                 const __half *__restrict__ scale_x, const __half *__restrict__ scale_y,
                                                                 __half *__restrict__ out, int bx, int by) {
    const int64_t g = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (g >= total) return;
    const int64_t row = g / m;
    const int c = (int)(g - row * m);
    const int b = (int)(row / n);
    const int r = (int)(row - (int64_t)b * n);
    float v = (float)mat[g];
    if (MODE == 0) v = __fmul_rn(__fmul_rn(v, __half2float(scale_x[bx ? r : row])), __half2float(scale_y[(by ? 0 : (int64_t)b * m) + c]));
    else if (MODE == 1) v = __fmul_rn(__half2float(scale_x[row]), v);
    else v = __fmul_rn(v, __half2float(scale_y[(int64_t)b * m + c]));
    out[g] = __float2half_rn(v);
}

// ------------------------------------------------------------------------------------------------
// Backward helpers (cuda/gemm.cu:103-172): the operand is mat * scale, its absmax scale stays in
// fp32 for the division, so the division-free rule (which relies on fp16 operands) does not apply.
// One block per row / one thread per column, reference expressions.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock) backward_round_scale_kernel(int32_t batch, int32_t n, int32_t m, const __half *__restrict__ mat,
                                                                      const __half *__restrict__ scale_y, int8_t *__restrict__ out,
                                                                      __half *__restrict__ scale_x, int by) {
    __shared__ float warp_max[kBlock / 32];
    __shared__ float row_scale;
    const int64_t rows = (int64_t)batch * n;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = (int)(row / n);
        const __half *src = mat + row * (int64_t)m;
        const __half *sy = scale_y + (by ? 0 : (int64_t)b * m);
        float amax = 0.f;
        for (int i = threadIdx.x; i < m; i += kBlock)
            amax = fmaxf(fabsf(__fmul_rn(__half2float(src[i]), __half2float(__ldg(sy + i)))), amax);
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < kBlock / 32; ++w) amax = fmaxf(amax, warp_max[w]);
            const float s = __fdiv_rn(amax, 127.0f);
            row_scale = s;
            scale_x[row] = __float2half_rn(s);
        }
        __syncthreads();
        const float s = row_scale;
        for (int i = threadIdx.x; i < m; i += kBlock)
            out[row * (int64_t)m + i] = (int8_t)nearbyintf(__fdiv_rn(__fmul_rn(__half2float(src[i]), __half2float(__ldg(sy + i))), s));
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kBlock) backward_scale_round_kernel(int32_t batch, int32_t n, int32_t m, const __half *__restrict__ mat,
                                                                      const __half *__restrict__ scale_x, int8_t *__restrict__ out,
                                                                      __half *__restrict__ scale_y, int bx) {
    const int64_t idx = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (idx >= (int64_t)batch * m) return;
    const int b = (int)(idx / m), c = (int)(idx % m);
    const __half *base = mat + (int64_t)b * n * m + c;
    const __half *sx = scale_x + (bx ? 0 : (int64_t)b * n);
    float amax = 0.f;
    for (int r = 0; r < n; ++r) amax = fmaxf(fabsf(__fmul_rn(__half2float(base[(int64_t)r * m]), __half2float(__ldg(sx + r)))), amax);
    const float s = __fdiv_rn(amax, 127.0f);
    scale_y[idx] = __float2half_rn(s);
    for (int r = 0; r < n; ++r)
        out[(int64_t)b * n * m + (int64_t)r * m + c] =
            (int8_t)nearbyintf(__fdiv_rn(__fmul_rn(__half2float(base[(int64_t)r * m]), __half2float(__ldg(sx + r))), s));
}

// ------------------------------------------------------------------------------------------------
// host-side dispatch
// ------------------------------------------------------------------------------------------------
int32_t check_shape(int32_t batch, int32_t n, int32_t m) {
    CPMK_REQUIRE(batch >= 0 && n >= 0 && m >= 0, "negative size: batch=%d n=%d m=%d", batch, n, m);
    CPMK_REQUIRE((int64_t)batch * n * m < (int64_t(1) << 40), "tensor too large: batch=%d n=%d m=%d", batch, n, m);
    return CPMK_OK;
}

template <int MODE>
int32_t launch_quant_rows(int32_t batch, int32_t n, int32_t m, const void *mat, void *scale, void *out, cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_shape(batch, n, m);
    if (rc) return rc;
    const int64_t rows = (int64_t)batch * n;
    if (rows == 0 || m == 0) {
        if (MODE != 2 && rows > 0) CPMK_CUDA_TRY(cudaMemsetAsync(scale, 0, rows * sizeof(__half), stream));
        return CPMK_OK;
    }
    CPMK_REQUIRE(mat && (MODE == 1 || out) && scale, "null tensor pointer");
    const __half *src = static_cast<const __half *>(mat);
    __half *sc = static_cast<__half *>(scale);
    int8_t *dst = static_cast<int8_t *>(out);
    const bool vec_ok = (m % 8 == 0) && aligned16(mat) && (MODE == 1 || (reinterpret_cast<uintptr_t>(out) & 7u) == 0) && m <= 256 * 8 * 8;
    if (!vec_ok) {
        const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
        quant_rows_generic_kernel<MODE><<<grid, kBlock, 0, stream>>>(rows, m, src, sc, dst);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    const int nvec = m / 8;
    // four vectors (32 elements) per thread where the row is long enough: measured best on B200 (fewer threads
    // per row means fewer shuffle / barrier steps per byte, and more bytes in flight per thread)
    int group = 8;
    while (group < 256 && group * 4 < nvec) group <<= 1;
    const int nv = (nvec + group - 1) / group;                  // 1..8
    const int rows_per_block = kBlock / group;
    const int64_t blocks = ceil_div64(rows, rows_per_block);
    CPMK_REQUIRE(blocks < (int64_t(1) << 31), "too many rows: %lld", (long long)rows);
    const dim3 grid((unsigned)blocks);
    const bool full = (rows % rows_per_block == 0) && (nvec == group * nv) && (nv == 1 || nv == 2 || nv == 4 || nv == 6 || nv == 8);
#define CPMK_LAUNCH_ROWS(NVT)                                                                                        \
    do {                                                                                                             \
        if (full) quant_rows_kernel<NVT, MODE, true><<<grid, kBlock, 0, stream>>>(rows, m, group, src, sc, dst);     \
        else quant_rows_kernel<NVT, MODE, false><<<grid, kBlock, 0, stream>>>(rows, m, group, src, sc, dst);         \
    } while (0)
    if (nv <= 1) CPMK_LAUNCH_ROWS(1);
    else if (nv <= 2) CPMK_LAUNCH_ROWS(2);
    else if (nv <= 4) CPMK_LAUNCH_ROWS(4);
    else if (nv <= 6) CPMK_LAUNCH_ROWS(6);
    else CPMK_LAUNCH_ROWS(8);
#undef CPMK_LAUNCH_ROWS
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

// Fused scale + round of two operands with rows of the same length in one launch (see SecondOperand).
// `multi`: when given, the first operand's scales and codes go to its destinations (see MultiDst) and the second
// operand may be empty (rows1 == 0).
int32_t launch_quant_rows_pair(int64_t rows0, const void *mat0, void *scale0, void *out0, int64_t rows1, const void *mat1, void *scale1,
                               void *out1, int32_t m, cudaStream_t stream, bool *done, const MultiDst *multi = nullptr) {
    *done = false;
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    if (rows0 <= 0 || (rows1 <= 0 && !multi) || rows1 < 0 || m <= 0) return CPMK_OK;
    bool vec_ok = (m % 8 == 0) && m <= 256 * 8 * 8 && aligned16(mat0) && (rows1 == 0 || (aligned16(mat1) && (reinterpret_cast<uintptr_t>(out1) & 7u) == 0));
    if (multi) {
        for (int d = 0; d < multi->n; ++d) vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(multi->codes[d]) & 7u) == 0;
    } else {
        vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(out0) & 7u) == 0;
    }
    if (!vec_ok) return CPMK_OK;
    const int nvec = m / 8;
    int group = 8;
    while (group < 256 && group * 4 < nvec) group <<= 1;
    const int nv = (nvec + group - 1) / group;
    const int rows_per_block = kBlock / group;
    const int64_t blocks0 = ceil_div64(rows0, rows_per_block), blocks1 = ceil_div64(rows1, rows_per_block);
    if (blocks0 + blocks1 >= (int64_t(1) << 31)) return CPMK_OK;
    SecondOperand second;
    second.rows = rows1;
    second.mat = static_cast<const __half *>(mat1);
    second.scale = static_cast<__half *>(scale1);
    second.out = static_cast<int8_t *>(out1);
    second.first_block = (unsigned)blocks0;
    const dim3 grid((unsigned)(blocks0 + blocks1));
    const bool full = (rows0 % rows_per_block == 0) && (rows1 % rows_per_block == 0) && (nvec == group * nv) &&
                      (nv == 1 || nv == 2 || nv == 4 || nv == 6 || nv == 8);
    const __half *src = static_cast<const __half *>(mat0);
    __half *sc = static_cast<__half *>(scale0);
    int8_t *dst = static_cast<int8_t *>(out0);
#define CPMK_LAUNCH_ROWS_PAIR(NVT)                                                                                               \
    do {                                                                                                                         \
        if (multi) {                                                                                                             \
            if (full) quant_rows_kernel<NVT, 0, true, true, true><<<grid, kBlock, 0, stream>>>(rows0, m, group, src, sc, dst, second, *multi);  \
            else quant_rows_kernel<NVT, 0, false, true, true><<<grid, kBlock, 0, stream>>>(rows0, m, group, src, sc, dst, second, *multi);      \
        } else if (full) quant_rows_kernel<NVT, 0, true, true><<<grid, kBlock, 0, stream>>>(rows0, m, group, src, sc, dst, second);     \
        else quant_rows_kernel<NVT, 0, false, true><<<grid, kBlock, 0, stream>>>(rows0, m, group, src, sc, dst, second);         \
    } while (0)
    if (nv <= 1) CPMK_LAUNCH_ROWS_PAIR(1);
    else if (nv <= 2) CPMK_LAUNCH_ROWS_PAIR(2);
    else if (nv <= 4) CPMK_LAUNCH_ROWS_PAIR(4);
    else if (nv <= 6) CPMK_LAUNCH_ROWS_PAIR(6);
    else CPMK_LAUNCH_ROWS_PAIR(8);
#undef CPMK_LAUNCH_ROWS_PAIR
    CPMK_LAUNCH_CHECK();
    *done = true;
    return CPMK_OK;
}

struct ColPlan {
    int strips, splits, rows_per_split;
};

ColPlan plan_cols(int32_t batch, int32_t n, int32_t m, int sm_count, size_t partial_elem_bytes, size_t scratch_bytes) {
    ColPlan p;
    p.strips = (m + kStripCols - 1) / kStripCols;
    const int64_t target = (int64_t)sm_count * 8;
    int64_t splits = target / ((int64_t)p.strips * batch);
    const int64_t max_by_rows = (n + kStripRows - 1) / kStripRows;
    if (splits > max_by_rows) splits = max_by_rows;
    if (splits > 64) splits = 64;
    const int64_t max_by_scratch = (int64_t)(scratch_bytes / (partial_elem_bytes * (size_t)batch * (size_t)m));
    if (splits > max_by_scratch) splits = max_by_scratch;
    if (splits < 1) splits = 1;
    int rps = (int)((n + splits - 1) / splits);
    rps = (rps + kStripRows - 1) / kStripRows * kStripRows;
    p.rows_per_split = rps;
    p.splits = (n + rps - 1) / rps;
    return p;
}

// Launches quant_cols_resident_kernel when the shape and the device admit it (*done says whether it did).
int32_t launch_quant_cols_resident(int32_t batch, int32_t n, int32_t m, const __half *src, __half *sc, int8_t *dst, cudaStream_t stream,
                                   const DeviceInfo &info, const Workspace &ws, bool *done) {
    *done = false;
    int cluster = 1;
    while (cluster <= kRsMaxCluster && (n + cluster - 1) / cluster > kRsMaxChunks * kRsChunkRows) cluster <<= 1;
    if (cluster > kRsMaxCluster) return CPMK_OK;
    const int rows_per_cta = ((n + cluster - 1) / cluster + kRsChunkRows - 1) / kRsChunkRows * kRsChunkRows;
    const int chunks = rows_per_cta / kRsChunkRows;
    const size_t smem = (size_t)rows_per_cta * kRsCols * 2;
    if (info.max_smem_optin < (int)smem + 8192 || batch > 65535) return CPMK_OK;
    const int dev = info.device & 63;
    static std::once_flag attr_once[64];
    static cudaError_t attr_err[64];
    std::call_once(attr_once[dev], [dev] {
        cudaError_t e = cudaFuncSetAttribute(quant_cols_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRsMaxChunks * kRsChunkBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(quant_cols_resident_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        attr_err[dev] = e;
        (void)cudaGetLastError();
    });
    if (attr_err[dev] != cudaSuccess) return CPMK_OK;
    const int64_t strips = (m + kRsCols - 1) / kRsCols;
    if (strips * cluster >= (int64_t(1) << 31)) return CPMK_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(strips * cluster), (unsigned)batch, 1);
    cfg.blockDim = dim3(kBlock, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // a cluster of this size and footprint must fit the device (asked once per device and cluster size)
    static int fits[64][kRsMaxCluster + 1];                  // 0: not asked, 1: fits, -1: does not
    static std::mutex fits_mutex;
    {
        std::lock_guard<std::mutex> lock(fits_mutex);
        if (fits[dev][cluster] == 0) {
            int clusters = 0;
            cudaLaunchConfig_t probe = cfg;
            probe.dynamicSmemBytes = kRsMaxChunks * kRsChunkBytes;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, quant_cols_resident_kernel, &probe);
            fits[dev][cluster] = (e == cudaSuccess && clusters > 0) ? 1 : -1;
            (void)cudaGetLastError();
        }
        if (fits[dev][cluster] < 0) return CPMK_OK;
    }
    CUtensorMap tmap;
    const uint64_t dims[3] = {(uint64_t)m, (uint64_t)n, (uint64_t)batch};
    const uint64_t strides[2] = {(uint64_t)m * 2, (uint64_t)n * (uint64_t)m * 2};
    const uint32_t box[3] = {(uint32_t)kRsCols, (uint32_t)kRsChunkRows, 1u};
    if (!encode_tiled_3d(&tmap, 2, src, dims, strides, box, false)) return CPMK_OK;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, quant_cols_resident_kernel, tmap, n, m, (int32_t)rows_per_cta, (int32_t)chunks, sc, dst, ws.status());
    if (e != cudaSuccess) {
        set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e), __FILE__, __LINE__);
        return CPMK_ECUDA;
    }
    *done = true;
    return CPMK_OK;
}

// MODE 0: fused; 1: scale only; 2: round only with the caller's scale
template <int MODE>
int32_t launch_quant_cols(int32_t batch, int32_t n, int32_t m, const void *mat, void *scale, void *out, cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_shape(batch, n, m);
    if (rc) return rc;
    if (batch == 0 || m == 0) return CPMK_OK;
    if (n == 0) {
        if (MODE != 2) CPMK_CUDA_TRY(cudaMemsetAsync(scale, 0, (size_t)batch * m * sizeof(__half), stream));
        return CPMK_OK;
    }
    CPMK_REQUIRE(mat && (MODE == 1 || out) && scale, "null tensor pointer");
    const __half *src = static_cast<const __half *>(mat);
    __half *sc = static_cast<__half *>(scale);
    int8_t *dst = static_cast<int8_t *>(out);
    const bool vec_ok = (m % 8 == 0) && aligned16(mat) && aligned16(scale) && (MODE == 1 || (reinterpret_cast<uintptr_t>(out) & 7u) == 0) &&
                        batch <= 65535 && (size_t)batch * m * sizeof(__half) <= Workspace::kScratchBytes;
    if (!vec_ok) {
        const int64_t blocks = ceil_div64((int64_t)batch * m, kBlock);
        quant_cols_generic_kernel<MODE><<<(unsigned)blocks, kBlock, 0, stream>>>(batch, n, m, src, sc, dst);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    if (MODE == 2) {
        const ColPlan p = plan_cols(batch, n, m, info.sm_count, sizeof(__half), Workspace::kScratchBytes);
        const dim3 grid(p.strips, p.splits, batch);
        quant_cols_round_kernel<1><<<grid, kBlock, 0, stream>>>(n, m, p.rows_per_split, p.splits, 0, src, nullptr, sc, dst);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    Workspace ws;
    rc = get_workspace(stream, &ws);
    if (rc) return rc;
    __half *partial = reinterpret_cast<__half *>(ws.scratch());
    if (MODE == 1) {
        const ColPlan p = plan_cols(batch, n, m, info.sm_count, sizeof(__half), Workspace::kScratchBytes);
        const dim3 grid(p.strips, p.splits, batch);
        colmax_partial_kernel<<<grid, kBlock, 0, stream>>>(n, m, p.rows_per_split, 0, src, partial);
        CPMK_LAUNCH_CHECK();
        const int64_t blocks = ceil_div64((int64_t)batch * m, kBlock);
        colmax_finish_kernel<<<(unsigned)blocks, kBlock, 0, stream>>>(batch, m, p.splits, partial, sc);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    // The resident-strip kernel reads the operand once: any operand whose rows fit 8 CTAs of 768 rows, big enough to
    // fill the machine.
    if ((int64_t)batch * n * m >= (int64_t(1) << 21) && n <= 8 * kRsMaxChunks * kRsChunkRows && !getenv("CPMK_QUANT_NO_RESIDENT")) {
        bool done = false;
        rc = launch_quant_cols_resident(batch, n, m, src, sc, dst, stream, info, ws, &done);
        if (rc) return rc;
        if (done) return CPMK_OK;
    }
    // Operands of 64 MB and more (below that the register-staged kernels measured faster): the streaming kernels
    // (96 KiB ring, two blocks per SM).
    if ((int64_t)batch * n * m >= (int64_t(1) << 25) && n >= 64 && m >= 1024 && info.max_smem_optin >= kCsRingBytes + 1024 && !getenv("CPMK_QUANT_NO_STREAM")) {
        static std::once_flag attr_once[64];
        static cudaError_t attr_err[64];
        const int dev = info.device & 63;
        std::call_once(attr_once[dev], [dev] {
            cudaError_t e = cudaFuncSetAttribute(quant_cols_stream_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCsRingBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(quant_cols_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCsRingBytes);
            attr_err[dev] = e;
        });
        if (attr_err[dev] == cudaSuccess) {
            // strips of equal width, at most 2048 columns (narrower strips mean bulk copies of 1 KiB and less: measured slower)
            const int64_t by_rows = (n + 63) / 64;
            const int64_t target = (int64_t)info.sm_count * 2;
            int strips = (m + kCsCols - 1) / kCsCols;
            const int strip_cols = ((m + strips - 1) / strips + 7) / 8 * 8;
            strips = (m + strip_cols - 1) / strip_cols;
            int64_t sp = target / ((int64_t)strips * batch);
            if (sp > by_rows) sp = by_rows;
            // (folding the per-range maxima once in a small kernel between the passes, instead of in each block's prologue
            // of the rounding pass, measured no faster: the extra kernel boundary costs what the prologues save)
            const int64_t by_scratch = (int64_t)(Workspace::kScratchBytes / (sizeof(__half) * (size_t)batch * (size_t)m));
            if (sp > by_scratch) sp = by_scratch;
            if (sp > 65535) sp = 65535;
            if (sp < 1) sp = 1;
            int rps = (int)((n + sp - 1) / sp);
            rps = (rps + kCsRows - 1) / kCsRows * kCsRows;
            const int nsp = (n + rps - 1) / rps;
            const dim3 grid(strips, nsp, batch);
            quant_cols_stream_kernel<0><<<grid, kCsThreads, kCsRingBytes, stream>>>(n, m, rps, nsp, strip_cols, src, partial, sc, dst, ws.status());
            CPMK_LAUNCH_CHECK();
            quant_cols_stream_kernel<1><<<grid, kCsThreads, kCsRingBytes, stream>>>(n, m, rps, nsp, strip_cols, src, partial, sc, dst, ws.status());
            CPMK_LAUNCH_CHECK();
            return CPMK_OK;
        }
    }
    // Fused form: absmax pass, then rounding pass over the same operand in the opposite row order.  (Walking the
    // operand in L2-sized column panels, so that the second read never reaches HBM, was tried and measured slower:
    // the per-panel launches are too small to fill the machine.)
    const ColPlan p = plan_cols(batch, n, m, info.sm_count, sizeof(__half), Workspace::kScratchBytes);
    const dim3 grid(p.strips, p.splits, batch);
    colmax_partial_kernel<<<grid, kBlock, 0, stream>>>(n, m, p.rows_per_split, 0, src, partial);
    CPMK_LAUNCH_CHECK();
    quant_cols_round_kernel<0><<<grid, kBlock, 0, stream>>>(n, m, p.rows_per_split, p.splits, 0, src, partial, sc, dst);
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

template <int MODE>
int32_t launch_dequant(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, const void *scale_y, void *out,
                       int bx, int by, cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_shape(batch, n, m);
    if (rc) return rc;
    const int64_t total = (int64_t)batch * n * m;
    if (total == 0) return CPMK_OK;
    CPMK_REQUIRE(mat && out && (MODE == 2 || scale_x) && (MODE == 1 || scale_y), "null tensor pointer");
    const int32_t *acc = static_cast<const int32_t *>(mat);
    const __half *sx = static_cast<const __half *>(scale_x);
    const __half *sy = static_cast<const __half *>(scale_y);
    __half *dst = static_cast<__half *>(out);
    const bool vec_ok = (m % 8 == 0) && aligned16(mat) && aligned16(out) && (MODE == 1 || aligned16(scale_y));
    if (vec_ok) {
        const int64_t total_vec = total / 8;
        const int64_t blocks = ceil_div64(total_vec, kBlock);
        CPMK_REQUIRE(blocks < (int64_t(1) << 31), "tensor too large");
        dequant_kernel<MODE><<<(unsigned)blocks, kBlock, 0, stream>>>(total_vec, n, m, acc, sx, sy, dst, bx, by);
    } else {
        const int64_t blocks = ceil_div64(total, kBlock);
        CPMK_REQUIRE(blocks < (int64_t(1) << 31), "tensor too large");
        dequant_generic_kernel<MODE><<<(unsigned)blocks, kBlock, 0, stream>>>(total, n, m, acc, sx, sy, dst, bx, by);
    }
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

}  // namespace
}  // namespace cpmk

using namespace cpmk;

extern "C" {

int32_t cpmk_gemm_calc_scale(int32_t batch, int32_t n, int32_t m, const void *mat, void *out, cpmk_stream_t stream) {
    return launch_quant_rows<1>(batch, n, m, mat, out, nullptr, as_stream(stream));
}

int32_t cpmk_gemm_round(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale, void *out, cpmk_stream_t stream) {
    return launch_quant_rows<2>(batch, n, m, mat, const_cast<void *>(scale), out, as_stream(stream));
}

int32_t cpmk_quantize_rows(int32_t batch, int32_t n, int32_t m, const void *mat, void *scale_out, void *q_out, cpmk_stream_t stream) {
    return launch_quant_rows<0>(batch, n, m, mat, scale_out, q_out, as_stream(stream));
}

int32_t cpmk_quantize_rows_pair(int32_t batch0, int32_t n0, const void *mat0, void *scale_out0, void *q_out0, int32_t batch1, int32_t n1,
                                const void *mat1, void *scale_out1, void *q_out1, int32_t m, cpmk_stream_t stream) {
    int32_t rc = check_shape(batch0, n0, m);
    if (rc) return rc;
    rc = check_shape(batch1, n1, m);
    if (rc) return rc;
    bool done = false;
    if ((int64_t)batch0 * n0 > 0 && (int64_t)batch1 * n1 > 0 && m > 0) {
        CPMK_REQUIRE(mat0 && mat1 && scale_out0 && scale_out1 && q_out0 && q_out1, "null tensor pointer");
        rc = launch_quant_rows_pair((int64_t)batch0 * n0, mat0, scale_out0, q_out0, (int64_t)batch1 * n1, mat1, scale_out1, q_out1, m,
                                    as_stream(stream), &done);
        if (rc) return rc;
    }
    if (done) return CPMK_OK;
    // shapes the vector kernel does not take, or an empty operand: one call per operand
    rc = launch_quant_rows<0>(batch0, n0, m, mat0, scale_out0, q_out0, as_stream(stream));
    if (rc) return rc;
    return launch_quant_rows<0>(batch1, n1, m, mat1, scale_out1, q_out1, as_stream(stream));
}

int32_t cpmk_quantize_rows_pair_scatter(int32_t n0, const void *mat0, int32_t n_dst, void *const *scale_dst0, void *const *q_dst0,
                                        int32_t n1, const void *mat1, void *scale_out1, void *q_out1, int32_t m, cpmk_stream_t stream) {
    int32_t rc = check_shape(1, n0, m);
    if (rc) return rc;
    rc = check_shape(1, n1, m);
    if (rc) return rc;
    CPMK_REQUIRE(n_dst >= 1 && n_dst <= kMaxQuantDst, "number of destinations must be 1..%d (got %d)", kMaxQuantDst, n_dst);
    CPMK_REQUIRE(scale_dst0 && q_dst0, "null destination list");
    if (n0 == 0 && n1 == 0) return CPMK_OK;
    CPMK_REQUIRE(n0 > 0 && m > 0, "the scattered operand must not be empty (n0=%d m=%d)", n0, m);
    CPMK_REQUIRE(mat0 && (n1 == 0 || (mat1 && scale_out1 && q_out1)), "null tensor pointer");
    MultiDst multi;
    multi.n = n_dst;
    for (int d = 0; d < kMaxQuantDst; ++d) {
        multi.codes[d] = d < n_dst ? static_cast<int8_t *>(q_dst0[d]) : nullptr;
        multi.scale[d] = d < n_dst ? static_cast<__half *>(scale_dst0[d]) : nullptr;
        if (d < n_dst) CPMK_REQUIRE(multi.codes[d] && multi.scale[d], "destination %d is null", d);
    }
    bool done = false;
    rc = launch_quant_rows_pair(n0, mat0, nullptr, nullptr, n1, mat1, scale_out1, q_out1, m, as_stream(stream), &done, &multi);
    if (rc) return rc;
    CPMK_REQUIRE(done, "scattered quantisation needs rows of a multiple of 8 and at most 16384 elements, a 16-byte aligned operand and "
                       "8-byte aligned destinations (m=%d)", m);
    return CPMK_OK;
}

int32_t cpmk_gemm_calc_scale_transpose(int32_t batch, int32_t n, int32_t m, const void *inp, void *out, cpmk_stream_t stream) {
    return launch_quant_cols<1>(batch, n, m, inp, out, nullptr, as_stream(stream));
}

int32_t cpmk_gemm_round_transpose(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale, void *out, cpmk_stream_t stream) {
    return launch_quant_cols<2>(batch, n, m, mat, const_cast<void *>(scale), out, as_stream(stream));
}

int32_t cpmk_quantize_cols(int32_t batch, int32_t n, int32_t m, const void *mat, void *scale_out, void *q_out, cpmk_stream_t stream) {
    return launch_quant_cols<0>(batch, n, m, mat, scale_out, q_out, as_stream(stream));
}

int32_t cpmk_gemm_scale(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, const void *scale_y, void *out,
                        int32_t broad_cast_x, int32_t broad_cast_y, cpmk_stream_t stream) {
    return launch_dequant<0>(batch, n, m, mat, scale_x, scale_y, out, broad_cast_x != 0, broad_cast_y != 0, as_stream(stream));
}

int32_t cpmk_gemm_scale_x(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, void *out, cpmk_stream_t stream) {
    return launch_dequant<1>(batch, n, m, mat, scale_x, nullptr, out, 0, 0, as_stream(stream));
}

int32_t cpmk_gemm_scale_y(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_y, void *out, cpmk_stream_t stream) {
    return launch_dequant<2>(batch, n, m, mat, nullptr, scale_y, out, 0, 0, as_stream(stream));
}

int32_t cpmk_gemm_backward_round_scale(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_y, void *out, void *scale_x,
                                       int32_t broad_cast_y, cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_shape(batch, n, m);
    if (rc) return rc;
    const int64_t rows = (int64_t)batch * n;
    if (rows == 0) return CPMK_OK;
    CPMK_REQUIRE(mat && scale_y && out && scale_x, "null tensor pointer");
    const int grid = (int)(rows < (int64_t)info.sm_count * 16 ? rows : (int64_t)info.sm_count * 16);
    backward_round_scale_kernel<<<grid, kBlock, 0, as_stream(stream)>>>(batch, n, m, static_cast<const __half *>(mat),
                                                                         static_cast<const __half *>(scale_y), static_cast<int8_t *>(out),
                                                                         static_cast<__half *>(scale_x), broad_cast_y != 0);
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

int32_t cpmk_gemm_backward_scale_round(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, void *out, void *scale_y,
                                       int32_t broad_cast_x, cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_shape(batch, n, m);
    if (rc) return rc;
    if ((int64_t)batch * m == 0) return CPMK_OK;
    CPMK_REQUIRE(mat && scale_x && out && scale_y, "null tensor pointer");
    const int64_t blocks = ceil_div64((int64_t)batch * m, kBlock);
    backward_scale_round_kernel<<<(unsigned)blocks, kBlock, 0, as_stream(stream)>>>(batch, n, m, static_cast<const __half *>(mat),
                                                                                    static_cast<const __half *>(scale_x), static_cast<int8_t *>(out),
                                                                                    static_cast<__half *>(scale_y), broad_cast_x != 0);
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

}  // extern "C"
