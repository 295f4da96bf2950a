// fp16 decode GEMV for sm_100a: HBM-bound streaming of the weight matrix with 128-bit loads and fp32
// accumulation.
//
// Replaces cuda/gemv.cu:57-164 of the reference (one block per output element with half2 accumulation;
// 32x32 blocks reading 64-byte row segments for the transposed form) and the cublasLt n=1 GEMMs of
// cpm_kernels/kernels/gemv.py:82-262.
#include <stdlib.h>

#include <mutex>

#include <cuda.h>
#include "cpmk_common.cuh"
#include "cpmk_ptx.cuh"

namespace cpmk {
namespace {

constexpr int kBlock = 256;
constexpr int kWarps = kBlock / 32;

__device__ __forceinline__ float dot8(const uint4 &a, const uint4 &b, float acc) {
    const __half2 *x = reinterpret_cast<const __half2 *>(&a);
    const __half2 *y = reinterpret_cast<const __half2 *>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fx = __half22float2(x[i]);
        const float2 fy = __half22float2(y[i]);
        acc = fmaf(fx.x, fy.x, acc);
        acc = fmaf(fx.y, fy.y, acc);
    }
    return acc;
}

// the same with the second operand already widened to fp32 (four float2)
__device__ __forceinline__ float dot8f(const uint4 &a, const float2 *y, float acc) {
    const __half2 *x = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fx = __half22float2(x[i]);
        acc = fmaf(fx.x, y[i].x, acc);
        acc = fmaf(fx.y, y[i].y, acc);
    }
    return acc;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------------------------------------
// out[b, o] = sum_i mat[b?, o, i] * vec[b, i]: one warp per matrix row, NB vectors per pass.
// SHARED = false: mat is (batch, dim_out, dim_in) and NB == 1 (gemv_fp16);
// SHARED = true : mat is (dim_out, dim_in), read once for NB vectors (gemv_broadcast_mat_fp16).
// ------------------------------------------------------------------------------------------------
template <int NB, bool SHARED>
__global__ void __launch_bounds__(kBlock) gemv_rows_kernel(int32_t batch, int32_t dim_out, int32_t dim_in, int32_t batch_begin,
                                                           const __half *__restrict__ mat, const __half *__restrict__ vec,
                                                           __half *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_id = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t total_rows = SHARED ? (int64_t)dim_out : (int64_t)batch * dim_out;
    if (warp_id >= total_rows) return;
    const int nvec = dim_in >> 3;
    const uint4 *row = reinterpret_cast<const uint4 *>(mat + warp_id * (int64_t)dim_in);
    const int b0 = SHARED ? batch_begin : (int)(warp_id / dim_out);
    const int o = SHARED ? (int)warp_id : (int)(warp_id - (int64_t)b0 * dim_out);

    float acc[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j] = 0.f;

    int i = lane;
    // four independent 128-bit loads in flight per lane
    for (; i + 96 < nvec; i += 128) {
        uint4 w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) w[u] = __ldcs(row + i + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const uint4 x = __ldg(reinterpret_cast<const uint4 *>(vec + (int64_t)(b0 + j) * dim_in) + i + 32 * u);
                acc[j] = dot8(w[u], x, acc[j]);
            }
        }
    }
    for (; i < nvec; i += 32) {
        const uint4 w = __ldcs(row + i);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const uint4 x = __ldg(reinterpret_cast<const uint4 *>(vec + (int64_t)(b0 + j) * dim_in) + i);
            acc[j] = dot8(w, x, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const float v = warp_sum(acc[j]);
        if (lane == 0) out[(int64_t)(b0 + j) * dim_out + o] = __float2half_rn(v);
    }
}

// ------------------------------------------------------------------------------------------------
// Streaming form of the row-major GEMV for decode-sized rows (2 KiB .. 12.5 KiB): one persistent block per SM
// owns a contiguous range of matrix rows and pulls them through a shared-memory ring with 1-d bulk asynchronous
// copies (one producer thread), eight rows per stage, so that 100-200 KiB per SM are in flight without costing
// registers; eight consumer warps take one row of each stage apiece (128-bit shared loads, fp32 accumulation).
// ------------------------------------------------------------------------------------------------
constexpr int kStreamRows = 8;                      // rows per stage = consumer warps
constexpr int kStreamThreads = (kStreamRows + 1) * 32;
constexpr int kStreamRingBytes = 200 * 1024;
constexpr int kStreamVecBytes = 13 * 1024;           // the vector behind the ring (rows of up to 12.5 KiB)
constexpr int kXregPieces = 16;                     // 16-byte pieces of the vector per lane in the register-resident form: rows of <= 4096 halves
constexpr uint32_t kErrGemvProducer = 0x201;
constexpr uint32_t kErrGemvConsumer = 0x202;

// Rows longer than one stage slot are streamed in chunks of `chunk` halves (<= 4096): a stage then holds the
// same chunk of eight consecutive rows, and each warp carries its row's sum across the chunks.
// PROBE: the same copy pipeline with the arithmetic left out (no vector loads, no sums): how long the matrix takes to
// arrive through this launch shape; the consumers only fold one word per 16 bytes so that the reads are not elided.
// XREG: ONE matrix per block (the caller guarantees it: one matrix, or a grid row per batch entry) with rows of at most 4096 halves in one chunk: every consumer lane keeps
// its share of the vector (the 16-byte pieces lane, lane + 32, ... of it, widened to fp32) in 128 registers for the
// whole kernel, so the consumers read only the matrix out of shared memory (batch 1: 17.7 -> 15.6 us on 10240 x 4096).
// With per-batch matrices the launcher gives every batch entry its own row of the grid (sm_count / batch blocks), so that no
// block's rows belong to two entries (batch 4 on 10240 x 4096: 59.5 -> 53.6 us; letting blocks straddle entries and fall back to
// global loads of the vector measured 70 us).
template <bool SHARED, bool PROBE = false, bool XREG = false>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_rows_stream_kernel(int64_t rows_base, int64_t rows_extra, int32_t dim_out, int32_t dim_in, int32_t chunk,
                                                                             int32_t stages, const __half *__restrict__ mat,
                                                                             const __half *__restrict__ vec, __half *__restrict__ out,
                                                                             uint32_t *status) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t bars[32];       // full[stages], empty[stages]
    __shared__ uint32_t abort_word;
    // the vector of the batch entry the consumers are working on, copied once per block (per batch entry) behind the
    // ring: read out of shared memory it costs the consumers a short wait instead of a global load per 16 bytes of matrix
    __half *xs = reinterpret_cast<__half *>(ring + (size_t)stages * chunk * 2 * kStreamRows);
    const uint32_t slot_bytes = (uint32_t)chunk * 2u;             // one row's chunk
    const uint32_t stage_bytes = slot_bytes * kStreamRows;
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + 16);
    const uint32_t ring_base = smem_u32(ring);
    volatile uint32_t *abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = (dim_in + chunk - 1) / chunk;
    // gridDim.y > 1: per-batch matrices with the blocks of row blockIdx.y of the grid sharing out the rows of entry
    // blockIdx.y, so that no block's rows belong to two entries and each block sees one matrix and one vector
    mat += (int64_t)blockIdx.y * dim_out * dim_in;
    vec += (int64_t)blockIdx.y * dim_in;
    out += (int64_t)blockIdx.y * dim_out;

    // this block's rows [r0, r1): total_rows = rows_base * gridDim.x + rows_extra, the first rows_extra blocks take one more
    // (host-computed: a 64-bit division here would sit in front of the first copy)
    const int64_t bx = blockIdx.x;
    const int64_t r0 = bx * rows_base + (bx < rows_extra ? bx : rows_extra), r1 = r0 + rows_base + (bx < rows_extra ? 1 : 0);
    const int groups = (int)((r1 - r0 + kStreamRows - 1) / kStreamRows);
    bool x_in_smem = false;
    float2 xf[XREG ? 4 * kXregPieces : 1];

    // Producer warp.  A single thread issuing eight copies one after another takes over a microsecond per stage
    // (measured), which delays the first stage and barely keeps up afterwards: whole rows of a group are contiguous in
    // memory and in the ring, so they travel as ONE copy; chunks of long rows are issued by one lane each.
    // copy number t = g * chunks + c goes to stage t % stages
    auto issue_copy = [&](int g, int c, uint32_t stage) {
        const int64_t row = r0 + (int64_t)g * kStreamRows;
        const int n = (int)((r1 - row) < kStreamRows ? (r1 - row) : kStreamRows);
        const int c0 = c * chunk;
        const uint32_t bytes = (uint32_t)((dim_in - c0) < chunk ? (dim_in - c0) : chunk) * 2u;
        if (lane == 0) mbar_expect_tx(full_bar + 8 * stage, (uint32_t)n * bytes);
        if (chunks == 1) {
            if (lane == 0) bulk_load_1d(ring_base + stage * stage_bytes, mat + row * (int64_t)dim_in, (uint32_t)n * bytes, full_bar + 8 * stage);
        } else {
            __syncwarp();
            if (lane < n)
                bulk_load_1d(ring_base + stage * stage_bytes + (uint32_t)lane * slot_bytes, mat + (row + lane) * (int64_t)dim_in + c0, bytes,
                             full_bar + 8 * stage);
        }
    };
    const int total_copies = groups * chunks;
    const int prologue = total_copies < stages ? total_copies : stages;
    if (warp == kStreamRows) {
        // the producer initialises the barriers itself and fills the whole ring before the block's first barrier, so the
        // first bytes are on their way while the other warps are still setting up
        if (lane == 0) {
            for (int s = 0; s < stages; ++s) {
                mbar_init(full_bar + 8 * s, 1);
                mbar_init(empty_bar + 8 * s, kStreamRows);
            }
            abort_word = 0u;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        for (int t = 0; t < prologue; ++t) issue_copy(t / chunks, t % chunks, (uint32_t)t);
    } else if (XREG) {
        const uint4 *srcv = reinterpret_cast<const uint4 *>(vec);
        const int nv = dim_in >> 3;
#pragma unroll
        for (int j = 0; j < kXregPieces; ++j) {
            const int idx = lane + 32 * j;
            const uint4 v = idx < nv ? __ldg(srcv + idx) : make_uint4(0u, 0u, 0u, 0u);
            const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) xf[4 * j + e] = __half22float2(h[e]);
        }
    } else if (!PROBE && r1 > r0) {
        // When all rows of the block belong to one batch entry (always, for a single matrix) its vector is copied into
        // shared memory once; a block that straddles two entries reads the vectors from global memory as it goes.
        const bool one_matrix = SHARED || rows_base * gridDim.x + rows_extra == dim_out;
        const int64_t b_lo = one_matrix ? 0 : r0 / dim_out, b_hi = one_matrix ? 0 : (r1 - 1) / dim_out;
        if (b_lo == b_hi) {
            x_in_smem = true;
            const uint4 *srcv = reinterpret_cast<const uint4 *>(vec + b_lo * dim_in);
            for (int i = threadIdx.x; i < (dim_in >> 3); i += kStreamRows * 32) reinterpret_cast<uint4 *>(xs)[i] = __ldg(srcv + i);
        }
    }
    __syncthreads();

    if (warp == kStreamRows) {
        uint32_t stage = prologue == stages ? 0u : (uint32_t)prologue, phase = prologue == stages ? 1u : 0u;
        bool alive = true;
        for (int t = prologue; alive && t < total_copies; ++t) {
            int ok = 1;
            if (lane == 0) ok = mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kErrGemvProducer) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { alive = false; break; }
            issue_copy(t / chunks, t % chunks, stage);
            if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
    } else {
        uint32_t stage = 0, phase = 0;
        bool alive = true;
        for (int g = 0; alive && g < groups; ++g) {
            const int64_t row = r0 + (int64_t)g * kStreamRows + warp;
            // (one matrix: every row belongs to batch entry 0; otherwise one division per group, overlapped with the copy)
            const int b = (SHARED || rows_base * gridDim.x + rows_extra == dim_out) ? 0 : (int)((row < r1 ? row : r0) / dim_out);
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
            for (int c = 0; c < chunks; ++c) {
                if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, status, kErrGemvConsumer)) { alive = false; break; }
                if (row < r1) {
                    const int c0 = c * chunk;
                    const int nvec = ((dim_in - c0) < chunk ? (dim_in - c0) : chunk) >> 3;
                    const uint4 *w = reinterpret_cast<const uint4 *>(ring + (size_t)stage * stage_bytes + (size_t)warp * slot_bytes);
                    const uint4 *x = x_in_smem ? reinterpret_cast<const uint4 *>(xs + c0) : reinterpret_cast<const uint4 *>(vec + (int64_t)b * dim_in + c0);
                    int i = lane;
                    if (XREG) {
                        // four pieces at a time: their shared-memory loads are issued together, four independent sums
#pragma unroll
                        for (int j = 0; j < kXregPieces; j += 4) {
                            uint4 wv[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) wv[u] = lane + 32 * (j + u) < nvec ? w[lane + 32 * (j + u)] : make_uint4(0u, 0u, 0u, 0u);
                            acc0 = dot8f(wv[0], &xf[4 * j], acc0);
                            acc1 = dot8f(wv[1], &xf[4 * j + 4], acc1);
                            acc2 = dot8f(wv[2], &xf[4 * j + 8], acc2);
                            acc3 = dot8f(wv[3], &xf[4 * j + 12], acc3);
                        }
                    } else if (PROBE) {
                        uint32_t fold = 0u;
                        for (; i < nvec; i += 32) {
                            const uint4 w0 = w[i];
                            fold ^= w0.x ^ w0.y ^ w0.z ^ w0.w;
                        }
                        acc0 += fold == 0x9e3779b9u ? 1.f : 0.f;
                    } else {
                        // (generic loads: x is in shared memory, or in global memory when the block's rows span two batch entries)
                        for (; i + 32 < nvec; i += 64) {
                            const uint4 w0 = w[i], w1 = w[i + 32];
                            const uint4 x0 = x[i], x1 = x[i + 32];
                            acc0 = dot8(w0, x0, acc0);
                            acc1 = dot8(w1, x1, acc1);
                        }
                        if (i < nvec) acc0 = dot8(w[i], x[i], acc0);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
                if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
            }
            if (alive && row < r1) {
                const float v = warp_sum((acc0 + acc1) + (acc2 + acc3));
                if (lane == 0 && (!PROBE || v != 0.f)) out[row] = __float2half_rn(v);     // (the probe writes nothing unless a fold hits the magic word)
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);     // let copies in flight land before the ring is released
    }
}

// ------------------------------------------------------------------------------------------------
// Streaming form of the transposed GEMV (mat (dim_in, dim_out) row-major, out[o] = sum_i mat[i, o] * vec[i]).
// A block owns a strip of up to 2048 columns (4 KiB row segments) and a range of rows; the producer thread pulls
// eight row segments per stage through a 3-stage ring (two blocks per SM keep ~190 KiB per SM in flight); each
// of the 256 consumer threads owns eight columns and eight fp32 sums.  Row ranges are combined as in the
// non-streaming kernel: fp32 partials in scratch, added in range order by the block that takes the last ticket.
// ------------------------------------------------------------------------------------------------
constexpr int kTsCols = 2048;
constexpr int kTsStages = 3;
constexpr int kTsStageBytes = kStreamRows * kTsCols * 2;       // 32 KiB
constexpr int kTsRingBytes = kTsStages * kTsStageBytes;        // 96 KiB
constexpr int kTsVecFloats = 2048;                             // rows of the vector a block may keep in shared memory (8 KiB)

__global__ void __launch_bounds__(kStreamThreads, 2) gemv_transpose_stream_kernel(int32_t dim_out, int32_t dim_in, int32_t rows_per_split,
                                                                                  int32_t splits, int32_t x_in_smem, const __half *__restrict__ mat,
                                                                                  const __half *__restrict__ vec, __half *__restrict__ out,
                                                                                  float *__restrict__ partial, uint32_t *__restrict__ tickets,
                                                                                  uint32_t *status) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t bars[2 * kTsStages];
    __shared__ uint32_t abort_word;
    __shared__ uint32_t is_last;
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + kTsStages);
    const uint32_t ring_base = smem_u32(ring);
    float *xs = reinterpret_cast<float *>(ring + kTsRingBytes);    // x_in_smem: this block's rows of the vector, as fp32
    volatile uint32_t *abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strip = blockIdx.x, split = blockIdx.y, b = blockIdx.z, batch = gridDim.z;
    const int c0 = strip * kTsCols;
    const int width = (dim_out - c0) < kTsCols ? (dim_out - c0) : kTsCols;       // multiple of 8
    const uint32_t seg_bytes = (uint32_t)width * 2u;
    const int i0 = split * rows_per_split;
    const int i1 = min(dim_in, i0 + rows_per_split);
    const int groups = (i1 - i0 + kStreamRows - 1) / kStreamRows;
    const __half *base = mat + (int64_t)b * dim_in * dim_out + c0;
    const __half *x = vec + (int64_t)b * dim_in;

    // one lane per row segment: a single thread issuing the eight copies of a stage takes over a microsecond
    auto issue_group = [&](int g, uint32_t stage) {
        const int row = i0 + g * kStreamRows;
        const int n = (i1 - row) < kStreamRows ? (i1 - row) : kStreamRows;
        if (lane == 0) mbar_expect_tx(full_bar + 8 * stage, (uint32_t)n * seg_bytes);
        __syncwarp();
        if (lane < n)
            bulk_load_1d(ring_base + stage * kTsStageBytes + (uint32_t)lane * (kTsCols * 2), base + (int64_t)(row + lane) * dim_out, seg_bytes,
                         full_bar + 8 * stage);
    };
    const int prologue = groups < kTsStages ? groups : kTsStages;
    if (warp == kStreamRows) {
        // the producer initialises the barriers itself and fills the ring before the block's first barrier
        if (lane == 0) {
            for (int s = 0; s < kTsStages; ++s) {
                mbar_init(full_bar + 8 * s, 1);
                mbar_init(empty_bar + 8 * s, kStreamRows);
            }
            abort_word = 0u;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        for (int g = 0; g < prologue; ++g) issue_group(g, (uint32_t)g);
    } else if (x_in_smem) {
        for (int i = threadIdx.x; i < i1 - i0; i += kStreamRows * 32) xs[i] = __half2float(__ldg(x + i0 + i));
    }
    __syncthreads();

    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;

    if (warp == kStreamRows) {
        uint32_t stage = prologue == kTsStages ? 0u : (uint32_t)prologue, phase = prologue == kTsStages ? 1u : 0u;
        for (int g = prologue; g < groups; ++g) {
            int ok = 1;
            if (lane == 0) ok = mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kErrGemvProducer) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            issue_group(g, stage);
            if (++stage == kTsStages) { stage = 0; phase ^= 1u; }
        }
    } else {
        const int t = threadIdx.x;                       // 0..255: columns c0 + 8 t .. + 7
        const bool col_ok = t * 8 < width;
        uint32_t stage = 0, phase = 0;
        for (int g = 0; g < groups; ++g) {
            const int row = i0 + g * kStreamRows;
            const int n = (i1 - row) < kStreamRows ? (i1 - row) : kStreamRows;
            float xv[kStreamRows];
            if (x_in_smem) {
#pragma unroll
                for (int r = 0; r < kStreamRows; ++r) xv[r] = r < n ? xs[g * kStreamRows + r] : 0.f;
            } else {
#pragma unroll
                for (int r = 0; r < kStreamRows; ++r) xv[r] = r < n ? __half2float(__ldg(x + row + r)) : 0.f;
            }
            if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, status, kErrGemvConsumer)) break;
            if (col_ok) {
                const uint8_t *src = ring + (size_t)stage * kTsStageBytes + (size_t)t * 16;
#pragma unroll
                for (int r = 0; r < kStreamRows; ++r) {
                    if (r < n) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(src + (size_t)r * (kTsCols * 2));
                        const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __half22float2(h[j]);
                            acc[2 * j] = fmaf(f.x, xv[r], acc[2 * j]);
                            acc[2 * j + 1] = fmaf(f.y, xv[r], acc[2 * j + 1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
            if (++stage == kTsStages) { stage = 0; phase ^= 1u; }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        return;
    }
    const int t = threadIdx.x;
    const bool writer = t < kStreamRows * 32 && t * 8 < width;
    const int c = c0 + t * 8;
    if (splits == 1) {
        if (writer) {
            __align__(16) __half o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(acc[j]);
            *reinterpret_cast<uint4 *>(out + (int64_t)b * dim_out + c) = *reinterpret_cast<const uint4 *>(o);
        }
        return;
    }
    if (writer) {
        float4 *dst = reinterpret_cast<float4 *>(partial + ((int64_t)split * batch + b) * dim_out + c);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    if (tickets == nullptr) return;                      // a separate kernel adds the row ranges (many of them)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t tk = atomicAdd(&tickets[b * gridDim.x + strip], 1u);
        is_last = (tk == (uint32_t)splits - 1u);
        if (is_last) tickets[b * gridDim.x + strip] = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (writer) {
        float sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
            const float4 *src = reinterpret_cast<const float4 *>(partial + ((int64_t)sp * batch + b) * dim_out + c);
            const float4 p0 = __ldcg(src), p1 = __ldcg(src + 1);
            sum[0] += p0.x; sum[1] += p0.y; sum[2] += p0.z; sum[3] += p0.w;
            sum[4] += p1.x; sum[5] += p1.y; sum[6] += p1.z; sum[7] += p1.w;
        }
        __align__(16) __half o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(sum[j]);
        *reinterpret_cast<uint4 *>(out + (int64_t)b * dim_out + c) = *reinterpret_cast<const uint4 *>(o);
    }
}

// ------------------------------------------------------------------------------------------------
// Transposed form for ONE matrix without partial sums: a block owns a strip of `width` columns (a multiple of 16, chosen
// so that the strips just cover the SMs: 80 columns of a 10240-column matrix, 128 strips on 148 SMs) over ALL rows, so nothing
// has to be added across blocks and no second kernel runs.  The strip's 160-byte row segments are gathered by tiled TMA
// loads, 256 rows per box (the largest box a tiled copy takes: the fewer copies per byte the better), into a ring of three
// to sixteen boxes (one elected thread issues one copy per box); 8 consumer warps: thread t owns 8 columns (t mod width/8)
// and every (256 / (width/8))-th row, keeps 8 fp32 sums, and the block adds its row lanes through shared memory at the
// end in a fixed order.  The vector sits in shared memory.
// ------------------------------------------------------------------------------------------------
constexpr int kTpRows = 256;                       // rows per box (the largest extent a tiled copy takes)
constexpr int kTpMaxWidth = 256;                   // columns per strip (the largest inner extent of a box)
constexpr int kTpMaxStages = 16;
constexpr int kTpRedBytes = 256 * 8 * 4;           // one fp32 sum per consumer thread and column
constexpr uint32_t kErrGemvStripProducer = 0x203;
constexpr uint32_t kErrGemvStripConsumer = 0x204;

__global__ void __launch_bounds__(kStreamThreads, 1) gemv_transpose_strip_kernel(const __grid_constant__ CUtensorMap tmap, int32_t dim_out, int32_t dim_in,
                                                                                 int32_t width, int32_t stages, int32_t box_rows, const __half *__restrict__ vec,
                                                                                 __half *__restrict__ out, uint32_t *status) {
    extern __shared__ __align__(128) uint8_t ring[];               // stages boxes, then the vector (fp16), then the row lanes' sums
    __shared__ __align__(8) uint64_t bars[2 * kTpMaxStages];
    __shared__ uint32_t abort_word;
    const uint32_t full_bar = smem_u32(bars), empty_bar = smem_u32(bars + kTpMaxStages);
    const uint32_t ring_base = smem_u32(ring);
    volatile uint32_t *abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strip = blockIdx.x, b = blockIdx.y;
    const int c0 = strip * width;
    const uint32_t stage_bytes = (uint32_t)(box_rows * width * 2);
    const int x_halves = (dim_in + 63) / 64 * 64;                  // keeps what follows 128-byte aligned
    __half *xs = reinterpret_cast<__half *>(ring + (size_t)stages * stage_bytes);
    float *red = reinterpret_cast<float *>(xs + x_halves);
    const int groups = (dim_in + box_rows - 1) / box_rows;
    const int prologue = groups < stages ? groups : stages;

    if (warp == kStreamRows) {
        if (lane == 0) {
            for (int s = 0; s < stages; ++s) {
                mbar_init(full_bar + 8 * s, 1);
                mbar_init(empty_bar + 8 * s, kStreamRows);
            }
            abort_word = 0u;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // rows beyond dim_in and columns beyond dim_out are filled with zeros by the copy and count towards its bytes
            for (int g = 0; g < prologue; ++g) {
                mbar_expect_tx(full_bar + 8 * g, stage_bytes);
                tma_load_tile_3d(ring_base + (uint32_t)g * stage_bytes, &tmap, c0, g * box_rows, b, full_bar + 8 * g);
            }
        }
    } else {
        const __half *x = vec + (int64_t)b * dim_in;
        for (int i = threadIdx.x; i < dim_in; i += kStreamRows * 32) xs[i] = __ldg(x + i);
    }
    __syncthreads();

    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const int col_groups = width >> 3;
    const int row_lanes = (kStreamRows * 32) / col_groups;
    const int t = threadIdx.x;
    const int rl = t / col_groups, cg = t - rl * col_groups;
    const bool active = warp < kStreamRows && rl < row_lanes;

    if (warp == kStreamRows) {
        if (lane == 0) {
            uint32_t stage = prologue == stages ? 0u : (uint32_t)prologue, phase = prologue == stages ? 1u : 0u;
            for (int g = prologue; g < groups; ++g) {
                if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kErrGemvStripProducer)) break;
                mbar_expect_tx(full_bar + 8 * stage, stage_bytes);
                tma_load_tile_3d(ring_base + stage * stage_bytes, &tmap, c0, g * box_rows, b, full_bar + 8 * stage);
                if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        uint32_t stage = 0, phase = 0;
        for (int g = 0; g < groups; ++g) {
            if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, status, kErrGemvStripConsumer)) break;
            if (active) {
                const uint8_t *src = ring + (size_t)stage * stage_bytes + (size_t)cg * 16;
                const int row0 = g * box_rows;
#pragma unroll 4
                for (int r = rl; r < box_rows; r += row_lanes) {
                    // (rows beyond dim_in hold zeros; the vector is not read there)
                    const float xv = row0 + r < dim_in ? __half2float(xs[row0 + r]) : 0.f;
                    const uint4 w = *reinterpret_cast<const uint4 *>(src + (size_t)r * (size_t)(width * 2));
                    const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]);
                        acc[2 * j] = fmaf(f.x, xv, acc[2 * j]);
                        acc[2 * j + 1] = fmaf(f.y, xv, acc[2 * j + 1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
            if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);          // let copies in flight land before the ring is released
        return;
    }
    if (active) {
#pragma unroll
        for (int j = 0; j < 8; ++j) red[rl * width + cg * 8 + j] = acc[j];
    }
    __syncthreads();
    if (t < width && c0 + t < dim_out) {
        float total = 0.f;
        for (int r = 0; r < row_lanes; ++r) total += red[r * width + t];
        out[(int64_t)b * dim_out + c0 + t] = __float2half_rn(total);
    }
}

// Any dim_in / alignment: one warp per row, scalar loads.
__global__ void __launch_bounds__(kBlock) gemv_rows_generic_kernel(int32_t batch, int32_t dim_out, int32_t dim_in, int shared,
                                                                   const __half *__restrict__ mat, const __half *__restrict__ vec,
                                                                   __half *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_id = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (warp_id >= (int64_t)batch * dim_out) return;
    const int b = (int)(warp_id / dim_out);
    const int o = (int)(warp_id - (int64_t)b * dim_out);
    const __half *row = mat + (shared ? (int64_t)o : warp_id) * dim_in;
    const __half *x = vec + (int64_t)b * dim_in;
    float acc = 0.f;
    for (int i = lane; i < dim_in; i += 32) acc = fmaf(__half2float(row[i]), __half2float(x[i]), acc);
    acc = warp_sum(acc);
    if (lane == 0) out[warp_id] = __float2half_rn(acc);
}

// ------------------------------------------------------------------------------------------------
// Transposed form: out[b, o] = sum_i mat[b, i, o] * vec[b, i], mat (batch, dim_in, dim_out).
// A block owns a strip of 256 columns (32 lanes x 8 halves) and a chunk of rows; its 8 warps take
// rows w, w+8, ...  Chunks are combined through fp32 partials in scratch; the block that takes the
// last ticket of a strip adds them in chunk order (deterministic) and writes the fp16 result.
// ------------------------------------------------------------------------------------------------
constexpr int kTStripCols = 256;

__global__ void __launch_bounds__(kBlock) gemv_transpose_kernel(int32_t dim_out, int32_t dim_in, int32_t rows_per_split, int32_t splits,
                                                                const __half *__restrict__ mat, const __half *__restrict__ vec,
                                                                __half *__restrict__ out, float *__restrict__ partial,
                                                                uint32_t *__restrict__ tickets) {
    __shared__ float red[kWarps][kTStripCols];
    __shared__ uint32_t is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int strip = blockIdx.x, split = blockIdx.y, b = blockIdx.z, batch = gridDim.z;
    const int col = strip * kTStripCols + lane * 8;
    const int r_begin = split * rows_per_split;
    const int r_end = min(dim_in, r_begin + rows_per_split);
    const __half *base = mat + (int64_t)b * dim_in * dim_out;
    const __half *x = vec + (int64_t)b * dim_in;

    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (col < dim_out) {
        int r = r_begin + warp;
        for (; r + 3 * kWarps < r_end; r += 4 * kWarps) {
            uint4 w[4];
            float xv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                w[u] = __ldcs(reinterpret_cast<const uint4 *>(base + (int64_t)(r + u * kWarps) * dim_out + col));
                xv[u] = __half2float(__ldg(x + r + u * kWarps));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const __half2 *h = reinterpret_cast<const __half2 *>(&w[u]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    acc[2 * j] = fmaf(f.x, xv[u], acc[2 * j]);
                    acc[2 * j + 1] = fmaf(f.y, xv[u], acc[2 * j + 1]);
                }
            }
        }
        for (; r < r_end; r += kWarps) {
            const uint4 w = __ldcs(reinterpret_cast<const uint4 *>(base + (int64_t)r * dim_out + col));
            const float xv = __half2float(__ldg(x + r));
            const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                acc[2 * j] = fmaf(f.x, xv, acc[2 * j]);
                acc[2 * j + 1] = fmaf(f.y, xv, acc[2 * j + 1]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = acc[j];
    __syncthreads();
    const int c = strip * kTStripCols + threadIdx.x;
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total += red[w][threadIdx.x];

    if (splits == 1) {
        if (c < dim_out) out[(int64_t)b * dim_out + c] = __float2half_rn(total);
        return;
    }
    // partial[(split * batch + b) * dim_out + c]
    if (c < dim_out) partial[((int64_t)split * batch + b) * dim_out + c] = total;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(&tickets[b * gridDim.x + strip], 1u);
        is_last = (t == (uint32_t)splits - 1u);
        if (is_last) tickets[b * gridDim.x + strip] = 0u;          // leave the ticket at zero for the next call
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (c < dim_out) {
        float sum = 0.f;
        for (int s = 0; s < splits; ++s) sum += __ldcg(partial + ((int64_t)s * batch + b) * dim_out + c);
        out[(int64_t)b * dim_out + c] = __float2half_rn(sum);
    }
}

// out[b, c] = half(sum over row ranges of partial[(range * batch + b) * dim_out + c]), ranges added in order within each
// of blockDim.x / 32 interleaved groups and the groups in order: deterministic.  32 columns per block.
constexpr int kReduceThreads = 512;
__global__ void __launch_bounds__(1024) gemv_reduce_partials_kernel(int32_t dim_out, int32_t splits, const float *__restrict__ partial,
                                                                    __half *__restrict__ out) {
    // blockDim.x / 32 warps (up to 32) share the row ranges of 32 columns; with 16 warps and 57 ranges every thread has
    // four loads, all in flight at once (measured on 10240 x 4096: 19.5 us for the whole GEMV with 8 warps and two loads
    // in flight, 18.8 with 16 warps, 19.2 with 32)
    __shared__ float red[32][32];
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int b = blockIdx.y, batch = gridDim.y;
    const int c = blockIdx.x * 32 + lane;
    float sum = 0.f;
    if (c < dim_out) {
        int sp = g;
        for (; sp + 3 * nw < splits; sp += 4 * nw) {
            const float p0 = __ldcg(partial + ((int64_t)sp * batch + b) * dim_out + c);
            const float p1 = __ldcg(partial + ((int64_t)(sp + nw) * batch + b) * dim_out + c);
            const float p2 = __ldcg(partial + ((int64_t)(sp + 2 * nw) * batch + b) * dim_out + c);
            const float p3 = __ldcg(partial + ((int64_t)(sp + 3 * nw) * batch + b) * dim_out + c);
            sum += p0; sum += p1; sum += p2; sum += p3;
        }
        if (sp + nw < splits) {
            const float p0 = __ldcg(partial + ((int64_t)sp * batch + b) * dim_out + c);
            const float p1 = __ldcg(partial + ((int64_t)(sp + nw) * batch + b) * dim_out + c);
            sum += p0; sum += p1;
            sp += 2 * nw;
        }
        for (; sp < splits; sp += nw) sum += __ldcg(partial + ((int64_t)sp * batch + b) * dim_out + c);
    }
    red[g][lane] = sum;
    __syncthreads();
    if (g == 0 && c < dim_out) {
        float total = 0.f;
        for (int w = 0; w < nw; ++w) total += red[w][lane];
        out[(int64_t)b * dim_out + c] = __float2half_rn(total);
    }
}

__global__ void __launch_bounds__(kBlock) gemv_transpose_generic_kernel(int32_t batch, int32_t dim_out, int32_t dim_in,
                                                                        const __half *__restrict__ mat, const __half *__restrict__ vec,
                                                                        __half *__restrict__ out) {
    const int64_t idx = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (idx >= (int64_t)batch * dim_out) return;
    const int b = (int)(idx / dim_out), o = (int)(idx % dim_out);
    const __half *base = mat + (int64_t)b * dim_in * dim_out + o;
    const __half *x = vec + (int64_t)b * dim_in;
    float acc = 0.f;
    for (int i = 0; i < dim_in; ++i) acc = fmaf(__half2float(base[(int64_t)i * dim_out]), __half2float(x[i]), acc);
    out[idx] = __float2half_rn(acc);
}

// ------------------------------------------------------------------------------------------------
// int8 shared-matrix GEMV: out[b,o] = half(((float)sum_i mat[o,i]*vec[b,i]) * scale_vec[b] * scale_mat[o])
// One warp per matrix row, dp4a on 128-bit loads, NB vectors per pass.
// ------------------------------------------------------------------------------------------------
template <int NB>
__global__ void __launch_bounds__(kBlock) gemv_int8_kernel(int32_t dim_out, int32_t dim_in, int32_t batch_begin,
                                                           const __half *__restrict__ scale_mat, const int8_t *__restrict__ mat,
                                                           const __half *__restrict__ scale_vec, const int8_t *__restrict__ vec,
                                                           __half *__restrict__ out, int vec16) {
    const int lane = threadIdx.x & 31;
    const int64_t o = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (o >= dim_out) return;
    int32_t acc[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j] = 0;
    if (vec16) {
        const int nvec = dim_in >> 4;
        const int4 *row = reinterpret_cast<const int4 *>(mat + o * (int64_t)dim_in);
        for (int i = lane; i < nvec; i += 32) {
            const int4 w = __ldcs(row + i);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int4 x = __ldg(reinterpret_cast<const int4 *>(vec + (int64_t)(batch_begin + j) * dim_in) + i);
                acc[j] = __dp4a(w.x, x.x, acc[j]);
                acc[j] = __dp4a(w.y, x.y, acc[j]);
                acc[j] = __dp4a(w.z, x.z, acc[j]);
                acc[j] = __dp4a(w.w, x.w, acc[j]);
            }
        }
    } else {
        const int nword = dim_in >> 2;
        const int *row = reinterpret_cast<const int *>(mat + o * (int64_t)dim_in);
        for (int i = lane; i < nword; i += 32) {
            const int w = __ldg(row + i);
#pragma unroll
            for (int j = 0; j < NB; ++j)
                acc[j] = __dp4a(w, __ldg(reinterpret_cast<const int *>(vec + (int64_t)(batch_begin + j) * dim_in) + i), acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        int32_t v = acc[j];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0) {
            const float f = __fmul_rn(__fmul_rn((float)v, __half2float(scale_vec[batch_begin + j])), __half2float(scale_mat[o]));
            out[(int64_t)(batch_begin + j) * dim_out + o] = __float2half_rn(f);
        }
    }
}

// Reads `nvec` 16-byte vectors once, grid-stride, four loads in flight per thread, and folds them: the time any kernel
// needs to pull that many bytes out of HBM (the floor the GEMVs are compared with).
__global__ void __launch_bounds__(kBlock) read_probe_kernel(int64_t nvec, const uint4 *__restrict__ src, uint32_t *__restrict__ sink) {
    uint32_t fold = 0u;
    const int64_t stride = (int64_t)gridDim.x * kBlock;
    int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        const uint4 a = __ldcs(src + i), b = __ldcs(src + i + stride), c = __ldcs(src + i + 2 * stride), d = __ldcs(src + i + 3 * stride);
        fold ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < nvec; i += stride) {
        const uint4 a = __ldcs(src + i);
        fold ^= a.x ^ a.y ^ a.z ^ a.w;
    }
    if (fold == 0x9e3779b9u) atomicAdd(sink, 1u);           // practically never: keeps the loads alive
}

int32_t check_gemv(int32_t batch, int32_t dim_out, int32_t dim_in) {
    CPMK_REQUIRE(batch >= 0 && dim_out >= 0 && dim_in >= 0, "negative size: batch=%d dim_out=%d dim_in=%d", batch, dim_out, dim_in);
    return CPMK_OK;
}

template <bool SHARED>
int32_t launch_gemv_rows(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out, cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_gemv(batch, dim_out, dim_in);
    if (rc) return rc;
    if ((int64_t)batch * dim_out == 0) return CPMK_OK;
    CPMK_REQUIRE(mat && vec && out, "null tensor pointer");
    const __half *w = static_cast<const __half *>(mat);
    const __half *x = static_cast<const __half *>(vec);
    __half *y = static_cast<__half *>(out);
    const bool vec_ok = dim_in % 8 == 0 && aligned16(mat) && aligned16(vec);
    if (!vec_ok) {
        const int64_t blocks = ceil_div64((int64_t)batch * dim_out, kWarps);
        gemv_rows_generic_kernel<<<(unsigned)blocks, kBlock, 0, stream>>>(batch, dim_out, dim_in, SHARED ? 1 : 0, w, x, y);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    // rows of at least 2 KiB in a matrix that gives every SM a few dozen rows: the streaming kernel
    const int64_t total_rows = SHARED ? (int64_t)dim_out : (int64_t)batch * dim_out;
    const int64_t row_bytes = (int64_t)dim_in * 2;
    // (rows that do not fit a stage slot could be streamed in chunks -- the kernel supports it -- but measured slower
    // than the register-staged kernel on a 4096 x 10240 matrix, so such shapes stay with that kernel)
    if ((!SHARED || batch == 1) && row_bytes >= 2048 && row_bytes * kStreamRows * 2 <= kStreamRingBytes && total_rows >= (int64_t)info.sm_count * 16 &&
        info.max_smem_optin >= kStreamRingBytes + kStreamVecBytes + 1024 && !getenv("CPMK_GEMV_NO_STREAM")) {
        static std::once_flag attr_once[64];
        static cudaError_t attr_err[64];
        const int dev = info.device & 63;
        std::call_once(attr_once[dev], [dev] {
            cudaError_t e = cudaFuncSetAttribute(gemv_rows_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes + kStreamVecBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_rows_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes + kStreamVecBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_rows_stream_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes + kStreamVecBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_rows_stream_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes + kStreamVecBytes);
            attr_err[dev] = e;
        });
        if (attr_err[dev] == cudaSuccess) {
            Workspace ws;
            rc = get_workspace(stream, &ws);
            if (rc) return rc;
            // chunk: the whole row when it fits 8 KiB, else equal parts of at most 4096 halves (multiples of 8)
            int chunk = dim_in;
            if (chunk > 4096) {
                const int parts = (dim_in + 4095) / 4096;
                chunk = ((dim_in + parts - 1) / parts + 7) / 8 * 8;
            }
            int stages = (int)(kStreamRingBytes / ((int64_t)chunk * 2 * kStreamRows));
            if (stages > 16) stages = 16;
            const size_t smem = (size_t)stages * chunk * 2 * kStreamRows + (size_t)dim_in * 2;        // ring + the vector
            // one matrix with rows of at most 4096 halves: the vector lives in the consumers' registers (CPMK_GEMV_NO_XREG=1: in shared memory)
            const bool xreg = dim_in <= 32 * 8 * kXregPieces && !getenv("CPMK_GEMV_NO_XREG");
            // per-batch matrices: sm_count / batch blocks per entry (a 2-d grid), each entry's rows shared out among its own
            // blocks, so that every block works on one matrix with one vector
            const int per_entry = SHARED ? 0 : info.sm_count / batch;
            if (xreg && !SHARED && batch > 1 && per_entry >= 4 && dim_out >= per_entry * 16 && !getenv("CPMK_GEMV_NO_ENTRY_GRID"))
                gemv_rows_stream_kernel<false, false, true><<<dim3(per_entry, batch), kStreamThreads, smem, stream>>>(dim_out / per_entry, dim_out % per_entry, dim_out, dim_in,
                                                                                                                  chunk, stages, w, x, y, ws.status());
            else if (xreg && (SHARED || batch == 1))
                gemv_rows_stream_kernel<SHARED, false, true><<<info.sm_count, kStreamThreads, smem, stream>>>(total_rows / info.sm_count, total_rows % info.sm_count,
                                                                                                             dim_out, dim_in, chunk, stages, w, x, y, ws.status());
            else
                gemv_rows_stream_kernel<SHARED><<<info.sm_count, kStreamThreads, smem, stream>>>(total_rows / info.sm_count, total_rows % info.sm_count,
                                                                                                dim_out, dim_in, chunk, stages, w, x, y, ws.status());
            CPMK_LAUNCH_CHECK();
            return CPMK_OK;
        }
    }
    if (!SHARED) {
        const int64_t blocks = ceil_div64((int64_t)batch * dim_out, kWarps);
        CPMK_REQUIRE(blocks < (int64_t(1) << 31), "too many rows");
        gemv_rows_kernel<1, false><<<(unsigned)blocks, kBlock, 0, stream>>>(batch, dim_out, dim_in, 0, w, x, y);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    const unsigned blocks = (unsigned)ceil_div64(dim_out, kWarps);
    int b = 0;
    while (b < batch) {
        const int left = batch - b;
        if (left >= 8) { gemv_rows_kernel<8, true><<<blocks, kBlock, 0, stream>>>(batch, dim_out, dim_in, b, w, x, y); b += 8; }
        else if (left >= 4) { gemv_rows_kernel<4, true><<<blocks, kBlock, 0, stream>>>(batch, dim_out, dim_in, b, w, x, y); b += 4; }
        else if (left >= 2) { gemv_rows_kernel<2, true><<<blocks, kBlock, 0, stream>>>(batch, dim_out, dim_in, b, w, x, y); b += 2; }
        else { gemv_rows_kernel<1, true><<<blocks, kBlock, 0, stream>>>(batch, dim_out, dim_in, b, w, x, y); b += 1; }
        CPMK_LAUNCH_CHECK();
    }
    return CPMK_OK;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the transposed GEMV: its split partial sums and tickets live in a
// file-scope device array instead of the library's cudaMalloc'ed workspace.
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticTicketBytes = 16 * 1024;
constexpr size_t kStaticPartialBytes = 4u << 20;
constexpr size_t kStaticScratchBytes = kStaticTicketBytes + kStaticPartialBytes;

// [0, kStaticTicketBytes): tickets; [kStaticTicketBytes, end): fp32 partial sums.  One copy per GPU that loads
// the library, held until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address it stands for is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mutex;
unsigned char *g_static_ptr[64] = {nullptr};

// Device address of g_static_scratch on the current device (looked up on the first call per device).
int32_t static_scratch_address(int device, unsigned char **out) {
    CPMK_REQUIRE(device >= 0 && device < 64, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[device]) {
        void *p = nullptr;
        CPMK_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        g_static_ptr[device] = static_cast<unsigned char *>(p);
    }
    *out = g_static_ptr[device];
    return CPMK_OK;
}

}  // namespace
}  // namespace cpmk

using namespace cpmk;

extern "C" {

int32_t cpmk_gemv_fp16(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out, cpmk_stream_t stream) {
    return launch_gemv_rows<false>(batch, dim_out, dim_in, mat, vec, out, as_stream(stream));
}

int32_t cpmk_gemv_broadcast_mat_fp16(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out,
                                     cpmk_stream_t stream) {
    return launch_gemv_rows<true>(batch, dim_out, dim_in, mat, vec, out, as_stream(stream));
}

int32_t cpmk_gemv_fp16_transpose(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out,
                                 cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_gemv(batch, dim_out, dim_in);
    if (rc) return rc;
    if ((int64_t)batch * dim_out == 0) return CPMK_OK;
    CPMK_REQUIRE(mat && vec && out, "null tensor pointer");
    cudaStream_t st = as_stream(stream);
    const __half *w = static_cast<const __half *>(mat);
    const __half *x = static_cast<const __half *>(vec);
    __half *y = static_cast<__half *>(out);
    if (dim_in == 0) {
        CPMK_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)batch * dim_out * sizeof(__half), st));
        return CPMK_OK;
    }
    const int strips = (dim_out + kTStripCols - 1) / kTStripCols;
    const bool vec_ok = dim_out % 8 == 0 && aligned16(mat) && batch <= 65535 &&
                        (size_t)batch * strips * sizeof(uint32_t) <= Workspace::kTicketBytes;
    if (!vec_ok) {
        const int64_t blocks = ceil_div64((int64_t)batch * dim_out, kBlock);
        gemv_transpose_generic_kernel<<<(unsigned)blocks, kBlock, 0, st>>>(batch, dim_out, dim_in, w, x, y);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    // matrices of a few MB and more: whole columns per block, no partial sums (CPMK_GEMV_NO_STRIP=1: off)
    if ((int64_t)dim_in * dim_out >= (int64_t(1) << 21) && dim_in >= 1024 && dim_in <= 16384 && aligned16(out) && batch <= 65535 && !getenv("CPMK_GEMV_NO_STRIP") &&
        !getenv("CPMK_GEMV_NO_STREAM") && info.max_smem_optin >= kStreamRingBytes + 1024) {
        // Strips of a multiple of 16 columns: row segments that start and end on 32-byte sectors (with multiples of 8 the
        // segments of neighbouring strips share sectors, and a fifth more bytes crossed L2: 18.6 against 17.3 us).  Among the
        // widths of 32 to 256 columns, the one whose strips x batch entries fill whole waves of the SMs best (the widest one
        // within two percent of the best): 80 columns for one 10240-column matrix (128 blocks), 144 for four (288 blocks).
        // Boxes of 256 rows (the most a tiled copy takes) when three of them fit the ring, else 128: the larger the box the
        // fewer copies per byte (10240 x 4096 with 80-column strips: 25.4 us with 64-row boxes, 17.9 with 128, 15.5 with 256).
        const size_t tail_bytes = (size_t)((dim_in + 63) / 64 * 64) * 2 + kTpRedBytes;
        int width = 0, box_rows = 0, stages = 0;
        double best = 0.0;
        for (int w_try = 32; w_try <= kTpMaxWidth; w_try += 16) {
            const int rows_try = (kStreamRingBytes - tail_bytes) / ((size_t)kTpRows * w_try * 2) < 3 ? kTpRows / 2 : kTpRows;
            int stages_try = (int)((kStreamRingBytes - tail_bytes) / ((size_t)rows_try * w_try * 2));
            if (stages_try > kTpMaxStages) stages_try = kTpMaxStages;
            if (stages_try < 3) break;
            const int64_t blocks = (int64_t)((dim_out + w_try - 1) / w_try) * batch;
            const int64_t waves = (blocks + info.sm_count - 1) / info.sm_count;
            const double fill = (double)blocks / (double)(waves * info.sm_count);
            if (fill > best) best = fill;
            if (fill >= best - 0.02) { width = w_try; box_rows = rows_try; stages = stages_try; }
        }
        // (the loop keeps the last width within two percent of the best fill seen SO FAR; a later, better fill replaces it)
        const size_t stage_bytes = (size_t)box_rows * width * 2;
        const int strips_tp = width ? (dim_out + width - 1) / width : 0;
        if (width && best >= 0.75) {
            static std::once_flag attr_once[64];
            static cudaError_t attr_err[64];
            const int dev = info.device & 63;
            std::call_once(attr_once[dev], [dev] {
                attr_err[dev] = cudaFuncSetAttribute(gemv_transpose_strip_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes);
            });
            CUtensorMap tmap;
            const uint64_t dims[3] = {(uint64_t)dim_out, (uint64_t)dim_in, (uint64_t)batch};
            const uint64_t strides[2] = {(uint64_t)dim_out * 2, (uint64_t)dim_in * (uint64_t)dim_out * 2};
            const uint32_t box[3] = {(uint32_t)width, (uint32_t)box_rows, 1u};
            if (attr_err[dev] == cudaSuccess && encode_tiled_3d(&tmap, 2, mat, dims, strides, box, false)) {
                Workspace ws;
                rc = get_workspace(st, &ws);
                if (rc) return rc;
                gemv_transpose_strip_kernel<<<dim3(strips_tp, batch), kStreamThreads, (size_t)stages * stage_bytes + tail_bytes, st>>>(tmap, dim_out, dim_in, width,
                                                                                                                                        stages, box_rows, x, y, ws.status());
                CPMK_LAUNCH_CHECK();
                return CPMK_OK;
            }
        }
    }
    // matrices of a few MB and more: the streaming kernel, two blocks per SM
    if ((int64_t)dim_in * dim_out >= (int64_t(1) << 21) && dim_in >= 256 && aligned16(out) && info.max_smem_optin >= kTsRingBytes + kTsVecFloats * 4 + 1024 &&
        !getenv("CPMK_GEMV_NO_STREAM")) {
        static std::once_flag attr_once[64];
        static cudaError_t attr_err[64];
        const int dev = info.device & 63;
        std::call_once(attr_once[dev], [dev] {
            attr_err[dev] = cudaFuncSetAttribute(gemv_transpose_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTsRingBytes + kTsVecFloats * 4);
        });
        const int ts_strips = (dim_out + kTsCols - 1) / kTsCols;
        if (attr_err[dev] == cudaSuccess && (size_t)batch * ts_strips * sizeof(uint32_t) <= Workspace::kTicketBytes) {
            int64_t sp = ((int64_t)info.sm_count * 2) / ((int64_t)ts_strips * batch);
            const int64_t by_rows = (dim_in + 63) / 64;
            if (sp > by_rows) sp = by_rows;
            const int64_t by_scratch = (int64_t)(Workspace::kScratchBytes / (sizeof(float) * (size_t)batch * (size_t)dim_out));
            if (sp > by_scratch) sp = by_scratch;
            if (sp > 65535) sp = 65535;
            if (sp < 1) sp = 1;
            int rps = (int)((dim_in + sp - 1) / sp);
            rps = (rps + kStreamRows - 1) / kStreamRows * kStreamRows;
            const int nsp = (dim_in + rps - 1) / rps;
            // up to 24 row ranges: the block that takes the last ticket of a strip adds them; more than that (one
            // matrix of a few thousand columns) and that serial tail would dominate, so a second, wide kernel adds them
            {
                Workspace ws;
                rc = get_workspace(st, &ws);
                if (rc) return rc;
                const dim3 grid(ts_strips, nsp, batch);
                float *partial = reinterpret_cast<float *>(ws.scratch());
                const bool two_kernels = nsp > 24;
                // this block's rows of the vector go to shared memory (as fp32) when they fit behind the ring
                const int x_in_smem = rps <= kTsVecFloats ? 1 : 0;
                gemv_transpose_stream_kernel<<<grid, kStreamThreads, kTsRingBytes + (x_in_smem ? rps * 4 : 0), st>>>(dim_out, dim_in, rps, nsp, x_in_smem, w, x, y, partial,
                                                                                         two_kernels ? nullptr : ws.tickets(), ws.status());
                CPMK_LAUNCH_CHECK();
                if (two_kernels) {
                    gemv_reduce_partials_kernel<<<dim3((dim_out + 31) / 32, batch), kReduceThreads, 0, st>>>(dim_out, nsp, partial, y);
                    CPMK_LAUNCH_CHECK();
                }
                return CPMK_OK;
            }
        }
    }
    // enough blocks to keep ~6 per SM streaming; at least 8 rows per warp in a chunk
    int64_t splits = ((int64_t)info.sm_count * 6) / ((int64_t)strips * batch);
    const int64_t max_by_rows = (dim_in + 63) / 64;
    if (splits > max_by_rows) splits = max_by_rows;
    const int64_t max_by_scratch = (int64_t)(Workspace::kScratchBytes / (sizeof(float) * (size_t)batch * (size_t)dim_out));
    if (splits > max_by_scratch) splits = max_by_scratch;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
    int rps = (int)((dim_in + splits - 1) / splits);
    rps = (rps + kWarps - 1) / kWarps * kWarps;
    const int nsplit = (dim_in + rps - 1) / rps;
    Workspace ws;
    ws.base = nullptr;
    if (nsplit > 1) {
        rc = get_workspace(st, &ws);
        if (rc) return rc;
    }
    const dim3 grid(strips, nsplit, batch);
    gemv_transpose_kernel<<<grid, kBlock, 0, st>>>(dim_out, dim_in, rps, nsplit, w, x, y,
                                                   nsplit > 1 ? reinterpret_cast<float *>(ws.scratch()) : nullptr,
                                                   nsplit > 1 ? ws.tickets() : nullptr);
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

int32_t cpmk_gemv_calc_scale(int32_t batch, int32_t n, const void *vec, void *out, cpmk_stream_t stream) {
    return cpmk_gemm_calc_scale(1, batch, n, vec, out, stream);
}

int32_t cpmk_gemv_round(int32_t batch, int32_t n, const void *vec, const void *scale, void *out, cpmk_stream_t stream) {
    return cpmk_gemm_round(1, batch, n, vec, scale, out, stream);
}

int32_t cpmk_gemv_broadcast_mat_int8(int32_t batch, int32_t dim_out, int32_t dim_in, const void *scale_mat, const void *mat,
                                     const void *scale_vec, const void *vec, void *out, cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_gemv(batch, dim_out, dim_in);
    if (rc) return rc;
    if ((int64_t)batch * dim_out == 0) return CPMK_OK;
    CPMK_REQUIRE(scale_mat && mat && scale_vec && vec && out, "null tensor pointer");
    // kernels/gemv.py:65
    CPMK_REQUIRE(dim_in % 4 == 0, "dim_in must be a multiple of 4 (got %d)", dim_in);
    CPMK_REQUIRE((reinterpret_cast<uintptr_t>(mat) & 3u) == 0 && (reinterpret_cast<uintptr_t>(vec) & 3u) == 0, "int8 tensors must be 4-byte aligned");
    cudaStream_t st = as_stream(stream);
    const int vec16 = (dim_in % 16 == 0 && aligned16(mat) && aligned16(vec)) ? 1 : 0;
    const unsigned blocks = (unsigned)ceil_div64(dim_out, kWarps);
    const __half *sm = static_cast<const __half *>(scale_mat);
    const __half *sv = static_cast<const __half *>(scale_vec);
    const int8_t *w = static_cast<const int8_t *>(mat);
    const int8_t *x = static_cast<const int8_t *>(vec);
    __half *y = static_cast<__half *>(out);
    int b = 0;
    while (b < batch) {
        const int left = batch - b;
        if (left >= 8) { gemv_int8_kernel<8><<<blocks, kBlock, 0, st>>>(dim_out, dim_in, b, sm, w, sv, x, y, vec16); b += 8; }
        else if (left >= 4) { gemv_int8_kernel<4><<<blocks, kBlock, 0, st>>>(dim_out, dim_in, b, sm, w, sv, x, y, vec16); b += 4; }
        else if (left >= 2) { gemv_int8_kernel<2><<<blocks, kBlock, 0, st>>>(dim_out, dim_in, b, sm, w, sv, x, y, vec16); b += 2; }
        else { gemv_int8_kernel<1><<<blocks, kBlock, 0, st>>>(dim_out, dim_in, b, sm, w, sv, x, y, vec16); b += 1; }
        CPMK_LAUNCH_CHECK();
    }
    return CPMK_OK;
}

int32_t cpmk_probe_read(int32_t mode, int32_t rows, int32_t row_elems, const void *src, void *sink, cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    CPMK_REQUIRE(rows > 0 && row_elems > 0 && row_elems % 8 == 0 && src && sink && aligned16(src), "bad arguments (rows=%d row_elems=%d)", rows, row_elems);
    cudaStream_t st = as_stream(stream);
    if (mode == 0) {
        const int64_t nvec = (int64_t)rows * row_elems / 8;
        read_probe_kernel<<<info.sm_count * 8, kBlock, 0, st>>>(nvec, static_cast<const uint4 *>(src), static_cast<uint32_t *>(sink));
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    CPMK_REQUIRE(mode == 1, "mode must be 0 (plain read) or 1 (the row GEMV's copy pipeline)");
    const int64_t row_bytes = (int64_t)row_elems * 2;
    CPMK_REQUIRE(row_bytes >= 2048 && row_bytes * kStreamRows * 2 <= kStreamRingBytes && rows >= info.sm_count * 16,
                 "mode 1 takes the shapes the streaming row GEMV takes (rows of 2 KiB to 12.5 KiB, at least %d rows)", info.sm_count * 16);
    static std::once_flag attr_once[64];
    static cudaError_t attr_err[64];
    const int dev = info.device & 63;
    std::call_once(attr_once[dev], [dev] {
        attr_err[dev] = cudaFuncSetAttribute(gemv_rows_stream_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes + kStreamVecBytes);
    });
    CPMK_CUDA_TRY(attr_err[dev]);
    Workspace ws;
    rc = get_workspace(st, &ws);
    if (rc) return rc;
    int chunk = row_elems;
    if (chunk > 4096) {
        const int parts = (row_elems + 4095) / 4096;
        chunk = ((row_elems + parts - 1) / parts + 7) / 8 * 8;
    }
    int stages = (int)(kStreamRingBytes / ((int64_t)chunk * 2 * kStreamRows));
    if (stages > 16) stages = 16;
    const size_t smem = (size_t)stages * chunk * 2 * kStreamRows + (size_t)row_elems * 2;
    gemv_rows_stream_kernel<false, true><<<info.sm_count, kStreamThreads, smem, st>>>(rows / info.sm_count, rows % info.sm_count, rows, row_elems, chunk, stages,
                                                                                        static_cast<const __half *>(src), static_cast<const __half *>(src),
                                                                                        static_cast<__half *>(sink), ws.status());
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

int32_t cpmk_gemv_fp16_transpose_noalloc(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out,
                                         cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    rc = check_gemv(batch, dim_out, dim_in);
    if (rc) return rc;
    if ((int64_t)batch * dim_out == 0) return CPMK_OK;
    CPMK_REQUIRE(mat && vec && out, "null tensor pointer");
    CPMK_REQUIRE(dim_in > 0, "dim_in must be positive");
    CPMK_REQUIRE(dim_out % 8 == 0 && aligned16(mat), "the allocation-free GEMV needs dim_out %% 8 == 0 and a 16-byte aligned matrix");
    CPMK_REQUIRE(batch <= 65535, "batch %d exceeds 65535", batch);
    const int strips = (dim_out + kTStripCols - 1) / kTStripCols;
    // the fixed scratch must hold at least two row chunks of partial sums and one ticket per (batch, strip)
    if ((size_t)batch * strips * sizeof(uint32_t) > kStaticTicketBytes ||
        2 * sizeof(float) * (size_t)batch * (size_t)dim_out > kStaticPartialBytes) {
        set_error("cpmk_gemv_fp16_transpose_noalloc: batch * dim_out = %lld exceeds the fixed scratch (limit: batch * dim_out <= %zu "
                  "and batch * ceil(dim_out / 256) <= %zu); use cpmk_gemv_fp16_transpose",
                  (long long)batch * dim_out, kStaticPartialBytes / (2 * sizeof(float)), kStaticTicketBytes / sizeof(uint32_t));
        return CPMK_ENOMEM;
    }
    unsigned char *scratch = nullptr;
    rc = static_scratch_address(info.device, &scratch);
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    int64_t splits = ((int64_t)info.sm_count * 6) / ((int64_t)strips * batch);
    const int64_t max_by_rows = (dim_in + 63) / 64;
    if (splits > max_by_rows) splits = max_by_rows;
    const int64_t max_by_scratch = (int64_t)(kStaticPartialBytes / (sizeof(float) * (size_t)batch * (size_t)dim_out));
    if (splits > max_by_scratch) splits = max_by_scratch;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
    int rps = (int)((dim_in + splits - 1) / splits);
    rps = (rps + kWarps - 1) / kWarps * kWarps;
    const int nsplit = (dim_in + rps - 1) / rps;
    uint32_t *tickets = reinterpret_cast<uint32_t *>(scratch);
    float *partial = reinterpret_cast<float *>(scratch + kStaticTicketBytes);
    // the array keeps whatever the previous call left: the tickets this call counts on must start at zero
    if (nsplit > 1) CPMK_CUDA_TRY(cudaMemsetAsync(tickets, 0, (size_t)batch * strips * sizeof(uint32_t), st));
    const dim3 grid(strips, nsplit, batch);
    gemv_transpose_kernel<<<grid, kBlock, 0, st>>>(dim_out, dim_in, rps, nsplit, static_cast<const __half *>(mat),
                                                   static_cast<const __half *>(vec), static_cast<__half *>(out), partial, tickets);
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

}  // extern "C"
