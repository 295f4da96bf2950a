// int8 x int8 -> int32 GEMM for sm_100a with the fp16 dequantisation fused into its epilogue.
//
// Replaces the cublasLtMatmul call of cpm_kernels/kernels/gemm.py:127-186 (and, when fused, the
// cu_gemm_scale pass of cuda/gemm.cu:37-57 that follows it in cpm_kernels/torch/gemm.py:40-64).
//
// Three kernels:
//   * gemm_i8_tc2_kernel -- the main one: a cluster of two CTAs computes a 256 x 256 output tile with
//     tcgen05.mma.cta_group::2.kind::i8, accumulators in tensor memory (two per CTA, so the epilogue of tile i overlaps
//     the main loop of tile i+1), operands staged by TMA through a 5-stage mbarrier ring, persistent grid with
//     warp-specialised roles (TMA producer / MMA issuer / 8 epilogue warps), output through swizzled shared-memory
//     staging tiles and TMA stores (to one or several destinations).  Takes all four storage orders of the operands.
//   * gemm_i8_tc_kernel  -- one CTA per 128 x 256 tile (cta_group::1, 4 stages, 4 epilogue warps, register epilogue),
//     for outputs of at most 128 rows with both operands contiguous along k.
//   * gemm_i8_simt_kernel -- dp4a, any layout, any size that the interface admits.
// gemm_f16_tc2_kernel is the first kernel's pipeline with kind::f16 (the int8=False branch of bmm).
//
// Every device-side wait is bounded: when one runs out the CTA records a code in the status word,
// raises its abort flag, lets copies in flight land, frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "cpmk_common.cuh"
#include "cpmk_ptx.cuh"

namespace cpmk {
namespace {

// ------------------------------------------------------------------------------------------------
// tile configuration of the tensor-core kernel
// ------------------------------------------------------------------------------------------------
constexpr int kBM = 128;                 // output rows per tile   (UMMA M; TMEM lanes)
constexpr int kBN = 256;                 // output cols per tile   (UMMA N; TMEM columns per accumulator)
constexpr int kBK = 128;                 // int8 elements (= bytes) of k per stage: one 128-byte swizzle row
constexpr int kUmmaK = 32;               // k per tcgen05.mma kind::i8
constexpr int kStages = 4;
constexpr int kPBytes = kBM * kBK;       // 16 KiB
constexpr int kQBytes = kBN * kBK;       // 32 KiB
constexpr int kStageBytes = kPBytes + kQBytes;
constexpr int kTmemCols = 512;           // two 256-column accumulators
constexpr int kTcThreads = 192;          // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int kBarrierBytes = 256;
constexpr int kTcSmemBytes = kStages * kStageBytes + 1024 + kBarrierBytes;


// status codes written to the status word (first failure wins)
constexpr uint32_t kErrProducerWait = 0x101;
constexpr uint32_t kErrMmaWaitFull = 0x102;
constexpr uint32_t kErrMmaWaitTmem = 0x103;
constexpr uint32_t kErrEpilogueWait = 0x104;
constexpr uint32_t kErrForwardWaitTile = 0x105;
constexpr uint32_t kErrForwardWaitLoad = 0x106;

struct GemmParams {
    int32_t R, C, K;              // out is (batch, R, C); reduction length K
    int32_t batch;
    int32_t p_batched, q_batched; // 0: operand has a single batch that is broadcast
    int32_t tiles_r, tiles_c, num_kb;
    int32_t total_tiles;
    void *out;
    const __half *scale_r;        // (bcast_r ? 1 : batch, R)   multiplies first
    const __half *scale_c;        // (bcast_c ? 1 : batch, C)
    int32_t bcast_r, bcast_c;
    int32_t tma_store;            // the two-CTA kernel writes its output with TMA stores (needs 16-byte row pitch)
    int32_t n_dst;                // number of destinations of the output (1, or one per GPU when scattering)
    int32_t n_store;              // destinations the computing CTAs store to themselves: n_dst, or 1 when forwarding CTAs serve the others
    int32_t send_pairs;           // > 0: the last `send_pairs` CTA pairs of the grid forward finished tiles from destination 0 to the others
    uint32_t *flags;              // send_pairs > 0: one counter per (pair tile, CTA of the pair), zero at launch; 8 = all epilogue warps have stored
    __half *fwd_dst[8];           // send_pairs > 0: element (0, 0, 0) of every destination (0: this GPU's own, where the computing CTAs store)
    int64_t out_ld;               // row pitch of the destinations in elements
    int32_t multicast;            // send_pairs > 0: destination 1 is a multicast address (one multimem store reaches every GPU)
    uint32_t *status;
    // tile index -> (batch, column block, row block) without integer division: multipliers and shifts for
    // tiles_r * tiles_c and for tiles_r (set_tile_divisors)
    uint32_t per_batch, per_batch_mul, per_batch_shr, tiles_r_mul, tiles_r_shr;
};

// Division of a 31-bit value by a constant through a multiply-high: q = umulhi(x, mul) >> shr with
// mul = ceil(2^(31 + ceil(log2 d)) / d), shr = ceil(log2 d) - 1; exact for 0 <= x < 2^31 (d = 1: q = x).
inline void find_divisor(uint32_t d, uint32_t *mul, uint32_t *shr) {
    if (d <= 1) {
        *mul = 0;
        *shr = 0;
        return;
    }
    uint32_t lg = 0;
    while ((1ull << lg) < d) ++lg;
    const uint32_t p = 31 + lg;
    *mul = (uint32_t)(((1ull << p) + d - 1) / d);
    *shr = p - 32;
}
__host__ __device__ __forceinline__ uint32_t fast_div(uint32_t x, uint32_t d, uint32_t mul, uint32_t shr) {
#if defined(__CUDA_ARCH__)
    return d == 1 ? x : (__umulhi(x, mul) >> shr);
#else
    return d == 1 ? x : (uint32_t)(((uint64_t)x * mul) >> 32) >> shr;
#endif
}
inline void set_tile_divisors(GemmParams *prm) {
    prm->per_batch = (uint32_t)prm->tiles_r * (uint32_t)prm->tiles_c;
    find_divisor(prm->per_batch, &prm->per_batch_mul, &prm->per_batch_shr);
    find_divisor((uint32_t)prm->tiles_r, &prm->tiles_r_mul, &prm->tiles_r_shr);
}
__device__ __forceinline__ void tile_coords(const GemmParams &prm, int tile, int &b, int &c_blk, int &r_blk) {
    b = (int)fast_div((uint32_t)tile, prm.per_batch, prm.per_batch_mul, prm.per_batch_shr);
    const int rem = tile - b * (int)prm.per_batch;
    c_blk = (int)fast_div((uint32_t)rem, (uint32_t)prm.tiles_r, prm.tiles_r_mul, prm.tiles_r_shr);
    r_blk = rem - c_blk * prm.tiles_r;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int32_t c0, int32_t c1, int32_t c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, int8 operands, int32 accumulator
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on `bar` once all tcgen05.mma issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a k-major tile whose rows are 128 bytes, stored with the 128-byte
// swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): 8-row groups are 1024 bytes apart.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (unused here: 1)
//   bits [32,46) stride byte offset >> 4   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1u << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1u << 46;
    d |= (uint64_t)2u << 61;
    return d;
}

// Shared-memory matrix descriptor of an MN-major tile (the operand's rows, not k, are contiguous in memory): what
// TMA writes for a box of 128 elements (one 128-byte swizzle row) by kBK k-rows.  Eight k-rows form a 1024-byte
// swizzle atom (stride byte offset); a further block of 128 elements along M/N, when an MMA spans more than
// one, lies `mn_block_bytes` away (leading byte offset).
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t mn_block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((mn_block_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1u << 46;
    d |= (uint64_t)2u << 61;
    return d;
}

// Instruction descriptor of tcgen05.mma kind::i8: int32 accumulator (bits 4-5 = 2), signed 8-bit A and B
// (bits 7-9 = 1, 10-12 = 1), both k-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// One epilogue warp's share of a finished accumulator: TMEM lanes [32*quarter, 32*quarter+32) = output rows
// row_base + 32*quarter + lane, all kBN columns from col_base, 32 columns per tcgen05.ld.
template <bool DEQUANT>
__device__ __forceinline__ void epilogue_rows(const GemmParams &prm, uint32_t tmem_base, uint32_t acc, int quarter, int lane, int b,
                                              int row_base, int col_base, int chunk_begin = 0, int chunk_end = kBN / 32) {
    const int row = row_base + quarter * 32 + lane;
    const bool row_ok = row < prm.R;
    const int64_t out_row = ((int64_t)b * prm.R + (row_ok ? row : 0)) * prm.C;
    float sr = 0.f;
    if (DEQUANT && row_ok) sr = __half2float(__ldg(prm.scale_r + (prm.bcast_r ? 0 : (int64_t)b * prm.R) + row));
    const __half *sc = DEQUANT ? prm.scale_c + (prm.bcast_c ? 0 : (int64_t)b * prm.C) : nullptr;
#pragma unroll 1
    for (int chunk = chunk_begin; chunk < chunk_end; ++chunk) {
        const int col0 = col_base + chunk * 32;
        if (col0 >= prm.C) break;                    // uniform across the warp
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBN + chunk * 32, v);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (DEQUANT) {
            __half *dst = static_cast<__half *>(prm.out) + out_row + col0;
            if ((prm.C & 7) == 0) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (col0 + g * 8 < prm.C) {
                        const uint4 s8 = __ldg(reinterpret_cast<const uint4 *>(sc + col0 + g * 8));
                        const __half2 *sh = reinterpret_cast<const __half2 *>(&s8);
                        uint4 o;
                        uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 s2 = __half22float2(sh[e]);
                            const float a0 = __fmul_rn(__fmul_rn((float)(int32_t)v[g * 8 + 2 * e], sr), s2.x);
                            const float a1 = __fmul_rn(__fmul_rn((float)(int32_t)v[g * 8 + 2 * e + 1], sr), s2.y);
                            ow[e] = pack_half2(a0, a1);
                        }
                        *reinterpret_cast<uint4 *>(dst + g * 8) = o;
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    if (col0 + e < prm.C) {
                        const float a = __fmul_rn(__fmul_rn((float)(int32_t)v[e], sr), __half2float(__ldg(sc + col0 + e)));
                        dst[e] = __float2half_rn(a);
                    }
                }
            }
        } else {
            int32_t *dst = static_cast<int32_t *>(prm.out) + out_row + col0;
            if ((prm.C & 3) == 0) {
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if (col0 + g * 4 < prm.C)
                        *reinterpret_cast<uint4 *>(dst + g * 4) = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    if (col0 + e < prm.C) dst[e] = (int32_t)v[e];
            }
        }
    }
}

template <bool DEQUANT>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q, const GemmParams prm) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars_base = tiles_base + kStages * kStageBytes;
    // barrier block: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then tmem slot, abort flag
    const uint32_t full_bar = bars_base;
    const uint32_t empty_bar = bars_base + 8 * kStages;
    const uint32_t tmem_full_bar = bars_base + 16 * kStages;
    const uint32_t tmem_empty_bar = tmem_full_bar + 16;
    uint8_t *bars_generic = smem_raw + (bars_base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars_generic + 16 * kStages + 32);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full_bar + 8 * a, 1);
            mbar_init(tmem_empty_bar + 8 * a, 4);      // one arrival per epilogue warp
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_per_batch = prm.tiles_r * prm.tiles_c;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < prm.total_tiles; tile += gridDim.x) {
                int b, c_blk, r_blk;
                tile_coords(prm, tile, b, c_blk, r_blk);
                for (int kb = 0; kb < prm.num_kb; ++kb) {
                    if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, prm.status, kErrProducerWait)) { alive = false; break; }
                    const uint32_t p_dst = tiles_base + stage * kStageBytes;
                    mbar_expect_tx(full_bar + 8 * stage, kStageBytes);
                    tma_load_3d(p_dst, &tmap_p, kb * kBK, r_blk * kBM, prm.p_batched ? b : 0, full_bar + 8 * stage);
                    tma_load_3d(p_dst + kPBytes, &tmap_q, kb * kBK, c_blk * kBN, prm.q_batched ? b : 0, full_bar + 8 * stage);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < prm.total_tiles; tile += gridDim.x) {
                if (!mbar_wait(tmem_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, prm.status, kErrMmaWaitTmem)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int kb = 0; kb < prm.num_kb; ++kb) {
                    if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, prm.status, kErrMmaWaitFull)) { alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t p_src = tiles_base + stage * kStageBytes;
                    const uint64_t p_desc = make_kmajor_sw128_desc(p_src);
                    const uint64_t q_desc = make_kmajor_sw128_desc(p_src + kPBytes);
#pragma unroll
                    for (int j = 0; j < kBK / kUmmaK; ++j) {
                        // advancing k inside the swizzle row: +32 bytes = +2 in the (address >> 4) field
                        umma_i8(d_tmem, p_desc + (uint64_t)(2 * j), q_desc + (uint64_t)(2 * j), kInstrDesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar + 8 * stage);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!alive) break;
                umma_commit(tmem_full_bar + 8 * acc);
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> (dequantise) -> global ----------------
        const int quarter = warp & 3;                       // TMEM lanes [32*quarter, 32*quarter + 32)
        uint32_t acc = 0, acc_phase = 0;
        for (int tile = blockIdx.x; tile < prm.total_tiles; tile += gridDim.x) {
            int b, c_blk, r_blk;
            tile_coords(prm, tile, b, c_blk, r_blk);
            if (!mbar_wait(tmem_full_bar + 8 * acc, acc_phase, abort_flag, prm.status, kErrEpilogueWait)) break;
            tcgen05_fence_after();
            epilogue_rows<DEQUANT>(prm, tmem_base, acc, quarter, lane, b, r_blk * kBM, c_blk * kBN);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty_bar + 8 * acc);
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    // ---------------- teardown ----------------
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies and MMAs that were in flight when the CTA gave up time to land before the
        // shared and tensor memory they target are released
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// Two-CTA form: a cluster of two CTAs on neighbouring SMs computes a 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of the row operand and 128 of the 256 rows of
// the column operand (the tensor cores of the pair read both halves), so per MMA a CTA's shared memory serves
// 8 KiB instead of 12 KiB and receives 8 KiB instead of 12 KiB from TMA: the shared-memory port stops being
// the limiter.  Stages shrink to 32 KiB; the ring holds 5 of them, and 64 KiB stage the output of eight epilogue
// warps (two per TMEM lane quarter, 128 columns each) on its way to TMA stores.
//   - both CTAs run a producer warp; every load signals the full barrier of CTA 0 (the leader), whose producer
//     posts the expected byte count of both CTAs;
//   - only the leader issues MMAs; its commits arrive on the empty / accumulator-full barriers of both CTAs;
//   - the epilogue warps of both CTAs arrive on the leader's accumulator-empty barrier.
// ------------------------------------------------------------------------------------------------
constexpr int kStages2 = 5;
constexpr int kEpiWarps2 = 8;                          // two epilogue warps per TMEM lane quarter, 128 columns each
constexpr int kTcThreads2 = (2 + kEpiWarps2) * 32;
constexpr int kHalfBN = kBN / 2;                       // rows of the column operand staged per CTA
constexpr int kQBytes2 = kHalfBN * kBK;                // 16 KiB
constexpr int kStageBytes2 = kPBytes + kQBytes2;       // 32 KiB
constexpr int kOutStageBytes = 32 * 128;                // one epilogue warp's staging tile: 32 rows x 128 bytes
constexpr int kOutStagingBytes = 8 * 2 * kOutStageBytes; // eight epilogue warps, two tiles each: 64 KiB (with five operand stages)
constexpr int kTc2SmemBytes = kStages2 * kStageBytes2 + kOutStagingBytes + 1024 + kBarrierBytes;
constexpr uint32_t kInstrDesc2 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)((2 * kBM) >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
// Arrive on a barrier of either CTA of the pair.  The arrival only hands a resource back (an accumulator that has been
// read); nothing written by this thread is published through it, so the default CTA-scope release is enough -- a
// cluster-scope release made every epilogue warp wait ~1000 cycles per tile for its earlier writes to drain.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load issued by one CTA of a pair; the completion bytes go to `bar`, a shared::cluster barrier address
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int32_t c0, int32_t c1, int32_t c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same for fp16 operands with an fp32 accumulator (k = 16 per instruction)
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor of kind::f16: fp32 accumulator (bits 4-5 = 1), fp16 A and B (bits 7-9 = 0, 10-12 = 0).
constexpr uint32_t kInstrDescF16 = (1u << 4) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)((2 * kBM) >> 4) << 24);
constexpr int kBKf16 = kBK / 2;                        // fp16 elements of k per stage (one 128-byte swizzle row)
constexpr int kMnBlockF16 = 64 * kBKf16 * 2;           // an MN-major fp16 tile is two blocks of 64 rows x kBKf16 k-rows: 8 KiB each

// arrives on the barrier at offset `bar` in every CTA of `cta_mask` once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask) : "memory");
}

// Up to eight destinations of the output (this GPU's buffer and, when the output is scattered, its peers').
constexpr int kMaxDst = 8;
struct OutMaps {
    CUtensorMap m[kMaxDst];
};

// TMA store of a staged 32-row x 128-byte tile (128-byte swizzle) to the 3-d output map; out-of-range rows and
// columns are clipped by the hardware.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// The dequantisation scales one epilogue warp needs for one tile, held in registers: the scale of the lane's output
// row, and the 128 column scales of the warp's half of the tile spread over the lanes (lane l holds columns
// 4 l .. 4 l + 3 as two half2 words; the epilogue broadcasts them with shuffles).  Loaded one tile ahead.
// The values stay as loaded (fp16 bits) until the epilogue uses them: nothing here depends on the loads' results, so
// the warp does not wait for them.
struct TileScales {
    unsigned short row;
    uint2 cols;
};
__device__ __forceinline__ TileScales load_tile_scales(const GemmParams &prm, int b, int row, int warp_col, int lane) {
    TileScales ts;
    ts.row = row < prm.R ? __ldg(reinterpret_cast<const unsigned short *>(prm.scale_r) + (prm.bcast_r ? 0 : (int64_t)b * prm.R) + row) : (unsigned short)0;
    const int c = warp_col + 4 * lane;                       // C % 8 == 0 on this path: the four columns are in or out together
    ts.cols = c < prm.C ? __ldg(reinterpret_cast<const uint2 *>(prm.scale_c + (prm.bcast_c ? 0 : (int64_t)b * prm.C) + c)) : make_uint2(0u, 0u);
    return ts;
}

// Epilogue of one warp for one finished accumulator, written through shared memory with TMA stores: the warp's
// 32 rows x 256 columns leave as 128-byte-wide pieces (64 fp16 or 32 int32 columns): each lane converts its row,
// writes it into a swizzled 32 x 128-byte staging tile (16-byte chunk j of row r at chunk j ^ (r & 7): no bank
// conflicts, and what the store's 128-byte swizzle expects), and lane 0 issues the store.  Two staging tiles per
// warp alternate, so converting piece i+1 overlaps the store of piece i; the stores are full lines and need no
// edge predicates.
// NB staging tiles per warp (2 or 4) form two groups of NB / 2: the pieces of a group are staged, made visible to the
// TMA unit with ONE proxy fence, and stored together, while the other group's stores drain.
template <bool DEQUANT, bool F16, int NB>
__device__ __forceinline__ void epilogue_rows_tma(const GemmParams &prm, const OutMaps *tmap_o, uint32_t staging, uint32_t &buf,
                                                  uint32_t tmem_base, uint32_t acc, int quarter, int lane, int b, int row_base, int col_base,
                                                  int half, const TileScales &ts) {
    const float sr = __half2float(__ushort_as_half(ts.row));
    const int warp_col = col_base + half * (kBN / 2);                // this warp's 128 columns
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBN + half * (kBN / 2);
    const uint32_t sw = (uint32_t)(lane & 7);
    constexpr int kSteps = (kBN / 2) / 32;                           // four steps of 32 columns
    constexpr int kStepsPerPiece = DEQUANT ? 2 : 1;                  // a stored piece is 128 bytes wide: 64 fp16 / 32 int32

    // Software pipeline over the steps: the tensor-memory load of step i+1 is requested before step i is converted,
    // so its latency hides behind the arithmetic and the shared-memory writes.  No global load happens in here: the
    // scales were fetched a tile ahead (TileScales), so the proxy fence before each store has nothing slow to wait for.
    uint32_t v[2][32];
    auto request = [&](int st, int slot) { tmem_ld_32x32b_x32(taddr + st * 32, v[slot]); };
    if (warp_col >= prm.C) return;                                   // uniform across the warp
    constexpr int kGroup = NB >= 2 ? NB / 2 : 1;                     // pieces per fence and commit group
    constexpr int kPendingGroups = NB / kGroup - 1;                  // commit groups that may still be reading when a group is reused
    int staged = 0, staged_col0 = 0, staged_col1 = 0;                // pieces of the current group waiting to be stored
    auto flush = [&]() {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            // one store per piece and destination (peers' buffers are reached over NVLink)
            for (int i = 0; i < staged; ++i)
                for (int d = 0; d < prm.n_store; ++d)
                    tma_store_3d(&tmap_o->m[d], staging + (buf + (uint32_t)i) * kOutStageBytes, i == 0 ? staged_col0 : staged_col1,
                                 row_base + quarter * 32, b);
            bulk_commit();
        }
        buf = (buf + kGroup) % NB;
        staged = 0;
    };
    request(0, 0);
#pragma unroll
    for (int st = 0; st < kSteps; ++st) {
        const int slot = st & 1;
        const int col0 = warp_col + st * 32;
        tmem_ld_wait();                                              // step st has arrived
        if (st + 1 < kSteps) request(st + 1, slot ^ 1);
        const bool first_of_piece = (st % kStepsPerPiece) == 0;
        const bool last_of_piece = (st % kStepsPerPiece) == kStepsPerPiece - 1;
        const int piece_col = col0 - (st % kStepsPerPiece) * 32;
        if (piece_col >= prm.C) continue;                            // nothing of this piece is inside the output (uniform)
        const uint32_t tile = staging + (buf + (uint32_t)staged) * kOutStageBytes;
        const uint32_t my_row = tile + (uint32_t)lane * 128u;
        if (first_of_piece && staged == 0) {
            // the stores committed two groups ago read these tiles: they must have finished reading
            if (lane == 0) bulk_wait_read<kPendingGroups>();
            __syncwarp();
        }
        if (F16) {
            // fp32 accumulators of the fp16 GEMM: one rounding to fp16, no scales
            const uint32_t chunk0 = (uint32_t)(st % kStepsPerPiece) * 4u;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    o[e] = pack_half2(__uint_as_float(v[slot][g * 8 + 2 * e]), __uint_as_float(v[slot][g * 8 + 2 * e + 1]));
                st_shared_v4(my_row + (((chunk0 + (uint32_t)g) ^ sw) << 4), o[0], o[1], o[2], o[3]);
            }
        } else if (DEQUANT) {
            const uint32_t chunk0 = (uint32_t)(st % kStepsPerPiece) * 4u;      // 16-byte chunks 0-3 or 4-7 of the 128-byte row
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                // columns 32 st + 8 g .. + 7 of the warp's 128: their scales sit in lanes 8 st + 2 g and 8 st + 2 g + 1
                const int src = 8 * st + 2 * g;
                uint32_t c4[4];
                c4[0] = __shfl_sync(0xffffffffu, ts.cols.x, src);
                c4[1] = __shfl_sync(0xffffffffu, ts.cols.y, src);
                c4[2] = __shfl_sync(0xffffffffu, ts.cols.x, src + 1);
                c4[3] = __shfl_sync(0xffffffffu, ts.cols.y, src + 1);
                const __half2 *sh = reinterpret_cast<const __half2 *>(c4);
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 s2 = __half22float2(sh[e]);
                    const float a0 = __fmul_rn(__fmul_rn((float)(int32_t)v[slot][g * 8 + 2 * e], sr), s2.x);
                    const float a1 = __fmul_rn(__fmul_rn((float)(int32_t)v[slot][g * 8 + 2 * e + 1], sr), s2.y);
                    o[e] = pack_half2(a0, a1);
                }
                st_shared_v4(my_row + (((chunk0 + (uint32_t)g) ^ sw) << 4), o[0], o[1], o[2], o[3]);
            }
        } else {
#pragma unroll
            for (int g = 0; g < 8; ++g)                              // eight 16-byte chunks = 32 int32 columns
                st_shared_v4(my_row + (((uint32_t)g ^ sw) << 4), v[slot][4 * g], v[slot][4 * g + 1], v[slot][4 * g + 2], v[slot][4 * g + 3]);
        }
        if (last_of_piece) {
            if (staged == 0) staged_col0 = piece_col;
            else staged_col1 = piece_col;
            if (++staged == kGroup) flush();
        }
    }
    if (staged > 0) flush();
}

// ------------------------------------------------------------------------------------------------
// Forwarding CTAs.  When the output goes to several GPUs, stores that cross NVLink are slow to drain: issued by the
// CTAs that compute, they sit in the same per-SM TMA queue as the operand loads and in the same staging tiles the
// epilogue wants back, and the main loop ends up waiting for the link (measured: GEMM time = compute + transfer).
// So the computing CTAs can store only to destination 0 -- this GPU's own buffer -- and signal each finished 128 x 256
// CTA tile through a counter; the last `send_pairs` CTA pairs of the same grid do nothing but wait for those counters
// and copy finished tiles from destination 0 (out of L2, where they were just written) to every other destination.
// Each forwarding warp keeps a ring of 4 KiB pieces (32 rows x 128 bytes) filled by TMA loads, which run ahead
// unhindered because nothing else shares that SM's TMA queue, and empties it with ordinary 16-byte stores by all of its
// lanes (a store that waits for the link then holds up nothing but the next store).  Transfer and arithmetic overlap
// tile by tile inside one kernel.  Only stores cross the link (no load touches a peer's memory, nothing is multicast
// by TMA).  The waits for a tile and for a load are bounded.
// ------------------------------------------------------------------------------------------------
constexpr int kFwdSlots = 6;                            // 4 KiB pieces per forwarding warp (8 warps: 192 KiB of the CTA's shared memory)

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
// one 16-byte store that the NVLink switch replicates into every GPU's copy of a multicast-mapped buffer
__device__ __forceinline__ void multimem_st_v4(void *mc_addr, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void forward_tiles(const OutMaps &tmap_o, const GemmParams &prm, int send_pair, uint32_t rank) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t ring_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars_base = ring_base + kEpiWarps2 * kFwdSlots * kOutStageBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ uint32_t fwd_abort;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kEpiWarps2 * kFwdSlots; ++i) mbar_init(bars_base + 8 * i, 1);
        fwd_abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (warp < 2) return;                                // as many forwarding warps as there are epilogue warps
    const int w = warp - 2, quarter = w & 3, half = w >> 2;
    const uint32_t my_ring = ring_base + (uint32_t)w * kFwdSlots * kOutStageBytes;
    const uint32_t my_bars = bars_base + 8u * (uint32_t)(w * kFwdSlots);
    volatile uint32_t *abort_flag = &fwd_abort;
    const int64_t ld = prm.out_ld;

    // pieces are numbered in the order they are forwarded; piece q lives in slot q % kFwdSlots (all lanes keep the same counts)
    int issued = 0, finished = 0;
    int piece_col[kFwdSlots], piece_row[kFwdSlots], piece_b[kFwdSlots];
    bool alive = true;
    auto finish_one = [&]() {
        const int slot = finished % kFwdSlots;
        const uint32_t parity = (uint32_t)(finished / kFwdSlots) & 1u;
        int ok = 1;
        if (lane == 0) ok = mbar_wait(my_bars + 8 * slot, parity, abort_flag, prm.status, kErrForwardWaitLoad) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { alive = false; return; }
        (void)mbar_try_wait(my_bars + 8 * slot, parity);  // every lane observes the completed phase before it reads the piece
        // lane l: 16-byte chunk l & 7 of rows (l >> 3), (l >> 3) + 4, ...: four 128-byte row segments per instruction;
        // the piece lies in shared memory as TMA wrote it (chunk c of row r at chunk c ^ (r & 7))
        const int chunk = lane & 7;
        const int col = piece_col[slot] + chunk * 8;
        const uint32_t src = my_ring + (uint32_t)slot * kOutStageBytes;
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r = j * 4 + (lane >> 3);
            v[j] = ld_shared_v4(src + (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4));
        }
        if (col < prm.C) {
            const int64_t offset = ((int64_t)piece_b[slot] * prm.R + piece_row[slot] + (lane >> 3)) * ld + col;
#pragma unroll
            for (int d = 1; d < kMaxDst; ++d) {
                if (d < prm.n_dst) {
                    __half *dst = prm.fwd_dst[d] + offset;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (piece_row[slot] + j * 4 + (lane >> 3) < prm.R) {
                            if (prm.multicast) multimem_st_v4(dst + (int64_t)(j * 4) * ld, v[j]);
                            else *reinterpret_cast<uint4 *>(dst + (int64_t)(j * 4) * ld) = v[j];
                        }
                    }
                }
            }
        }
        __syncwarp();                                    // every lane has read the slot before it is loaded again
        ++finished;
    };
    for (int tile = send_pair; alive && tile < prm.total_tiles; tile += prm.send_pairs) {
        int b, c_blk, r_blk;
        tile_coords(prm, tile, b, c_blk, r_blk);
        const int row0 = r_blk * (2 * kBM) + (int)rank * kBM + quarter * 32;
        const int col0 = c_blk * kBN + half * (kBN / 2);
        if (row0 >= prm.R || col0 >= prm.C) continue;     // nothing of this warp's block is inside the output (uniform)
        {
            const uint32_t *flag = prm.flags + ((size_t)tile * 2 + rank);
            int ready = 0;
            if (lane == 0) ready = ld_acquire_gpu(flag) >= (uint32_t)kEpiWarps2 ? 1 : 0;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) {
                // not finished yet: what is loaded ahead belongs to tiles that are complete, forward it before waiting
                while (alive && finished < issued) finish_one();
                if (!alive) break;
                int ok = 1;
                if (lane == 0) {
                    uint64_t t0 = 0;
                    for (uint32_t spin = 0; ld_acquire_gpu(flag) < (uint32_t)kEpiWarps2; ++spin) {
                        __nanosleep(64);
                        if ((spin & 0x3ffu) == 0x3ffu) {
                            const uint64_t now = global_timer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > kWaitLimitNs) {
                                atomicCAS(prm.status, 0u, kErrForwardWaitTile);
                                ok = 0;
                                break;
                            }
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
            }
        }
#pragma unroll 1
        for (int piece = 0; piece < 2 && alive; ++piece) {
            const int col = col0 + piece * 64;
            if (col >= prm.C) break;
            if (issued - finished >= kFwdSlots) finish_one();      // the slot's previous piece has been forwarded
            if (!alive) break;
            const int slot = issued % kFwdSlots;
            piece_col[slot] = col;
            piece_row[slot] = row0;
            piece_b[slot] = b;
            if (lane == 0) {
                // the slot was last read through the generic proxy: order those reads against the load that overwrites it
                // (a fence over shared memory only: one over all state spaces would wait for the stores to the peers)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(my_bars + 8 * slot, kOutStageBytes);
                tma_load_3d(my_ring + (uint32_t)slot * kOutStageBytes, &tmap_o.m[0], col, row0, b, my_bars + 8 * slot);
            }
            ++issued;
        }
    }
    while (alive && finished < issued) finish_one();
    if (prm.multicast) __threadfence_system();
    if (!alive) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // loads in flight land before the ring is released
    }
}

// P_MN / Q_MN: the row / column operand is stored with its rows contiguous (k is the slow axis) instead of k:
// the reference's bT / !aT layouts.  Their tensor maps then have (rows, k, batch) extents and 128 x kBK boxes, the
// shared-memory tiles are MN-major, and bits 15 / 16 of the instruction descriptor say so.
// F16: fp16 operands (kBKf16 elements of k per stage, kind::f16, fp32 accumulators) and an fp16 result with no
// scales; everything else -- stage bytes, barriers, tile walk, epilogue staging -- is the int8 pipeline's.
// STAGES operand stages of 32 KiB and 7 - STAGES output staging tiles per epilogue warp share the same 224 KiB.
// Five stages and two tiles are used; three and four (half as many proxy fences in the epilogue) measured the same on
// reductions of a single stage, where the epilogue is all there is.
// EG: groups of eight epilogue warps.  With two groups (reductions of one or two stages, where the epilogue is all there
// is) group g drains accumulator g, so the epilogues of two consecutive tiles run side by side; three operand stages and
// two staging tiles per warp then fill the same shared memory.
template <bool DEQUANT, bool P_MN, bool Q_MN, bool F16, int STAGES, int EG = 1>
__device__ __forceinline__ void tc2_pipeline(const CUtensorMap &tmap_p, const CUtensorMap &tmap_q, const OutMaps &tmap_o, const GemmParams &prm) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging_base = tiles_base + STAGES * kStageBytes2;       // 1024-byte aligned: swizzle atoms
    constexpr int kOutBufs = (7 - STAGES) / EG;                   // staging tiles per epilogue warp
    const uint32_t bars_base = staging_base + EG * kEpiWarps2 * kOutBufs * kOutStageBytes;
    const uint32_t full_bar = bars_base;                          // used in the leader only
    const uint32_t empty_bar = bars_base + 8 * STAGES;
    const uint32_t tmem_full_bar = bars_base + 16 * STAGES;
    const uint32_t tmem_empty_bar = tmem_full_bar + 16;           // used in the leader only
    uint8_t *bars_generic = smem_raw + (bars_base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars_generic + 16 * STAGES + 32);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    // the last send_pairs pairs of the grid forward finished tiles to the other destinations instead of computing
    const int pair = blockIdx.x >> 1, num_pairs = (gridDim.x >> 1) - prm.send_pairs;
    if (prm.send_pairs > 0 && pair >= num_pairs) {
        forward_tiles(tmap_o, prm, pair - num_pairs, rank);
        return;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full_bar + 8 * a, 1);
            mbar_init(tmem_empty_bar + 8 * a, 2 * kEpiWarps2);   // the epilogue warps of both CTAs
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tcgen05_fence_before();
    cluster_sync_all();                                // barriers of both CTAs are initialised before anyone signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;


    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (int tile = pair; alive && tile < prm.total_tiles; tile += num_pairs) {
                int b, c_blk, r_blk;
                tile_coords(prm, tile, b, c_blk, r_blk);
                const int row0 = r_blk * (2 * kBM) + (int)rank * kBM;
                const int col0 = c_blk * kBN + (int)rank * kHalfBN;
                for (int kb = 0; kb < prm.num_kb; ++kb) {
                    if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, prm.status, kErrProducerWait)) { alive = false; break; }
                    const uint32_t p_dst = tiles_base + stage * kStageBytes2;
                    if (leader) mbar_expect_tx(full_bar + 8 * stage, 2 * kStageBytes2);
                    const uint32_t leader_full = map_to_cta(full_bar + 8 * stage, 0);
                    constexpr int kKe = F16 ? kBKf16 : kBK;          // k elements per stage
                    if (P_MN && F16) {
                        // two boxes of 64 rows x 64 k-rows (a 16-bit swizzle row holds 64 elements)
                        tma_load_3d_pair(p_dst, &tmap_p, row0, kb * kKe, prm.p_batched ? b : 0, leader_full);
                        tma_load_3d_pair(p_dst + kMnBlockF16, &tmap_p, row0 + 64, kb * kKe, prm.p_batched ? b : 0, leader_full);
                    } else if (P_MN) tma_load_3d_pair(p_dst, &tmap_p, row0, kb * kKe, prm.p_batched ? b : 0, leader_full);
                    else tma_load_3d_pair(p_dst, &tmap_p, kb * kKe, row0, prm.p_batched ? b : 0, leader_full);
                    if (Q_MN && F16) {
                        tma_load_3d_pair(p_dst + kPBytes, &tmap_q, col0, kb * kKe, prm.q_batched ? b : 0, leader_full);
                        tma_load_3d_pair(p_dst + kPBytes + kMnBlockF16, &tmap_q, col0 + 64, kb * kKe, prm.q_batched ? b : 0, leader_full);
                    } else if (Q_MN) tma_load_3d_pair(p_dst + kPBytes, &tmap_q, col0, kb * kKe, prm.q_batched ? b : 0, leader_full);
                    else tma_load_3d_pair(p_dst + kPBytes, &tmap_q, kb * kKe, col0, prm.q_batched ? b : 0, leader_full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (leader && lane == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool alive = true;
            for (int tile = pair; alive && tile < prm.total_tiles; tile += num_pairs) {
                if (!mbar_wait(tmem_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, prm.status, kErrMmaWaitTmem)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int kb = 0; kb < prm.num_kb; ++kb) {
                    if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, prm.status, kErrMmaWaitFull)) { alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t p_src = tiles_base + stage * kStageBytes2;
                    // k advances by 32 per MMA: 32 bytes inside the swizzle row of a k-major tile (+2 in the
                    // address field), 32 rows of 128 bytes in an MN-major tile (+256)
                    // (fp16: k advances by 16 per MMA -- still 32 bytes of a k-major row, 16 rows = +128 MN-major)
                    const uint64_t p_desc = P_MN ? make_mnmajor_sw128_desc(p_src, F16 ? kMnBlockF16 : kPBytes) : make_kmajor_sw128_desc(p_src);
                    const uint64_t q_desc = Q_MN ? make_mnmajor_sw128_desc(p_src + kPBytes, F16 ? kMnBlockF16 : kQBytes2)
                                                 : make_kmajor_sw128_desc(p_src + kPBytes);
                    constexpr uint32_t idesc = (F16 ? kInstrDescF16 : kInstrDesc2) | (P_MN ? (1u << 15) : 0u) | (Q_MN ? (1u << 16) : 0u);
                    constexpr int kMnStep = F16 ? 128 : 256;
#pragma unroll
                    for (int j = 0; j < kBK / kUmmaK; ++j) {
                        const uint64_t pd = p_desc + (uint64_t)((P_MN ? kMnStep : 2) * j), qd = q_desc + (uint64_t)((Q_MN ? kMnStep : 2) * j);
                        if (F16) umma_f16_pair(d_tmem, pd, qd, idesc, (kb | j) != 0 ? 1u : 0u);
                        else umma_i8_pair(d_tmem, pd, qd, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar + 8 * stage, 3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!alive) break;
                umma_commit_pair(tmem_full_bar + 8 * acc, 3);
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue (both CTAs; each owns 128 of the tile's 256 rows) ----------------
        const int quarter = warp & 3;
        const int group = EG == 1 ? 0 : (warp - 2) >> 3; // which accumulator this warp's group drains (EG == 2)
        const int half = ((warp - 2) & 7) >> 2;          // which 128 of the tile's 256 columns this warp writes
        constexpr bool kScales = DEQUANT && !F16;
        const int tile_step = EG * num_pairs, first_tile = pair + group * num_pairs;
        uint32_t acc = (uint32_t)group, acc_phase = 0, out_buf = 0;
        auto scales_of = [&](int tile) {
            int b, c_blk, r_blk;
            tile_coords(prm, tile, b, c_blk, r_blk);
            return load_tile_scales(prm, b, r_blk * (2 * kBM) + (int)rank * kBM + quarter * 32 + lane, c_blk * kBN + half * (kBN / 2), lane);
        };
        TileScales ts = {(unsigned short)0, make_uint2(0u, 0u)}, ts_next = ts;
        if (kScales && prm.tma_store && first_tile < prm.total_tiles) ts = scales_of(first_tile);
        for (int tile = first_tile; tile < prm.total_tiles; tile += tile_step) {
            int b, c_blk, r_blk;
            tile_coords(prm, tile, b, c_blk, r_blk);
            // the next tile's scales travel while this tile is converted
            if (kScales && prm.tma_store && tile + tile_step < prm.total_tiles) ts_next = scales_of(tile + tile_step);
            if (!mbar_wait(tmem_full_bar + 8 * acc, acc_phase, abort_flag, prm.status, kErrEpilogueWait)) break;
            tcgen05_fence_after();
            if (F16 || prm.tma_store) {                  // (the fp16 GEMM is only launched with TMA stores)
                epilogue_rows_tma<DEQUANT, F16, kOutBufs>(prm, &tmap_o, staging_base + (uint32_t)(warp - 2) * kOutBufs * kOutStageBytes, out_buf, tmem_base, acc, quarter,
                                           lane, b, r_blk * (2 * kBM) + (int)rank * kBM, c_blk * kBN, half, ts);
                ts = ts_next;
            } else
                epilogue_rows<DEQUANT>(prm, tmem_base, acc, quarter, lane, b, r_blk * (2 * kBM) + (int)rank * kBM, c_blk * kBN, half * 4, half * 4 + 4);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar + 8 * acc, 0));
            if (prm.send_pairs > 0 && lane == 0) {
                // tell the forwarding CTAs that this warp's part of the tile is in destination 0: its stores have completed
                // (not merely been read out of shared memory), then a release at GPU scope, then the count
                bulk_wait_all();
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __threadfence();
                atomicAdd(prm.flags + ((size_t)tile * 2 + rank), 1u);
            }
            if (EG == 1) {
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            } else {
                acc_phase ^= 1u;                         // the group keeps its accumulator
            }
        }
        if (lane == 0) bulk_wait_all();                  // this warp's output stores have completed
    }

    // ---------------- teardown: neither CTA may leave while its partner can still touch its memory ----------------
    __syncwarp();
    tcgen05_fence_before();
    cluster_sync_all();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

template <bool DEQUANT, bool P_MN, bool Q_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads2, 1)
gemm_i8_tc2_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ OutMaps tmap_o, const GemmParams prm) {
    tc2_pipeline<DEQUANT, P_MN, Q_MN, false, kStages2>(tmap_p, tmap_q, tmap_o, prm);
}

// The same kernel with two groups of epilogue warps (18 warps), for reductions of at most two stages (K <= 256): the
// attention-score shape, whose time is its epilogue.
constexpr int kTcThreads2E = (2 + 2 * kEpiWarps2) * 32;
template <bool P_MN, bool Q_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads2E, 1)
gemm_i8_tc2e_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ OutMaps tmap_o, const GemmParams prm) {
    tc2_pipeline<true, P_MN, Q_MN, false, 3, 2>(tmap_p, tmap_q, tmap_o, prm);
}

// fp16 x fp16 -> fp16 with fp32 accumulation on the same pipeline (the reference's gemm_fp16, kernels/gemm.py:188-256)
template <bool P_MN, bool Q_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads2, 1)
gemm_f16_tc2_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ OutMaps tmap_o, const GemmParams prm) {
    tc2_pipeline<true, P_MN, Q_MN, true, kStages2>(tmap_p, tmap_q, tmap_o, prm);
}

// ------------------------------------------------------------------------------------------------
// Generic kernel: out[b, j, i] = sum_l Aop[b, l, i] * Bop[b, j, l] for any layout.
// 64 x 64 output tile per 256-thread block, 4 x 4 outputs per thread, k in chunks of 32 packed four to a
// word so that the inner product is dp4a.
// ------------------------------------------------------------------------------------------------
constexpr int kSimtTile = 64;
constexpr int kSimtK = 32;

template <bool DEQUANT>
__global__ void __launch_bounds__(256) gemm_i8_simt_kernel(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int aT, int bT,
                                                           const int8_t *__restrict__ A, const int8_t *__restrict__ B, void *__restrict__ out,
                                                           const __half *__restrict__ scale_x, const __half *__restrict__ scale_y, int bx, int by) {
    __shared__ int32_t As[kSimtK / 4][kSimtTile + 4];   // [k4][i]
    __shared__ int32_t Bs[kSimtK / 4][kSimtTile + 4];   // [k4][j]
    const int b = blockIdx.z;
    const int i0 = blockIdx.x * kSimtTile, j0 = blockIdx.y * kSimtTile;
    const int8_t *a = A + (batchA == 1 ? 0 : (int64_t)b * m * k);
    const int8_t *bb = B + (batchB == 1 ? 0 : (int64_t)b * n * k);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    int32_t acc[4][4];
#pragma unroll
    for (int y = 0; y < 4; ++y)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[y][x] = 0;

    for (int l0 = 0; l0 < k; l0 += kSimtK) {
        // 8 x 64 words per operand, 2 per thread
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            const int idx = threadIdx.x + w * 256;
            const int kk = idx >> 6, c = idx & 63;
            const int l = l0 + kk * 4;
            int32_t wa = 0, wb = 0;
            const int i = i0 + c, j = j0 + c;
            if (i < m && l < k) {                            // k % 4 == 0: a word is wholly inside or outside
                if (aT) {
                    wa = *reinterpret_cast<const int32_t *>(a + (int64_t)i * k + l);
                } else {
                    const uint32_t e0 = (uint8_t)a[(int64_t)l * m + i], e1 = (uint8_t)a[(int64_t)(l + 1) * m + i];
                    const uint32_t e2 = (uint8_t)a[(int64_t)(l + 2) * m + i], e3 = (uint8_t)a[(int64_t)(l + 3) * m + i];
                    wa = (int32_t)(e0 | (e1 << 8) | (e2 << 16) | (e3 << 24));
                }
            }
            if (j < n && l < k) {
                if (!bT) {
                    wb = *reinterpret_cast<const int32_t *>(bb + (int64_t)j * k + l);
                } else {
                    const uint32_t e0 = (uint8_t)bb[(int64_t)l * n + j], e1 = (uint8_t)bb[(int64_t)(l + 1) * n + j];
                    const uint32_t e2 = (uint8_t)bb[(int64_t)(l + 2) * n + j], e3 = (uint8_t)bb[(int64_t)(l + 3) * n + j];
                    wb = (int32_t)(e0 | (e1 << 8) | (e2 << 16) | (e3 << 24));
                }
            }
            As[kk][c] = wa;
            Bs[kk][c] = wb;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kSimtK / 4; ++kk) {
            int32_t av[4], bv[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) av[x] = As[kk][tx * 4 + x];
#pragma unroll
            for (int y = 0; y < 4; ++y) bv[y] = Bs[kk][ty * 4 + y];
#pragma unroll
            for (int y = 0; y < 4; ++y)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[y][x] = __dp4a(av[x], bv[y], acc[y][x]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int y = 0; y < 4; ++y) {
        const int j = j0 + ty * 4 + y;
        if (j >= n) continue;
        float sx = 0.f;
        if (DEQUANT) sx = __half2float(scale_x[(bx ? 0 : (int64_t)b * n) + j]);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = i0 + tx * 4 + x;
            if (i >= m) continue;
            const int64_t o = ((int64_t)b * n + j) * m + i;
            if (DEQUANT) {
                const float v = __fmul_rn(__fmul_rn((float)acc[y][x], sx), __half2float(scale_y[(by ? 0 : (int64_t)b * m) + i]));
                static_cast<__half *>(out)[o] = __float2half_rn(v);
            } else {
                static_cast<int32_t *>(out)[o] = acc[y][x];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        (void)cudaGetLastError();
    });
    return fn;
}

// Encoding a tensor map costs a microsecond or two of host time and a GEMM needs three or more; callers reuse the same
// buffers call after call (weights, and whatever the framework's caching allocator hands back), so encodings are kept
// per thread in a hash table keyed by everything that went into them.  A model of 48 layers with four weights each,
// activations, outputs and one output map per peer GPU stays well inside kMapCacheEntries; when the table is full it
// is emptied and refills.
struct MapKey {
    const void *ptr;
    int32_t a, b, c, kind;
    bool operator==(const MapKey &o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= ((uint64_t)(uint32_t)k.a << 32 | (uint32_t)k.b) * 0xC2B2AE3D27D4EB4Full;
        h ^= ((uint64_t)(uint32_t)k.c << 32 | (uint32_t)k.kind) * 0x165667B19E3779F9ull;
        return (size_t)(h ^ (h >> 29));
    }
};
constexpr size_t kMapCacheEntries = 4096;
struct MapCache {
    std::unordered_map<MapKey, CUtensorMap, MapKeyHash> table;
    const CUtensorMap *find(const MapKey &k) const {
        auto it = table.find(k);
        return it == table.end() ? nullptr : &it->second;
    }
    void put(const MapKey &k, const CUtensorMap &m) {
        if (table.size() >= kMapCacheEntries) table.clear();
        table.emplace(k, m);
    }
};
thread_local MapCache g_map_cache;

bool encode_operand_raw(CUtensorMap *map, const void *ptr, int32_t rows, int32_t k, int32_t batch, int32_t box_rows, int esz);
bool encode_operand_mn_raw(CUtensorMap *map, const void *ptr, int32_t rows, int32_t k, int32_t batch, int esz);
bool encode_output_raw(CUtensorMap *map, void *ptr, int32_t R, int32_t C, int64_t ld, int32_t batch, bool fp16);

template <typename F>
bool cached_encode(CUtensorMap *map, const MapKey &key, F &&encode) {
    if (const CUtensorMap *hit = g_map_cache.find(key)) {
        *map = *hit;
        return true;
    }
    if (!encode()) return false;
    g_map_cache.put(key, *map);
    return true;
}

// esz: bytes per operand element (1: int8, 2: fp16)
bool encode_operand(CUtensorMap *map, const void *ptr, int32_t rows, int32_t k, int32_t batch, int32_t box_rows, int esz = 1) {
    return cached_encode(map, MapKey{ptr, rows, k, batch, 0x100 + box_rows + 0x1000 * esz},
                         [&] { return encode_operand_raw(map, ptr, rows, k, batch, box_rows, esz); });
}
bool encode_operand_mn(CUtensorMap *map, const void *ptr, int32_t rows, int32_t k, int32_t batch, int esz = 1) {
    return cached_encode(map, MapKey{ptr, rows, k, batch, 1 + 0x1000 * esz}, [&] { return encode_operand_mn_raw(map, ptr, rows, k, batch, esz); });
}
bool encode_output(CUtensorMap *map, void *ptr, int32_t R, int32_t C, int64_t ld, int32_t batch, bool fp16) {
    if (ld != C) return encode_output_raw(map, ptr, R, C, ld, batch, fp16);       // pitched views are not cached
    return cached_encode(map, MapKey{ptr, R, C, batch, fp16 ? 2 : 3}, [&] { return encode_output_raw(map, ptr, R, C, ld, batch, fp16); });
}

// Operand (batch, rows, k) with k contiguous, as a 3-d tensor map whose box is box_rows x 128 bytes.
bool encode_operand_raw(CUtensorMap *map, const void *ptr, int32_t rows, int32_t k, int32_t batch, int32_t box_rows, int esz) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)k * esz, (cuuint64_t)rows * (cuuint64_t)k * esz};
    const cuuint32_t box[3] = {(cuuint32_t)(kBK / esz), (cuuint32_t)box_rows, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = enc(map, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Operand stored (batch, k, rows) with the rows contiguous, as a 3-d tensor map whose box is one 128-byte swizzle row
// of rows (128 int8 / 64 fp16) by one stage of k (128 int8 / 64 fp16).
bool encode_operand_mn_raw(CUtensorMap *map, const void *ptr, int32_t rows, int32_t k, int32_t batch, int esz) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)rows, (cuuint64_t)k, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)rows * esz, (cuuint64_t)rows * (cuuint64_t)k * esz};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / esz), (cuuint32_t)(kBK / esz), 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = enc(map, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Output (batch, R, C) with a row pitch of `ld` elements, as a 3-d tensor map whose box is 32 rows x 128 bytes,
// 128-byte swizzle (for TMA stores).
bool encode_output_raw(CUtensorMap *map, void *ptr, int32_t R, int32_t C, int64_t ld, int32_t batch, bool fp16) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t esz = fp16 ? 2 : 4;
    const cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)R, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * esz, (cuuint64_t)R * (cuuint64_t)ld * esz};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / esz), 32u, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = enc(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_INT32, 3, ptr, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

std::atomic<int> g_sm_margin{-1};
std::atomic<int> g_forward_sms{-1};
constexpr size_t kFlagBytes = 1u << 20;                 // tile counters of the forwarding CTAs: the last MiB of the workspace
thread_local int32_t g_last_path = 0;
thread_local int32_t g_last_variant = 0;

// CPMK_GEMM_VARIANT = auto (default) | 1cta | 2cta | generic; CPMK_FORCE_GENERIC_GEMM=1 is the same as "generic"
enum { kVariantAuto = 0, kVariantOneCta = 1, kVariantTwoCta = 2, kVariantGeneric = 3 };
int gemm_variant() {
    const char *e = getenv("CPMK_GEMM_VARIANT");
    if (e) {
        if (!strcmp(e, "1cta")) return kVariantOneCta;
        if (!strcmp(e, "2cta")) return kVariantTwoCta;
        if (!strcmp(e, "generic")) return kVariantGeneric;
    }
    const char *f = getenv("CPMK_FORCE_GENERIC_GEMM");
    if (f && f[0] && f[0] != '0') return kVariantGeneric;
    return kVariantAuto;
}

// Opt-in shared memory for the tensor-core kernels and the number of CTA pairs that can be resident at once
// (a persistent grid must not exceed it); once per device.
int g_max_pairs[64] = {0};
std::once_flag g_prepare_once[64];
cudaError_t g_prepare_err[64];

int32_t prepare_tc_kernels(int device) {
    const int dev = device & 63;
    std::call_once(g_prepare_once[dev], [dev] {
        cudaError_t e = cudaFuncSetAttribute(gemm_i8_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
#define CPMK_SET_TC2(D, P, Q) \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_tc2_kernel<D, P, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTc2SmemBytes)
        CPMK_SET_TC2(false, false, false); CPMK_SET_TC2(false, false, true); CPMK_SET_TC2(false, true, false); CPMK_SET_TC2(false, true, true);
        CPMK_SET_TC2(true, false, false); CPMK_SET_TC2(true, false, true); CPMK_SET_TC2(true, true, false); CPMK_SET_TC2(true, true, true);
#undef CPMK_SET_TC2
#define CPMK_SET_TC2E(P, Q) \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_tc2e_kernel<P, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTc2SmemBytes)
        CPMK_SET_TC2E(false, false); CPMK_SET_TC2E(false, true); CPMK_SET_TC2E(true, false); CPMK_SET_TC2E(true, true);
#undef CPMK_SET_TC2E
#define CPMK_SET_F16(P, Q) \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_f16_tc2_kernel<P, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTc2SmemBytes)
        CPMK_SET_F16(false, false); CPMK_SET_F16(false, true); CPMK_SET_F16(true, false); CPMK_SET_F16(true, true);
#undef CPMK_SET_F16
        g_prepare_err[dev] = e;
        if (e != cudaSuccess) return;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2, 1, 1);
        cfg.blockDim = dim3(kTcThreads2, 1, 1);
        cfg.dynamicSmemBytes = kTc2SmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_i8_tc2_kernel<true, false, false>, &cfg) == cudaSuccess && clusters > 0) {
            g_max_pairs[dev] = clusters;
        } else {
            // the query is advisory: a pair that is not resident at launch simply starts when a pair retires
            int sms = 0;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            g_max_pairs[dev] = sms / 2;
        }
        (void)cudaGetLastError();
    });
    if (g_prepare_err[dev] != cudaSuccess) {
        set_error("cudaFuncSetAttribute(max dynamic shared memory) failed: %s", cudaGetErrorString(g_prepare_err[dev]));
        return CPMK_ECUDA;
    }
    return CPMK_OK;
}

template <bool DEQUANT>
int32_t launch_gemm(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int aT, int bT, const void *A, const void *B,
                    const void *scale_x, const void *scale_y, int bx, int by, void *out, cudaStream_t stream, int n_dst = 1,
                    void *const *dsts = nullptr, int64_t dst_ld = 0, bool multicast = false) {
    // n_dst > 1 or dst_ld != m: the output tiles are scattered to several (possibly pitched) destinations; this is
    // implemented by the TMA-store epilogue of the two-CTA kernel only
    // multicast: dsts[1] is a multicast address (every GPU's copy of the buffer at once); it can only be written by the
    // forwarding CTAs' multimem stores
    const bool scatter = dsts != nullptr;
    if (!scatter) dst_ld = m;
    CPMK_REQUIRE(!multicast || (scatter && n_dst == 2), "a multicast destination needs exactly two destinations: the local buffer and the multicast address");
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    CPMK_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batchA >= 1 && batchB >= 1, "bad size: m=%d k=%d n=%d batchA=%d batchB=%d", m, k, n, batchA, batchB);
    // kernels/gemm.py:139-140
    CPMK_REQUIRE(m % 4 == 0 && n % 4 == 0 && k % 4 == 0, "m, n, k must be multiples of 4 (m=%d k=%d n=%d)", m, k, n);
    CPMK_REQUIRE(batchA == batchB || batchA == 1 || batchB == 1, "batch sizes must match or be 1 (batchA=%d batchB=%d)", batchA, batchB);
    const int32_t batch = batchA > batchB ? batchA : batchB;
    CPMK_REQUIRE(batch <= 65535, "batch %d exceeds 65535", batch);
    if (m == 0 || n == 0) return CPMK_OK;
    CPMK_REQUIRE(out || scatter, "null output pointer");
    if (scatter) {
        CPMK_REQUIRE(n_dst >= 1 && n_dst <= kMaxDst, "number of destinations must be 1..%d (got %d)", kMaxDst, n_dst);
        CPMK_REQUIRE(dst_ld >= m, "destination row pitch %lld is smaller than the row length %d", (long long)dst_ld, m);
        for (int d = 0; d < n_dst; ++d) CPMK_REQUIRE(dsts[d] && aligned16(dsts[d]), "destination %d is null or not 16-byte aligned", d);
        out = dsts[0];
    }
    const size_t out_elem = DEQUANT ? sizeof(__half) : sizeof(int32_t);
    if (k == 0) {
        CPMK_REQUIRE(!scatter, "k == 0 is not supported with scattered output");
        CPMK_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)batch * n * m * out_elem, stream));
        return CPMK_OK;
    }
    CPMK_REQUIRE(A && B, "null operand pointer");
    CPMK_REQUIRE((reinterpret_cast<uintptr_t>(A) & 3u) == 0 && (reinterpret_cast<uintptr_t>(B) & 3u) == 0, "operands must be 4-byte aligned");
    if (DEQUANT) CPMK_REQUIRE(scale_x && scale_y, "null scale pointer");

    // tensor-core paths.  Each operand is either k-major (k contiguous: aT for A, !bT for B) or MN-major; TMA needs
    // the contiguous extent to be a multiple of 16 bytes and 16-byte aligned base addresses.
    const int variant = gemm_variant();
    const bool q_mn = !aT, p_mn = bT;                       // column operand = A, row operand = B
    const bool strides_ok = (q_mn ? m % 16 == 0 : k % 16 == 0) && (p_mn ? n % 16 == 0 : k % 16 == 0);
    const bool tc_ok = variant != kVariantGeneric && strides_ok && aligned16(A) && aligned16(B) && aligned16(out) &&
                       (!DEQUANT || aligned16(scale_y)) && info.max_smem_optin >= kTcSmemBytes;
    if (tc_ok) {
        Workspace ws;
        rc = get_workspace(stream, &ws);
        if (rc) return rc;
        GemmParams prm;
        prm.R = n; prm.C = m; prm.K = k; prm.batch = batch;
        prm.p_batched = batchB > 1; prm.q_batched = batchA > 1;
        prm.num_kb = (k + kBK - 1) / kBK;
        prm.out = out;
        prm.scale_r = static_cast<const __half *>(scale_x); prm.scale_c = static_cast<const __half *>(scale_y);
        prm.bcast_r = bx; prm.bcast_c = by;
        prm.tma_store = 0;
        prm.send_pairs = 0;
        prm.flags = nullptr;
        prm.out_ld = 0;
        prm.multicast = 0;
        for (int d = 0; d < 8; ++d) prm.fwd_dst[d] = nullptr;
        prm.status = ws.status();
        rc = prepare_tc_kernels(info.device);
        if (rc) return rc;
        CUtensorMap tmap_p, tmap_q;
        // ---- two-CTA form: 256 x 256 tiles per CTA pair; worth it once there is more than one 128-row block ----
        // CPMK_GEMM_SM_MARGIN=n leaves n SMs free of the persistent GEMM grid, so that kernels of a concurrent stream
        // (the collective that gathers output slices across GPUs) find room to run beside it
        int max_pairs = g_max_pairs[info.device & 63];
        int margin = g_sm_margin.load(std::memory_order_relaxed);      // cpmk_set_gemm_sm_margin; negative: the environment
        if (margin < 0) {
            const char *mg = getenv("CPMK_GEMM_SM_MARGIN");
            margin = mg ? atoi(mg) : 0;
        }
        const int margin_pairs = (margin + 1) / 2;
        if (margin_pairs > 0 && max_pairs - margin_pairs >= 8) max_pairs -= margin_pairs;
        const bool any_mn = p_mn || q_mn;                   // MN-major operands are implemented in the two-CTA kernel only
        if ((variant != kVariantOneCta || scatter) && max_pairs > 0 && (n > kBM || variant == kVariantTwoCta || any_mn || scatter)) {
            const int64_t tiles_r = (n + 2 * kBM - 1) / (2 * kBM), tiles_c = (m + kBN - 1) / kBN;
            const int64_t total = tiles_r * tiles_c * batch;
            // rows of the output come from B (n x k), columns from A (m x k); each CTA stages 128 rows of either
            const bool enc_p = p_mn ? encode_operand_mn(&tmap_p, B, n, k, batchB) : encode_operand(&tmap_p, B, n, k, batchB, kBM);
            const bool enc_q = q_mn ? encode_operand_mn(&tmap_q, A, m, k, batchA) : encode_operand(&tmap_q, A, m, k, batchA, kHalfBN);
            if (total < (int64_t(1) << 31) && enc_p && enc_q) {
                prm.tiles_r = (int32_t)tiles_r; prm.tiles_c = (int32_t)tiles_c; prm.total_tiles = (int32_t)total;
                set_tile_divisors(&prm);
                // Several destinations: part of the grid can forward finished tiles from destination 0 to the others (see
                // forward_tiles).  CPMK_GEMM_FORWARD_SMS / cpmk_set_gemm_forward_sms: how many SMs do that (default 0: none,
                // every computing CTA stores to all destinations itself).
                int send_pairs = 0;
                if (scatter && n_dst > 1) {
                    int sms = g_forward_sms.load(std::memory_order_relaxed);
                    if (sms < 0) {
                        const char *fe = getenv("CPMK_GEMM_FORWARD_SMS");
                        sms = fe ? atoi(fe) : 0;
                    }
                    int want = (sms + 1) / 2;
                    if (multicast && want == 0) want = 8;               // a multicast address is only reachable through the forwarding CTAs
                    if (want > 0 && max_pairs - want >= 8 && (size_t)total * 2 * sizeof(uint32_t) <= kFlagBytes) send_pairs = want;
                    if (multicast && send_pairs == 0) {
                        set_error("the multicast form needs the forwarding CTAs (device too small or too many tiles: %lld)", (long long)total);
                        return CPMK_EINVAL;
                    }
                }
                const int compute_cap = max_pairs - send_pairs;
                const int pairs = (int)(total < compute_cap ? total : compute_cap);
                const dim3 grid(2 * (pairs + send_pairs));
                prm.send_pairs = send_pairs;
                prm.flags = nullptr;
                if (send_pairs > 0) {
                    for (int d = 0; d < kMaxDst; ++d) prm.fwd_dst[d] = d < n_dst ? static_cast<__half *>(dsts[d]) : nullptr;
                    prm.out_ld = dst_ld;
                    prm.multicast = multicast ? 1 : 0;
                    prm.flags = reinterpret_cast<uint32_t *>(ws.base + Workspace::kBytes - kFlagBytes);
                    CPMK_CUDA_TRY(cudaMemsetAsync(prm.flags, 0, (size_t)total * 2 * sizeof(uint32_t), stream));
                }
                OutMaps tmap_o;
                memset(&tmap_o, 0, sizeof(tmap_o));
                prm.n_dst = scatter ? n_dst : 1;
                prm.n_store = send_pairs > 0 ? 1 : prm.n_dst;
                prm.tma_store = (dst_ld * (DEQUANT ? 2 : 4)) % 16 == 0 && (scatter || !getenv("CPMK_GEMM_NO_TMA_STORE"));
                // (with forwarding CTAs only destination 0 is reached through a tensor map)
                for (int d = 0; prm.tma_store && d < (send_pairs > 0 ? 1 : prm.n_dst); ++d)
                    prm.tma_store = encode_output(&tmap_o.m[d], scatter ? dsts[d] : out, n, m, dst_ld, batch, DEQUANT);
                if (scatter && !prm.tma_store) {
                    set_error("scattered output needs a row pitch that is a multiple of 16 bytes and 16-byte aligned destinations");
                    return CPMK_EINVAL;
                }
                // short reductions are all epilogue: the form with two groups of epilogue warps (CPMK_GEMM_EPILOGUE_GROUPS=1: off)
                const char *eg = getenv("CPMK_GEMM_EPILOGUE_GROUPS");
                if (DEQUANT && prm.tma_store && !scatter && prm.num_kb <= 2 && !(eg && eg[0] == '1')) {
                    if (!p_mn && !q_mn) gemm_i8_tc2e_kernel<false, false><<<grid, kTcThreads2E, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                    else if (!p_mn && q_mn) gemm_i8_tc2e_kernel<false, true><<<grid, kTcThreads2E, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                    else if (p_mn && !q_mn) gemm_i8_tc2e_kernel<true, false><<<grid, kTcThreads2E, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                    else gemm_i8_tc2e_kernel<true, true><<<grid, kTcThreads2E, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                    CPMK_LAUNCH_CHECK();
                    g_last_path = 1;
                    g_last_variant = 2;
                    return CPMK_OK;
                }
                if (!p_mn && !q_mn) gemm_i8_tc2_kernel<DEQUANT, false, false><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                else if (!p_mn && q_mn) gemm_i8_tc2_kernel<DEQUANT, false, true><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                else if (p_mn && !q_mn) gemm_i8_tc2_kernel<DEQUANT, true, false><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                else gemm_i8_tc2_kernel<DEQUANT, true, true><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
                CPMK_LAUNCH_CHECK();
                g_last_path = 1;
                g_last_variant = 2;
                return CPMK_OK;
            }
        }
        if (scatter) {
            set_error("scattered output is only available on the two-CTA tensor-core kernel (shape m=%d k=%d n=%d not eligible)", m, k, n);
            return CPMK_EINVAL;
        }
        const int64_t tiles_r = (n + kBM - 1) / kBM, tiles_c = (m + kBN - 1) / kBN;
        const int64_t total_tiles = tiles_r * tiles_c * batch;
        if (!any_mn && variant != kVariantTwoCta && total_tiles < (int64_t(1) << 31) && encode_operand(&tmap_p, B, n, k, batchB, kBM) &&
            encode_operand(&tmap_q, A, m, k, batchA, kBN)) {
            prm.tiles_r = (int32_t)tiles_r; prm.tiles_c = (int32_t)tiles_c; prm.total_tiles = (int32_t)total_tiles;
            set_tile_divisors(&prm);
            const int grid = (int)(total_tiles < info.sm_count ? total_tiles : info.sm_count);
            gemm_i8_tc_kernel<DEQUANT><<<grid, kTcThreads, kTcSmemBytes, stream>>>(tmap_p, tmap_q, prm);
            CPMK_LAUNCH_CHECK();
            g_last_path = 1;
            g_last_variant = 1;
            return CPMK_OK;
        }
    }
    CPMK_REQUIRE(!scatter, "scattered output needs the tensor-core kernel: extents and pointers must be multiples of 16 bytes");
    const dim3 grid((m + kSimtTile - 1) / kSimtTile, (n + kSimtTile - 1) / kSimtTile, batch);
    CPMK_REQUIRE(grid.y <= 65535, "n = %d is too large for the generic kernel", n);
    gemm_i8_simt_kernel<DEQUANT><<<grid, 256, 0, stream>>>(m, k, n, batchA, batchB, aT, bT, static_cast<const int8_t *>(A),
                                                          static_cast<const int8_t *>(B), out, static_cast<const __half *>(scale_x),
                                                          static_cast<const __half *>(scale_y), bx, by);
    CPMK_LAUNCH_CHECK();
    g_last_path = 2;
    g_last_variant = 0;
    return CPMK_OK;
}

// ------------------------------------------------------------------------------------------------
// fp16 GEMM (the int8=False branch of bmm).  Generic kernel for shapes the tensor-core path does not take:
// 64 x 64 output tile per 256-thread block, 4 x 4 outputs per thread, k in chunks of 16, fp32 accumulation.
// ------------------------------------------------------------------------------------------------
constexpr int kF16SimtK = 16;

__global__ void __launch_bounds__(256) gemm_f16_simt_kernel(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int aT, int bT,
                                                            const __half *__restrict__ A, const __half *__restrict__ B, __half *__restrict__ out) {
    __shared__ float sa[kF16SimtK][kSimtTile + 1];    // [l][i]: columns of the output (from A)
    __shared__ float sb[kF16SimtK][kSimtTile + 1];    // [l][j]: rows of the output (from B)
    const int b = blockIdx.z;
    const int i0 = blockIdx.x * kSimtTile, j0 = blockIdx.y * kSimtTile;
    const __half *Ab = A + (batchA > 1 ? (int64_t)b * m * k : 0);
    const __half *Bb = B + (batchB > 1 ? (int64_t)b * n * k : 0);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int l0 = 0; l0 < k; l0 += kF16SimtK) {
        for (int e = threadIdx.x; e < kF16SimtK * kSimtTile; e += 256) {
            // A is (k, m) row-major, or (m, k) if aT: walk the contiguous axis with the fastest thread index
            const int l = aT ? e % kF16SimtK : e / kSimtTile, i = aT ? e / kF16SimtK : e % kSimtTile;
            const int gl = l0 + l, gi = i0 + i;
            sa[l][i] = (gl < k && gi < m) ? __half2float(aT ? Ab[(int64_t)gi * k + gl] : Ab[(int64_t)gl * m + gi]) : 0.f;
            // B is (n, k) row-major, or (k, n) if bT
            const int lb = bT ? e / kSimtTile : e % kF16SimtK, j = bT ? e % kSimtTile : e / kF16SimtK;
            const int glb = l0 + lb, gj = j0 + j;
            sb[lb][j] = (glb < k && gj < n) ? __half2float(bT ? Bb[(int64_t)glb * n + gj] : Bb[(int64_t)gj * k + glb]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < kF16SimtK; ++l) {
            float av[4], bv[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) av[x] = sa[l][tx + 16 * x];
#pragma unroll
            for (int y = 0; y < 4; ++y) bv[y] = sb[l][ty + 16 * y];
#pragma unroll
            for (int y = 0; y < 4; ++y)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[y][x] = fmaf(bv[y], av[x], acc[y][x]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int y = 0; y < 4; ++y) {
        const int j = j0 + ty + 16 * y;
        if (j >= n) continue;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = i0 + tx + 16 * x;
            if (i < m) out[((int64_t)b * n + j) * m + i] = __float2half_rn(acc[y][x]);
        }
    }
}

int32_t launch_gemm_f16(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int aT, int bT, const void *A, const void *B, void *out,
                        cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    CPMK_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batchA >= 1 && batchB >= 1, "bad size: m=%d k=%d n=%d batchA=%d batchB=%d", m, k, n, batchA, batchB);
    // kernels/gemm.py:200-201
    CPMK_REQUIRE(m % 2 == 0 && n % 2 == 0 && k % 2 == 0, "m, n, k must be even (m=%d k=%d n=%d)", m, k, n);
    CPMK_REQUIRE(batchA == batchB || batchA == 1 || batchB == 1, "batch sizes must match or be 1 (batchA=%d batchB=%d)", batchA, batchB);
    const int32_t batch = batchA > batchB ? batchA : batchB;
    CPMK_REQUIRE(batch <= 65535, "batch %d exceeds 65535", batch);
    if (m == 0 || n == 0) return CPMK_OK;
    CPMK_REQUIRE(out, "null output pointer");
    if (k == 0) {
        CPMK_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)batch * n * m * sizeof(__half), stream));
        return CPMK_OK;
    }
    CPMK_REQUIRE(A && B, "null operand pointer");
    CPMK_REQUIRE((reinterpret_cast<uintptr_t>(A) & 1u) == 0 && (reinterpret_cast<uintptr_t>(B) & 1u) == 0 && (reinterpret_cast<uintptr_t>(out) & 1u) == 0,
                 "operands must be 2-byte aligned");

    // tensor-core path: contiguous extents and the output's rows multiples of 16 bytes, 16-byte aligned pointers
    const int variant = gemm_variant();
    const bool q_mn = !aT, p_mn = bT;
    const bool strides_ok = (q_mn ? m % 8 == 0 : k % 8 == 0) && (p_mn ? n % 8 == 0 : k % 8 == 0) && m % 8 == 0;
    int max_pairs = 0;
    if (variant != kVariantGeneric && strides_ok && aligned16(A) && aligned16(B) && aligned16(out) && info.max_smem_optin >= kTc2SmemBytes) {
        Workspace ws;
        rc = get_workspace(stream, &ws);
        if (rc) return rc;
        rc = prepare_tc_kernels(info.device);
        if (rc) return rc;
        max_pairs = g_max_pairs[info.device & 63];
        const int64_t tiles_r = (n + 2 * kBM - 1) / (2 * kBM), tiles_c = (m + kBN - 1) / kBN;
        const int64_t total = tiles_r * tiles_c * batch;
        CUtensorMap tmap_p, tmap_q;
        OutMaps tmap_o;
        memset(&tmap_o, 0, sizeof(tmap_o));
        const bool enc_p = p_mn ? encode_operand_mn(&tmap_p, B, n, k, batchB, 2) : encode_operand(&tmap_p, B, n, k, batchB, kBM, 2);
        const bool enc_q = q_mn ? encode_operand_mn(&tmap_q, A, m, k, batchA, 2) : encode_operand(&tmap_q, A, m, k, batchA, kHalfBN, 2);
        if (max_pairs > 0 && total < (int64_t(1) << 31) && enc_p && enc_q && encode_output(&tmap_o.m[0], out, n, m, m, batch, true)) {
            GemmParams prm;
            memset(&prm, 0, sizeof(prm));
            prm.R = n; prm.C = m; prm.K = k; prm.batch = batch;
            prm.p_batched = batchB > 1; prm.q_batched = batchA > 1;
            prm.num_kb = (k + kBKf16 - 1) / kBKf16;
            prm.out = out;
            prm.tma_store = 1;
            prm.n_dst = 1;
            prm.n_store = 1;
            prm.status = ws.status();
            prm.tiles_r = (int32_t)tiles_r; prm.tiles_c = (int32_t)tiles_c; prm.total_tiles = (int32_t)total;
            set_tile_divisors(&prm);
            const int pairs = (int)(total < max_pairs ? total : max_pairs);
            const dim3 grid(2 * pairs);
            if (!p_mn && !q_mn) gemm_f16_tc2_kernel<false, false><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
            else if (!p_mn && q_mn) gemm_f16_tc2_kernel<false, true><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
            else if (p_mn && !q_mn) gemm_f16_tc2_kernel<true, false><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
            else gemm_f16_tc2_kernel<true, true><<<grid, kTcThreads2, kTc2SmemBytes, stream>>>(tmap_p, tmap_q, tmap_o, prm);
            CPMK_LAUNCH_CHECK();
            g_last_path = 1;
            g_last_variant = 2;
            return CPMK_OK;
        }
    }
    const dim3 grid((m + kSimtTile - 1) / kSimtTile, (n + kSimtTile - 1) / kSimtTile, batch);
    CPMK_REQUIRE(grid.y <= 65535, "n = %d is too large for the generic kernel", n);
    gemm_f16_simt_kernel<<<grid, 256, 0, stream>>>(m, k, n, batchA, batchB, aT, bT, static_cast<const __half *>(A), static_cast<const __half *>(B),
                                                   static_cast<__half *>(out));
    CPMK_LAUNCH_CHECK();
    g_last_path = 2;
    g_last_variant = 0;
    return CPMK_OK;
}

}  // namespace
}  // namespace cpmk

using namespace cpmk;

extern "C" {

int32_t cpmk_gemm_int8(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT, const void *A, const void *B,
                       void *out, cpmk_stream_t stream) {
    return launch_gemm<false>(m, k, n, batchA, batchB, aT != 0, bT != 0, A, B, nullptr, nullptr, 0, 0, out, as_stream(stream));
}

int32_t cpmk_gemm_int8_dequant(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT, const void *A,
                               const void *B, const void *scale_x, const void *scale_y, int32_t broad_cast_x, int32_t broad_cast_y, void *out,
                               cpmk_stream_t stream) {
    return launch_gemm<true>(m, k, n, batchA, batchB, aT != 0, bT != 0, A, B, scale_x, scale_y, broad_cast_x != 0, broad_cast_y != 0, out,
                             as_stream(stream));
}

int32_t cpmk_gemm_int8_dequant_scatter(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT, const void *A,
                                       const void *B, const void *scale_x, const void *scale_y, int32_t broad_cast_x, int32_t broad_cast_y,
                                       int32_t n_dst, void *const *dst, int64_t dst_row_pitch, cpmk_stream_t stream) {
    if (!dst) {
        set_error("dst is null");
        return CPMK_EINVAL;
    }
    return launch_gemm<true>(m, k, n, batchA, batchB, aT != 0, bT != 0, A, B, scale_x, scale_y, broad_cast_x != 0, broad_cast_y != 0, nullptr,
                             as_stream(stream), n_dst, dst, dst_row_pitch);
}

int32_t cpmk_gemm_int8_dequant_multicast(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT, const void *A,
                                         const void *B, const void *scale_x, const void *scale_y, int32_t broad_cast_x, int32_t broad_cast_y,
                                         void *dst_local, void *dst_multicast, int64_t dst_row_pitch, cpmk_stream_t stream) {
    void *dst[2] = {dst_local, dst_multicast};
    return launch_gemm<true>(m, k, n, batchA, batchB, aT != 0, bT != 0, A, B, scale_x, scale_y, broad_cast_x != 0, broad_cast_y != 0, nullptr,
                             as_stream(stream), 2, dst, dst_row_pitch, true);
}

int32_t cpmk_gemm_int8_dequant_gelu(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT, const void *A,
                                    const void *B, const void *scale_x, const void *scale_y, int32_t broad_cast_x, int32_t broad_cast_y, void *out,
                                    cpmk_stream_t stream) {
    const int32_t rc = launch_gemm<true>(m, k, n, batchA, batchB, aT != 0, bT != 0, A, B, scale_x, scale_y, broad_cast_x != 0, broad_cast_y != 0,
                                         out, as_stream(stream));
    if (rc != CPMK_OK) return rc;
    // The activation runs as a second kernel over the result while most of it is still in L2.  Applying it inside the
    // GEMM's epilogue was measured slower (182 us against 114 + 28 us on the 4096 x 10240 x 4096 feed-forward shape):
    // the exact expression costs ~45 instructions per element, more than the epilogue warps can hide behind the main
    // loop, and the 128 KiB table that makes the separate kernel cheap does not fit beside the GEMM's stages.
    const int64_t batch = batchA > batchB ? batchA : batchB;
    return launch_gelu(batch * n * m, out, out, as_stream(stream));
}

int32_t cpmk_gemm_fp16(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT, const void *A, const void *B,
                       void *out, cpmk_stream_t stream) {
    return launch_gemm_f16(m, k, n, batchA, batchB, aT != 0, bT != 0, A, B, out, as_stream(stream));
}

int32_t cpmk_set_gemm_sm_margin(int32_t sms) {
    g_sm_margin.store(sms < 0 ? -1 : sms, std::memory_order_relaxed);
    return CPMK_OK;
}

int32_t cpmk_set_gemm_forward_sms(int32_t sms) {
    g_forward_sms.store(sms < 0 ? -1 : sms, std::memory_order_relaxed);
    return CPMK_OK;
}

int32_t cpmk_last_gemm_path(void) { return g_last_path; }

int32_t cpmk_last_gemm_variant(void) { return g_last_path == 1 ? g_last_variant : 0; }

}  // extern "C"
