// Batched fp16 matrix transpose for sm_100a: out[b, c, r] = in[b, r, c], the step between the (batch, hidden, seq)
// activations of the layer-norm / attention kernels and a token-major (batch, seq, hidden) consumer.  Replaces
// cuda/transpose.cu:6-22 (32 x 32 tiles, one 2-byte load and one 2-byte store per thread, grid.y/z limited to 65535
// tiles).  Pure data movement: 2 bytes read + 2 bytes written per element, bound by HBM.
//
// transpose_tile64_kernel: 64 x 64 tiles, 256 threads.  A thread loads 16 bytes from each of two neighbouring rows,
// interleaves them into eight 32-bit words (two rows of one column = two neighbouring elements of an output row) and
// stores them into a 64 x 32-word tile of shared memory whose 16-byte groups are XOR-swizzled by the output row, so
// that the word stores and the 16-byte loads of the second phase are both free of bank conflicts; each thread then
// writes two 16-byte pieces of output rows.  Needs n and m multiples of 8 and 16-byte aligned pointers.
// transpose_generic_kernel: 32 x 32 tiles with 2-byte accesses for every other size.
#include "cpmk_common.cuh"

namespace cpmk {
namespace {

constexpr int kTile = 64;
constexpr int kTileThreads = 256;

__global__ void __launch_bounds__(kTileThreads) transpose_tile64_kernel(int32_t batch, int32_t n, int32_t m, int32_t tiles_r, int32_t tiles_c,
                                                                       int64_t total_tiles, const __half *__restrict__ in,
                                                                       __half *__restrict__ out) {
    __shared__ __align__(16) uint32_t tile[kTile * 32];        // [output row 0..63][32 words], 16-byte groups swizzled
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // load phase: column vector cv (8 columns) of row pair rp (rows 2rp, 2rp+1)
    const int cv = (lane & 3) + 4 * (warp & 1);
    const int rp = (lane >> 2) + 8 * (warp >> 1);
    // store phase: 16-byte group sq of output rows so and so + 32
    const int so = tid >> 3, sq = tid & 7;
    const int64_t plane = (int64_t)n * m;
    const int32_t per_batch = tiles_r * tiles_c;

    for (int64_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const int32_t b = (int32_t)(t / per_batch);
        const int32_t rest = (int32_t)(t - (int64_t)b * per_batch);
        const int32_t tr = rest / tiles_c, tc = rest - tr * tiles_c;
        const int32_t r0 = tr * kTile, c0 = tc * kTile;
        const __half *src = in + (int64_t)b * plane;
        __half *dst = out + (int64_t)b * plane;

        const int32_t r = r0 + 2 * rp, c = c0 + 8 * cv;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (r < n && c < m) {                                   // n is even: rows r and r + 1 exist together
            lo = __ldcs(reinterpret_cast<const uint4 *>(src + (int64_t)r * m + c));
            hi = __ldcs(reinterpret_cast<const uint4 *>(src + (int64_t)(r + 1) * m + c));
        }
        const uint32_t a[4] = {lo.x, lo.y, lo.z, lo.w}, d[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o0 = 8 * cv + 2 * j;                      // output rows o0, o0 + 1 of the tile
            const int grp = (rp >> 2) ^ (2 * (cv & 3));         // swizzle depends on (output row >> 3) only
            tile[o0 * 32 + grp * 4 + (rp & 3)] = __byte_perm(a[j], d[j], 0x5410);
            tile[(o0 + 1) * 32 + grp * 4 + (rp & 3)] = __byte_perm(a[j], d[j], 0x7632);
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int o = so + 32 * h;
            const int32_t orow = c0 + o, ocol = r0 + 8 * sq;
            if (orow < m && ocol < n) {
                const int grp = sq ^ (2 * ((o >> 3) & 3));
                const uint4 v = *reinterpret_cast<const uint4 *>(&tile[o * 32 + grp * 4]);
                __stcs(reinterpret_cast<uint4 *>(dst + (int64_t)orow * n + ocol), v);
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) transpose_generic_kernel(int32_t batch, int32_t n, int32_t m, int32_t tiles_r, int32_t tiles_c,
                                                                int64_t total_tiles, const __half *__restrict__ in,
                                                                __half *__restrict__ out) {
    __shared__ unsigned short tile[32 * 33];
    const int x = threadIdx.x & 31, y0 = threadIdx.x >> 5;    // 8 warps: each covers rows y0, y0 + 8, ...
    const int64_t plane = (int64_t)n * m;
    const int32_t per_batch = tiles_r * tiles_c;
    const unsigned short *src_all = reinterpret_cast<const unsigned short *>(in);
    unsigned short *dst_all = reinterpret_cast<unsigned short *>(out);
    for (int64_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const int32_t b = (int32_t)(t / per_batch);
        const int32_t rest = (int32_t)(t - (int64_t)b * per_batch);
        const int32_t tr = rest / tiles_c, tc = rest - tr * tiles_c;
        const int32_t r0 = tr * 32, c0 = tc * 32;
        const unsigned short *src = src_all + (int64_t)b * plane;
        unsigned short *dst = dst_all + (int64_t)b * plane;
#pragma unroll
        for (int y = y0; y < 32; y += 8)
            if (r0 + y < n && c0 + x < m) tile[y * 33 + x] = src[(int64_t)(r0 + y) * m + c0 + x];
        __syncthreads();
#pragma unroll
        for (int y = y0; y < 32; y += 8)
            if (c0 + y < m && r0 + x < n) dst[(int64_t)(c0 + y) * n + r0 + x] = tile[x * 33 + y];
        __syncthreads();
    }
}

int32_t launch_transpose(int32_t batch, int32_t n, int32_t m, const void *in, void *out, cudaStream_t stream) {
    DeviceInfo info;
    const int32_t rc = current_device_info(&info);
    if (rc) return rc;
    if (batch == 0 || n == 0 || m == 0) return CPMK_OK;
    CPMK_REQUIRE(in && out, "null pointer");
    CPMK_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 1u) == 0, "pointers must be 2-byte aligned");
    const bool fast = (n % 8 == 0) && (m % 8 == 0) && aligned16(in) && aligned16(out);
    const int edge = fast ? kTile : 32;
    const int32_t tiles_r = (n + edge - 1) / edge, tiles_c = (m + edge - 1) / edge;
    const int64_t total = (int64_t)batch * tiles_r * tiles_c;
    const int64_t cap = (int64_t)info.sm_count * 32;       // blocks beyond this walk the tiles in a grid-stride loop
    const unsigned grid = (unsigned)(total < cap ? total : cap);
    if (fast)
        transpose_tile64_kernel<<<grid, kTileThreads, 0, stream>>>(batch, n, m, tiles_r, tiles_c, total, static_cast<const __half *>(in),
                                                                  static_cast<__half *>(out));
    else
        transpose_generic_kernel<<<grid, 256, 0, stream>>>(batch, n, m, tiles_r, tiles_c, total, static_cast<const __half *>(in),
                                                           static_cast<__half *>(out));
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

}  // namespace
}  // namespace cpmk

using namespace cpmk;

extern "C" int32_t cpmk_transpose(int32_t batch, int32_t n, int32_t m, const void *in, void *out, cpmk_stream_t stream) {
    CPMK_REQUIRE(batch >= 0 && n >= 0 && m >= 0, "negative size: batch=%d n=%d m=%d", batch, n, m);
    CPMK_REQUIRE(in != out || (int64_t)batch * n * m == 0, "transpose cannot run in place");
    return launch_transpose(batch, n, m, in, out, as_stream(stream));
}
