// Element-wise GELU on fp16 for sm_100a: the activation between the two feed-forward linears, the step right
// after the int8 linear's dequantisation.  Replaces cuda/gelu.cu:6-17 (one 2-byte load, ~45 instructions of mixed
// binary64 / binary32 arithmetic and one 2-byte store per element, which is issue-bound far below HBM rate).
//
// GELU maps one fp16 value to one fp16 value, so large inputs go through a table of all 65536 results: the table is
// filled once per device by evaluating the reference expression on the device, copied into 128 KiB of shared memory
// by every block, and each element costs one shared-memory lookup between a 128-bit load and a 128-bit store.
// Small inputs evaluate the expression directly.
#include <mutex>

#include "cpmk_common.cuh"
#include "cpmk_gelu_device.cuh"

namespace cpmk {
namespace {

constexpr int kTableEntries = 65536;
constexpr int kTableBytes = kTableEntries * 2;
constexpr int kLutThreads = 1024;
constexpr int64_t kLutMinElements = int64_t(1) << 21;     // below this the table load per block outweighs the arithmetic

// All 65536 results; static storage in the library image (no allocation), filled by gelu_table_kernel.
__device__ __align__(16) __half g_gelu_table[kTableEntries];

__global__ void __launch_bounds__(256) gelu_table_kernel(__half *table) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < kTableEntries) table[i] = gelu_half(__ushort_as_half((unsigned short)i));
}

__global__ void __launch_bounds__(256) gelu_direct_kernel(int64_t count, const __half *__restrict__ in, __half *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (int64_t)gridDim.x * 256) out[i] = gelu_half(in[i]);
}

// grad[i] = gelu'(mat[i]) * grad_out[i]; eight elements per thread and step where the pointers allow 128-bit accesses
__global__ void __launch_bounds__(256) gelu_backward_kernel(int64_t count, int vec_ok, const __half *__restrict__ grad_out, const __half *__restrict__ mat,
                                                            __half *__restrict__ grad) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t nvec = count >> 3;
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nvec; i += stride) {
            const uint4 g = __ldcs(reinterpret_cast<const uint4 *>(grad_out) + i), x = __ldcs(reinterpret_cast<const uint4 *>(mat) + i);
            const __half *gh = reinterpret_cast<const __half *>(&g), *xh = reinterpret_cast<const __half *>(&x);
            __align__(16) __half o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = gelu_backward_half(gh[j], xh[j]);
            __stcs(reinterpret_cast<uint4 *>(grad) + i, *reinterpret_cast<const uint4 *>(o));
        }
        done = nvec << 3;
    }
    for (int64_t i = done + (int64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += stride) grad[i] = gelu_backward_half(grad_out[i], mat[i]);
}

// in == out is allowed (each element is read before it is written, by the same thread)
__global__ void __launch_bounds__(kLutThreads, 1) gelu_lut_kernel(int64_t count, const __half *in, __half *out, const __half *__restrict__ table) {
    extern __shared__ __align__(16) unsigned short lut[];
    for (int i = threadIdx.x; i < kTableBytes / 16; i += kLutThreads)
        reinterpret_cast<uint4 *>(lut)[i] = __ldg(reinterpret_cast<const uint4 *>(table) + i);
    __syncthreads();
    const int64_t nvec = count >> 3;
    const int64_t stride = (int64_t)gridDim.x * kLutThreads;
    constexpr int kUnroll = 4;                                  // 128-bit loads in flight per thread
    for (int64_t v0 = (int64_t)blockIdx.x * kLutThreads + threadIdx.x; v0 < nvec; v0 += stride * kUnroll) {
        uint4 x[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (v0 + u * stride < nvec) x[u] = __ldcs(reinterpret_cast<const uint4 *>(in) + v0 + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (v0 + u * stride >= nvec) break;
            const uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = (uint32_t)lut[w[j] & 0xffffu] | ((uint32_t)lut[w[j] >> 16] << 16);
            __stcs(reinterpret_cast<uint4 *>(out) + v0 + u * stride, make_uint4(o[0], o[1], o[2], o[3]));
        }
    }
    if (blockIdx.x == 0) {
        for (int64_t i = (nvec << 3) + threadIdx.x; i < count; i += kLutThreads)
            reinterpret_cast<unsigned short *>(out)[i] = lut[reinterpret_cast<const unsigned short *>(in)[i]];
    }
}

struct TableState {
    std::once_flag once;
    cudaError_t err = cudaSuccess;
    __half *table = nullptr;
    cudaEvent_t filled = nullptr;
    bool known_complete = false;
};
TableState g_table_state[64];
std::mutex g_table_mutex;

// The device address of the table of the current device; fills it on first use (on `stream`) and makes `stream`
// wait for the fill if it is still in flight on another stream.
int32_t gelu_table(int device, cudaStream_t stream, const __half **table_out) {
    TableState &st = g_table_state[device & 63];
    std::call_once(st.once, [&] {
        void *p = nullptr;
        st.err = cudaGetSymbolAddress(&p, g_gelu_table);
        if (st.err != cudaSuccess) return;
        st.table = static_cast<__half *>(p);
        st.err = cudaFuncSetAttribute(gelu_lut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTableBytes);
        if (st.err != cudaSuccess) return;
        st.err = cudaEventCreateWithFlags(&st.filled, cudaEventDisableTiming);
        if (st.err != cudaSuccess) return;
        gelu_table_kernel<<<kTableEntries / 256, 256, 0, stream>>>(st.table);
        st.err = cudaGetLastError();
        if (st.err == cudaSuccess) st.err = cudaEventRecord(st.filled, stream);
    });
    if (st.err != cudaSuccess) {
        set_error("setting up the GELU table failed: %s", cudaGetErrorString(st.err));
        return CPMK_ECUDA;
    }
    {
        std::lock_guard<std::mutex> lock(g_table_mutex);
        if (!st.known_complete) {
            if (cudaEventQuery(st.filled) == cudaSuccess) st.known_complete = true;
            else {
                (void)cudaGetLastError();
                CPMK_CUDA_TRY(cudaStreamWaitEvent(stream, st.filled, 0));
            }
        }
    }
    *table_out = st.table;
    return CPMK_OK;
}

}  // namespace

int32_t launch_gelu(int64_t count, const void *in, void *out, cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    if (count == 0) return CPMK_OK;
    CPMK_REQUIRE(in && out, "null pointer");
    CPMK_REQUIRE((reinterpret_cast<uintptr_t>(in) & 1u) == 0 && (reinterpret_cast<uintptr_t>(out) & 1u) == 0, "pointers must be 2-byte aligned");
    if (count >= kLutMinElements && aligned16(in) && aligned16(out) && info.max_smem_optin >= kTableBytes) {
        const __half *table = nullptr;
        rc = gelu_table(info.device, stream, &table);
        if (rc) return rc;
        gelu_lut_kernel<<<info.sm_count, kLutThreads, kTableBytes, stream>>>(count, static_cast<const __half *>(in), static_cast<__half *>(out), table);
        CPMK_LAUNCH_CHECK();
        return CPMK_OK;
    }
    const int64_t blocks = ceil_div64(count, 256);
    const int grid = (int)(blocks < (int64_t)info.sm_count * 16 ? blocks : (int64_t)info.sm_count * 16);
    gelu_direct_kernel<<<grid, 256, 0, stream>>>(count, static_cast<const __half *>(in), static_cast<__half *>(out));
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

int32_t launch_gelu_backward(int64_t count, const void *grad_out, const void *mat, void *grad, cudaStream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    if (count == 0) return CPMK_OK;
    CPMK_REQUIRE(grad_out && mat && grad, "null pointer");
    CPMK_REQUIRE(((reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(mat) | reinterpret_cast<uintptr_t>(grad)) & 1u) == 0,
                 "pointers must be 2-byte aligned");
    const int vec_ok = aligned16(grad_out) && aligned16(mat) && aligned16(grad);
    const int64_t blocks = ceil_div64(vec_ok ? (count + 7) / 8 : count, 256);
    const int grid = (int)(blocks < (int64_t)info.sm_count * 16 ? blocks : (int64_t)info.sm_count * 16);
    gelu_backward_kernel<<<grid, 256, 0, stream>>>(count, vec_ok, static_cast<const __half *>(grad_out), static_cast<const __half *>(mat),
                                                   static_cast<__half *>(grad));
    CPMK_LAUNCH_CHECK();
    return CPMK_OK;
}

}  // namespace cpmk

using namespace cpmk;

extern "C" int32_t cpmk_gelu_backward(int32_t batch, int32_t n, const void *grad_out, const void *mat, void *grad, cpmk_stream_t stream) {
    CPMK_REQUIRE(batch >= 0 && n >= 0, "negative size: batch=%d n=%d", batch, n);
    return launch_gelu_backward((int64_t)batch * n, grad_out, mat, grad, as_stream(stream));
}

extern "C" int32_t cpmk_gelu_forward(int32_t batch, int32_t n, const void *mat, void *out, cpmk_stream_t stream) {
    CPMK_REQUIRE(batch >= 0 && n >= 0, "negative size: batch=%d n=%d", batch, n);
    return launch_gelu((int64_t)batch * n, mat, out, as_stream(stream));
}
