// Self-test of the give-up path that every device-side wait of this library shares (mbar_wait, cpmk_ptx.cuh): a
// one-block kernel waits, with a short limit, on a barrier on which nothing ever arrives.  The wait must run out, the
// kernel must record its code in the stream's status word and return normally, and the context must stay usable.
// No fault, trap or unbounded loop is involved: the only thing that happens is that a bounded wait ends.
#include "cpmk_common.cuh"
#include "cpmk_ptx.cuh"

namespace cpmk {
namespace {

constexpr uint32_t kErrSelfTestWait = 0x901;

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(uint64_t limit_ns, uint32_t *status, uint32_t *result) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_word = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        // phase 0 of a barrier that expects one arrival and gets none: the wait can only end by running out
        const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_word, status, kErrSelfTestWait, limit_ns);
        // 1: the wait gave up and raised the abort flag (expected); 2: it returned true (a bug); 3: gave up without the flag
        *result = ok ? 2u : (abort_word ? 1u : 3u);
    }
}

}  // namespace
}  // namespace cpmk

using namespace cpmk;

extern "C" int32_t cpmk_selftest_bounded_wait(uint32_t limit_us, cpmk_stream_t stream) {
    DeviceInfo info;
    int32_t rc = current_device_info(&info);
    if (rc) return rc;
    CPMK_REQUIRE(limit_us >= 1 && limit_us <= 100000, "limit_us must be 1..100000 (got %u)", limit_us);
    cudaStream_t st = as_stream(stream);
    Workspace ws;
    rc = get_workspace(st, &ws);
    if (rc) return rc;
    // the kernel's own verdict goes to the second status word (the first one is the failure code that cpmk_check_stream reports)
    uint32_t *result = ws.status() + 1;
    CPMK_CUDA_TRY(cudaMemsetAsync(result, 0, sizeof(uint32_t), st));
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>((uint64_t)limit_us * 1000ull, ws.status(), result);
    CPMK_LAUNCH_CHECK();
    uint32_t verdict = 0;
    CPMK_CUDA_TRY(cudaMemcpyAsync(&verdict, result, sizeof(verdict), cudaMemcpyDeviceToHost, st));
    CPMK_CUDA_TRY(cudaStreamSynchronize(st));
    if (verdict != 1u) {
        set_error("bounded-wait self-test: the kernel reported %u (1 = the wait ran out as it should)", verdict);
        return CPMK_EDEVICE;
    }
    return CPMK_OK;
}
