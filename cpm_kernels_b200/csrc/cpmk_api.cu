// Host-side plumbing of the cpmk_b200 C-ABI library: thread-local error text, per-device
// capability check and the (device, stream)-keyed workspace.
#include <cuda.h>
#include <stdarg.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "cpmk_common.cuh"

namespace cpmk {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

static std::mutex g_mutex;
static std::map<int, DeviceInfo> g_devices;
static std::map<std::pair<int, cudaStream_t>, Workspace> g_workspaces;

int32_t current_device_info(DeviceInfo *info) {
    int dev = 0;
    CPMK_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_devices.find(dev);
    if (it == g_devices.end()) {
        DeviceInfo d;
        d.device = dev;
        int major = 0, minor = 0;
        CPMK_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        CPMK_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
        CPMK_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        CPMK_CUDA_TRY(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        d.arch = major * 10 + minor;
        it = g_devices.emplace(dev, d).first;
    }
    *info = it->second;
    if (info->arch / 10 != 10) {
        set_error("cpmk_b200 kernels are built for sm_100a only; device %d is compute capability %d.%d",
                  dev, info->arch / 10, info->arch % 10);
        return CPMK_EARCH;
    }
    return CPMK_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool encode_tiled_3d(void *map_out, int esz, const void *ptr, const uint64_t dims[3], const uint64_t strides[2], const uint32_t box[3], bool swizzle128) {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        (void)cudaGetLastError();
    });
    if (!fn) return false;
    const cuuint64_t d[3] = {dims[0], dims[1], dims[2]};
    const cuuint64_t st[2] = {strides[0], strides[1]};
    const cuuint32_t bx[3] = {box[0], box[1], box[2]};
    const cuuint32_t es[3] = {1u, 1u, 1u};
    const CUtensorMapDataType dt = esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : (esz == 4 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
    return fn(static_cast<CUtensorMap *>(map_out), dt, 3, const_cast<void *>(ptr), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// At most this many (stream) workspaces per device; a slot is given back with cpmk_release_workspace.
constexpr size_t kMaxWorkspacesPerDevice = 256;

int32_t get_workspace(cudaStream_t stream, Workspace *ws) {
    int dev = 0;
    CPMK_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mutex);
    auto key = std::make_pair(dev, stream);
    auto it = g_workspaces.find(key);
    if (it == g_workspaces.end()) {
        size_t on_device = 0;
        for (auto &kv : g_workspaces) on_device += kv.first.first == dev ? 1 : 0;
        if (on_device >= kMaxWorkspacesPerDevice) {
            set_error("more than %zu streams of device %d asked for a cpmk workspace; release those of destroyed streams with "
                      "cpmk_release_workspace", kMaxWorkspacesPerDevice, dev);
            return CPMK_ENOMEM;
        }
        Workspace w;
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, Workspace::kBytes);
        if (e != cudaSuccess) {
            set_error("workspace allocation of %zu bytes failed: %s", Workspace::kBytes, cudaGetErrorString(e));
            return CPMK_ENOMEM;
        }
        w.base = static_cast<char *>(p);
        // status words and tickets start at zero; kernels leave the tickets at zero when they finish
        CPMK_CUDA_TRY(cudaMemset(w.base, 0, Workspace::kScratchOffset));
        it = g_workspaces.emplace(key, w).first;
    }
    *ws = it->second;
    return CPMK_OK;
}

// Reads the status word of one workspace; when a kernel recorded a failure there, clears the word AND the ticket
// region: a kernel that gave up a wait leaves without taking its ticket, so the counters it shares with later calls
// are no longer at zero.  The caller holds g_mutex and has synchronised the work that uses the workspace.
static int32_t collect_status(const Workspace &w, uint32_t *word_out) {
    uint32_t word = 0;
    CPMK_CUDA_TRY(cudaMemcpy(&word, w.status(), sizeof(word), cudaMemcpyDeviceToHost));
    if (word != 0) CPMK_CUDA_TRY(cudaMemset(w.base, 0, Workspace::kScratchOffset));
    *word_out = word;
    return CPMK_OK;
}

}  // namespace cpmk

extern "C" {

int32_t cpmk_abi_version(void) { return CPMK_ABI_VERSION; }

const char *cpmk_last_error(void) { return cpmk::g_error; }

int32_t cpmk_check_device(int32_t *arch_out) {
    cpmk::DeviceInfo info;
    int32_t rc = cpmk::current_device_info(&info);
    if (arch_out) *arch_out = info.arch;
    return rc;
}

int32_t cpmk_read_status(uint32_t *status_out) {
    if (!status_out) {
        cpmk::set_error("status_out is null");
        return CPMK_EINVAL;
    }
    int dev = 0;
    CPMK_CUDA_TRY(cudaGetDevice(&dev));
    CPMK_CUDA_TRY(cudaDeviceSynchronize());
    uint32_t worst = 0;
    std::lock_guard<std::mutex> lock(cpmk::g_mutex);
    for (auto &kv : cpmk::g_workspaces) {
        if (kv.first.first != dev) continue;
        uint32_t word = 0;
        const int32_t rc = cpmk::collect_status(kv.second, &word);
        if (rc) return rc;
        if (word != 0 && worst == 0) worst = word;
    }
    *status_out = worst;
    return CPMK_OK;
}

int32_t cpmk_check_stream(cpmk_stream_t stream) {
    int dev = 0;
    CPMK_CUDA_TRY(cudaGetDevice(&dev));
    CPMK_CUDA_TRY(cudaStreamSynchronize(cpmk::as_stream(stream)));
    std::lock_guard<std::mutex> lock(cpmk::g_mutex);
    auto it = cpmk::g_workspaces.find(std::make_pair(dev, cpmk::as_stream(stream)));
    if (it == cpmk::g_workspaces.end()) return CPMK_OK;          // no kernel with a bounded wait ran on this stream
    uint32_t word = 0;
    const int32_t rc = cpmk::collect_status(it->second, &word);
    if (rc) return rc;
    if (word != 0) {
        cpmk::set_error("a kernel on this stream gave up a bounded wait (code 0x%x); its output is incomplete", word);
        return CPMK_EDEVICE;
    }
    return CPMK_OK;
}

int32_t cpmk_release_workspace(cpmk_stream_t stream) {
    int dev = 0;
    CPMK_CUDA_TRY(cudaGetDevice(&dev));
    cpmk::Workspace w;
    {
        std::lock_guard<std::mutex> lock(cpmk::g_mutex);
        auto it = cpmk::g_workspaces.find(std::make_pair(dev, cpmk::as_stream(stream)));
        if (it == cpmk::g_workspaces.end()) return CPMK_OK;
        w = it->second;
        cpmk::g_workspaces.erase(it);
    }
    CPMK_CUDA_TRY(cudaFree(w.base));                             // waits for the device to finish with the memory
    return CPMK_OK;
}

}  // extern "C"
