#include "host_util.h"
#include "nccl_dyn.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace efa {

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

const char* last_error() { return g_err; }

int check_cuda(cudaError_t e, const char* what, const char* file, int line)
{
    if (e == cudaSuccess) return 0;
    set_error("CUDA error %s:%d: %s: %s", file, line, what, cudaGetErrorString(e));
    return 1;
}

int check_cu(CUresult r, const char* what, const char* file, int line)
{
    if (r == CUDA_SUCCESS) return 0;
    const char* msg = nullptr;
    const DriverApi* api = driver_api();
    if (api && api->cuGetErrorString) api->cuGetErrorString(r, &msg);
    set_error("CUDA driver error %s:%d: %s: %s", file, line, what, msg ? msg : "?");
    return 1;
}

static int resolve(const char* name, void** fn)
{
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || *fn == nullptr) {
        set_error("driver entry point %s not available: %s", name,
                  e != cudaSuccess ? cudaGetErrorString(e) : "not found");
        (void)cudaGetLastError();
        return 1;
    }
    return 0;
}

const DriverApi* driver_api()
{
    static DriverApi api;
    static int state = 0;   // 0 unresolved, 1 ok, -1 failed
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (state == 1) return &api;
    if (state == -1) return nullptr;
    if (resolve("cuTensorMapEncodeTiled", (void**)&api.cuTensorMapEncodeTiled) ||
        resolve("cuStreamWaitValue32", (void**)&api.cuStreamWaitValue32) ||
        resolve("cuStreamWriteValue32", (void**)&api.cuStreamWriteValue32) ||
        resolve("cuGetErrorString", (void**)&api.cuGetErrorString) ||
        resolve("cuMemGetAddressRange", (void**)&api.cuMemGetAddressRange) ||
        resolve("cuCtxGetDevice", (void**)&api.cuCtxGetDevice) ||
        resolve("cuDeviceGetAttribute", (void**)&api.cuDeviceGetAttribute) ||
        resolve("cuMemGetAllocationGranularity", (void**)&api.cuMemGetAllocationGranularity) ||
        resolve("cuMemCreate", (void**)&api.cuMemCreate) ||
        resolve("cuMemRelease", (void**)&api.cuMemRelease) ||
        resolve("cuMemAddressReserve", (void**)&api.cuMemAddressReserve) ||
        resolve("cuMemAddressFree", (void**)&api.cuMemAddressFree) ||
        resolve("cuMemMap", (void**)&api.cuMemMap) ||
        resolve("cuMemUnmap", (void**)&api.cuMemUnmap) ||
        resolve("cuMemSetAccess", (void**)&api.cuMemSetAccess) ||
        resolve("cuMemExportToShareableHandle", (void**)&api.cuMemExportToShareableHandle) ||
        resolve("cuMemImportFromShareableHandle", (void**)&api.cuMemImportFromShareableHandle) ||
        resolve("cuMulticastCreate", (void**)&api.cuMulticastCreate) ||
        resolve("cuMulticastAddDevice", (void**)&api.cuMulticastAddDevice) ||
        resolve("cuMulticastBindMem", (void**)&api.cuMulticastBindMem) ||
        resolve("cuMulticastUnbind", (void**)&api.cuMulticastUnbind) ||
        resolve("cuMulticastGetGranularity", (void**)&api.cuMulticastGetGranularity)) {
        state = -1;
        return nullptr;
    }
    state = 1;
    return &api;
}

const NcclApi* nccl_api()
{
    static NcclApi api;
    static int state = 0;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (state == 1) return &api;
    if (state == -1) { set_error("NCCL (libnccl.so.2) could not be loaded"); return nullptr; }
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { set_error("dlopen(libnccl.so.2): %s", dlerror()); state = -1; return nullptr; }
    struct { const char* name; void** fn; } syms[] = {
        {"ncclGetUniqueId", (void**)&api.GetUniqueId}, {"ncclCommInitRank", (void**)&api.CommInitRank},
        {"ncclCommDestroy", (void**)&api.CommDestroy}, {"ncclAllReduce", (void**)&api.AllReduce},
        {"ncclGetErrorString", (void**)&api.GetErrorString},
    };
    for (auto& s : syms) {
        *s.fn = dlsym(h, s.name);
        if (!*s.fn) { set_error("dlsym(%s): %s", s.name, dlerror()); state = -1; return nullptr; }
    }
    state = 1;
    return &api;
}

int* kernel_status_word()
{
    constexpr int kMaxDev = 64;
    static int* words[kMaxDev] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, 4 * sizeof(int)) != cudaSuccess) return nullptr;
        if (cudaMemset(p, 0, 4 * sizeof(int)) != cudaSuccess) return nullptr;
        words[dev] = p;
    }
    return words[dev];
}

int* work_counter_slot()
{
    constexpr int kMaxDev = 64, kSlots = 256;
    static int* ring[kMaxDev] = {};
    static unsigned next[kMaxDev] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ring[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, kSlots * sizeof(int)) != cudaSuccess) return nullptr;
        ring[dev] = p;
    }
    return ring[dev] + (next[dev]++ % kSlots);
}

int make_tmap_f16(CUtensorMap* out, const void* base, int rank,
                  const unsigned long long* dims, const unsigned long long* strides_bytes,
                  const unsigned* box)
{
    const DriverApi* api = driver_api();
    if (!api) return 1;
    if (rank < 2 || rank > 3) { set_error("make_tmap_f16: rank %d unsupported", rank); return 1; }
    if (((uintptr_t)base & 15) != 0) { set_error("make_tmap_f16: base address not 16-byte aligned"); return 1; }
    const unsigned inner_bytes = box[0] * 2u;
    CUtensorMapSwizzle swz;
    switch (inner_bytes) {
        case 128: swz = CU_TENSOR_MAP_SWIZZLE_128B; break;
        case 64:  swz = CU_TENSOR_MAP_SWIZZLE_64B;  break;
        case 32:  swz = CU_TENSOR_MAP_SWIZZLE_32B;  break;
        default: set_error("make_tmap_f16: inner box of %u bytes has no swizzle mode", inner_bytes); return 1;
    }
    cuuint64_t gdim[3]; cuuint64_t gstr[2]; cuuint32_t bdim[3]; cuuint32_t estr[3];
    for (int i = 0; i < rank; i++) { gdim[i] = dims[i]; bdim[i] = box[i]; estr[i] = 1; }
    for (int i = 0; i + 1 < rank; i++) {
        if (strides_bytes[i] % 16 != 0) { set_error("make_tmap_f16: stride %d (%llu B) not a multiple of 16", i, strides_bytes[i]); return 1; }
        gstr[i] = strides_bytes[i];
    }
    CUresult r = api->cuTensorMapEncodeTiled(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank,
                                             const_cast<void*>(base), gdim, gstr, bdim, estr,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return check_cu(r, "cuTensorMapEncodeTiled", __FILE__, __LINE__);
}

}  // namespace efa
