// Host-side helpers shared by the translation units of the library: per-thread error string,
// CUDA error capture, driver entry points fetched at run time (the library does not link libcuda,
// so it can be loaded and its symbols inspected on a machine without a driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>

namespace efa {

void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
const char* last_error();

// Returns 0 when `e` is cudaSuccess; otherwise records "<what>: <cuda error string>" and returns 1.
int check_cuda(cudaError_t e, const char* what, const char* file, int line);
int check_cu(CUresult r, const char* what, const char* file, int line);

#define EFA_CUDA(call) do { if (::efa::check_cuda((call), #call, __FILE__, __LINE__)) return 1; } while (0)
#define EFA_CU(call)   do { if (::efa::check_cu((call), #call, __FILE__, __LINE__)) return 1; } while (0)

// Driver API entry points (resolved through cudaGetDriverEntryPoint on first use).
struct DriverApi {
    CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                       const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                       const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    CUresult (*cuStreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    CUresult (*cuStreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    CUresult (*cuGetErrorString)(CUresult, const char**);
    CUresult (*cuMemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
    // virtual memory management and NVLink multicast objects (nvls_reduce.cu)
    CUresult (*cuCtxGetDevice)(CUdevice*);
    CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
    CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
    CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
    CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
    CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
    CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
};
// nullptr (with the error recorded) when the driver is not available.
const DriverApi* driver_api();

// Device-side status word (int[4]) of the current device, allocated on first use.
int* kernel_status_word();

// A device int for one launch (work distribution of persistent kernels): slots of a small per-device
// ring handed out round-robin; the caller clears its slot on the launch stream.
int* work_counter_slot();

// fp16 tensor map over a row-major tensor viewed as up to 3 dimensions (dim 0 fastest).
// `box` rows x `box_cols` columns, swizzle chosen from box_cols * 2 bytes (32, 64 or 128).
int make_tmap_f16(CUtensorMap* out, const void* base, int rank,
                  const unsigned long long* dims, const unsigned long long* strides_bytes /* rank-1 */,
                  const unsigned* box);

}  // namespace efa
