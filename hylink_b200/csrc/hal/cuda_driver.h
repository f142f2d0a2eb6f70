// Lazily resolved CUDA driver entry points (virtual memory management,
// NVSwitch multicast objects, stream memory operations). The library links
// the CUDA runtime statically and never links libcuda, so it also loads on a
// machine without a GPU or driver (the CPU-only configuration).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "core/core.h"

namespace hl {

struct CudaDriver {
  bool ok = false;
  CUresult (*cuGetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*cuDeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*cuStreamWriteValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int) = nullptr;
  CUresult (*cuStreamWaitValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int) = nullptr;

  // nullptr when no driver is present.
  static const CudaDriver* get();
  const char* err(CUresult r) const;
};

// True when at least one CUDA device can be used by this process.
bool cudaAvailable();

#define HL_CUDA(expr)                                                                     \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) return ::hl::fail(hlDeviceError, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)
#define HL_CU(drv, expr)                                                                  \
  do {                                                                                    \
    CUresult _e = (drv)->expr;                                                            \
    if (_e != CUDA_SUCCESS) return ::hl::fail(hlDeviceError, "%s: %s", #expr, (drv)->err(_e)); \
  } while (0)

}  // namespace hl
