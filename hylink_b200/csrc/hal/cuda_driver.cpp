#include "hal/cuda_driver.h"

#include <mutex>

namespace hl {

template <typename F>
static bool resolve(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    *out = nullptr;
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

bool cudaAvailable() {
  static int state = -1;
  if (state < 0) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) cudaGetLastError();
    state = (e == cudaSuccess && n > 0) ? 1 : 0;
  }
  return state == 1;
}

const CudaDriver* CudaDriver::get() {
  static CudaDriver d;
  static std::once_flag once;
  std::call_once(once, [] {
    if (!cudaAvailable()) return;
    bool ok = true;
    ok &= resolve("cuGetErrorString", &d.cuGetErrorString);
    ok &= resolve("cuDeviceGet", &d.cuDeviceGet);
    ok &= resolve("cuDeviceGetAttribute", &d.cuDeviceGetAttribute);
    ok &= resolve("cuMemGetAllocationGranularity", &d.cuMemGetAllocationGranularity);
    ok &= resolve("cuMemCreate", &d.cuMemCreate);
    ok &= resolve("cuMemRelease", &d.cuMemRelease);
    ok &= resolve("cuMemExportToShareableHandle", &d.cuMemExportToShareableHandle);
    ok &= resolve("cuMemImportFromShareableHandle", &d.cuMemImportFromShareableHandle);
    ok &= resolve("cuMemAddressReserve", &d.cuMemAddressReserve);
    ok &= resolve("cuMemAddressFree", &d.cuMemAddressFree);
    ok &= resolve("cuMemMap", &d.cuMemMap);
    ok &= resolve("cuMemUnmap", &d.cuMemUnmap);
    ok &= resolve("cuMemSetAccess", &d.cuMemSetAccess);
    ok &= resolve("cuStreamWriteValue64", &d.cuStreamWriteValue64);
    ok &= resolve("cuStreamWaitValue64", &d.cuStreamWaitValue64);
    // multicast is optional (absent on drivers older than 12.1)
    resolve("cuMulticastCreate", &d.cuMulticastCreate);
    resolve("cuMulticastAddDevice", &d.cuMulticastAddDevice);
    resolve("cuMulticastBindMem", &d.cuMulticastBindMem);
    resolve("cuMulticastUnbind", &d.cuMulticastUnbind);
    resolve("cuMulticastGetGranularity", &d.cuMulticastGetGranularity);
    d.ok = ok;
  });
  return d.ok ? &d : nullptr;
}

const char* CudaDriver::err(CUresult r) const {
  const char* s = nullptr;
  if (cuGetErrorString && cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "unknown driver error";
}

}  // namespace hl
