#include "nvl/symm_mem.h"

#include <unistd.h>

#include <cstring>

namespace hl {

// All ranks learn whether every rank succeeded at a step; a failure anywhere
// makes everybody take the same fallback instead of meeting at a barrier that
// one rank never reaches.
static bool agree(Bootstrap* bs, bool mine, hlResult_t* err) {
  int32_t v = mine ? 1 : 0, all[kMaxRanks];
  hlResult_t r = bs->allGather(&v, sizeof(v), all);
  if (r != hlSuccess) {
    *err = r;
    return false;
  }
  for (int q = 0; q < bs->nranks(); ++q)
    if (!all[q]) return false;
  return true;
}

static size_t roundUp(size_t v, size_t g) { return g ? ((v + g - 1) / g) * g : v; }

static hlResult_t allocVmm(Bootstrap* bs, int device, size_t bytes, int want_mc, SymmRegion* out, bool* usable) {
  *usable = false;
  const CudaDriver* drv = CudaDriver::get();
  const int n = bs->nranks(), me = bs->rank();
  hlResult_t err = hlSuccess;
  bool ok = drv != nullptr;
  CUdevice cudev = 0;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  size_t gran = 0;
  int mc_supported = 0;
  if (ok) {
    ok = drv->cuDeviceGet(&cudev, device) == CUDA_SUCCESS;
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    ok = ok && drv->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS;
    if (ok && drv->cuMulticastCreate && want_mc != 0)
      drv->cuDeviceGetAttribute(&mc_supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev);
  }
  bool try_mc = agree(bs, ok && mc_supported && n > 1, &err);
  if (err != hlSuccess) return err;
  CUmulticastObjectProp mcprop;
  memset(&mcprop, 0, sizeof(mcprop));
  size_t size = roundUp(bytes, gran ? gran : (2u << 20));
  if (try_mc) {
    mcprop.numDevices = (unsigned)n;
    mcprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcprop.size = size;
    size_t mgran = 0;
    if (drv->cuMulticastGetGranularity(&mgran, &mcprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran) {
      size = roundUp(size, mgran);
      mcprop.size = size;
    }
  }
  CUmemGenericAllocationHandle mine = 0;
  int my_fd = -1;
  if (ok) {
    CUresult r = drv->cuMemCreate(&mine, size, &prop, 0);
    if (r != CUDA_SUCCESS) {
      HL_INFO("cuMemCreate(%zu, posix-fd) failed: %s", size, drv->err(r));
      ok = false;
    } else {
      r = drv->cuMemExportToShareableHandle(&my_fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) {
        HL_INFO("cuMemExportToShareableHandle failed: %s", drv->err(r));
        ok = false;
      }
    }
  }
  if (!agree(bs, ok, &err)) {
    if (my_fd >= 0) close(my_fd);
    if (mine) drv->cuMemRelease(mine);
    return err;  // hlSuccess with *usable == false: caller falls back
  }
  int fds[kMaxRanks];
  HL_CHECK(bs->exchangeFds(my_fd, fds));
  out->handle[me] = mine;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int q = 0; q < n && ok; ++q) {
    CUmemGenericAllocationHandle h = mine;
    if (q != me) {
      CUresult r = drv->cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fds[q], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) {
        HL_WARN("import of rank %d's allocation failed: %s", q, drv->err(r));
        ok = false;
        break;
      }
      out->handle[q] = h;
    }
    CUdeviceptr va = 0;
    CUresult r = drv->cuMemAddressReserve(&va, size, gran, 0, 0);
    if (r == CUDA_SUCCESS) r = drv->cuMemMap(va, size, 0, h, 0);
    if (r == CUDA_SUCCESS) r = drv->cuMemSetAccess(va, size, &acc, 1);
    if (r != CUDA_SUCCESS) {
      HL_WARN("mapping rank %d's allocation failed: %s", q, drv->err(r));
      ok = false;
      break;
    }
    out->ptr[q] = (void*)va;
  }
  for (int q = 0; q < n; ++q)
    if (fds[q] >= 0) close(fds[q]);
  if (!agree(bs, ok, &err)) return err != hlSuccess ? err : fail(hlDeviceError, "peer mapping of symmetric memory failed on some rank");
  out->mode = kSymmVmm;
  out->map_bytes = size;
  *usable = true;

  // ---- multicast object (NVLS)
  if (try_mc) {
    CUmemGenericAllocationHandle mch = 0;
    int mc_fd = -1;
    bool mok = true;
    if (me == 0) {
      CUresult r = drv->cuMulticastCreate(&mch, &mcprop);
      if (r == CUDA_SUCCESS) r = drv->cuMemExportToShareableHandle(&mc_fd, mch, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) {
        HL_INFO("multicast object not available: %s", drv->err(r));
        mok = false;
      }
    }
    if (!agree(bs, mok, &err)) {
      if (mc_fd >= 0) close(mc_fd);
      if (mch) drv->cuMemRelease(mch);
      if (err != hlSuccess) return err;
      if (want_mc == 1) return fail(hlUnsupported, "NVLS requested but no multicast object could be created");
      return hlSuccess;
    }
    int got = -1;
    HL_CHECK(bs->broadcastFd(0, mc_fd, &got));
    if (me != 0) {
      CUresult r = drv->cuMemImportFromShareableHandle(&mch, (void*)(uintptr_t)got, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) {
        HL_WARN("multicast import failed: %s", drv->err(r));
        mok = false;
      }
    }
    if (got >= 0) close(got);
    if (mok) {
      CUresult r = drv->cuMulticastAddDevice(mch, cudev);
      if (r != CUDA_SUCCESS) {
        HL_WARN("cuMulticastAddDevice failed: %s", drv->err(r));
        mok = false;
      }
    }
    // every device must be added before anyone binds
    bool all_ok = agree(bs, mok, &err);
    if (err != hlSuccess) return err;
    if (all_ok) {
      CUresult r = drv->cuMulticastBindMem(mch, 0, mine, 0, size, 0);
      if (r != CUDA_SUCCESS) {
        HL_WARN("cuMulticastBindMem failed: %s", drv->err(r));
        mok = false;
      } else {
        out->mc_bound = true;
      }
      CUdeviceptr va = 0;
      if (mok) {
        r = drv->cuMemAddressReserve(&va, size, gran, 0, 0);
        if (r == CUDA_SUCCESS) r = drv->cuMemMap(va, size, 0, mch, 0);
        if (r == CUDA_SUCCESS) r = drv->cuMemSetAccess(va, size, &acc, 1);
        if (r != CUDA_SUCCESS) {
          HL_WARN("mapping the multicast object failed: %s", drv->err(r));
          mok = false;
        }
      }
      all_ok = agree(bs, mok, &err);
      if (err != hlSuccess) return err;
      if (all_ok) {
        out->mc = (void*)va;
        out->mc_handle = mch;
      } else {
        if (va) {
          drv->cuMemUnmap(va, size);
          drv->cuMemAddressFree(va, size);
        }
        if (out->mc_bound) drv->cuMulticastUnbind(mch, cudev, 0, size);
        out->mc_bound = false;
      }
    }
    if (!out->mc) {
      if (mch) drv->cuMemRelease(mch);
      if (want_mc == 1) return fail(hlUnsupported, "NVLS requested but the multicast mapping failed");
    }
  } else if (want_mc == 1 && n > 1) {
    return fail(hlUnsupported, "NVLS requested but multicast is not supported on every rank");
  }
  return hlSuccess;
}

static hlResult_t allocIpc(Bootstrap* bs, int device, size_t bytes, SymmRegion* out) {
  const int n = bs->nranks(), me = bs->rank();
  (void)device;
  void* p = nullptr;
  const size_t size = roundUp(bytes, 2u << 20);
  HL_CUDA(cudaMalloc(&p, size));
  out->ptr[me] = p;
  out->map_bytes = size;
  if (bs->singleProcess()) {
    struct Pub { void* p; int dev; } mine = {p, device}, all[kMaxRanks];
    HL_CHECK(bs->allGather(&mine, sizeof(mine), all));
    for (int q = 0; q < n; ++q) {
      out->ptr[q] = all[q].p;
      if (q != me && all[q].dev != device) {
        cudaError_t e = cudaDeviceEnablePeerAccess(all[q].dev, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          return fail(hlDeviceError, "peer access %d->%d: %s", device, all[q].dev, cudaGetErrorString(e));
        cudaGetLastError();
      }
    }
    out->mode = kSymmInProcess;
    return hlSuccess;
  }
  cudaIpcMemHandle_t h, all[kMaxRanks];
  HL_CUDA(cudaIpcGetMemHandle(&h, p));
  HL_CHECK(bs->allGather(&h, sizeof(h), all));
  bool ok = true;
  for (int q = 0; q < n; ++q) {
    if (q == me) continue;
    void* rp = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&rp, all[q], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      HL_WARN("cudaIpcOpenMemHandle(rank %d): %s", q, cudaGetErrorString(e));
      cudaGetLastError();
      ok = false;
      break;
    }
    out->ptr[q] = rp;
  }
  hlResult_t err = hlSuccess;
  if (!agree(bs, ok, &err)) return err != hlSuccess ? err : fail(hlDeviceError, "CUDA IPC mapping of symmetric memory failed");
  out->mode = kSymmIpc;
  return hlSuccess;
}

hlResult_t symmAlloc(Bootstrap* bs, int device, size_t bytes, int want_mc, const std::string& mode_pref, SymmRegion* out) {
  *out = SymmRegion();
  out->bytes = bytes;
  out->device = device;
  out->nranks = bs->nranks();
  out->rank = bs->rank();
  HL_CUDA(cudaSetDevice(device));
  HL_CUDA(cudaFree(0));  // make sure the primary context exists before driver calls
  const bool allow_vmm = mode_pref != "ipc" && !bs->singleProcess();
  if (allow_vmm) {
    bool usable = false;
    HL_CHECK(allocVmm(bs, device, bytes, want_mc, out, &usable));
    if (usable) return hlSuccess;
    if (mode_pref == "vmm") return fail(hlUnsupported, "HYLINK_SYMM_MODE=vmm but cuMem file-descriptor sharing is unavailable");
    HL_INFO("falling back to CUDA IPC for symmetric memory");
    *out = SymmRegion();
    out->bytes = bytes;
    out->device = device;
    out->nranks = bs->nranks();
    out->rank = bs->rank();
  }
  if (want_mc == 1 && bs->nranks() > 1) return fail(hlUnsupported, "NVLS requires the cuMem mode of symmetric memory");
  return allocIpc(bs, device, bytes, out);
}

void symmFree(Bootstrap* bs, SymmRegion* r, bool peers_gone) {
  if (r->mode == kSymmNone) return;
  cudaSetDevice(r->device);
  cudaDeviceSynchronize();
  if (!peers_gone && bs) bs->barrier(kBarSymm, 10000);
  const CudaDriver* drv = CudaDriver::get();
  if (r->mode == kSymmVmm && drv) {
    if (r->mc) {
      drv->cuMemUnmap((CUdeviceptr)r->mc, r->map_bytes);
      drv->cuMemAddressFree((CUdeviceptr)r->mc, r->map_bytes);
    }
    if (r->mc_handle) {
      CUdevice cudev = 0;
      drv->cuDeviceGet(&cudev, r->device);
      if (r->mc_bound) drv->cuMulticastUnbind((CUmemGenericAllocationHandle)r->mc_handle, cudev, 0, r->map_bytes);
      drv->cuMemRelease((CUmemGenericAllocationHandle)r->mc_handle);
    }
    for (int q = 0; q < r->nranks; ++q) {
      if (r->ptr[q]) {
        drv->cuMemUnmap((CUdeviceptr)r->ptr[q], r->map_bytes);
        drv->cuMemAddressFree((CUdeviceptr)r->ptr[q], r->map_bytes);
      }
      if (r->handle[q]) drv->cuMemRelease((CUmemGenericAllocationHandle)r->handle[q]);
    }
  } else if (r->mode == kSymmIpc) {
    // (the reference leaves this to process exit by default: pcie-ccl-cuda/src/core/process_state.cpp:512-525)
    for (int q = 0; q < r->nranks && Config::get().ipc_close_on_finalize; ++q)
      if (q != r->rank && r->ptr[q]) cudaIpcCloseMemHandle(r->ptr[q]);
    if (!peers_gone && bs) bs->barrier(kBarSymm, 10000);
    cudaFree(r->ptr[r->rank]);
  } else if (r->mode == kSymmInProcess) {
    if (!peers_gone && bs) bs->barrier(kBarSymm, 10000);
    cudaFree(r->ptr[r->rank]);
  }
  cudaGetLastError();
  *r = SymmRegion();
}

}  // namespace hl
