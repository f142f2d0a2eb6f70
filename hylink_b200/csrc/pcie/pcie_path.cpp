#include "pcie/pcie_path.h"
namespace hl {
PciePath::~PciePath() {}
size_t PciePath::ctrlBytes(int) { return 0; }
hlResult_t PciePath::create(Bootstrap*, int, void*, PciePath**) { return fail(hlUnsupported, "PCIe path not built yet"); }
hlResult_t PciePath::allReduce(const void*, void*, size_t, hlDataType_t, hlRedOp_t, float, hlStream_t) { return hlUnsupported; }
hlResult_t PciePath::reduceScatter(const void*, void*, size_t, size_t, hlDataType_t, hlRedOp_t, float, hlStream_t) { return hlUnsupported; }
hlResult_t PciePath::allGather(const void*, void*, size_t, size_t, hlDataType_t, hlStream_t) { return hlUnsupported; }
hlResult_t PciePath::allToAll(const void*, void*, size_t, size_t, hlDataType_t, hlStream_t) { return hlUnsupported; }
hlResult_t PciePath::broadcast(const void*, void*, size_t, hlDataType_t, int, hlStream_t) { return hlUnsupported; }
hlResult_t PciePath::submitIr(const char*, const void*, void*, size_t, size_t, int, int, hlDataType_t, hlRedOp_t, hlStream_t) { return hlUnsupported; }
hlResult_t PciePath::drain() { return hlSuccess; }
hlResult_t PciePath::lastResult() const { return hlSuccess; }
uint64_t PciePath::kernelLaunches() const { return 0; }
uint64_t PciePath::copyOps() const { return 0; }
}
