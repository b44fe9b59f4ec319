// Host-side launch helpers shared by the kernel files.
#include <mutex>
#include <set>
#include <utility>

#include "kernels.h"

namespace lq {

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-DEVICE attribute of a kernel: a process
// that drives several GPUs has to set it once on each of them.  Remembers (device, kernel) pairs
// under a lock so that concurrent contexts on different threads and devices all get it.
cudaError_t set_max_dyn_smem(const void* func, int bytes) {
    static std::mutex mu;
    static std::set<std::pair<int, const void*>> done;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair(dev, func);
    if (done.count(key)) return cudaSuccess;
    e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done.insert(key);
    return e;
}

}  // namespace lq
