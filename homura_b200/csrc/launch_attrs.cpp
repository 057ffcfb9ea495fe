#include "launch_attrs.h"

#include <map>
#include <mutex>
#include <utility>

namespace hm {
namespace {
std::mutex g_mu;
// (device, kernel) -> dynamic shared memory limit set there; kernels start at the 48 KB default, of which
// static shared memory takes its share, so anything above 40 KB is requested explicitly
std::map<std::pair<int, const void*>, size_t> g_smem;
std::map<std::pair<int, const void*>, bool> g_nonportable;
constexpr size_t kDefaultDynSmem = 40 * 1024;
}  // namespace

cudaError_t ensure_dyn_smem(const void* func, size_t bytes) {
    if (bytes <= kDefaultDynSmem) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lk(g_mu);
    size_t& have = g_smem[{dev, func}];
    if (bytes <= have) return cudaSuccess;
    e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) have = bytes;
    return e;
}

cudaError_t ensure_nonportable_clusters(const void* func) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lk(g_mu);
    bool& have = g_nonportable[{dev, func}];
    if (have) return cudaSuccess;
    e = cudaFuncSetAttribute(func, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) have = true;
    return e;
}

}  // namespace hm
