// Per-device kernel attributes.
//
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize / NonPortableClusterSizeAllowed) applies to the
// device that is current when it is called.  One host process may drive several engines, one per
// GPU and each from its own thread (Homura is a single process, src/hf/model.rs:17-31), so what
// has been set is remembered per (device, kernel) under a lock -- never in a process-wide flag.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace hm {

// Makes sure `func` may be launched with `bytes` of dynamic shared memory on the current device.
// The limit is only ever raised, so launches already captured in a graph stay valid.
cudaError_t ensure_dyn_smem(const void* func, size_t bytes);
// Allows cluster sizes above 8 for `func` on the current device.
cudaError_t ensure_nonportable_clusters(const void* func);

template <typename F>
inline cudaError_t ensure_dyn_smem(F* func, size_t bytes) { return ensure_dyn_smem(reinterpret_cast<const void*>(func), bytes); }
template <typename F>
inline cudaError_t ensure_nonportable_clusters(F* func) { return ensure_nonportable_clusters(reinterpret_cast<const void*>(func)); }

}  // namespace hm
