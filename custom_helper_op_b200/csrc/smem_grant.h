// Opt-in to more than 48 KB of dynamic shared memory is a per-(device, kernel) attribute.  grant_smem sets it
// the first time a launch of that kernel on that device needs that much, not on every call; the table of what
// has been granted is the only state it keeps (process-wide, guarded by a mutex, a few entries).
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

namespace chop {

template <typename K>
inline int grant_smem(K kernel, size_t smem) {
  if (smem <= 48 * 1024) return 0;
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, size_t> granted;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  const std::pair<int, const void*> key(dev, reinterpret_cast<const void*>(kernel));
  std::lock_guard<std::mutex> lock(mu);
  auto it = granted.find(key);
  if (it != granted.end() && it->second >= smem) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  granted[key] = smem;
  return 0;
}

}  // namespace chop
