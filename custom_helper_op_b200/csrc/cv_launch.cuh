// Typed kernel selection for the cost-volume kernels.  Each cv_<dtype>.cu instantiates this header
// for one feature type so the three translation units compile in parallel.
#pragma once
#include "cv_bwd.cuh"
#include "cv_fwd.cuh"

namespace chop {

struct CvPlan {
  int cpl;    // channels per lane
  int kind;   // 1 CostVolume, 2 CostVolumeV2, 3 CostAggregate
  int mode;   // forward: 0 fast MEAN, 1 unfused MEAN, 2 MIN
  int rmin;   // backward: MIN
  int nv;     // backward: source views tracked per pass
  int blocks;
  FwdCfg fwd;
  BwdCfg bwd;
};

template <typename T, typename R, int CPL, int KIND, int MODE>
inline int fwd_go(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  auto k = cv_fwd_kernel<T, R, CPL, KIND, MODE>;
  const size_t smem = p.fwd.smem_per_warp * p.fwd.warps;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  k<<<p.blocks, p.fwd.warps * 32, smem, st>>>(a, p.fwd);
  return (int)cudaGetLastError();
}

template <typename T, typename R, int CPL, int KIND>
inline int fwd_mode(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  switch (p.mode) {
    case 0: return fwd_go<T, R, CPL, KIND, 0>(a, p, st);
    case 1: return fwd_go<T, R, CPL, KIND, 1>(a, p, st);
    default: return fwd_go<T, R, CPL, KIND, 2>(a, p, st);
  }
}

template <typename T, typename R, int CPL>
inline int fwd_kind(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  switch (p.kind) {
    case 1: return fwd_mode<T, R, CPL, 1>(a, p, st);
    case 2: return fwd_mode<T, R, CPL, 2>(a, p, st);
    default: return fwd_mode<T, R, CPL, 3>(a, p, st);
  }
}

template <typename T, typename R, int CPL, int KIND, bool RMIN, int NV>
inline int bwd_go(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  auto k = cv_bwd_kernel<T, R, CPL, KIND, RMIN, NV>;
  const size_t smem = p.bwd.smem_per_warp * p.bwd.warps;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  k<<<p.blocks, p.bwd.warps * 32, smem, st>>>(a, p.bwd);
  return (int)cudaGetLastError();
}

template <typename T, typename R, int CPL, int KIND, bool RMIN>
inline int bwd_nv(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  if constexpr (RMIN) {
    return bwd_go<T, R, CPL, KIND, RMIN, 2>(a, p, st);  // MIN is not a tuned path: one variant
  } else {
  switch (p.nv) {
    case 1: return bwd_go<T, R, CPL, KIND, RMIN, 1>(a, p, st);
    case 2: return bwd_go<T, R, CPL, KIND, RMIN, 2>(a, p, st);
    case 3: return bwd_go<T, R, CPL, KIND, RMIN, 3>(a, p, st);
    default: return bwd_go<T, R, CPL, KIND, RMIN, 4>(a, p, st);
  }
  }
}

template <typename T, typename R, int CPL>
inline int bwd_kind(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  switch (p.kind) {
    case 1: return p.rmin ? bwd_nv<T, R, CPL, 1, true>(a, p, st) : bwd_nv<T, R, CPL, 1, false>(a, p, st);
    case 2: return p.rmin ? bwd_nv<T, R, CPL, 2, true>(a, p, st) : bwd_nv<T, R, CPL, 2, false>(a, p, st);
    default: return p.rmin ? bwd_nv<T, R, CPL, 3, true>(a, p, st) : bwd_nv<T, R, CPL, 3, false>(a, p, st);
  }
}

}  // namespace chop
