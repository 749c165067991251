// Typed kernel selection for the cost-volume kernels.  Each cv_<dtype>.cu instantiates this header
// for one feature type so the three translation units compile in parallel.
#pragma once
#include "cv_bwd.cuh"
#include "cv_fwd.cuh"
#include "cv_packed.cuh"
#include "cv_tuned.cuh"
#include "smem_grant.h"

namespace chop {

struct CvPlan {
  int cpl;    // channels per lane
  int kind;   // 1 CostVolume, 2 CostVolumeV2, 3 CostAggregate
  int mode;   // forward: 0 fast MEAN, 1 unfused MEAN, 2 MIN
  int rmin;   // backward: MIN
  int nv;     // backward: source views tracked per pass
  int blocks;
  int use_tuned;  // allow the compile-time-C kernels of cv_tuned.cuh where one exists
  int use_packed; // allow the packed-pair kernels of cv_packed.cuh where one exists
  FwdCfg fwd;
  BwdCfg bwd;
};

template <typename T, typename R, int CPL, int KIND, int MODE>
inline int fwd_go(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  auto k = cv_fwd_kernel<T, R, CPL, KIND, MODE>;
  const size_t smem = p.fwd.smem_per_warp * p.fwd.warps;
  if (int e = grant_smem(k, smem)) return e;
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
  if (int e = grant_smem(k, smem)) return e;
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

// ---- compile-time-C kernels -------------------------------------------------------------------------
inline int tuned_warps(size_t smem_per_warp) {
  int w = 8;
  while (w > 1 && smem_per_warp * w > 96 * 1024) w >>= 1;
  return w;
}

template <typename T, int C, int CPL, bool AGG = false>
inline int fwd_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv_fwd_tuned<T, C, CPL, AGG>;
  const size_t spw = tuned_fwd_smem_per_warp<T>(a.N, 32 / (C / CPL));
  const int warps = tuned_warps(spw);
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int CPL>
inline int fwd_min_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv_fwd_min_tuned<T, C, CPL>;
  const size_t spw = tuned_fwd_smem_per_warp<T>(a.N, 32 / (C / CPL));
  const int warps = tuned_warps(spw);
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int CPL>
inline int agg_min_fwd_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv_agg_min_fwd_tuned<T, C, CPL>;
  const size_t spw = tuned_fwd_smem_per_warp<T>(a.N, 32 / (C / CPL)) + (size_t)32 * (C + 4) * sizeof(float);
  const int warps = tuned_warps(spw);
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int CPL, bool AGG = false, bool RMIN = false>
inline int bwd_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv_bwd_tuned<T, C, CPL, AGG, RMIN>;
  const size_t spw = tuned_bwd_smem_per_warp<C>(a.N, 32 / (C / CPL), (RMIN && !AGG) ? 2 : 1);
  const int warps = 4;
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int SUB>
inline int fwd2_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv2_fwd_tuned<T, C, SUB>;
  const size_t spw = tuned_fwd_smem_per_warp<T>(a.N, 32 / (C / 4));
  const int warps = tuned_warps(spw);
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int SUB>
inline int fwd2_min_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv2_fwd_min_tuned<T, C, SUB>;
  const size_t spw = tuned_fwd_smem_per_warp<T>(a.N, 32 / (C / 4));
  const int warps = tuned_warps(spw);
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int SUB, bool RMIN>
inline int bwd2_tuned_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv2_bwd_tuned<T, C, SUB, RMIN>;
  const size_t spw = tuned2_bwd_smem_per_warp<T>(a.N, 32 / (C / 4));
  const int warps = 4;
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

// ---- packed-pair kernels (cv_packed.cuh) ----------------------------------------------------------------
template <typename T, int C, int NV, bool AGG = false>
inline int fwd_pm_go(const CvArgs& a, cudaStream_t st);

template <typename T, int C>
inline int fwd_packed_go(const CvArgs& a, cudaStream_t st) {
#ifndef CHOP_NO_PM
  if (a.N == 1) return fwd_pm_go<T, C, 1>(a, st);
  if (a.N == 2) return fwd_pm_go<T, C, 2>(a, st);
#endif
  auto k = cv_fwd_packed<T, C>;
  const size_t spw = packed_fwd_smem_per_warp(a.N, 32 / (C / 4));
  const int warps = tuned_warps(spw);
  const size_t smem = spw * warps;
  if (smem > 200 * 1024) return -4;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, int C, int NV, bool AGG>
inline int fwd_pm_go(const CvArgs& a, cudaStream_t st) {
  auto k = cv_fwd_pm<T, C, NV, AGG>;
  const size_t spw = pm_fwd_smem_per_warp(NV);
  const int warps = CHOP_PM_FWD_WARPS;
  const size_t smem = spw * warps;
  if (int e = grant_smem(k, smem)) return e;
  const long long items = (long long)a.npb * a.nchunks;
  k<<<(unsigned)((items + warps - 1) / warps), warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

// CostAggregate MEAN with one or two source views on the plane-major packed kernel; -4: no such kernel
template <typename T, int C>
inline int fwd_agg_packed_go(const CvArgs& a, cudaStream_t st) {
#ifndef CHOP_NO_PM
  if (a.N == 1) return fwd_pm_go<T, C, 1, true>(a, st);
  if (a.N == 2) return fwd_pm_go<T, C, 2, true>(a, st);
#endif
  return -4;
}

// C in {8,16,32}, channels per group in {1,2,4}; returns -4 if there is no such kernel
template <typename T>
inline int tuned2_dispatch(bool backward, bool rmin, const CvArgs& a, cudaStream_t st) {
  const int sub = a.C / a.G;
  if (rmin && !backward && a.N > 254) return -4;   // the MIN forward packs the winning view into a byte
#define CHOP_V2_CASE(CC, SS)                                                                            \
  if (a.C == CC && sub == SS)                                                                           \
    return backward ? (rmin ? bwd2_tuned_go<T, CC, SS, true>(a, st) : bwd2_tuned_go<T, CC, SS, false>(a, st)) \
                    : (rmin ? fwd2_min_tuned_go<T, CC, SS>(a, st) : fwd2_tuned_go<T, CC, SS>(a, st));
  CHOP_V2_CASE(8, 1) CHOP_V2_CASE(8, 2) CHOP_V2_CASE(8, 4)
  CHOP_V2_CASE(16, 1) CHOP_V2_CASE(16, 2) CHOP_V2_CASE(16, 4)
  CHOP_V2_CASE(32, 1) CHOP_V2_CASE(32, 2) CHOP_V2_CASE(32, 4)
#undef CHOP_V2_CASE
  return -4;
}

}  // namespace chop
