// bfloat16 features with float32 arithmetic and outputs: channel slices of 1 or 8 per lane in the
// generic kernels, 4 per lane in the compile-time-C CostVolume MEAN kernels.
#include "cv_launch.cuh"
#include "cv_entry.h"

namespace chop {
int cv_fwd_bf16(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  if (p.use_tuned && p.use_packed && p.kind == 3 && p.mode == 0 && p.cpl == 4) {
    int r = -4;
    switch (a.C) {
      case 8: r = fwd_agg_packed_go<__nv_bfloat16, 8>(a, st); break;
      case 16: r = fwd_agg_packed_go<__nv_bfloat16, 16>(a, st); break;
      case 32: r = fwd_agg_packed_go<__nv_bfloat16, 32>(a, st); break;
      default: break;
    }
    if (r != -4) return r;
  }
  if (p.use_tuned && p.kind == 3 && p.mode == 0 && p.cpl == 4) {
    switch (a.C) {
      case 8: return fwd_tuned_go<__nv_bfloat16, 8, 4, true>(a, st);
      case 16: return fwd_tuned_go<__nv_bfloat16, 16, 4, true>(a, st);
      case 32: return fwd_tuned_go<__nv_bfloat16, 32, 4, true>(a, st);
      case 64: return fwd_tuned_go<__nv_bfloat16, 64, 4, true>(a, st);
      default: break;
    }
  }
  if (p.use_tuned && p.kind == 2 && p.mode != 1 && p.cpl == 4) {
    const int r = tuned2_dispatch<__nv_bfloat16>(false, p.mode == 2, a, st);
    if (r != -4) return r;  // -4: no compile-time-C kernel for this (C, groups): generic kernel below
  }
  if (p.use_tuned && p.kind == 3 && p.mode == 2 && p.cpl == 4) {
    switch (a.C) {
      case 8: return agg_min_fwd_tuned_go<__nv_bfloat16, 8, 4>(a, st);
      case 16: return agg_min_fwd_tuned_go<__nv_bfloat16, 16, 4>(a, st);
      case 32: return agg_min_fwd_tuned_go<__nv_bfloat16, 32, 4>(a, st);
      default: break;
    }
  }
  if (p.use_tuned && p.kind == 1 && p.mode == 2 && p.cpl == 4 && a.N <= 254) {
    switch (a.C) {
      case 8: return fwd_min_tuned_go<__nv_bfloat16, 8, 4>(a, st);
      case 16: return fwd_min_tuned_go<__nv_bfloat16, 16, 4>(a, st);
      case 32: return fwd_min_tuned_go<__nv_bfloat16, 32, 4>(a, st);
      default: break;
    }
  }
  if (p.use_tuned && p.use_packed && p.kind == 1 && p.mode == 0 && p.cpl == 4) {
    int r = -4;
    switch (a.C) {
      case 8: r = fwd_packed_go<__nv_bfloat16, 8>(a, st); break;
      case 16: r = fwd_packed_go<__nv_bfloat16, 16>(a, st); break;
      case 32: r = fwd_packed_go<__nv_bfloat16, 32>(a, st); break;
      default: break;
    }
    if (r != -4) return r;
  }
  if (p.use_tuned && p.kind == 1 && p.mode == 0 && p.cpl == 4) {
    switch (a.C) {
      case 8: return fwd_tuned_go<__nv_bfloat16, 8, 4>(a, st);
      case 16: return fwd_tuned_go<__nv_bfloat16, 16, 4>(a, st);
      case 32: return fwd_tuned_go<__nv_bfloat16, 32, 4>(a, st);
      case 64: return fwd_tuned_go<__nv_bfloat16, 64, 4>(a, st);
      default: break;
    }
  }
  return p.cpl == 8 ? fwd_kind<__nv_bfloat16, float, 8>(a, p, st) : fwd_kind<__nv_bfloat16, float, 1>(a, p, st);
}
int cv_bwd_bf16(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  if (p.use_tuned && p.kind == 3 && !p.rmin && p.cpl == 4) {
    switch (a.C) {
      case 8: return bwd_tuned_go<__nv_bfloat16, 8, 4, true>(a, st);
      case 16: return bwd_tuned_go<__nv_bfloat16, 16, 4, true>(a, st);
      case 32: return bwd_tuned_go<__nv_bfloat16, 32, 4, true>(a, st);
      case 64: return bwd_tuned_go<__nv_bfloat16, 64, 4, true>(a, st);
      default: break;
    }
  }
  if (p.use_tuned && p.kind == 3 && p.rmin && p.cpl == 4) {
    switch (a.C) {
      case 8: return bwd_tuned_go<__nv_bfloat16, 8, 4, true, true>(a, st);
      case 16: return bwd_tuned_go<__nv_bfloat16, 16, 4, true, true>(a, st);
      case 32: return bwd_tuned_go<__nv_bfloat16, 32, 4, true, true>(a, st);
      case 64: return bwd_tuned_go<__nv_bfloat16, 64, 4, true, true>(a, st);
      default: break;
    }
  }
  if (p.use_tuned && p.kind == 1 && p.rmin && p.cpl == 4) {
    switch (a.C) {
      case 8: return bwd_tuned_go<__nv_bfloat16, 8, 4, false, true>(a, st);
      case 16: return bwd_tuned_go<__nv_bfloat16, 16, 4, false, true>(a, st);
      case 32: return bwd_tuned_go<__nv_bfloat16, 32, 4, false, true>(a, st);
      case 64: return bwd_tuned_go<__nv_bfloat16, 64, 4, false, true>(a, st);
      default: break;
    }
  }
  if (p.use_tuned && p.kind == 2 && p.cpl == 4) {
    const int r = tuned2_dispatch<__nv_bfloat16>(true, p.rmin != 0, a, st);
    if (r != -4) return r;
  }
  if (p.use_tuned && p.kind == 1 && !p.rmin && p.cpl == 4) {
    switch (a.C) {
      case 8: return bwd_tuned_go<__nv_bfloat16, 8, 4>(a, st);
      case 16: return bwd_tuned_go<__nv_bfloat16, 16, 4>(a, st);
      case 32: return bwd_tuned_go<__nv_bfloat16, 32, 4>(a, st);
      case 64: return bwd_tuned_go<__nv_bfloat16, 64, 4>(a, st);
      default: break;
    }
  }
  return p.cpl == 8 ? bwd_kind<__nv_bfloat16, float, 8>(a, p, st) : bwd_kind<__nv_bfloat16, float, 1>(a, p, st);
}
}  // namespace chop
