// float64 everything: channel slices of 1 or 2 per lane.
#include "cv_launch.cuh"
#include "cv_entry.h"

namespace chop {
int cv_fwd_f64(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  return p.cpl == 2 ? fwd_kind<double, double, 2>(a, p, st) : fwd_kind<double, double, 1>(a, p, st);
}
int cv_bwd_f64(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  return p.cpl == 2 ? bwd_kind<double, double, 2>(a, p, st) : bwd_kind<double, double, 1>(a, p, st);
}
}  // namespace chop
