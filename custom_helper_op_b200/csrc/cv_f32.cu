// float32 features: channel slices of 1 or 4 per lane.
#include "cv_launch.cuh"
#include "cv_entry.h"

namespace chop {
int cv_fwd_f32(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  return p.cpl == 4 ? fwd_kind<float, float, 4>(a, p, st) : fwd_kind<float, float, 1>(a, p, st);
}
int cv_bwd_f32(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  return p.cpl == 4 ? bwd_kind<float, float, 4>(a, p, st) : bwd_kind<float, float, 1>(a, p, st);
}
}  // namespace chop
