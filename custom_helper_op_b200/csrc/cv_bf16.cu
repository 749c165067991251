// bfloat16 features with float32 arithmetic and outputs: channel slices of 1 or 8 per lane.
#include "cv_launch.cuh"
#include "cv_entry.h"

namespace chop {
int cv_fwd_bf16(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  return p.cpl == 8 ? fwd_kind<__nv_bfloat16, float, 8>(a, p, st) : fwd_kind<__nv_bfloat16, float, 1>(a, p, st);
}
int cv_bwd_bf16(const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  return p.cpl == 8 ? bwd_kind<__nv_bfloat16, float, 8>(a, p, st) : bwd_kind<__nv_bfloat16, float, 1>(a, p, st);
}
}  // namespace chop
