// Typed launch entry points implemented by cv_f32.cu / cv_f64.cu / cv_bf16.cu.
#pragma once
#include <cuda_runtime.h>

namespace chop {
struct CvArgs;
struct CvPlan;
int cv_fwd_f32(const CvArgs&, const CvPlan&, cudaStream_t);
int cv_bwd_f32(const CvArgs&, const CvPlan&, cudaStream_t);
int cv_fwd_f64(const CvArgs&, const CvPlan&, cudaStream_t);
int cv_bwd_f64(const CvArgs&, const CvPlan&, cudaStream_t);
int cv_fwd_bf16(const CvArgs&, const CvPlan&, cudaStream_t);
int cv_bwd_bf16(const CvArgs&, const CvPlan&, cudaStream_t);
}  // namespace chop
