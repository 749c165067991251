// Launch entry points of the CostVolumeV3 kernels (cv_v3.cu).
#pragma once
#include <cuda_runtime.h>

namespace chop {
struct CvArgs;
int cv3_fwd_launch(int dtype, bool rmin, const CvArgs& a, cudaStream_t st);
int cv3_bwd_launch(int dtype, bool rmin, const CvArgs& a, cudaStream_t st);
}  // namespace chop
