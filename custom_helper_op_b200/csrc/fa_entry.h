// Launch entry points of the FeatureAggregate and IndexInitializer kernels (fa.cu).
#pragma once
#include <cuda_runtime.h>

namespace chop {
struct CvArgs;
// dtype: 0 float32, 1 float64, 2 bfloat16 features (float32 everything else); cpl: channels per lane
int fa_fwd_launch(int dtype, int cpl, const CvArgs& a, cudaStream_t st);
int fa_bwd_launch(int dtype, int cpl, const CvArgs& a, cudaStream_t st);
int index_init_launch(int dtype, int half_centor, int H, int W, void* out, cudaStream_t st);
}  // namespace chop
