// TEST INFRASTRUCTURE ONLY.  C entry points around the reference's own kernel bodies compiled as
// host code (see build_ref.py).  Each entry point replays what the reference's functor does around
// the kernel launch - the int32/int64 index choice, MEAN/MIN dispatch and the zero fill of the
// gradient outputs (custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:289-335,590-655 and
// the v2 / aggregate twins) - and sweeps the voxel range on host threads.
//
// nthreads <= 1 runs one thread over the voxels in ascending order, which makes the atomic sums of
// the gradient kernels deterministic (used when minting fixtures).
#include <omp.h>

#include <cstring>
#include <type_traits>

#include "ref_shim.h"

namespace ref_shim {
thread_local int64 lo = 0;
thread_local int64 hi = 0;
}  // namespace ref_shim

#include "ref_cost_volume_v1.inc"
#include "ref_cost_volume_v2.inc"
#include "ref_cost_aggregate.inc"
#include "ref_sparse_conv_macros.inc"
#include "ref_sparse_conv3d.inc"
#include "ref_cost_volume_v3_macros.inc"
#include "ref_cost_volume_v3.inc"
#include "ref_feature_aggregate.inc"
#include "ref_index_initializer.inc"
#include "ref_sparse_pad_macros.inc"
#include "ref_sparse_pad.inc"

namespace {

template <typename F>
void sweep(int64 count, int nthreads, F body) {
  if (nthreads <= 1) {
    ref_shim::lo = 0;
    ref_shim::hi = count;
    body();
    return;
  }
  const int64 chunk = 2048;
  const int64 nchunks = (count + chunk - 1) / chunk;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
  for (int64 c = 0; c < nchunks; ++c) {
    ref_shim::lo = c * chunk;
    ref_shim::hi = std::min(count, (c + 1) * chunk);
    body();
  }
}

struct Dims {
  int64 B, H, W, C, D, N, Hs, Ws;
};

bool needs_int64(const Dims& s, int64 out_channels) {
  const int64 in_ref = s.B * s.H * s.W * s.C;
  const int64 in_src = s.B * s.N * s.Hs * s.Ws * s.C;
  const int64 out = s.B * s.H * s.W * s.D * out_channels;
  return in_ref > INT32_MAX || in_src > INT32_MAX || out > INT32_MAX;
}

#define V1_ARGS(I)                                                                                 \
  (I) count, (I)s.B, (I)s.H, (I)s.W, (I)s.C, (I)s.D, (I)s.N, (I)s.Hs, (I)s.Ws, ref, src, depth, \
      offsets, Rs, Ts
#define V3_ARGS(I)                                                                                 \
  (I) count, (I)s.B, (I)s.H, (I)s.W, (I)s.C, (I)s.D, (I)s.N, (I)s.Hs, (I)s.Ws, (int32)groups,   \
      ref, src, depth, offsets, Rs, Ts
#define V2_ARGS(I)                                                                                 \
  (I) count, (I)s.B, (I)s.H, (I)s.W, (I)s.C, (I)s.D, (I)s.N, (I)s.Hs, (I)s.Ws, (int32)groups,   \
      ref, src, depth, Rs, Ts

// kind: 1 = CostVolume, 2 = CostVolumeV2, 3 = CostAggregate, 4 = CostVolumeV3
template <typename T, typename I, bool HC>
void fwd_t(int kind, int reduce_min, const Dims& s, int groups, const T* ref, const T* src,
           const T* depth, const T* offsets, const T* Rs, const T* Ts, T* cost, int32* mask,
           int nthreads) {
  const int64 count = s.B * s.H * s.W * s.D;
  if (kind == 1) {
    if (!reduce_min)
      sweep(count, nthreads, [&] { CostMeanVolumeKernel<T, I, HC>(V1_ARGS(I), cost, mask); });
    else
      sweep(count, nthreads, [&] { CostMinVolumeKernel<T, I, HC>(V1_ARGS(I), cost, mask); });
  } else if (kind == 2) {
    if (!reduce_min)
      sweep(count, nthreads, [&] { CostMeanVolumeV2Kernel<T, I, HC>(V2_ARGS(I), cost, mask); });
    else
      sweep(count, nthreads, [&] { CostMinVolumeV2Kernel<T, I, HC>(V2_ARGS(I), cost, mask); });
  } else if (kind == 4) {
    if (!reduce_min)
      sweep(count, nthreads, [&] { CostMeanVolumeV3Kernel<T, I, HC>(V3_ARGS(I), cost, mask); });
    else
      sweep(count, nthreads, [&] { CostMinVolumeV3Kernel<T, I, HC>(V3_ARGS(I), cost, mask); });
  } else {
    if (!reduce_min)
      sweep(count, nthreads, [&] { CostMeanAggregateKernel<T, I, HC>(V1_ARGS(I), cost, mask); });
    else
      sweep(count, nthreads, [&] { CostMinAggregateKernel<T, I, HC>(V1_ARGS(I), cost, mask); });
  }
}

template <typename T, typename I, bool HC>
void bwd_t(int kind, int reduce_min, const Dims& s, int groups, const T* ref, const T* src,
           const T* depth, const T* offsets, const T* Rs, const T* Ts, const T* cost_grad,
           const int32* mask, T* ref_grad, T* src_grad, T* depth_grad, int nthreads) {
  const int64 count = s.B * s.H * s.W * s.D;
  std::memset(ref_grad, 0, sizeof(T) * s.B * s.H * s.W * s.C);
  std::memset(src_grad, 0, sizeof(T) * s.B * s.N * s.Hs * s.Ws * s.C);
  if (kind != 2) std::memset(depth_grad, 0, sizeof(T) * s.B * s.H * s.W);
  if (kind == 1) {
    if (!reduce_min)
      sweep(count, nthreads, [&] {
        CostMeanVolumeGradKernel<T, I, HC>(V1_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
    else
      sweep(count, nthreads, [&] {
        CostMinVolumeGradKernel<T, I, HC>(V1_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
  } else if (kind == 2) {
    if (!reduce_min)
      sweep(count, nthreads, [&] {
        CostMeanVolumeGradV2Kernel<T, I, HC>(V2_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
    else
      sweep(count, nthreads, [&] {
        CostMinVolumeGradV2Kernel<T, I, HC>(V2_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
  } else if (kind == 4) {
    if (!reduce_min)
      sweep(count, nthreads, [&] {
        CostMeanVolumeGradV3Kernel<T, I, HC>(V3_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
    else
      sweep(count, nthreads, [&] {
        CostMinVolumeGradV3Kernel<T, I, HC>(V3_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
  } else {
    if (!reduce_min)
      sweep(count, nthreads, [&] {
        CostMeanAggregateGradKernel<T, I, HC>(V1_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
    else
      sweep(count, nthreads, [&] {
        CostMinAggregateGradKernel<T, I, HC>(V1_ARGS(I), cost_grad, mask, ref_grad, src_grad, depth_grad);
      });
  }
}

int64 out_channels_of(int kind, const Dims& s, int groups) {
  return kind == 1 ? s.C : (kind == 2 ? groups : 1);
}

template <typename T>
void fwd_d(int kind, int reduce_min, int hc, const Dims& s, int groups, const void* ref,
           const void* src, const void* depth, const void* offsets, const void* Rs, const void* Ts,
           void* cost, int32* mask, int nthreads) {
  const bool big = needs_int64(s, out_channels_of(kind, s, groups));
#define CALL(I, HC)                                                                               \
  fwd_t<T, I, HC>(kind, reduce_min, s, groups, (const T*)ref, (const T*)src, (const T*)depth,     \
                  (const T*)offsets, (const T*)Rs, (const T*)Ts, (T*)cost, mask, nthreads)
  if (big) { if (hc) CALL(int64, true); else CALL(int64, false); }
  else     { if (hc) CALL(int32, true); else CALL(int32, false); }
#undef CALL
}

template <typename T>
void bwd_d(int kind, int reduce_min, int hc, const Dims& s, int groups, const void* ref,
           const void* src, const void* depth, const void* offsets, const void* Rs, const void* Ts,
           const void* cost_grad, const int32* mask, void* ref_grad, void* src_grad,
           void* depth_grad, int nthreads) {
  const bool big = needs_int64(s, out_channels_of(kind, s, groups));
#define CALL(I, HC)                                                                               \
  bwd_t<T, I, HC>(kind, reduce_min, s, groups, (const T*)ref, (const T*)src, (const T*)depth,     \
                  (const T*)offsets, (const T*)Rs, (const T*)Ts, (const T*)cost_grad, mask,       \
                  (T*)ref_grad, (T*)src_grad, (T*)depth_grad, nthreads)
  if (big) { if (hc) CALL(int64, true); else CALL(int64, false); }
  else     { if (hc) CALL(int32, true); else CALL(int32, false); }
#undef CALL
}

}  // namespace

extern "C" {

// dtype: 0 = float32, 1 = float64.  dims = {B,H,W,C,D,N,Hs,Ws}.
int ref_cost_fwd(int kind, int dtype, int reduce_min, int half_centor, const int64* dims,
                 int groups, const void* ref, const void* src, const void* depth,
                 const void* offsets, const void* Rs, const void* Ts, void* cost, int32* mask,
                 int nthreads) {
  Dims s{dims[0], dims[1], dims[2], dims[3], dims[4], dims[5], dims[6], dims[7]};
  if (dtype == 0)
    fwd_d<float>(kind, reduce_min, half_centor, s, groups, ref, src, depth, offsets, Rs, Ts, cost, mask, nthreads);
  else
    fwd_d<double>(kind, reduce_min, half_centor, s, groups, ref, src, depth, offsets, Rs, Ts, cost, mask, nthreads);
  return 0;
}

int ref_cost_bwd(int kind, int dtype, int reduce_min, int half_centor, const int64* dims,
                 int groups, const void* ref, const void* src, const void* depth,
                 const void* offsets, const void* Rs, const void* Ts, const void* cost_grad,
                 const int32* mask, void* ref_grad, void* src_grad, void* depth_grad,
                 int nthreads) {
  Dims s{dims[0], dims[1], dims[2], dims[3], dims[4], dims[5], dims[6], dims[7]};
  if (dtype == 0)
    bwd_d<float>(kind, reduce_min, half_centor, s, groups, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, ref_grad, src_grad, depth_grad, nthreads);
  else
    bwd_d<double>(kind, reduce_min, half_centor, s, groups, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, ref_grad, src_grad, depth_grad, nthreads);
  return 0;
}

// The reference's older thread-per-voxel manifold convolution (runtime filter/stride/dilation
// instantiation <-1,...>), custom_helper_op/cc/kernels/sparse_conv3d_kernels_gpu.cu.cc:75-163.
// p = {stride h,w,d, dilation h,w,d, filter h,w,d, B, H, W, D, Cin, outH, outW, outD, Cout}.
int ref_sparse_conv3d_fwd(int dtype, const int* p, const void* images, const void* filter,
                          const void* default_value, const int32* base_plane, void* out,
                          int nthreads) {
  const int64 count = (int64)p[9] * p[14] * p[15] * p[16];
#define SC_ARGS p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7], p[8], p[9], p[10], p[11], p[12], p[13], p[14], p[15], p[16], p[17]
  if (dtype == 0)
    sweep(count, nthreads, [&] {
      SparseConv3DKernel<float, int64, -1, -1, -1, -1, -1, -1, -1, -1, -1>(
          count, SC_ARGS, (const float*)images, (const float*)filter, (const float*)default_value,
          base_plane, (float*)out);
    });
  else
    sweep(count, nthreads, [&] {
      SparseConv3DKernel<double, int64, -1, -1, -1, -1, -1, -1, -1, -1, -1>(
          count, SC_ARGS, (const double*)images, (const double*)filter,
          (const double*)default_value, base_plane, (double*)out);
    });
#undef SC_ARGS
  return 0;
}

// SparsePad / SparsePadGrad (custom_helper_op/cc/kernels/sparse_pad_kernels_gpu.cu.cc:36-64, 82-104).
// q = {stride h,w,d, B, coarse H,W,D, C, fine H,W,D}.
int ref_sparse_pad_fwd(int dtype, const int* q, const void* images, const int32* base_plane, void* out) {
  const int32 count = q[3] * q[8] * q[9] * q[10];
#define PAD_ARGS q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7], q[8], q[9], q[10]
  if (dtype == 0)
    sweep(count, 1, [&] { SparsePadKernel<float, int32>(count, PAD_ARGS, (const float*)images, base_plane, (float*)out); });
  else
    sweep(count, 1, [&] { SparsePadKernel<double, int32>(count, PAD_ARGS, (const double*)images, base_plane, (double*)out); });
  return 0;
}
int ref_sparse_pad_bwd(int dtype, const int* q, const void* images, const int32* base_plane, const void* out_grad,
                       void* images_grad) {
  const int32 count = q[3] * q[4] * q[5] * q[6];
  if (dtype == 0)
    sweep(count, 1, [&] {
      SparsePadGradKernel<float, int32>(count, PAD_ARGS, (const float*)images, base_plane, (const float*)out_grad,
                                        (float*)images_grad);
    });
  else
    sweep(count, 1, [&] {
      SparsePadGradKernel<double, int32>(count, PAD_ARGS, (const double*)images, base_plane, (const double*)out_grad,
                                         (double*)images_grad);
    });
#undef PAD_ARGS
  return 0;
}

// FeatureAggregate / FeatureAggregateGrad (custom_helper_op/cc/kernels/feature_aggregate_kernels_gpu.cu.cc:33-121,
// 219-317), with the int32/int64 choice and the zero fill of the gradient functor (:337-383).
// dims = {B, H, W, C, D, N, Hs, Ws}: (H, W) is the output grid (base_plane), (Hs, Ws) the source images.
int ref_feature_aggregate_fwd(int dtype, int half_centor, const int64* dims, const void* src, const void* base,
                              const void* offsets, const void* Rs, const void* Ts, void* mapped, int32* mask, int nthreads) {
  Dims s{dims[0], dims[1], dims[2], dims[3], dims[4], dims[5], dims[6], dims[7]};
  const int64 count = s.B * s.H * s.W * s.D;
  const bool big = s.B * s.H * s.W * s.C > INT32_MAX || s.B * s.N * s.Hs * s.Ws * s.C > INT32_MAX || count > INT32_MAX;
#define FA_ARGS(I, T) (I) count, (I)s.B, (I)s.H, (I)s.W, (I)s.C, (I)s.D, (I)s.N, (I)s.Hs, (I)s.Ws, (const T*)src, (const T*)base, \
                      (const T*)offsets, (const T*)Rs, (const T*)Ts
#define FA_FWD(T, I, HC) sweep(count, nthreads, [&] { FeatureAggregateKernel<T, I, HC>(FA_ARGS(I, T), (T*)mapped, mask); })
#define FA_PICK(M, T)                                                                  \
  do {                                                                                 \
    if (big) { if (half_centor) M(T, int64, true); else M(T, int64, false); }          \
    else     { if (half_centor) M(T, int32, true); else M(T, int32, false); }          \
  } while (0)
  if (dtype == 0) FA_PICK(FA_FWD, float); else FA_PICK(FA_FWD, double);
  return 0;
}

int ref_feature_aggregate_bwd(int dtype, int half_centor, const int64* dims, const void* src, const void* base,
                              const void* offsets, const void* Rs, const void* Ts, const void* mapped_grad,
                              const int32* mask, void* src_grad, void* base_grad, int nthreads) {
  Dims s{dims[0], dims[1], dims[2], dims[3], dims[4], dims[5], dims[6], dims[7]};
  const int64 count = s.B * s.H * s.W * s.D;
  const bool big = s.B * s.H * s.W * s.C > INT32_MAX || s.B * s.N * s.Hs * s.Ws * s.C > INT32_MAX || count > INT32_MAX;
  const size_t el = dtype == 0 ? 4 : 8;
  std::memset(src_grad, 0, el * s.B * s.N * s.Hs * s.Ws * s.C);
  std::memset(base_grad, 0, el * s.B * s.H * s.W);
#define FA_BWD(T, I, HC)                                                                                            \
  sweep(count, nthreads, [&] {                                                                                      \
    FeatureAggregateGradKernel<T, I, HC>(FA_ARGS(I, T), (const T*)mapped_grad, mask, (T*)src_grad, (T*)base_grad);  \
  })
  if (dtype == 0) FA_PICK(FA_BWD, float); else FA_PICK(FA_BWD, double);
#undef FA_BWD
#undef FA_FWD
#undef FA_PICK
#undef FA_ARGS
  return 0;
}

// IndexInitializer (custom_helper_op/cc/kernels/index_initializer_kernels_gpu.cu.cc:21-29): out [H,W,3] = (column, row, 1),
// plus 0.5 on the first two when half_centor.
int ref_index_initializer(int dtype, int half_centor, int H, int W, void* out) {
  const int32 count = H * W;
  if (dtype == 0) {
    if (half_centor) sweep(count, 1, [&] { SetToIndex<float, true>(count, (float*)out, W); });
    else sweep(count, 1, [&] { SetToIndex<float, false>(count, (float*)out, W); });
  } else {
    if (half_centor) sweep(count, 1, [&] { SetToIndex<double, true>(count, (double*)out, W); });
    else sweep(count, 1, [&] { SetToIndex<double, false>(count, (double*)out, W); });
  }
  return 0;
}

int ref_max_threads(void) { return omp_get_max_threads(); }
}
