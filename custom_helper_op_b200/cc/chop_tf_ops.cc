// TensorFlow binding of libchop_b200.so: op registrations and GPU OpKernels for the cost-volume path,
// written against the C ABI in include/chop.h.  Built only where TensorFlow headers exist:
//
//   g++ -std=c++17 -shared -fPIC chop_tf_ops.cc -o _custom_helper_ops.so \
//       $(python -c 'import tensorflow as tf; print(" ".join(tf.sysconfig.get_compile_flags()+tf.sysconfig.get_link_flags()))') \
//       -I<repo>/include -L<repo>/custom_helper_op_b200 -lchop_b200 -DGOOGLE_CUDA=1
//
// Op names, input order, attrs and output shapes are those of the reference project
// (custom_helper_op/cc/ops/custom_helper_ops.cc:190-307 CostVolume*, :311-371 CostVolumeV3*, :374-411
// CostAggregate*, :498-535 SparsePad*, :590-641 SparseConv3DFast*, :644-715 SparseConv3DTransposeFast*), so its
// Python wrapper and its tf.RegisterGradient functions work unchanged.  The
// As in the reference only DEVICE_GPU kernels are registered (DecodePfm is a host op there and here).
#include <string>
#include <vector>

#include "chop.h"
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/shape_inference.h"
#include "tensorflow/core/util/gpu_kernel_helper.h"

namespace tensorflow {
namespace chop_b200 {

using shape_inference::InferenceContext;
using shape_inference::ShapeHandle;

// ---- schema ---------------------------------------------------------------------------------------------
namespace {

// cost [B,H,W,D,last], mask [B,H,W,D,1 (MEAN) | last (MIN)]
Status CostShapes(InferenceContext* c, bool v2, bool aggregate) {
  ShapeHandle ref, depth;
  TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 4, &ref));
  std::string reduce;
  TF_RETURN_IF_ERROR(c->GetAttr("reduce_method", &reduce));
  shape_inference::DimensionHandle planes, last;
  if (v2) {
    TF_RETURN_IF_ERROR(c->WithRank(c->input(2), 4, &depth));
    planes = c->Dim(depth, 3);
    int groups;
    TF_RETURN_IF_ERROR(c->GetAttr("groups", &groups));
    last = c->MakeDim(groups);
  } else {
    TF_RETURN_IF_ERROR(c->WithRank(c->input(3), 2, &depth));
    planes = c->Dim(depth, 1);
    last = c->Dim(ref, 3);
  }
  std::vector<shape_inference::DimensionHandle> dims = {c->Dim(ref, 0), c->Dim(ref, 1), c->Dim(ref, 2), planes};
  if (aggregate) {
    c->set_output(0, c->MakeShape(dims));
    c->set_output(1, c->MakeShape(dims));
    return Status::OK();
  }
  auto cost = dims, mask = dims;
  cost.push_back(last);
  mask.push_back(reduce == "MEAN" ? c->MakeDim(1) : last);
  c->set_output(0, c->MakeShape(cost));
  c->set_output(1, c->MakeShape(mask));
  return Status::OK();
}

Status GradLikeInputs(InferenceContext* c) {
  for (int i = 0; i < 3; ++i) c->set_output(i, c->input(i));
  return Status::OK();
}

}  // namespace

// The reference's dtype list.  bfloat16 features are reachable through the C ABI and the torch wrapper only: that
// mode keeps depths, cameras, cost and all gradients in float32 (include/chop.h), which a schema with one type
// attribute cannot express, and this binding registers no kernel for it.
#define CHOP_FLOAT_TYPES "{float, double}"

REGISTER_OP("CostVolume")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype")
    .Input("rs: dtype").Input("ts: dtype")
    .Output("cost: dtype").Output("cost_mask: int32")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("half_centor: bool = true")
    .SetShapeFn([](InferenceContext* c) { return CostShapes(c, false, false); });

REGISTER_OP("CostVolumeGrad")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype")
    .Input("rs: dtype").Input("ts: dtype").Input("cost_grad: dtype").Input("cost_mask: int32")
    .Output("ref_image_grad: dtype").Output("src_images_grad: dtype").Output("base_plane_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("half_centor: bool = true")
    .SetShapeFn(GradLikeInputs);

REGISTER_OP("CostVolumeV2")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("depth_grid: dtype").Input("rs: dtype").Input("ts: dtype")
    .Output("cost: dtype").Output("cost_mask: int32")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("groups: int")
    .Attr("half_centor: bool = true")
    .SetShapeFn([](InferenceContext* c) { return CostShapes(c, true, false); });

REGISTER_OP("CostVolumeGradV2")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("depth_grid: dtype").Input("rs: dtype").Input("ts: dtype")
    .Input("cost_grad: dtype").Input("cost_mask: int32")
    .Output("ref_image_grad: dtype").Output("src_images_grad: dtype").Output("base_plane_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("groups: int")
    .Attr("half_centor: bool = true")
    .SetShapeFn(GradLikeInputs);

REGISTER_OP("CostAggregate")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype")
    .Input("rs: dtype").Input("ts: dtype")
    .Output("cost: dtype").Output("cost_mask: int32")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("half_centor: bool = true")
    .SetShapeFn([](InferenceContext* c) { return CostShapes(c, false, true); });

REGISTER_OP("CostAggregateGrad")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype")
    .Input("rs: dtype").Input("ts: dtype").Input("cost_grad: dtype").Input("cost_mask: int32")
    .Output("ref_image_grad: dtype").Output("src_images_grad: dtype").Output("base_plane_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("half_centor: bool = true")
    .SetShapeFn(GradLikeInputs);

REGISTER_OP("CostVolumeV3")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype")
    .Input("rs: dtype").Input("ts: dtype")
    .Output("cost: dtype").Output("cost_mask: int32")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("groups: int")
    .Attr("half_centor: bool = true")
    .SetShapeFn([](InferenceContext* c) {
      // cost [B,H,W,D,1]; mask [B,H,W,D,1] (MEAN) or [B,H,W,D,3] (MIN): custom_helper_ops.cc:311-371 of the reference
      std::string reduce;
      TF_RETURN_IF_ERROR(c->GetAttr("reduce_method", &reduce));
      ShapeHandle ref, offs;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 4, &ref));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(3), 2, &offs));
      c->set_output(0, c->MakeShape({c->Dim(ref, 0), c->Dim(ref, 1), c->Dim(ref, 2), c->Dim(offs, 1), c->MakeDim(1)}));
      c->set_output(1, c->MakeShape({c->Dim(ref, 0), c->Dim(ref, 1), c->Dim(ref, 2), c->Dim(offs, 1),
                                     c->MakeDim(reduce == "MIN" ? 3 : 1)}));
      return Status::OK();
    });

REGISTER_OP("CostVolumeGradV3")
    .Input("ref_image: dtype").Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype")
    .Input("rs: dtype").Input("ts: dtype").Input("cost_grad: dtype").Input("cost_mask: int32")
    .Output("ref_image_grad: dtype").Output("src_images_grad: dtype").Output("base_plane_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("reduce_method: {'MEAN', 'MIN'}").Attr("groups: int")
    .Attr("half_centor: bool = true")
    .SetShapeFn(GradLikeInputs);

REGISTER_OP("SparseConv3DTransposeFast")
    .Input("images: dtype").Input("filters: dtype").Input("default_value: dtype").Input("base_plane: int32")
    .Input("output_size: int32")
    .Output("output: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("strides: list(int)").Attr("dilations: list(int)")
    .Attr("dynamic_default: bool").Attr("data_format: { 'NDHWC' }")
    .SetShapeFn([](InferenceContext* c) {
      ShapeHandle img, flt, size;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 5, &img));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 5, &flt));
      TF_RETURN_IF_ERROR(c->MakeShapeFromShapeTensor(4, &size));
      TF_RETURN_IF_ERROR(c->WithRank(size, 3, &size));
      c->set_output(0, c->MakeShape({c->Dim(img, 0), c->Dim(size, 0), c->Dim(size, 1), c->Dim(size, 2), c->Dim(flt, 3)}));
      return Status::OK();
    });

REGISTER_OP("SparseConv3DTransposeFastGrad")
    .Input("images: dtype").Input("filters: dtype").Input("default_value: dtype").Input("base_plane: int32")
    .Input("output_size: int32").Input("out_grad: dtype")
    .Output("images_grad: dtype").Output("filter_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("strides: list(int)").Attr("dilations: list(int)")
    .Attr("dynamic_default: bool").Attr("data_format: { 'NDHWC' }")
    .SetShapeFn([](InferenceContext* c) {
      c->set_output(0, c->input(0));
      c->set_output(1, c->input(1));
      return Status::OK();
    });

REGISTER_OP("SparsePad")
    .Input("images: dtype").Input("base_plane: int32")
    .Output("output: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("strides: list(int)").Attr("dilations: list(int)")
    .SetShapeFn([](InferenceContext* c) {
      std::vector<int32> s;
      TF_RETURN_IF_ERROR(c->GetAttr("strides", &s));
      ShapeHandle img;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 5, &img));
      std::vector<shape_inference::DimensionHandle> out = {c->Dim(img, 0)};
      for (int i = 0; i < 3; ++i) {
        const int64 n = c->Value(c->Dim(img, 1 + i));
        out.push_back(n < 0 ? c->UnknownDim() : c->MakeDim(n * s[i]));
      }
      out.push_back(c->Dim(img, 4));
      c->set_output(0, c->MakeShape(out));
      return Status::OK();
    });

REGISTER_OP("SparsePadGrad")
    .Input("images: dtype").Input("base_plane: int32").Input("out_grad: dtype")
    .Output("images_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("strides: list(int)").Attr("dilations: list(int)")
    .SetShapeFn([](InferenceContext* c) {
      c->set_output(0, c->input(0));
      return Status::OK();
    });

REGISTER_OP("SparseConv3DFast")
    .Input("images: dtype").Input("filters: dtype").Input("default_value: dtype").Input("base_plane: int32")
    .Output("output: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("strides: list(int)").Attr("dilations: list(int)")
    .Attr("dynamic_default: bool").Attr("data_format: { 'NDHWC' }")
    .SetShapeFn([](InferenceContext* c) {
      std::vector<int32> s;
      TF_RETURN_IF_ERROR(c->GetAttr("strides", &s));
      ShapeHandle img, flt;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 5, &img));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 5, &flt));
      std::vector<shape_inference::DimensionHandle> out = {c->Dim(img, 0)};
      for (int i = 0; i < 3; ++i) {
        const int64 n = c->Value(c->Dim(img, 1 + i));
        out.push_back(n < 0 ? c->UnknownDim() : c->MakeDim((n + s[i] - 1) / s[i]));
      }
      out.push_back(c->Dim(flt, 4));
      c->set_output(0, c->MakeShape(out));
      return Status::OK();
    });

REGISTER_OP("SparseConv3DFastGrad")
    .Input("images: dtype").Input("filters: dtype").Input("default_value: dtype").Input("base_plane: int32")
    .Input("out_grad: dtype")
    .Output("images_grad: dtype").Output("filter_grad: dtype").Output("default_value_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("strides: list(int)").Attr("dilations: list(int)")
    .Attr("dynamic_default: bool").Attr("data_format: { 'NDHWC' }")
    .SetShapeFn(GradLikeInputs);

#if GOOGLE_CUDA
REGISTER_OP("FeatureAggregate")
    .Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype").Input("rs: dtype").Input("ts: dtype")
    .Output("mapped_feature: dtype").Output("mapped_mask: int32")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("half_centor: bool")
    .SetShapeFn([](InferenceContext* c) {
      // [B,H,W,D,N,C] and [B,H,W,D,N,1]: custom_helper_ops.cc:414-441 of the reference
      ShapeHandle src, base, offs;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 5, &src));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 4, &base));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(2), 2, &offs));
      c->set_output(0, c->MakeShape({c->Dim(src, 0), c->Dim(base, 1), c->Dim(base, 2), c->Dim(offs, 1), c->Dim(src, 1),
                                     c->Dim(src, 4)}));
      c->set_output(1, c->MakeShape({c->Dim(src, 0), c->Dim(base, 1), c->Dim(base, 2), c->Dim(offs, 1), c->Dim(src, 1),
                                     c->MakeDim(1)}));
      return Status::OK();
    });

REGISTER_OP("FeatureAggregateGrad")
    .Input("src_images: dtype").Input("base_plane: dtype").Input("offsets: dtype").Input("rs: dtype").Input("ts: dtype")
    .Input("mapped_feature_grad: dtype").Input("mapped_mask: int32")
    .Output("src_images_grad: dtype").Output("base_plane_grad: dtype")
    .Attr("dtype: " CHOP_FLOAT_TYPES).Attr("half_centor: bool")
    .SetShapeFn([](InferenceContext* c) {
      c->set_output(0, c->input(0));
      c->set_output(1, c->input(1));
      return Status::OK();
    });

REGISTER_OP("IndexInitializer")
    .Input("output_shape: int32")
    .Output("output: dtype")
    .Attr("half_centor: bool").Attr("dtype: " CHOP_FLOAT_TYPES)
    .SetShapeFn([](InferenceContext* c) {
      ShapeHandle out;
      TF_RETURN_IF_ERROR(c->MakeShapeFromShapeTensor(0, &out));   // (height, width, 3)
      TF_RETURN_IF_ERROR(c->WithRank(out, 3, &out));
      c->set_output(0, out);
      return Status::OK();
    });

REGISTER_OP("DecodePfm")
    .Input("input: string")
    .Output("image: float")
    .SetShapeFn([](InferenceContext* c) {
      ShapeHandle unused;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 0, &unused));
      c->set_output(0, c->MakeShape({c->UnknownDim(), c->UnknownDim(), c->MakeDim(1)}));
      return Status::OK();
    });

// ---- kernels ---------------------------------------------------------------------------------------------
namespace {

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = CHOP_F32; };
template <> struct DtypeOf<double> { static constexpr int value = CHOP_F64; };
inline const void* In(OpKernelContext* ctx, int i) { return ctx->input(i).tensor_data().data(); }
inline void* Out(Tensor* t) { return const_cast<char*>(t->tensor_data().data()); }
inline void* StreamOf(OpKernelContext* ctx) { return ctx->eigen_device<Eigen::GpuDevice>().stream(); }

}  // namespace

// kind: CHOP_COST_VOLUME / _V2 / _AGGREGATE / _V3;  gradient: the *Grad op
template <typename T, int KIND, bool GRADIENT>
class CostOp : public OpKernel {
 public:
  explicit CostOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    std::string reduce;
    OP_REQUIRES_OK(ctx, ctx->GetAttr("reduce_method", &reduce));
    OP_REQUIRES(ctx, reduce == "MEAN" || reduce == "MIN",
                errors::InvalidArgument("Invalid reduce method ", reduce, ". Supported types: MEAN, MIN"));
    min_ = reduce == "MIN";
    OP_REQUIRES_OK(ctx, ctx->GetAttr("half_centor", &half_centor_));
    if (KIND == CHOP_COST_VOLUME_V2 || KIND == CHOP_COST_VOLUME_V3) OP_REQUIRES_OK(ctx, ctx->GetAttr("groups", &groups_));
  }

  void Compute(OpKernelContext* ctx) override {
    constexpr bool V2 = KIND == CHOP_COST_VOLUME_V2;
    const Tensor& ref = ctx->input(0);
    const Tensor& src = ctx->input(1);
    const Tensor& depth = ctx->input(2);
    const int cam0 = V2 ? 3 : 4;  // index of rs
    OP_REQUIRES(ctx, ref.dims() == 4, errors::InvalidArgument("ref image must have rank 4"));
    const int64 B = ref.dim_size(0), H = ref.dim_size(1), W = ref.dim_size(2), C = ref.dim_size(3);
    OP_REQUIRES(ctx, src.dims() == 5 && src.dim_size(0) == B && src.dim_size(2) == H && src.dim_size(3) == W &&
                         src.dim_size(4) == C,
                errors::InvalidArgument("src_images must have rank 5, and must compate to ref_image"));
    const int64 N = src.dim_size(1);
    int64 D;
    if (V2) {
      OP_REQUIRES(ctx, depth.dims() == 4 && depth.dim_size(0) == B && depth.dim_size(1) == H && depth.dim_size(2) == W,
                  errors::InvalidArgument("depth_grid must have rank 4, and must compate to ref_image"));
      D = depth.dim_size(3);
      OP_REQUIRES(ctx, groups_ > 0 && C % groups_ == 0, errors::InvalidArgument("channels must be divisible by groups"));
    } else {
      const Tensor& offsets = ctx->input(3);
      OP_REQUIRES(ctx, depth.dims() == 4 && depth.dim_size(0) == B && depth.dim_size(1) == H && depth.dim_size(2) == W &&
                           depth.dim_size(3) == 1,
                  errors::InvalidArgument("base_plane must have rank 4, and must compate to ref_image"));
      OP_REQUIRES(ctx, offsets.dims() == 2 && offsets.dim_size(0) == B,
                  errors::InvalidArgument("offsets must have rank 2, and must compate to ref_image"));
      D = offsets.dim_size(1);
      if (KIND == CHOP_COST_VOLUME_V3) {   // cost_volume_kernels_v3.cc:107-111
        OP_REQUIRES(ctx, groups_ > 0 && C % groups_ == 0, errors::InvalidArgument("image_channels and groups_ must match"));
        OP_REQUIRES(ctx, C / groups_ <= 8, errors::InvalidArgument("image_channels / groups_ less than MAX_SUBCHANNELS_SIZE(8)"));
      }
    }
    const Tensor& Rs = ctx->input(cam0);
    const Tensor& Ts = ctx->input(cam0 + 1);
    OP_REQUIRES(ctx, Rs.dims() == 4 && Rs.dim_size(0) == B && Rs.dim_size(1) == N && Rs.dim_size(2) == 3 && Rs.dim_size(3) == 3,
                errors::InvalidArgument("Rs must have rank 4, and must compate to ref_image"));
    OP_REQUIRES(ctx, Ts.dims() == 3 && Ts.dim_size(0) == B && Ts.dim_size(1) == N && Ts.dim_size(2) == 3,
                errors::InvalidArgument("Ts must have rank 3, and must compate to ref_image"));

    chop_cv_desc d = {};
    d.kind = KIND;
    d.dtype = DtypeOf<T>::value;
    d.reduce = min_ ? CHOP_REDUCE_MIN : CHOP_REDUCE_MEAN;
    d.half_centor = half_centor_;
    d.groups = groups_;
    d.B = B; d.H = H; d.W = W; d.C = C; d.D = D; d.N = N; d.Hs = src.dim_size(2); d.Ws = src.dim_size(3);
    const int64 last = KIND == CHOP_COST_VOLUME ? C : (V2 ? groups_ : 1);
    const int64 mask_last = !min_ ? 1 : (KIND == CHOP_COST_VOLUME_V3 ? 3 : last);
    const void* offsets = V2 ? nullptr : In(ctx, 3);
    int status;
    if (!GRADIENT) {
      TensorShape cs({B, H, W, D}), ms({B, H, W, D});
      if (KIND != CHOP_COST_AGGREGATE) {
        cs.AddDim(last);
        ms.AddDim(mask_last);
      }
      Tensor *cost = nullptr, *mask = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, cs, &cost));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(1, ms, &mask));
      status = chop_cost_volume_fwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), offsets, In(ctx, cam0), In(ctx, cam0 + 1), Out(cost),
                                    static_cast<int32_t*>(Out(mask)), StreamOf(ctx));
    } else {
      const Tensor& cost_grad = ctx->input(cam0 + 2);
      const Tensor& cost_mask = ctx->input(cam0 + 3);
      OP_REQUIRES(ctx, cost_grad.NumElements() == B * H * W * D * last,
                  errors::InvalidArgument("cost_grad must have rank 5, and must compate to ref_image"));
      OP_REQUIRES(ctx, cost_mask.NumElements() == B * H * W * D * mask_last,
                  errors::InvalidArgument("cost_mask must be the mask returned by the forward op"));
      Tensor *rg = nullptr, *sg = nullptr, *dg = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, ref.shape(), &rg));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(1, src.shape(), &sg));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(2, depth.shape(), &dg));
      status = chop_cost_volume_bwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), offsets, In(ctx, cam0), In(ctx, cam0 + 1),
                                    In(ctx, cam0 + 2), static_cast<const int32_t*>(In(ctx, cam0 + 3)), Out(rg), Out(sg), Out(dg),
                                    StreamOf(ctx));
    }
    OP_REQUIRES(ctx, status == 0, errors::Internal("libchop_b200: ", chop_status_string(status)));
  }

 private:
  bool min_ = false;
  bool half_centor_ = true;
  int groups_ = 1;
};

template <typename T, bool GRADIENT>
class ManifoldConvOp : public OpKernel {
 public:
  explicit ManifoldConvOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("strides", &strides_));
    OP_REQUIRES_OK(ctx, ctx->GetAttr("dilations", &dilations_));
    OP_REQUIRES_OK(ctx, ctx->GetAttr("dynamic_default", &dynamic_default_));
    OP_REQUIRES(ctx, strides_.size() == 3, errors::InvalidArgument("strides must be a vector have 3 element"));
    OP_REQUIRES(ctx, dilations_.size() == 3, errors::InvalidArgument("dilations must be a vector have 3 element"));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& images = ctx->input(0);
    const Tensor& filters = ctx->input(1);
    const Tensor& defv = ctx->input(2);
    const Tensor& base_plane = ctx->input(3);
    OP_REQUIRES(ctx, TensorShapeUtils::IsScalar(defv.shape()), errors::InvalidArgument("default_value must be scalar"));
    OP_REQUIRES(ctx, images.dims() == 5, errors::InvalidArgument("images must have rank 5"));
    OP_REQUIRES(ctx, filters.dims() == 5, errors::InvalidArgument("filter must have rank 5"));
    OP_REQUIRES(ctx, images.dim_size(4) == filters.dim_size(3), errors::InvalidArgument("images channel size wrong"));
    chop_sc_desc d = {};
    d.dtype = DtypeOf<T>::value;
    d.dynamic_default = dynamic_default_;
    d.B = images.dim_size(0); d.H = images.dim_size(1); d.W = images.dim_size(2); d.D = images.dim_size(3);
    d.Cin = images.dim_size(4); d.Cout = filters.dim_size(4);
    for (int i = 0; i < 3; ++i) {
      d.filter[i] = filters.dim_size(i);
      d.strides[i] = strides_[i];
      d.dilations[i] = dilations_[i];
    }
    OP_REQUIRES(ctx, base_plane.dims() == 4 && base_plane.dim_size(0) == d.B && base_plane.dim_size(1) == d.H &&
                         base_plane.dim_size(2) == d.W && base_plane.dim_size(3) == 1,
                errors::InvalidArgument("base_plane must have rank 4, and must compate to ref_image"));
    TensorShape out_shape({d.B, (d.H + strides_[0] - 1) / strides_[0], (d.W + strides_[1] - 1) / strides_[1],
                           (d.D + strides_[2] - 1) / strides_[2], d.Cout});
    int status;
    if (!GRADIENT) {
      Tensor* out = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, out_shape, &out));
      status = chop_sparse_conv3d_fwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), static_cast<const int32_t*>(In(ctx, 3)), Out(out),
                                      StreamOf(ctx));
    } else {
      const Tensor& out_grad = ctx->input(4);
      OP_REQUIRES(ctx, out_grad.shape() == out_shape, errors::InvalidArgument("out_grad must have rank 5, and must compate to ref_image"));
      Tensor *ig = nullptr, *fg = nullptr, *dg = nullptr, ws;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, images.shape(), &ig));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(1, filters.shape(), &fg));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(2, defv.shape(), &dg));
      const int64 ws_bytes = chop_sparse_conv3d_bwd_workspace_size(&d);
      OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_UINT8, TensorShape({ws_bytes}), &ws));
      status = chop_sparse_conv3d_bwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), static_cast<const int32_t*>(In(ctx, 3)), In(ctx, 4),
                                      Out(ig), Out(fg), Out(dg), Out(&ws), ws_bytes, StreamOf(ctx));
    }
    OP_REQUIRES(ctx, status == 0, errors::Internal("libchop_b200: ", chop_status_string(status)));
  }

 private:
  std::vector<int32> strides_, dilations_;
  bool dynamic_default_ = false;
};

// SparseConv3DTransposeFast / ...Grad (reference: sparse_conv3d_fast_op.cc:346-411, 427-505).  The descriptor is that of
// the forward convolution whose transpose is taken: its input grid is output_size, its output grid the op's images.
template <typename T, bool GRADIENT>
class ManifoldConvTransposeOp : public OpKernel {
 public:
  explicit ManifoldConvTransposeOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("strides", &strides_));
    OP_REQUIRES_OK(ctx, ctx->GetAttr("dilations", &dilations_));
    OP_REQUIRES(ctx, strides_.size() == 3, errors::InvalidArgument("strides must be a vector have 3 element"));
    OP_REQUIRES(ctx, dilations_.size() == 3, errors::InvalidArgument("dilations must be a vector have 3 element"));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& images = ctx->input(0);
    const Tensor& filters = ctx->input(1);
    const Tensor& defv = ctx->input(2);
    const Tensor& base_plane = ctx->input(3);
    const Tensor& size = ctx->input(4);   // host memory
    OP_REQUIRES(ctx, TensorShapeUtils::IsScalar(defv.shape()), errors::InvalidArgument("default_value must be scalar"));
    OP_REQUIRES(ctx, images.dims() == 5, errors::InvalidArgument("images must have rank 5"));
    OP_REQUIRES(ctx, filters.dims() == 5, errors::InvalidArgument("filter must have rank 5"));
    OP_REQUIRES(ctx, size.dims() == 1 && size.dim_size(0) == 3,
                errors::InvalidArgument("output_shape must be an 1-D vector of (height, width, depth)"));
    OP_REQUIRES(ctx, images.dim_size(4) == filters.dim_size(4), errors::InvalidArgument("images channel size wrong"));
    const auto sv = size.vec<int32>();
    chop_sc_desc d = {};
    d.dtype = DtypeOf<T>::value;
    d.B = images.dim_size(0); d.H = sv(0); d.W = sv(1); d.D = sv(2);
    d.Cin = filters.dim_size(3); d.Cout = filters.dim_size(4);
    for (int i = 0; i < 3; ++i) {
      d.filter[i] = filters.dim_size(i);
      d.strides[i] = strides_[i];
      d.dilations[i] = dilations_[i];
    }
    OP_REQUIRES(ctx, base_plane.dims() == 4 && base_plane.dim_size(0) == d.B && base_plane.dim_size(1) == d.H &&
                         base_plane.dim_size(2) == d.W && base_plane.dim_size(3) == 1,
                errors::InvalidArgument("base_plane must have rank 4, and must compate to ref_image"));
    OP_REQUIRES(ctx, images.dim_size(1) == (d.H + strides_[0] - 1) / strides_[0] &&
                         images.dim_size(2) == (d.W + strides_[1] - 1) / strides_[1] &&
                         images.dim_size(3) == (d.D + strides_[2] - 1) / strides_[2],
                errors::InvalidArgument("images shape and output_shape does not compate"));
    const TensorShape fine({d.B, d.H, d.W, d.D, d.Cin});
    int status;
    if (!GRADIENT) {
      Tensor* out = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, fine, &out));
      status = chop_sparse_conv3d_transpose_fwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), static_cast<const int32_t*>(In(ctx, 3)),
                                                Out(out), StreamOf(ctx));
    } else {
      const Tensor& out_grad = ctx->input(5);
      OP_REQUIRES(ctx, out_grad.shape() == fine, errors::InvalidArgument("out_grad must have rank 5, and must compate to ref_image"));
      Tensor *ig = nullptr, *fg = nullptr, ws;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, images.shape(), &ig));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(1, filters.shape(), &fg));
      const int64 ws_bytes = chop_sparse_conv3d_transpose_bwd_workspace_size(&d);
      OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_UINT8, TensorShape({ws_bytes}), &ws));
      status = chop_sparse_conv3d_transpose_bwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), static_cast<const int32_t*>(In(ctx, 3)),
                                                In(ctx, 5), Out(ig), Out(fg), Out(&ws), ws_bytes, StreamOf(ctx));
    }
    OP_REQUIRES(ctx, status == 0, errors::Internal("libchop_b200: ", chop_status_string(status)));
  }

 private:
  std::vector<int32> strides_, dilations_;
};

// SparsePad / SparsePadGrad (reference: sparse_pad_kernels.cc:76-130, 150-210).
template <typename T, bool GRADIENT>
class ManifoldPadOp : public OpKernel {
 public:
  explicit ManifoldPadOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("strides", &strides_));
    OP_REQUIRES(ctx, strides_.size() == 3, errors::InvalidArgument("strides must be a vector have 3 element"));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& images = ctx->input(0);
    const Tensor& base_plane = ctx->input(1);
    OP_REQUIRES(ctx, images.dims() == 5, errors::InvalidArgument("images must have rank 5"));
    const int64 B = images.dim_size(0), h = images.dim_size(1), w = images.dim_size(2), dd = images.dim_size(3),
                C = images.dim_size(4);
    const int32_t s[3] = {strides_[0], strides_[1], strides_[2]};
    OP_REQUIRES(ctx, base_plane.dims() == 4 && base_plane.dim_size(0) == B && base_plane.dim_size(1) == h * s[0] &&
                         base_plane.dim_size(2) == w * s[1] && base_plane.dim_size(3) == 1,
                errors::InvalidArgument("base_plane must have rank 4, and must compate to ref_image"));
    const TensorShape fine({B, h * s[0], w * s[1], dd * s[2], C});
    int status;
    if (!GRADIENT) {
      Tensor* out = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, fine, &out));
      status = chop_sparse_pad_fwd(DtypeOf<T>::value, B, h, w, dd, C, s, In(ctx, 0), static_cast<const int32_t*>(In(ctx, 1)),
                                   Out(out), StreamOf(ctx));
    } else {
      OP_REQUIRES(ctx, ctx->input(2).shape() == fine, errors::InvalidArgument("out_grad must compate to the padded shape"));
      Tensor* ig = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, images.shape(), &ig));
      status = chop_sparse_pad_bwd(DtypeOf<T>::value, B, h, w, dd, C, s, static_cast<const int32_t*>(In(ctx, 1)), In(ctx, 2),
                                   Out(ig), StreamOf(ctx));
    }
    OP_REQUIRES(ctx, status == 0, errors::Internal("libchop_b200: ", chop_status_string(status)));
  }

 private:
  std::vector<int32> strides_;
};

// FeatureAggregate / FeatureAggregateGrad (reference kernels: feature_aggregate_kernels.cc:60-130,170-250)
template <typename T, bool GRADIENT>
class FeatureAggregateOp : public OpKernel {
 public:
  explicit FeatureAggregateOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("half_centor", &half_centor_));
  }
  void Compute(OpKernelContext* ctx) override {
    const Tensor& src = ctx->input(0);
    const Tensor& base = ctx->input(1);
    const Tensor& offsets = ctx->input(2);
    const Tensor& Rs = ctx->input(3);
    const Tensor& Ts = ctx->input(4);
    OP_REQUIRES(ctx, src.dims() == 5, errors::InvalidArgument("src image must have rank 5"));
    const int64 B = src.dim_size(0), N = src.dim_size(1), C = src.dim_size(4);
    OP_REQUIRES(ctx, base.dims() == 4 && base.dim_size(0) == B && base.dim_size(3) == 1,
                errors::InvalidArgument("base_plane must have rank 4, and must compate to src_images"));
    OP_REQUIRES(ctx, offsets.dims() == 2 && offsets.dim_size(0) == B,
                errors::InvalidArgument("offsets must have rank 2, and must compate to src_images"));
    OP_REQUIRES(ctx, Rs.dims() == 4 && Rs.dim_size(0) == B && Rs.dim_size(1) == N && Rs.dim_size(2) == 3 && Rs.dim_size(3) == 3,
                errors::InvalidArgument("Rs must have rank 4, and must compate to src_images"));
    OP_REQUIRES(ctx, Ts.dims() == 3 && Ts.dim_size(0) == B && Ts.dim_size(1) == N && Ts.dim_size(2) == 3,
                errors::InvalidArgument("Ts must have rank 3, and must compate to src_images"));
    const int64 H = base.dim_size(1), W = base.dim_size(2), D = offsets.dim_size(1);
    chop_cv_desc d = {};
    d.dtype = DtypeOf<T>::value;
    d.half_centor = half_centor_;
    d.groups = 1;
    d.B = B; d.H = H; d.W = W; d.C = C; d.D = D; d.N = N; d.Hs = src.dim_size(2); d.Ws = src.dim_size(3);
    int status;
    if (!GRADIENT) {
      Tensor *mapped = nullptr, *mask = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({B, H, W, D, N, C}), &mapped));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(1, TensorShape({B, H, W, D, N, 1}), &mask));
      status = chop_feature_aggregate_fwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), In(ctx, 3), In(ctx, 4), Out(mapped),
                                          static_cast<int32_t*>(Out(mask)), StreamOf(ctx));
    } else {
      const Tensor& mg = ctx->input(5);
      const Tensor& mm = ctx->input(6);
      OP_REQUIRES(ctx, mg.NumElements() == B * H * W * D * N * C,
                  errors::InvalidArgument("mapped_feature_grad must have rank 6, and must compate to src_images"));
      OP_REQUIRES(ctx, mm.NumElements() == B * H * W * D * N,
                  errors::InvalidArgument("mapped_mask must be the mask returned by the forward op"));
      Tensor *sg = nullptr, *bg = nullptr;
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, src.shape(), &sg));
      OP_REQUIRES_OK(ctx, ctx->allocate_output(1, base.shape(), &bg));
      status = chop_feature_aggregate_bwd(&d, In(ctx, 0), In(ctx, 1), In(ctx, 2), In(ctx, 3), In(ctx, 4), In(ctx, 5),
                                          static_cast<const int32_t*>(In(ctx, 6)), Out(sg), Out(bg), StreamOf(ctx));
    }
    OP_REQUIRES(ctx, status == 0, errors::Internal("libchop_b200: ", chop_status_string(status)));
  }

 private:
  bool half_centor_ = true;
};

// IndexInitializer (index_initializer_kernels.cc:52-100): output_shape = (height, width, 3) in host memory
template <typename T>
class IndexInitializerOp : public OpKernel {
 public:
  explicit IndexInitializerOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("half_centor", &half_centor_));
  }
  void Compute(OpKernelContext* ctx) override {
    const Tensor& shape = ctx->input(0);
    OP_REQUIRES(ctx, shape.dims() == 1 && shape.NumElements() == 3,
                errors::InvalidArgument("output_shape must be a 1-D vector of 3 elements (height, width, 3)"));
    const auto v = shape.vec<int32>();
    OP_REQUIRES(ctx, v(0) > 0 && v(1) > 0 && v(2) == 3, errors::InvalidArgument("output_shape must be (height > 0, width > 0, 3)"));
    Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({v(0), v(1), 3}), &out));
    const int status = chop_index_initializer(DtypeOf<T>::value, half_centor_, v(0), v(1), Out(out), StreamOf(ctx));
    OP_REQUIRES(ctx, status == 0, errors::Internal("libchop_b200: ", chop_status_string(status)));
  }

 private:
  bool half_centor_ = true;
};

// DecodePfm (pfm_decoder_kernels.cc:30-118): a host op; the parser reports the reference's error texts
class DecodePfmOp : public OpKernel {
 public:
  explicit DecodePfmOp(OpKernelConstruction* ctx) : OpKernel(ctx) {}
  void Compute(OpKernelContext* ctx) override {
    const Tensor& contents = ctx->input(0);
    OP_REQUIRES(ctx, TensorShapeUtils::IsScalar(contents.shape()), errors::InvalidArgument("contents must be scalar"));
    const tstring& data = contents.scalar<tstring>()();
    int64_t h = 0, w = 0, ch = 0;
    char msg[256] = {0};
    int status = chop_decode_pfm(data.data(), data.size(), &h, &w, &ch, nullptr, 0, msg, sizeof(msg));
    OP_REQUIRES(ctx, status == 0, errors::InvalidArgument(msg[0] ? msg : chop_status_string(status)));
    Tensor* image = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({h, w, ch}), &image));
    status = chop_decode_pfm(data.data(), data.size(), &h, &w, &ch, image->flat<float>().data(), (size_t)(h * w * ch), msg,
                             sizeof(msg));
    OP_REQUIRES(ctx, status == 0, errors::InvalidArgument(msg[0] ? msg : chop_status_string(status)));
  }
};
REGISTER_KERNEL_BUILDER(Name("DecodePfm").Device(DEVICE_CPU), DecodePfmOp);

#define CHOP_REGISTER(T)                                                                                                   \
  REGISTER_KERNEL_BUILDER(Name("CostVolume").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_VOLUME, false>);      \
  REGISTER_KERNEL_BUILDER(Name("CostVolumeGrad").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_VOLUME, true>);   \
  REGISTER_KERNEL_BUILDER(Name("CostVolumeV2").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_VOLUME_V2, false>); \
  REGISTER_KERNEL_BUILDER(Name("CostVolumeGradV2").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_VOLUME_V2, true>); \
  REGISTER_KERNEL_BUILDER(Name("CostAggregate").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_AGGREGATE, false>); \
  REGISTER_KERNEL_BUILDER(Name("CostAggregateGrad").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_AGGREGATE, true>); \
  REGISTER_KERNEL_BUILDER(Name("SparseConv3DFast").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), ManifoldConvOp<T, false>);          \
  REGISTER_KERNEL_BUILDER(Name("SparseConv3DFastGrad").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), ManifoldConvOp<T, true>);         \
  REGISTER_KERNEL_BUILDER(Name("CostVolumeV3").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_VOLUME_V3, false>); \
  REGISTER_KERNEL_BUILDER(Name("CostVolumeGradV3").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), CostOp<T, CHOP_COST_VOLUME_V3, true>); \
  REGISTER_KERNEL_BUILDER(Name("SparseConv3DTransposeFast").Device(DEVICE_GPU).TypeConstraint<T>("dtype").HostMemory("output_size"), \
                          ManifoldConvTransposeOp<T, false>);                                                                         \
  REGISTER_KERNEL_BUILDER(Name("SparseConv3DTransposeFastGrad").Device(DEVICE_GPU).TypeConstraint<T>("dtype").HostMemory("output_size"), \
                          ManifoldConvTransposeOp<T, true>);                                                                          \
  REGISTER_KERNEL_BUILDER(Name("SparsePad").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), ManifoldPadOp<T, false>);                  \
  REGISTER_KERNEL_BUILDER(Name("SparsePadGrad").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), ManifoldPadOp<T, true>);                \
  REGISTER_KERNEL_BUILDER(Name("FeatureAggregate").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), FeatureAggregateOp<T, false>);     \
  REGISTER_KERNEL_BUILDER(Name("FeatureAggregateGrad").Device(DEVICE_GPU).TypeConstraint<T>("dtype"), FeatureAggregateOp<T, true>);  \
  REGISTER_KERNEL_BUILDER(Name("IndexInitializer").Device(DEVICE_GPU).TypeConstraint<T>("dtype").HostMemory("output_shape"),         \
                          IndexInitializerOp<T>);

CHOP_REGISTER(float)
CHOP_REGISTER(double)
#undef CHOP_REGISTER
#endif  // GOOGLE_CUDA

}  // namespace chop_b200
}  // namespace tensorflow
