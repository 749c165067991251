"""Python surface of the cost-volume ops, mirroring the reference wrapper
custom_helper_op/python/ops/custom_helper_ops.py: same function names, positional order, defaults
and return values (cost_volume :32-38, cost_volume_v2 :65-71, cost_aggregate), same gradient
contract (gradients for the two feature inputs and the depth input, None for offsets/Rs/Ts,
:41-61 and :74-94).

The reference wrapper feeds TensorFlow tensors to a TensorFlow op library.  TensorFlow is not a
dependency here: the functions take torch CUDA tensors and call the C ABI of libchop_b200.so on the
current CUDA stream; torch only supplies device memory, streams and autograd plumbing.  Every call
runs the CUDA kernels - a CPU tensor or a missing library raises.
"""
import ctypes

import torch

from custom_helper_op_b200 import _lib

_DT = {torch.float32: _lib.F32, torch.float64: _lib.F64, torch.bfloat16: _lib.BF16}


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require(cond, msg):
    # the reference reports these through OP_REQUIRES -> InvalidArgumentError
    if not cond:
        raise ValueError(msg)


def _prep(ref_image, src_images, depth, offsets, Rs, Ts, kind):
    _require(ref_image.is_cuda, "cost volume ops run on CUDA tensors only (no CPU kernel is registered)")
    _require(ref_image.dtype in _DT, "dtype must be float32, float64 or bfloat16")
    real = torch.float32 if ref_image.dtype == torch.bfloat16 else ref_image.dtype
    dev = ref_image.device

    def cv(t, dt):
        # the common case costs no torch dispatch: already a contiguous tensor of the right type on the right device
        if torch.is_tensor(t) and t.dtype == dt and t.device == dev and t.is_contiguous():
            return t
        return torch.as_tensor(t, device=dev).to(dt).contiguous()

    ref_image = ref_image.contiguous()
    src_images = cv(src_images, ref_image.dtype)
    depth = cv(depth, real)
    offsets = cv(offsets, real) if offsets is not None else None
    Rs = cv(Rs, real)
    Ts = cv(Ts, real)
    _require(ref_image.dim() == 4, "ref image must have rank 4")
    B, H, W, C = ref_image.shape
    _require(src_images.dim() == 5 and src_images.shape[0] == B and tuple(src_images.shape[2:]) == (H, W, C),
             "src_images must have rank 5, and must compate to ref_image")
    N = src_images.shape[1]
    if kind == _lib.KIND_V2:
        _require(depth.dim() == 4 and tuple(depth.shape[:3]) == (B, H, W),
                 "depth_grid must have rank 4, and must compate to ref_image")
        D = depth.shape[3]
    else:
        _require(depth.dim() == 4 and tuple(depth.shape) == (B, H, W, 1),
                 "base_plane must have rank 4, and must compate to ref_image")
        _require(offsets.dim() == 2 and offsets.shape[0] == B,
                 "offsets must have rank 2, and must compate to ref_image")
        D = offsets.shape[1]
    _require(tuple(Rs.shape) == (B, N, 3, 3), "Rs must have rank 4, and must compate to ref_image")
    _require(tuple(Ts.shape) == (B, N, 3), "Ts must have rank 3, and must compate to ref_image")
    return ref_image, src_images, depth, offsets, Rs, Ts, (B, H, W, C, D, N), real


def _desc(kind, dtype, reduce_method, half_centor, groups, dims, flags=0, d_range=None):
    _require(reduce_method in ("MEAN", "MIN"),
             "Invalid reduce method %s. Supported types: MEAN, MIN" % reduce_method)
    B, H, W, C, D, N = dims
    d = _lib.CvDesc()
    d.kind, d.dtype = kind, _DT[dtype]
    d.reduce = _lib.REDUCE_MIN if reduce_method == "MIN" else _lib.REDUCE_MEAN
    d.half_centor = int(bool(half_centor))
    d.groups = int(groups or 1)
    d.flags = flags
    d.B, d.H, d.W, d.C, d.D, d.N, d.Hs, d.Ws = B, H, W, C, D, N, H, W
    d.d_begin, d.d_end = d_range if d_range is not None else (0, 0)
    return d


def _out_channels(kind, C, groups):
    return C if kind == _lib.KIND_V1 else (groups if kind == _lib.KIND_V2 else 1)


def _mask_channels(kind, CO, reduce_method):
    if reduce_method != "MIN":
        return 1
    return 3 if kind == _lib.KIND_V3 else CO   # v3 MIN: (view, reference group, source group)


def _check_groups(kind, C, groups):
    if kind in (_lib.KIND_V2, _lib.KIND_V3):
        _require(groups is not None and groups >= 1 and C % groups == 0, "channels must be divisible by groups")
    if kind == _lib.KIND_V3:   # cost_volume_kernels_v3.cc:110-111
        _require(C // groups <= 8, "image_channels / groups_ less than MAX_SUBCHANNELS_SIZE(8)")


def cost_forward(kind, ref_image, src_images, depth, offsets, Rs, Ts, reduce_method="MEAN", groups=None,
                 half_centor=True, strict=False, d_range=None, out=None):
    """Raw forward op (CostVolume / CostVolumeV2 / CostAggregate).  Returns (cost, cost_mask).
    ``d_range=(d0,d1)`` computes only those depth planes (into ``out=(cost, mask)`` if given)."""
    ref_image, src_images, depth, offsets, Rs, Ts, dims, real = _prep(ref_image, src_images, depth, offsets, Rs, Ts, kind)
    B, H, W, C, D, N = dims
    _check_groups(kind, C, groups)
    CO = _out_channels(kind, C, groups)
    MC = _mask_channels(kind, CO, reduce_method)
    if out is None:
        alloc = torch.empty if d_range is None else torch.zeros
        cost = alloc((B, H, W, D, CO), dtype=real, device=ref_image.device)
        mask = alloc((B, H, W, D, MC), dtype=torch.int32, device=ref_image.device)
    else:
        cost, mask = out
    d = _desc(kind, ref_image.dtype, reduce_method, half_centor, groups, dims,
              _lib.FLAG_STRICT if strict else 0, d_range)
    st = _lib.lib().chop_cost_volume_fwd(ctypes.byref(d), _ptr(ref_image), _ptr(src_images), _ptr(depth),
                                         _ptr(offsets), _ptr(Rs), _ptr(Ts), _ptr(cost), _ptr(mask), _stream())
    _lib.check(st, "chop_cost_volume_fwd")
    if kind == _lib.KIND_AGG and out is None:
        return cost.view(B, H, W, D), mask.view(B, H, W, D)
    return cost, mask


def cost_backward(kind, ref_image, src_images, depth, offsets, Rs, Ts, cost_grad, cost_mask,
                  reduce_method="MEAN", groups=None, half_centor=True, d_range=None, accumulate_into=None,
                  zero_into=None):
    """Raw gradient op (CostVolumeGrad / CostVolumeGradV2 / CostAggregateGrad).
    Returns (ref_image_grad, src_images_grad, depth_grad)."""
    ref_image, src_images, depth, offsets, Rs, Ts, dims, real = _prep(ref_image, src_images, depth, offsets, Rs, Ts, kind)
    B, H, W, C, D, N = dims
    _check_groups(kind, C, groups)
    CO = _out_channels(kind, C, groups)
    MC = _mask_channels(kind, CO, reduce_method)
    cost_grad = cost_grad.to(real).contiguous()
    cost_mask = cost_mask.contiguous()
    _require(cost_grad.numel() == B * H * W * D * CO, "cost_grad must have rank 5, and must compate to ref_image")
    _require(cost_mask.dtype == torch.int32 and cost_mask.numel() == B * H * W * D * MC,
             "cost_mask must be the int32 mask returned by the forward op")
    flags = 0
    if zero_into is not None:          # caller-owned output buffers, zero-filled by the library
        ref_grad, src_grad, depth_grad = zero_into
    elif accumulate_into is None:
        ref_grad = torch.empty((B, H, W, C), dtype=real, device=ref_image.device)
        src_grad = torch.empty((B, N, H, W, C), dtype=real, device=ref_image.device)
        depth_grad = torch.empty_like(depth) if d_range is None else torch.zeros_like(depth)
    else:
        ref_grad, src_grad, depth_grad = accumulate_into
        flags |= _lib.FLAG_ACCUMULATE
    d = _desc(kind, ref_image.dtype, reduce_method, half_centor, groups, dims, flags, d_range)
    st = _lib.lib().chop_cost_volume_bwd(ctypes.byref(d), _ptr(ref_image), _ptr(src_images), _ptr(depth),
                                         _ptr(offsets), _ptr(Rs), _ptr(Ts), _ptr(cost_grad), _ptr(cost_mask),
                                         _ptr(ref_grad), _ptr(src_grad), _ptr(depth_grad), _stream())
    _lib.check(st, "chop_cost_volume_bwd")
    return ref_grad, src_grad, depth_grad


class _CostFn(torch.autograd.Function):
    """Glue between torch autograd and the two raw ops; the counterpart of the reference's
    @tf.RegisterGradient functions."""

    @staticmethod
    def forward(ctx, kind, reduce_method, groups, half_centor, ref_image, src_images, depth, offsets, Rs, Ts):
        cost, mask = cost_forward(kind, ref_image, src_images, depth, offsets, Rs, Ts, reduce_method, groups,
                                  half_centor)
        ctx.save_for_backward(ref_image, src_images, depth, offsets, Rs, Ts, mask)
        ctx.conf = (kind, reduce_method, groups, half_centor)
        ctx.feature_dtype = ref_image.dtype
        ctx.mark_non_differentiable(mask)
        return cost, mask

    @staticmethod
    def backward(ctx, grad_out, grad_mask):
        ref_image, src_images, depth, offsets, Rs, Ts, mask = ctx.saved_tensors
        kind, reduce_method, groups, half_centor = ctx.conf
        rg, sg, dg = cost_backward(kind, ref_image, src_images, depth, offsets, Rs, Ts, grad_out, mask,
                                   reduce_method, groups, half_centor)
        rg = rg.to(ctx.feature_dtype)
        sg = sg.to(ctx.feature_dtype)
        return None, None, None, None, rg, sg, dg.view_as(depth), None, None, None


def cost_volume(ref_image, src_images, base_plane, offsets, Rs, Ts, reduce_method="MEAN", half_centor=True,
                name=None):
    """cost [B,H,W,D,C], cost_mask [B,H,W,D,1|C] (reference: custom_helper_ops.py:32-38)."""
    dev = ref_image.device
    return _CostFn.apply(_lib.KIND_V1, reduce_method, None, half_centor, ref_image, src_images, base_plane,
                         torch.as_tensor(offsets, device=dev), torch.as_tensor(Rs, device=dev),
                         torch.as_tensor(Ts, device=dev))


def cost_volume_v2(ref_image, src_images, depth_grid, Rs, Ts, reduce_method="MEAN", groups=None, half_centor=True,
                   name=None):
    """cost [B,H,W,D,G], cost_mask [B,H,W,D,1|G] (reference: custom_helper_ops.py:65-71)."""
    dev = ref_image.device
    return _CostFn.apply(_lib.KIND_V2, reduce_method, groups, half_centor, ref_image, src_images,
                         torch.as_tensor(depth_grid, device=dev), None, torch.as_tensor(Rs, device=dev),
                         torch.as_tensor(Ts, device=dev))


def cost_volume_v3(ref_image, src_images, base_plane, offsets, Rs, Ts, reduce_method="MEAN", groups=None,
                   half_centor=True, name=None):
    """cost [B,H,W,D,1], cost_mask [B,H,W,D,1|3]: the largest correlation between any group of the sampled
    source feature and any group of the reference feature (reference: custom_helper_ops.py:98-104)."""
    dev = ref_image.device
    return _CostFn.apply(_lib.KIND_V3, reduce_method, groups, half_centor, ref_image, src_images, base_plane,
                         torch.as_tensor(offsets, device=dev), torch.as_tensor(Rs, device=dev),
                         torch.as_tensor(Ts, device=dev))


def cost_aggregate(ref_image, src_images, base_plane, offsets, Rs, Ts, reduce_method="MEAN", half_centor=True,
                   name=None):
    """cost [B,H,W,D], cost_mask [B,H,W,D]: the channel-averaged form of cost_volume the reference's
    CostMapLayer uses (custom_helper_ops.py cost_aggregate)."""
    dev = ref_image.device
    return _CostFn.apply(_lib.KIND_AGG, reduce_method, None, half_centor, ref_image, src_images, base_plane,
                         torch.as_tensor(offsets, device=dev), torch.as_tensor(Rs, device=dev),
                         torch.as_tensor(Ts, device=dev))


# ---- manifold ("sparse") 3-D convolution --------------------------------------------------------------
def _sc_desc(images, filters, strides, dilations, dynamic_default):
    _require(images.is_cuda, "sparse_conv3d_fast runs on CUDA tensors only (no CPU kernel is registered)")
    _require(images.dtype in _DT, "dtype must be float32, float64 or bfloat16")
    _require(images.dim() == 5, "images must have rank 5")
    _require(filters.dim() == 5, "filter must have rank 5")
    _require(len(strides) == 3, "strides must be a vector have 3 element")
    _require(len(dilations) == 3, "dilations must be a vector have 3 element")
    _require(images.shape[4] == filters.shape[3], "images channel size wrong")
    d = _lib.ScDesc()
    d.dtype = _DT[images.dtype]
    d.dynamic_default = int(bool(dynamic_default))
    d.B, d.H, d.W, d.D, d.Cin = images.shape
    d.Cout = filters.shape[4]
    for i in range(3):
        d.filter[i] = int(filters.shape[i])
        d.strides[i] = int(strides[i])
        d.dilations[i] = int(dilations[i])
    out_shape = (d.B, (d.H + d.strides[0] - 1) // d.strides[0], (d.W + d.strides[1] - 1) // d.strides[1],
                 (d.D + d.strides[2] - 1) // d.strides[2], d.Cout)
    return d, out_shape


def _scalar(value, like):
    """default_value as a device scalar of the images' dtype (python floats keep full precision)."""
    if torch.is_tensor(value):
        return value.to(device=like.device, dtype=like.dtype).reshape(())
    # a fill kernel on the current stream, not a synchronous host-to-device copy; float64 keeps the python float exactly
    return torch.full((), float(value), dtype=like.dtype, device=like.device)


def _umma_watch(images):
    """Before a tensor-core (bfloat16) manifold-convolution call: raise if a kernel of an EARLIER call gave up a
    bounded wait on its MMA barrier - the outputs of the calls since the last check are then incomplete.  Reads one
    int of pinned host memory (chop_umma_watch); only the first call per device synchronises."""
    if images.dtype != torch.bfloat16:
        return
    with torch.cuda.device(images.device):
        n = _lib.lib().chop_umma_watch()
    if n > 0:
        raise RuntimeError("custom_helper_op: %d tensor-core convolution wait(s) timed out on the device; results of "
                           "the manifold-convolution calls since the previous check are incomplete" % n)


def sparse_conv3d_forward(images, filters, default_value, base_plane, strides=(1, 1, 1), dilations=(1, 1, 1)):
    """Raw op SparseConv3DFast."""
    images = images.contiguous()
    filters = filters.to(images.dtype).contiguous()
    default_value = _scalar(default_value, images)
    base_plane = base_plane.contiguous()
    d, out_shape = _sc_desc(images, filters, strides, dilations, False)
    _require(base_plane.dtype == torch.int32 and tuple(base_plane.shape) == (d.B, d.H, d.W, 1),
             "base_plane must have rank 4, and must compate to ref_image")
    out = torch.empty(out_shape, dtype=images.dtype, device=images.device)
    _umma_watch(images)
    st = _lib.lib().chop_sparse_conv3d_fwd(ctypes.byref(d), _ptr(images), _ptr(filters), _ptr(default_value),
                                           _ptr(base_plane), _ptr(out), _stream())
    _lib.check(st, "chop_sparse_conv3d_fwd")
    return out


def sparse_conv3d_backward(images, filters, default_value, base_plane, out_grad, strides=(1, 1, 1),
                           dilations=(1, 1, 1), dynamic_default=False):
    """Raw op SparseConv3DFastGrad: (images_grad, filter_grad, default_value_grad)."""
    images = images.contiguous()
    filters = filters.to(images.dtype).contiguous()
    default_value = _scalar(default_value, images)
    base_plane = base_plane.contiguous()
    out_grad = out_grad.to(images.dtype).contiguous()
    d, out_shape = _sc_desc(images, filters, strides, dilations, dynamic_default)
    _require(tuple(out_grad.shape) == out_shape, "out_grad must have rank 5, and must compate to ref_image")
    wdt = torch.float32 if images.dtype == torch.bfloat16 else images.dtype
    images_grad = torch.empty_like(images)
    filter_grad = torch.empty(filters.shape, dtype=wdt, device=images.device)
    default_grad = torch.empty((), dtype=wdt, device=images.device)
    nbytes = _lib.lib().chop_sparse_conv3d_bwd_workspace_size(ctypes.byref(d))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=images.device)
    _umma_watch(images)
    st = _lib.lib().chop_sparse_conv3d_bwd(ctypes.byref(d), _ptr(images), _ptr(filters), _ptr(default_value),
                                           _ptr(base_plane), _ptr(out_grad), _ptr(images_grad), _ptr(filter_grad),
                                           _ptr(default_grad), _ptr(ws), ctypes.c_size_t(ws.numel()), _stream())
    _lib.check(st, "chop_sparse_conv3d_bwd")
    return images_grad, filter_grad, default_grad


class _SparseConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, images, filters, default_value, base_plane, strides, dilations, dynamic_default):
        out = sparse_conv3d_forward(images, filters, default_value, base_plane, strides, dilations)
        ctx.save_for_backward(images, filters, default_value, base_plane)
        ctx.conf = (tuple(strides), tuple(dilations), bool(dynamic_default))
        return out

    @staticmethod
    def backward(ctx, out_grad):
        images, filters, default_value, base_plane = ctx.saved_tensors
        strides, dilations, dynamic_default = ctx.conf
        ig, fg, dg = sparse_conv3d_backward(images, filters, default_value, base_plane, out_grad, strides, dilations,
                                            dynamic_default)
        # the reference drops the default-value gradient unless dynamic_default (custom_helper_ops.py:284-286)
        dg = dg.to(default_value.dtype) if dynamic_default else None
        return ig, fg.to(filters.dtype), dg, None, None, None, None


def sparse_conv3d_fast(images, filters, default_value, base_plane, data_format='NDHWC', strides=(1, 1, 1),
                       dilations=(1, 1, 1), dynamic_default=False, name=None):
    """output [B,ceil(H/s),ceil(W/s),ceil(D/s),Cout] (reference: custom_helper_ops.py:263-267)."""
    _require(data_format == 'NDHWC', "data_format must be NDHWC")
    default_value = _scalar(default_value, images)
    return _SparseConvFn.apply(images, filters, default_value, base_plane, strides, dilations, dynamic_default)


# ---- transposed manifold convolution ------------------------------------------------------------------
def _sct_desc(images, filters, output_size, strides, dilations):
    """Descriptor of the forward convolution whose transpose is taken, derived as the reference op derives it
    (sparse_conv3d_fast_op.cc:78-146): output_size is the fine grid, images the coarse one."""
    _require(images.is_cuda, "sparse_conv3d_transpose_fast runs on CUDA tensors only (no CPU kernel is registered)")
    _require(images.dtype in _DT, "dtype must be float32, float64 or bfloat16")
    _require(images.dim() == 5, "images must have rank 5")
    _require(filters.dim() == 5, "filter must have rank 5")
    _require(len(strides) == 3, "strides must be a vector have 3 element")
    _require(len(dilations) == 3, "dilations must be a vector have 3 element")
    output_size = [int(x) for x in (output_size.tolist() if torch.is_tensor(output_size) else output_size)]
    _require(len(output_size) == 3, "output_shape must be an 1-D vector of (height, width, depth)")
    _require(images.shape[4] == filters.shape[4], "images channel size wrong")
    d = _lib.ScDesc()
    d.dtype = _DT[images.dtype]
    d.dynamic_default = 0
    d.B = images.shape[0]
    d.H, d.W, d.D = output_size
    d.Cin, d.Cout = filters.shape[3], filters.shape[4]
    for i in range(3):
        d.filter[i] = int(filters.shape[i])
        d.strides[i] = int(strides[i])
        d.dilations[i] = int(dilations[i])
    coarse = tuple((n + s - 1) // s for n, s in zip(output_size, d.strides))
    _require(tuple(images.shape[1:4]) == coarse, "images shape and output_shape does not compate")
    return d, (d.B, d.H, d.W, d.D, d.Cin)


def sparse_conv3d_transpose_forward(images, filters, default_value, base_plane, output_size, strides=(1, 1, 1),
                                    dilations=(1, 1, 1)):
    """Raw op SparseConv3DTransposeFast: images [B,oH,oW,oD,Cout] -> [B,H,W,D,Cin]."""
    images = images.contiguous()
    filters = filters.to(images.dtype).contiguous()
    default_value = _scalar(default_value, images)
    base_plane = base_plane.contiguous()
    d, out_shape = _sct_desc(images, filters, output_size, strides, dilations)
    _require(base_plane.dtype == torch.int32 and tuple(base_plane.shape) == (d.B, d.H, d.W, 1),
             "base_plane must have rank 4, and must compate to ref_image")
    out = torch.empty(out_shape, dtype=images.dtype, device=images.device)
    _umma_watch(images)
    st = _lib.lib().chop_sparse_conv3d_transpose_fwd(ctypes.byref(d), _ptr(images), _ptr(filters), _ptr(default_value),
                                                     _ptr(base_plane), _ptr(out), _stream())
    _lib.check(st, "chop_sparse_conv3d_transpose_fwd")
    return out


def sparse_conv3d_transpose_backward(images, filters, default_value, base_plane, output_size, out_grad,
                                     strides=(1, 1, 1), dilations=(1, 1, 1)):
    """Raw op SparseConv3DTransposeFastGrad: (images_grad, filter_grad), both the derivatives of the forward op."""
    images = images.contiguous()
    filters = filters.to(images.dtype).contiguous()
    default_value = _scalar(default_value, images)
    base_plane = base_plane.contiguous()
    out_grad = out_grad.to(images.dtype).contiguous()
    d, out_shape = _sct_desc(images, filters, output_size, strides, dilations)
    _require(tuple(out_grad.shape) == out_shape, "out_grad must have rank 5, and must compate to ref_image")
    wdt = torch.float32 if images.dtype == torch.bfloat16 else images.dtype
    images_grad = torch.empty_like(images)
    filter_grad = torch.empty(filters.shape, dtype=wdt, device=images.device)
    nbytes = _lib.lib().chop_sparse_conv3d_transpose_bwd_workspace_size(ctypes.byref(d))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=images.device)
    _umma_watch(images)
    st = _lib.lib().chop_sparse_conv3d_transpose_bwd(ctypes.byref(d), _ptr(images), _ptr(filters), _ptr(default_value),
                                                     _ptr(base_plane), _ptr(out_grad), _ptr(images_grad),
                                                     _ptr(filter_grad), _ptr(ws), ctypes.c_size_t(ws.numel()), _stream())
    _lib.check(st, "chop_sparse_conv3d_transpose_bwd")
    return images_grad, filter_grad


class _SparseConvTransposeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, images, filters, default_value, base_plane, output_size, strides, dilations):
        out = sparse_conv3d_transpose_forward(images, filters, default_value, base_plane, output_size, strides, dilations)
        ctx.save_for_backward(images, filters, default_value, base_plane)
        ctx.conf = (tuple(int(x) for x in output_size), tuple(strides), tuple(dilations))
        return out

    @staticmethod
    def backward(ctx, out_grad):
        images, filters, default_value, base_plane = ctx.saved_tensors
        output_size, strides, dilations = ctx.conf
        ig, fg = sparse_conv3d_transpose_backward(images, filters, default_value, base_plane, output_size, out_grad,
                                                  strides, dilations)
        # gradients for images and filters only (reference: custom_helper_ops.py:313)
        return ig, fg.to(filters.dtype), None, None, None, None, None


def sparse_conv3d_transpose_fast(images, filters, default_value, base_plane, output_size, data_format='NDHWC',
                                 strides=(1, 1, 1), dilations=(1, 1, 1), dynamic_default=False, name=None):
    """output [B,*output_size,Cin] for filters [fh,fw,fd,Cin,Cout] (reference: custom_helper_ops.py:290-294)."""
    _require(data_format == 'NDHWC', "data_format must be NDHWC")
    default_value = _scalar(default_value, images)
    output_size = [int(x) for x in (output_size.tolist() if torch.is_tensor(output_size) else output_size)]
    return _SparseConvTransposeFn.apply(images, filters, default_value, base_plane, output_size, strides, dilations)


# ---- SparsePad ----------------------------------------------------------------------------------------
def _pad_args(images, base_plane, strides):
    _require(images.is_cuda, "sparse_pad runs on CUDA tensors only")
    _require(images.dtype in _DT, "dtype must be float32, float64 or bfloat16")
    _require(images.dim() == 5, "images must have rank 5")
    _require(len(strides) == 3, "strides must be a vector have 3 element")
    B, h, w, d, C = images.shape
    st = (ctypes.c_int32 * 3)(*[int(x) for x in strides])
    fine = (B, h * st[0], w * st[1], d * st[2], C)
    _require(base_plane.dtype == torch.int32 and tuple(base_plane.shape) == (B, fine[1], fine[2], 1),
             "base_plane must have rank 4, and must compate to ref_image")
    return st, fine


def sparse_pad_forward(images, base_plane, strides=(1, 1, 1)):
    """Raw op SparsePad."""
    images = images.contiguous()
    base_plane = base_plane.contiguous()
    st, fine = _pad_args(images, base_plane, strides)
    out = torch.empty(fine, dtype=images.dtype, device=images.device)
    B, h, w, d, C = images.shape
    rc = _lib.lib().chop_sparse_pad_fwd(_DT[images.dtype], B, h, w, d, C, st, _ptr(images), _ptr(base_plane), _ptr(out),
                                        _stream())
    _lib.check(rc, "chop_sparse_pad_fwd")
    return out


def sparse_pad_backward(images, base_plane, out_grad, strides=(1, 1, 1)):
    """Raw op SparsePadGrad (images is used for its shape only, as in the reference)."""
    base_plane = base_plane.contiguous()
    st, fine = _pad_args(images, base_plane, strides)
    out_grad = out_grad.to(images.dtype).contiguous()
    _require(tuple(out_grad.shape) == fine, "out_grad must compate to the padded shape")
    images_grad = torch.empty(images.shape, dtype=images.dtype, device=images.device)
    B, h, w, d, C = images.shape
    rc = _lib.lib().chop_sparse_pad_bwd(_DT[images.dtype], B, h, w, d, C, st, _ptr(base_plane), _ptr(out_grad),
                                        _ptr(images_grad), _stream())
    _lib.check(rc, "chop_sparse_pad_bwd")
    return images_grad


class _SparsePadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, images, base_plane, strides):
        ctx.save_for_backward(images, base_plane)
        ctx.strides = tuple(strides)
        return sparse_pad_forward(images, base_plane, strides)

    @staticmethod
    def backward(ctx, out_grad):
        images, base_plane = ctx.saved_tensors
        return sparse_pad_backward(images, base_plane, out_grad, ctx.strides), None, None


def sparse_pad(images, base_plane, strides=(1, 1, 1), dilations=(1, 1, 1), name=None):
    """Zero insertion of a coarse band into the fine band (reference: custom_helper_ops.py:220-234)."""
    _require(len(dilations) == 3, "dilations must be a vector have 3 element")
    return _SparsePadFn.apply(images, base_plane, strides)


# ---- FeatureAggregate ---------------------------------------------------------------------------------
def _fa_prep(src_images, base_plane, offsets, Rs, Ts):
    _require(src_images.is_cuda, "feature_aggregate runs on CUDA tensors only (no CPU kernel is registered)")
    _require(src_images.dtype in _DT, "dtype must be float32, float64 or bfloat16")
    _require(src_images.dim() == 5, "src image must have rank 5")
    real = torch.float32 if src_images.dtype == torch.bfloat16 else src_images.dtype
    dev = src_images.device
    src_images = src_images.contiguous()
    base_plane = base_plane.to(real).contiguous()
    offsets = torch.as_tensor(offsets, device=dev).to(real).contiguous()
    Rs = torch.as_tensor(Rs, device=dev).to(real).contiguous()
    Ts = torch.as_tensor(Ts, device=dev).to(real).contiguous()
    B, N, Hs, Ws, C = src_images.shape
    _require(base_plane.dim() == 4 and base_plane.shape[0] == B and base_plane.shape[3] == 1,
             "base_plane must have rank 4, and must compate to src_images")
    H, W = base_plane.shape[1], base_plane.shape[2]
    _require(offsets.dim() == 2 and offsets.shape[0] == B, "offsets must have rank 2, and must compate to src_images")
    D = offsets.shape[1]
    _require(tuple(Rs.shape) == (B, N, 3, 3), "Rs must have rank 4, and must compate to src_images")
    _require(tuple(Ts.shape) == (B, N, 3), "Ts must have rank 3, and must compate to src_images")
    d = _lib.CvDesc()
    d.kind, d.dtype, d.reduce, d.groups, d.flags = 0, _DT[src_images.dtype], 0, 1, 0
    d.B, d.H, d.W, d.C, d.D, d.N, d.Hs, d.Ws = B, H, W, C, D, N, Hs, Ws
    d.d_begin, d.d_end = 0, 0
    return src_images, base_plane, offsets, Rs, Ts, d, real


def feature_aggregate_forward(src_images, base_plane, offsets, Rs, Ts, half_centor=True):
    """Raw op FeatureAggregate: (mapped_feature [B,H,W,D,N,C], mapped_mask int32 [B,H,W,D,N,1])."""
    src_images, base_plane, offsets, Rs, Ts, d, real = _fa_prep(src_images, base_plane, offsets, Rs, Ts)
    d.half_centor = int(bool(half_centor))
    shape = (d.B, d.H, d.W, d.D, d.N)
    mapped = torch.empty(shape + (d.C,), dtype=real, device=src_images.device)
    mask = torch.empty(shape + (1,), dtype=torch.int32, device=src_images.device)
    st = _lib.lib().chop_feature_aggregate_fwd(ctypes.byref(d), _ptr(src_images), _ptr(base_plane), _ptr(offsets), _ptr(Rs),
                                               _ptr(Ts), _ptr(mapped), _ptr(mask), _stream())
    _lib.check(st, "chop_feature_aggregate_fwd")
    return mapped, mask


def feature_aggregate_backward(src_images, base_plane, offsets, Rs, Ts, mapped_feature_grad, mapped_mask, half_centor=True):
    """Raw op FeatureAggregateGrad: (src_images_grad, base_plane_grad)."""
    src_images, base_plane, offsets, Rs, Ts, d, real = _fa_prep(src_images, base_plane, offsets, Rs, Ts)
    d.half_centor = int(bool(half_centor))
    n = d.B * d.H * d.W * d.D * d.N
    mapped_feature_grad = mapped_feature_grad.to(real).contiguous()
    mapped_mask = mapped_mask.contiguous()
    _require(mapped_feature_grad.numel() == n * d.C, "mapped_feature_grad must compate to the forward output")
    _require(mapped_mask.dtype == torch.int32 and mapped_mask.numel() == n,
             "mapped_mask must be the int32 mask returned by the forward op")
    src_grad = torch.empty(src_images.shape, dtype=real, device=src_images.device)
    base_grad = torch.empty_like(base_plane)
    st = _lib.lib().chop_feature_aggregate_bwd(ctypes.byref(d), _ptr(src_images), _ptr(base_plane), _ptr(offsets), _ptr(Rs),
                                               _ptr(Ts), _ptr(mapped_feature_grad), _ptr(mapped_mask), _ptr(src_grad),
                                               _ptr(base_grad), _stream())
    _lib.check(st, "chop_feature_aggregate_bwd")
    return src_grad, base_grad


class _FeatureAggregateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, half_centor, src_images, base_plane, offsets, Rs, Ts):
        mapped, mask = feature_aggregate_forward(src_images, base_plane, offsets, Rs, Ts, half_centor)
        ctx.save_for_backward(src_images, base_plane, offsets, Rs, Ts, mask)
        ctx.half_centor = half_centor
        ctx.mark_non_differentiable(mask)
        return mapped, mask

    @staticmethod
    def backward(ctx, grad_out, grad_mask):
        src_images, base_plane, offsets, Rs, Ts, mask = ctx.saved_tensors
        sg, bg = feature_aggregate_backward(src_images, base_plane, offsets, Rs, Ts, grad_out, mask, ctx.half_centor)
        # gradients for src_images and base_plane only (reference: custom_helper_ops.py:192)
        return None, sg.to(src_images.dtype), bg.to(base_plane.dtype), None, None, None


def feature_aggregate(src_images, base_plane, offsets, Rs, Ts, half_centor=True, name=None):
    """Warped source features of every view at every voxel (reference: custom_helper_ops.py:166-171)."""
    dev = src_images.device
    return _FeatureAggregateFn.apply(half_centor, src_images, base_plane, torch.as_tensor(offsets, device=dev),
                                     torch.as_tensor(Rs, device=dev), torch.as_tensor(Ts, device=dev))


# ---- IndexInitializer, DecodePfm ----------------------------------------------------------------------
def index_initializer(output_shape, half_centor=True, dtype=torch.float32, device="cuda"):
    """[H,W,3] = (column, row, 1) per pixel, +0.5 on the first two when half_centor (reference:
    custom_helper_ops.py:329-330; output_shape = (H, W, 3))."""
    output_shape = [int(x) for x in (output_shape.tolist() if torch.is_tensor(output_shape) else output_shape)]
    _require(len(output_shape) == 3, "output shape must have 3 elements")
    _require(output_shape[2] == 3, "last dimsion must be 3")
    _require(dtype in (torch.float32, torch.float64), "dtype must be float32 or float64")
    out = torch.empty(output_shape, dtype=dtype, device=device)
    _require(out.is_cuda, "index_initializer fills a CUDA tensor")
    with torch.cuda.device(out.device):
        st = _lib.lib().chop_index_initializer(_DT[dtype], int(bool(half_centor)), output_shape[0], output_shape[1], _ptr(out),
                                               _stream())
    _lib.check(st, "chop_index_initializer")
    return out


class IndexInitializer:
    """Initializer object form of index_initializer (reference: custom_helper_ops.py:332-344)."""

    def __call__(self, output_shape, half_centor=True, dtype=torch.float32, device="cuda"):
        return index_initializer(output_shape, half_centor, dtype, device)


def decode_pfm(contents, name=None):
    """Decode an in-memory single-channel PFM file to a float32 CPU tensor [height, width, 1] (reference:
    custom_helper_ops.py:317-326; a host op there too).  Raises ValueError with the reference's message for
    contents it rejects."""
    contents = bytes(contents)
    h, w, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    msg = ctypes.create_string_buffer(256)
    L = _lib.lib()
    st = L.chop_decode_pfm(contents, len(contents), ctypes.byref(h), ctypes.byref(w), ctypes.byref(c), None, 0, msg, 256)
    if st == _lib.ERR_FORMAT:
        raise ValueError(msg.value.decode(errors="replace"))
    _lib.check(st, "chop_decode_pfm")
    out = torch.empty((h.value, w.value, c.value), dtype=torch.float32)
    st = L.chop_decode_pfm(contents, len(contents), ctypes.byref(h), ctypes.byref(w), ctypes.byref(c),
                           ctypes.c_void_p(out.data_ptr()), out.numel(), msg, 256)
    _lib.check(st, "chop_decode_pfm")
    return out
