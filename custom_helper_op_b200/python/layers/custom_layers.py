"""The reference's layers over this library's ops (reference: custom_helper_op/python/layers/custom_layers.py:34-199,
Keras layers there; torch.nn.Module here, with the same constructor arguments, weights and call conventions).

Weights are created on first use from the input shapes, as Keras' ``build`` does.  ``default_type``:
'DYNAMIC' = a trainable scalar initialised to zero, 'CONSTANT' = a non-trainable zero, or a tensor to use as given.
"""
import math

import torch

from custom_helper_op_b200.python.ops.custom_helper_ops import (cost_aggregate, cost_volume_v2, sparse_conv3d_fast,
                                                                 sparse_conv3d_transpose_fast)


def _default_scalar(default_type, like):
    """(tensor, trainable) for a layer's default value."""
    if torch.is_tensor(default_type):
        return default_type.to(device=like.device, dtype=like.dtype), bool(default_type.requires_grad)
    assert default_type in ("CONSTANT", "DYNAMIC")
    trainable = default_type == "DYNAMIC"
    return torch.nn.Parameter(torch.zeros((), dtype=like.dtype, device=like.device), requires_grad=trainable), trainable


class CostMapLayer(torch.nn.Module):
    """cost_aggregate with the voxels no view saw replaced by a default cost (custom_layers.py:34-59).
    call: (ref_image, src_images, base_plane, offsets, Rs, Ts) -> (cost [B,H,W,D], cost_mask [B,H,W,D])."""

    def __init__(self, reduce_method="MIN", half_centor=True, default_type="DYNAMIC"):
        super().__init__()
        assert reduce_method in ["MEAN", "MIN"]
        self.reduce_method = reduce_method
        self.half_centor = half_centor
        self.default_type = default_type
        self.default_cost = None

    def _cost(self, inputs):
        return cost_aggregate(*inputs, reduce_method=self.reduce_method, half_centor=self.half_centor)

    def forward(self, inputs):
        if self.default_cost is None:
            self.default_cost, _ = _default_scalar(self.default_type, inputs[2])
        cost, cost_mask = self._cost(inputs)
        seen = cost_mask > 0 if self.reduce_method == "MEAN" else cost_mask >= 0
        if seen.dim() == cost.dim() and seen.shape != cost.shape:   # MIN masks of the v2 op carry one entry per group
            seen = seen.expand_as(cost)
        return torch.where(seen, cost, self.default_cost.to(cost.dtype)), cost_mask


class CostMapLayerV2(CostMapLayer):
    """The same over cost_volume_v2 (custom_layers.py:61-86).
    call: (ref_image, src_images, depth_grid, Rs, Ts) -> (cost [B,H,W,D,groups], cost_mask)."""

    def __init__(self, reduce_method="MIN", half_centor=True, default_type="DYNAMIC", groups=1):
        super().__init__(reduce_method, half_centor, default_type)
        self.groups = groups

    def _cost(self, inputs):
        return cost_volume_v2(*inputs, reduce_method=self.reduce_method, groups=self.groups, half_centor=self.half_centor)


def _glorot_uniform(shape, dtype, device):
    """Keras' glorot_uniform for a [*kernel, in, out] filter."""
    receptive = 1
    for k in shape[:-2]:
        receptive *= k
    limit = math.sqrt(6.0 / (receptive * (shape[-2] + shape[-1])))
    return (torch.rand(shape, dtype=torch.float32, device=device) * 2 - 1).mul_(limit).to(dtype)


class SparseConv3DLayer(torch.nn.Module):
    """sparse_conv3d_fast with its filter, optional bias and default value as weights (custom_layers.py:88-138).
    call: (images [B,H,W,D,Cin], base_plane [B,H,W,1] int32) -> [B,ceil(H/s),ceil(W/s),ceil(D/s),filters]."""

    def __init__(self, filters, kernel_size, default_type="CONSTANT", strides=(1, 1, 1), dilations=(1, 1, 1), use_bias=False):
        super().__init__()
        assert len(kernel_size) == 3 and len(strides) == 3 and len(dilations) == 3
        self.filters, self.kernel_size = filters, tuple(kernel_size)
        self.strides, self.dilations = tuple(strides), tuple(dilations)
        self.use_bias, self.default_type = use_bias, default_type
        self.kernel = self.bias = self.default_value = None
        self.dynamic_default = False

    def _build(self, images):
        self.kernel = torch.nn.Parameter(_glorot_uniform((*self.kernel_size, images.shape[-1], self.filters), images.dtype,
                                                         images.device))
        if self.use_bias:
            self.bias = torch.nn.Parameter(torch.zeros(self.filters, dtype=images.dtype, device=images.device))
        self.default_value, self.dynamic_default = _default_scalar(self.default_type, images)

    def forward(self, inputs):
        images, base_plane = inputs
        if self.kernel is None:
            self._build(images)
        out = sparse_conv3d_fast(images, self.kernel, self.default_value, base_plane, strides=self.strides,
                                 dilations=self.dilations, dynamic_default=self.dynamic_default)
        return out + self.bias if self.use_bias else out


class SparseConv3DTransposeLayer(torch.nn.Module):
    """sparse_conv3d_transpose_fast as an up-sampling layer (custom_layers.py:140-199): at least one stride above 1,
    unit dilations, a constant zero default.  The filter is [*kernel_size, filters, Cin of the input].
    call: (images, base_plane of the FINE grid [, output_size]); without output_size the fine grid is
    (base_plane rows, base_plane columns, coarse depth * depth stride)."""

    def __init__(self, filters, kernel_size, output_size=None, default_type="CONSTANT", strides=(1, 1, 1),
                 dilations=(1, 1, 1), use_bias=False):
        super().__init__()
        assert len(kernel_size) == 3 and len(strides) == 3 and len(dilations) == 3
        assert strides[0] > 1 or strides[1] > 1 or strides[2] > 1
        assert tuple(dilations) == (1, 1, 1)
        assert default_type == "CONSTANT"
        self.filters, self.kernel_size = filters, tuple(kernel_size)
        self.strides, self.dilations = tuple(strides), tuple(dilations)
        self.use_bias, self.output_size = use_bias, output_size
        self.kernel = self.bias = self.default_value = None

    def forward(self, inputs):
        if len(inputs) == 2:
            images, base_plane = inputs
            output_size = [base_plane.shape[1], base_plane.shape[2], images.shape[3] * self.strides[2]]
        else:
            assert len(inputs) == 3
            images, base_plane, output_size = inputs
        if self.kernel is None:
            self.kernel = torch.nn.Parameter(_glorot_uniform((*self.kernel_size, self.filters, images.shape[-1]),
                                                             images.dtype, images.device))
            if self.use_bias:
                self.bias = torch.nn.Parameter(torch.zeros(self.filters, dtype=images.dtype, device=images.device))
            self.default_value = torch.nn.Parameter(torch.zeros((), dtype=images.dtype, device=images.device),
                                                    requires_grad=False)
        out = sparse_conv3d_transpose_fast(images, self.kernel, self.default_value, base_plane, output_size,
                                           strides=self.strides, dilations=self.dilations, dynamic_default=False)
        return out + self.bias if self.use_bias else out
