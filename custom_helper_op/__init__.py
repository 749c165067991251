"""Drop-in module path of the reference package: `import custom_helper_op` resolves to the B200-native
implementation in custom_helper_op_b200, with the reference's export list
(custom_helper_op/__init__.py:20-36 of the reference) for every op and layer on the accelerated path.

Names the reference exports that are outside that path (sparse_conv2d, the older sparse_conv3d,
DepthProjectLayer, DeformableConv2D) are not provided: asking for one raises an AttributeError that
says so, instead of handing back something that fails later.
"""
from custom_helper_op.python.layers.custom_layers import (CostMapLayer, CostMapLayerV2,  # noqa: F401
                                                           SparseConv3DLayer, SparseConv3DTransposeLayer)
from custom_helper_op.python.ops.custom_helper_ops import (IndexInitializer, cost_aggregate,  # noqa: F401
                                                            cost_volume, cost_volume_v2, cost_volume_v3, decode_pfm,
                                                            feature_aggregate, index_initializer, sparse_conv3d_fast,
                                                            sparse_conv3d_transpose_fast, sparse_pad)

__all__ = ["cost_volume", "cost_volume_v2", "cost_volume_v3", "cost_aggregate", "feature_aggregate",
           "index_initializer", "decode_pfm", "IndexInitializer", "sparse_pad", "sparse_conv3d_fast",
           "sparse_conv3d_transpose_fast", "CostMapLayer", "CostMapLayerV2", "SparseConv3DLayer",
           "SparseConv3DTransposeLayer"]

NOT_ON_THE_ACCELERATED_PATH = ("sparse_conv2d", "sparse_conv3d", "DepthProjectLayer", "DeformableConv2D")


def __getattr__(name):
    if name in NOT_ON_THE_ACCELERATED_PATH:
        raise AttributeError("custom_helper_op.%s is outside the cost-volume / manifold-convolution path this build "
                             "replaces; use the reference package for it" % name)
    raise AttributeError("module 'custom_helper_op' has no attribute %r" % name)
