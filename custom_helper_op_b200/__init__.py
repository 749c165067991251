"""B200-native drop-in for the cost-volume path of custom_helper_op: the same op functions as the
reference package exports (custom_helper_op/__init__.py:20-31), backed by hand-written sm_100a CUDA
kernels behind a C ABI (include/chop.h)."""
from custom_helper_op_b200.python.layers.custom_layers import (CostMapLayer, CostMapLayerV2,  # noqa: F401
                                                               SparseConv3DLayer, SparseConv3DTransposeLayer)
from custom_helper_op_b200.python.ops.custom_helper_ops import (IndexInitializer, cost_aggregate,  # noqa: F401
                                                                 cost_volume, cost_volume_v2, cost_volume_v3, decode_pfm,
                                                                 feature_aggregate, index_initializer, sparse_conv3d_fast,
                                                                 sparse_conv3d_transpose_fast, sparse_pad)

__all__ = ["cost_volume", "cost_volume_v2", "cost_volume_v3", "cost_aggregate", "feature_aggregate", "index_initializer",
           "IndexInitializer", "decode_pfm", "sparse_conv3d_fast",
           "sparse_conv3d_transpose_fast", "sparse_pad", "CostMapLayer", "CostMapLayerV2", "SparseConv3DLayer",
           "SparseConv3DTransposeLayer"]
