"""custom_helper_op.python.layers.custom_layers - the reference's layer module path
(custom_helper_op/python/layers/custom_layers.py:33,59,85,132), re-exporting the torch.nn.Module layers of
custom_helper_op_b200.python.layers.custom_layers (same constructor arguments and weights)."""
from custom_helper_op_b200.python.layers.custom_layers import (  # noqa: F401
    CostMapLayer, CostMapLayerV2, SparseConv3DLayer, SparseConv3DTransposeLayer)

__all__ = ["CostMapLayer", "CostMapLayerV2", "SparseConv3DLayer", "SparseConv3DTransposeLayer"]
