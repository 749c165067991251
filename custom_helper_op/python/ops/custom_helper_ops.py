"""custom_helper_op.python.ops.custom_helper_ops - the reference's op module path
(custom_helper_op/python/ops/custom_helper_ops.py:33,66,99,133,166,221,264,291,317,329,332), re-exporting
the op functions of custom_helper_op_b200.python.ops.custom_helper_ops: same names, positional order and
defaults; torch CUDA tensors and torch.autograd in place of TensorFlow tensors and tf.RegisterGradient."""
from custom_helper_op_b200.python.ops.custom_helper_ops import (  # noqa: F401
    IndexInitializer, cost_aggregate, cost_volume, cost_volume_v2, cost_volume_v3, decode_pfm, feature_aggregate,
    index_initializer, sparse_conv3d_fast, sparse_conv3d_transpose_fast, sparse_pad)

__all__ = ["cost_volume", "cost_volume_v2", "cost_volume_v3", "cost_aggregate", "feature_aggregate", "sparse_pad",
           "sparse_conv3d_fast", "sparse_conv3d_transpose_fast", "decode_pfm", "index_initializer", "IndexInitializer"]
