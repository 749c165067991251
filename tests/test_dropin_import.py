"""`import custom_helper_op` - the reference's module path - resolves to this implementation: every name of the
reference's export list that is on the accelerated path is importable from the same three module paths with the
reference's signature, and the names outside the path fail with a message that says why."""
import inspect

import pytest

# name -> parameters of the reference signature (custom_helper_op/python/ops/custom_helper_ops.py of the reference)
OPS = {
    "cost_volume": ["ref_image", "src_images", "base_plane", "offsets", "Rs", "Ts", "reduce_method", "half_centor", "name"],
    "cost_volume_v2": ["ref_image", "src_images", "depth_grid", "Rs", "Ts", "reduce_method", "groups", "half_centor", "name"],
    "cost_volume_v3": ["ref_image", "src_images", "base_plane", "offsets", "Rs", "Ts", "reduce_method", "groups",
                       "half_centor", "name"],
    "cost_aggregate": ["ref_image", "src_images", "base_plane", "offsets", "Rs", "Ts", "reduce_method", "half_centor", "name"],
    "feature_aggregate": ["src_images", "base_plane", "offsets", "Rs", "Ts", "half_centor", "name"],
    "sparse_pad": ["images", "base_plane", "strides", "dilations", "name"],
    "sparse_conv3d_fast": ["images", "filters", "default_value", "base_plane", "data_format", "strides", "dilations",
                           "dynamic_default", "name"],
    "sparse_conv3d_transpose_fast": ["images", "filters", "default_value", "base_plane", "output_size", "data_format",
                                     "strides", "dilations", "dynamic_default", "name"],
    "decode_pfm": ["contents", "name"],
}
DEFAULTS = {"reduce_method": "MEAN", "half_centor": True, "groups": None, "name": None, "data_format": "NDHWC",
            "strides": (1, 1, 1), "dilations": (1, 1, 1), "dynamic_default": False}
LAYERS = ["CostMapLayer", "CostMapLayerV2", "SparseConv3DLayer", "SparseConv3DTransposeLayer"]


def test_reference_module_paths_and_signatures():
    import custom_helper_op
    from custom_helper_op.python.layers import custom_layers
    from custom_helper_op.python.ops import custom_helper_ops
    import custom_helper_op_b200.python.ops.custom_helper_ops as impl

    for name, params in OPS.items():
        f = getattr(custom_helper_op, name)
        assert f is getattr(custom_helper_ops, name) is getattr(impl, name)
        sig = inspect.signature(f)
        assert list(sig.parameters)[:len(params)] == params, name
        for p in params:
            if p in DEFAULTS:
                assert sig.parameters[p].default == DEFAULTS[p], (name, p)
    assert callable(custom_helper_op.index_initializer) and inspect.isclass(custom_helper_op.IndexInitializer)
    for name in LAYERS:
        assert getattr(custom_helper_op, name) is getattr(custom_layers, name)


@pytest.mark.parametrize("name", ["sparse_conv2d", "sparse_conv3d", "DepthProjectLayer", "DeformableConv2D"])
def test_names_outside_the_path_fail_loudly(name):
    import custom_helper_op
    with pytest.raises(AttributeError, match="outside the cost-volume"):
        getattr(custom_helper_op, name)
