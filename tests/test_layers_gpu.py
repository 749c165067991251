"""The layer classes (mirrors of the reference's Keras layers) on the GPU: masking by the default cost, weights
created on first use, gradients reaching every trainable weight."""
import numpy as np
import pytest
import torch

import oracle
from custom_helper_op_b200.python.layers.custom_layers import (CostMapLayer, CostMapLayerV2, SparseConv3DLayer,
                                                               SparseConv3DTransposeLayer)
from tests import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
def test_cost_map_layer(reduce):
    c = helpers.make_case(3, 71, 1, 2, 10, 12, 8, 6, "rot_y", np.float32)   # rot_y leaves many voxels unseen
    want, mask = oracle.cost_fwd(3, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], reduce)
    layer = CostMapLayer(reduce_method=reduce, default_type="DYNAMIC")
    ref = _t(c["ref"]).requires_grad_()
    cost, m = layer((ref, _t(c["src"]), _t(c["depth"]), _t(c["offsets"]), _t(c["Rs"]), _t(c["Ts"])))
    seen = mask > 0 if reduce == "MEAN" else mask >= 0
    assert 0 < seen.mean() < 1
    assert np.array_equal(m.cpu().numpy(), mask)
    got = cost.detach().cpu().numpy()
    assert helpers.rel_err(got[seen], want[seen]) <= 1e-5 and np.all(got[~seen] == 0)
    cost.sum().backward()
    assert float(layer.default_cost.grad) == float((~seen).sum())    # the default cost is trainable
    assert ref.grad is not None and torch.isfinite(ref.grad).all()


def test_cost_map_layer_v2():
    c = helpers.make_case(2, 72, 1, 2, 10, 12, 8, 6, "rot_y", np.float32)
    want, mask = oracle.cost_fwd(2, c["ref"], c["src"], c["depth"], None, c["Rs"], c["Ts"], "MEAN", 4)
    layer = CostMapLayerV2(reduce_method="MEAN", default_type=torch.tensor(-1.0), groups=4)
    cost, m = layer((_t(c["ref"]), _t(c["src"]), _t(c["depth"]), _t(c["Rs"]), _t(c["Ts"])))
    seen = np.broadcast_to(mask > 0, want.shape)
    got = cost.cpu().numpy()
    assert helpers.rel_err(got[seen], want[seen]) <= 1e-5 and np.all(got[~seen] == -1.0)


def test_sparse_conv_layers_down_and_up():
    rng = np.random.default_rng(73)
    B, H, W, D, C = 1, 8, 10, 6, 4
    x = _t(rng.standard_normal((B, H, W, D, C)).astype(np.float32))
    bp = _t(rng.integers(0, 4, (B, H, W, 1)).astype(np.int32))
    down = SparseConv3DLayer(6, (3, 3, 3), default_type="DYNAMIC", strides=(2, 2, 2), use_bias=True)
    up = SparseConv3DTransposeLayer(5, (3, 3, 3), strides=(2, 2, 2), use_bias=True)
    y = down((x, bp))
    assert tuple(y.shape) == (B, 4, 5, 3, 6) and tuple(down.kernel.shape) == (3, 3, 3, C, 6)
    z = up((y, bp))
    assert tuple(z.shape) == (B, H, W, D, 5) and tuple(up.kernel.shape) == (3, 3, 3, 5, 6)
    want_y = oracle.sparse_conv3d_fwd(x.cpu().numpy(), down.kernel.detach().cpu().numpy(), 0.0, bp.cpu().numpy(), (2, 2, 2))
    assert helpers.rel_err(y.detach().cpu().numpy(), want_y) <= 1e-5
    want_z = oracle.sparse_conv3d_transpose_fwd(want_y, up.kernel.detach().cpu().numpy(), 0.0, bp.cpu().numpy(), (H, W, D),
                                                (2, 2, 2))
    assert helpers.rel_err(z.detach().cpu().numpy(), want_z) <= 1e-4
    z.square().mean().backward()
    for p in (down.kernel, down.bias, down.default_value, up.kernel, up.bias):
        assert p.grad is not None and torch.isfinite(p.grad).all()
    assert up.default_value.grad is None and not up.default_value.requires_grad
    z2 = up((y.detach(), bp, (H, W, D)))       # explicit output_size
    assert torch.equal(z2, z.detach())
