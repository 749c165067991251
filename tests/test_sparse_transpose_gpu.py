"""Parity of the transposed manifold convolution, its gradient and SparsePad (CUDA, through the C ABI) with the
CPU oracle.  Tolerances as for the convolution: float32 1e-5 scale-relative, float64 1e-12, bfloat16 storage 1e-2
with float32 filter gradients at 2e-3; SparsePad moves data and is compared bit for bit."""
import numpy as np
import pytest
import torch

import oracle
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers
from tests.test_oracle_sparse import PAD_CASES, TCASES, make_pad_case, make_transpose_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, tdtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return x if tdtype is None else x.to(tdtype)


def _np(x):
    return x.float().cpu().numpy() if x.dtype == torch.bfloat16 else x.cpu().numpy()


@pytest.mark.parametrize("case", TCASES)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("default", [0.0, None])
def test_transpose_forward_and_gradient(case, dtype, default):
    B, H, W, D, Cin, Cout, ks, st, dl = case
    images, filters, defv, bp = make_transpose_case(31, B, H, W, D, Cin, Cout, ks, st, dtype=dtype, default=default)
    want = oracle.sparse_conv3d_transpose_fwd(images, filters, defv, bp, (H, W, D), st, dl, dtype)
    og = np.random.default_rng(32).uniform(-1, 1, want.shape).astype(dtype)
    ig_w, fg_w = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, st, dl, False, dtype)
    out = ops.sparse_conv3d_transpose_forward(_t(images), _t(filters), float(defv), _t(bp), (H, W, D), st, dl)
    ig, fg = ops.sparse_conv3d_transpose_backward(_t(images), _t(filters), float(defv), _t(bp), (H, W, D), _t(og), st, dl)
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == np.float32 else 1e-12
    assert helpers.rel_err(_np(out), want) <= tol
    assert helpers.rel_err(_np(ig), ig_w) <= tol
    assert helpers.rel_err(_np(fg), fg_w) <= tol


def test_transpose_wide_channels():
    """3x3x3 with 48 coarse channels: 1296 accumulator rows in the transposed filter gradient, more than one sweep."""
    B, H, W, D, Cin, Cout, ks, st, dl = 1, 6, 8, 4, 6, 48, (3, 3, 3), (2, 2, 1), (1, 1, 1)
    images, filters, defv, bp = make_transpose_case(35, B, H, W, D, Cin, Cout, ks, st, dtype=np.float32, default=None)
    want = oracle.sparse_conv3d_transpose_fwd(images, filters, defv, bp, (H, W, D), st, dl, np.float32)
    og = np.random.default_rng(36).uniform(-1, 1, want.shape).astype(np.float32)
    ig_w, fg_w = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, st, dl, False, np.float32)
    out = ops.sparse_conv3d_transpose_forward(_t(images), _t(filters), float(defv), _t(bp), (H, W, D), st, dl)
    ig, fg = ops.sparse_conv3d_transpose_backward(_t(images), _t(filters), float(defv), _t(bp), (H, W, D), _t(og), st, dl)
    torch.cuda.synchronize()
    assert helpers.rel_err(_np(out), want) <= 1e-5
    assert helpers.rel_err(_np(ig), ig_w) <= 1e-5
    assert helpers.rel_err(_np(fg), fg_w) <= 1e-5


@pytest.mark.parametrize("strides", [(1, 1, 1), (2, 2, 2), (2, 2, 1)])
@pytest.mark.parametrize("chans", [(16, 16), (32, 16), (16, 32), (8, 16), (8, 8)])
def test_transpose_bfloat16(strides, chans):
    """bf16 storage, float32 accumulation; 16/32-channel 3x3x3 filters run on the tensor cores, 8 channels on the
    register-tiled kernels."""
    Cin, Cout = chans
    B, H, W, D = 1, 10, 12, 8
    images, filters, defv, bp = make_transpose_case(33, B, H, W, D, Cin, Cout, (3, 3, 3), strides, dtype=np.float32)
    r = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    images, filters = r(images), r(filters * 0.3)
    defv = float(r(np.array([defv]))[0])
    want = oracle.sparse_conv3d_transpose_fwd(images, filters, defv, bp, (H, W, D), strides, (1, 1, 1), np.float32)
    og = r(np.random.default_rng(34).uniform(-1, 1, want.shape))
    ig_w, fg_w = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, strides, (1, 1, 1), False,
                                                    np.float32)
    from custom_helper_op_b200 import _lib
    bf = torch.bfloat16
    for umma in (1, 0):   # tensor-core kernels, then the generic ones
        try:
            _lib.set_tuning("umma", umma)
            out = ops.sparse_conv3d_transpose_forward(_t(images, bf), _t(filters, bf), defv, _t(bp), (H, W, D), strides)
            ig, fg = ops.sparse_conv3d_transpose_backward(_t(images, bf), _t(filters, bf), defv, _t(bp), (H, W, D),
                                                          _t(og, bf), strides)
            torch.cuda.synchronize()
        finally:
            _lib.set_tuning("umma", 1)
        assert helpers.rel_err(_np(out), want) <= 1e-2
        assert helpers.rel_err(_np(ig), ig_w) <= 1e-2
        assert fg.dtype == torch.float32 and helpers.rel_err(_np(fg), fg_w) <= 2e-3
    assert _lib.lib().chop_umma_timeouts() == 0


@pytest.mark.parametrize("strides", [(1, 1, 1), (2, 2, 2), (2, 2, 1)])
@pytest.mark.parametrize("chans", [(16, 16), (8, 16), (32, 16)])
@pytest.mark.parametrize("default", [0.0, None])
def test_transpose_float32_register_tiled(strides, chans, default):
    """float32 with 8/16/32 channels: the transposed forward and the image gradient run the register-tiled kernels."""
    Cin, Cout = chans
    B, H, W, D = 1, 9, 10, 6
    images, filters, defv, bp = make_transpose_case(36, B, H, W, D, Cin, Cout, (3, 3, 3), strides, dtype=np.float32,
                                                    default=default)
    want = oracle.sparse_conv3d_transpose_fwd(images, filters, defv, bp, (H, W, D), strides, (1, 1, 1), np.float32)
    og = np.random.default_rng(37).uniform(-1, 1, want.shape).astype(np.float32)
    ig_w, fg_w = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, strides, (1, 1, 1), False,
                                                    np.float32)
    out = ops.sparse_conv3d_transpose_forward(_t(images), _t(filters), float(defv), _t(bp), (H, W, D), strides)
    ig, fg = ops.sparse_conv3d_transpose_backward(_t(images), _t(filters), float(defv), _t(bp), (H, W, D), _t(og), strides)
    torch.cuda.synchronize()
    assert helpers.rel_err(_np(out), want) <= 1e-5
    assert helpers.rel_err(_np(ig), ig_w) <= 1e-5
    assert helpers.rel_err(_np(fg), fg_w) <= 1e-5


def test_transpose_autograd_and_up_down_round_trip():
    """The public function under autograd, and the shapes of a down-sampling convolution followed by the
    transposed one on the same base plane (the pair a coarse-to-fine network uses)."""
    B, H, W, D, C = 1, 9, 11, 7, 4
    st = (2, 2, 2)
    rng = np.random.default_rng(35)
    x = _t(rng.standard_normal((B, H, W, D, C)).astype(np.float32)).requires_grad_()
    bp = _t(rng.integers(0, 5, (B, H, W, 1)).astype(np.int32))
    wd = _t(rng.standard_normal((3, 3, 3, C, 6)).astype(np.float32) * 0.2).requires_grad_()
    wu = _t(rng.standard_normal((3, 3, 3, 5, 6)).astype(np.float32) * 0.2).requires_grad_()
    y = ops.sparse_conv3d_fast(x, wd, 0.0, bp, strides=st)
    assert tuple(y.shape) == (B, 5, 6, 4, 6)
    z = ops.sparse_conv3d_transpose_fast(y, wu, 0.0, bp, (H, W, D), strides=st)
    assert tuple(z.shape) == (B, H, W, D, 5)
    z.square().sum().backward()
    torch.cuda.synchronize()
    g = 2 * z.detach()
    ig_w, fg_w = oracle.sparse_conv3d_transpose_bwd(_np(y.detach()), _np(wu.detach()), 0.0, _np(bp), (H, W, D), _np(g), st)
    assert helpers.rel_err(_np(wu.grad), fg_w) <= 1e-5
    xg_w, wdg_w, _ = oracle.sparse_conv3d_bwd(_np(x.detach()), _np(wd.detach()), 0.0, _np(bp), ig_w, st)
    assert helpers.rel_err(_np(x.grad), xg_w) <= 1e-4
    assert helpers.rel_err(_np(wd.grad), wdg_w) <= 1e-4


def test_transpose_rejects_bad_arguments():
    x = torch.zeros((1, 3, 3, 2, 4), device=DEV)
    w = torch.zeros((3, 3, 3, 5, 4), device=DEV)
    bp = torch.zeros((1, 6, 6, 1), dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError):  # coarse shape does not match ceil(output_size / strides)
        ops.sparse_conv3d_transpose_forward(x, w, 0.0, bp, (6, 6, 8), (2, 2, 2))
    with pytest.raises(ValueError):  # image channels must equal the filter's last axis
        ops.sparse_conv3d_transpose_forward(x, torch.zeros((3, 3, 3, 4, 5), device=DEV), 0.0, bp, (6, 6, 4), (2, 2, 2))
    with pytest.raises(ValueError):
        ops.sparse_conv3d_transpose_forward(x.cpu(), w.cpu(), 0.0, bp.cpu(), (6, 6, 4), (2, 2, 2))


@pytest.mark.parametrize("case", PAD_CASES)
@pytest.mark.parametrize("tdtype", [torch.float32, torch.float64, torch.bfloat16])
def test_sparse_pad(case, tdtype):
    B, h, w, d, C, st = case
    ndt = np.float64 if tdtype == torch.float64 else np.float32
    images, bp, og = make_pad_case(41, B, h, w, d, C, st, ndt)
    if tdtype == torch.bfloat16:
        r = lambda a: torch.from_numpy(a).to(torch.bfloat16).float().numpy()
        images, og = r(images), r(og)
    want = oracle.sparse_pad_fwd(images, bp, st, ndt)
    ig_w = oracle.sparse_pad_bwd(images, bp, og, st, False, ndt)
    out = ops.sparse_pad_forward(_t(images, tdtype), _t(bp), st)
    ig = ops.sparse_pad_backward(_t(images, tdtype), _t(bp), _t(og, tdtype), st)
    torch.cuda.synchronize()
    assert np.array_equal(_np(out).astype(ndt), want)
    assert np.array_equal(_np(ig).astype(ndt), ig_w)


def test_sparse_pad_golden_and_autograd():
    for name in helpers.pad_golden_names():
        z = np.load(f"{helpers.GOLDEN_DIR}/{name}.npz")
        st = tuple(int(s) for s in z["in_strides"])
        x = _t(z["in_images"]).requires_grad_()
        out = ops.sparse_pad(x, _t(z["in_base_plane"]), st)
        assert np.array_equal(_np(out.detach()), z["out_output"])
        (out * _t(z["in_out_grad"])).sum().backward()
        if "out_images_grad" in z.files:
            assert np.array_equal(_np(x.grad), z["out_images_grad"])
