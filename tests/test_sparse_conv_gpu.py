"""Parity of the CUDA manifold-convolution kernels (through the C ABI) with the CPU oracle.
Tolerances: float32 1e-5 (scale-relative, the reference tests' rtol), float64 1e-12, bfloat16 storage 1e-2
(outputs are rounded to bf16: 2^-8 relative) with float32 filter gradients at 2e-3."""
import numpy as np
import pytest
import torch

import oracle
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers
from tests.test_oracle_sparse import CASES, make_case

pytestmark = pytest.mark.gpu


def run_gpu(images, filters, defv, bp, og, st, dl, dynamic_default, tdtype):
    dev = "cuda:0"
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(tdtype)
    out = ops.sparse_conv3d_forward(t(images), t(filters), float(defv), torch.from_numpy(bp).to(dev), st, dl)
    ig, fg, dg = ops.sparse_conv3d_backward(t(images), t(filters), float(defv), torch.from_numpy(bp).to(dev), t(og), st,
                                            dl, dynamic_default)
    torch.cuda.synchronize()
    f = lambda x: x.float().cpu().numpy() if x.dtype == torch.bfloat16 else x.cpu().numpy()
    return f(out), f(ig), f(fg), f(dg)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("dynamic_default", [False, True])
def test_generic_kernels(case, dtype, dynamic_default):
    B, H, W, D, Cin, Cout, ks, st, dl, vd = case
    images, filters, defv, bp, _ = make_case(7, B, H, W, D, Cin, Cout, ks, vd, dtype)
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, st, dl, dtype)
    og = np.random.default_rng(8).uniform(-1, 1, want.shape).astype(dtype)
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, st, dl, dynamic_default, dtype)
    out, ig, fg, dg = run_gpu(images, filters, defv, bp, og, st, dl, dynamic_default,
                              torch.float32 if dtype == np.float32 else torch.float64)
    tol = 1e-5 if dtype == np.float32 else 1e-12
    assert helpers.rel_err(out, want) <= tol
    assert helpers.rel_err(ig, ig_w) <= tol
    assert helpers.rel_err(fg, fg_w) <= tol
    assert abs(float(dg) - float(dg_w)) <= tol * max(1.0, abs(float(dg_w)))
    if not dynamic_default:
        assert float(dg) == 0.0


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("chan", [(64, 8), (40, 24)])
def test_wide_channels(chan, dtype):
    """3x3x3 with 64 (40) input channels: 1728 (1080) filter rows per output channel - more than one sweep of the
    generic filter-gradient kernel's accumulator rows.  The reference has no channel limit
    (sparse_conv3d_fast_op.cc:54-146)."""
    Cin, Cout = chan
    B, H, W, D = 1, 6, 7, 5
    images, filters, defv, bp, _ = make_case(31, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 6, dtype)
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, (1, 1, 1), (1, 1, 1), dtype)
    og = np.random.default_rng(32).uniform(-1, 1, want.shape).astype(dtype)
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, (1, 1, 1), (1, 1, 1), True, dtype)
    out, ig, fg, dg = run_gpu(images, filters, defv, bp, og, (1, 1, 1), (1, 1, 1), True,
                              torch.float32 if dtype == np.float32 else torch.float64)
    tol = 1e-5 if dtype == np.float32 else 1e-12
    assert helpers.rel_err(out, want) <= tol
    assert helpers.rel_err(ig, ig_w) <= tol
    assert helpers.rel_err(fg, fg_w) <= tol
    assert abs(float(dg) - float(dg_w)) <= tol * max(1.0, abs(float(dg_w)))


@pytest.mark.parametrize("shape", [(1, 12, 14, 9, 16, 16), (2, 9, 11, 9, 16, 16), (1, 8, 8, 5, 32, 16), (1, 7, 9, 9, 16, 32)])
def test_bfloat16(shape):
    """bf16 storage with float32 accumulation; oracle on the bf16-rounded inputs."""
    B, H, W, D, Cin, Cout = shape
    images, filters, defv, bp, _ = make_case(9, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 6, np.float32)
    r = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    images, filters = r(images - 0.5), r(filters * 0.3)
    defv = float(r(np.array([defv]))[0])
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, dtype=np.float32)
    og = r(np.random.default_rng(10).uniform(-1, 1, want.shape))
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, dynamic_default=True, dtype=np.float32)
    out, ig, fg, dg = run_gpu(images, filters, defv, bp, og, (1, 1, 1), (1, 1, 1), True, torch.bfloat16)
    assert helpers.rel_err(out, want) <= 1e-2
    assert helpers.rel_err(ig, ig_w) <= 1e-2
    assert helpers.rel_err(fg, fg_w) <= 2e-3
    assert abs(float(dg) - float(dg_w)) <= 2e-3 * max(1.0, abs(float(dg_w)))


@pytest.mark.parametrize("shape", [(1, 12, 14, 9, 16, 16), (2, 9, 11, 9, 16, 32), (1, 8, 8, 5, 32, 16), (1, 7, 9, 9, 32, 32),
                                   (1, 40, 48, 9, 16, 16)])
def test_tensor_core_kernel_matches_generic_kernel(shape):
    """The tcgen05 implicit-GEMM path (bf16, 3x3x3, stride 1) against the generic kernels on the same bf16
    inputs: both accumulate the same bf16 products in float32, so they agree to accumulation order, and
    after rounding the output to bf16 they may differ by one bf16 ulp at most."""
    from custom_helper_op_b200 import _lib
    B, H, W, D, Cin, Cout = shape
    images, filters, defv, bp, _ = make_case(13, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 6, np.float32)
    og = np.random.default_rng(14).uniform(-1, 1, (B, H, W, D, Cout)).astype(np.float32)
    res = {}
    for umma in (1, 0):
        try:
            _lib.set_tuning("umma", umma)
            res[umma] = run_gpu(images - 0.5, filters * 0.3, defv, bp, og, (1, 1, 1), (1, 1, 1), True, torch.bfloat16)
        finally:
            _lib.set_tuning("umma", 1)
    assert _lib.lib().chop_umma_timeouts() == 0
    for x, y in zip(res[1][:2], res[0][:2]):   # output and images_grad
        assert helpers.rel_err(x, y) <= 2.0 ** -7


@pytest.mark.parametrize("strides", [(2, 2, 2), (2, 2, 1), (1, 1, 2), (3, 2, 2)])
@pytest.mark.parametrize("chans", [(16, 16), (32, 16), (16, 32)])
def test_bfloat16_strided(strides, chans):
    """Strided 3x3x3 bf16 convolutions (the down-sampling step of a coarse-to-fine network) run on the tensor
    cores too; oracle on the bf16-rounded inputs, and the generic kernels on the same inputs."""
    from custom_helper_op_b200 import _lib
    Cin, Cout = chans
    B, H, W, D = 2, 11, 13, 9
    images, filters, defv, bp, _ = make_case(15, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 8, np.float32)
    r = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    images, filters = r(images - 0.5), r(filters * 0.3)
    defv = float(r(np.array([defv]))[0])
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, strides, dtype=np.float32)
    og = r(np.random.default_rng(16).uniform(-1, 1, want.shape))
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, strides, dynamic_default=True, dtype=np.float32)
    res = {}
    for umma in (1, 0):
        try:
            _lib.set_tuning("umma", umma)
            res[umma] = run_gpu(images, filters, defv, bp, og, strides, (1, 1, 1), True, torch.bfloat16)
        finally:
            _lib.set_tuning("umma", 1)
    assert _lib.lib().chop_umma_timeouts() == 0
    for out, ig, fg, dg in res.values():
        assert helpers.rel_err(out, want) <= 1e-2
        assert helpers.rel_err(ig, ig_w) <= 1e-2
        assert helpers.rel_err(fg, fg_w) <= 2e-3
        assert abs(float(dg) - float(dg_w)) <= 2e-3 * max(1.0, abs(float(dg_w)))


@pytest.mark.parametrize("D", [1, 2, 30, 62, 63, 126, 127])
def test_tensor_core_kernel_band_depths(D):
    """The stride-1 tensor-core forward / image gradient packs 128 // (D + 2) pixels into a tile (D <= 126) and falls
    back to one voxel per row above that; both against the oracle on bf16-rounded inputs."""
    from custom_helper_op_b200 import _lib
    B, H, W, Cin, Cout = 1, 5, 7, 16, 16
    images, filters, defv, bp, _ = make_case(17, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 6, np.float32)
    r = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    images, filters = r(images - 0.5), r(filters * 0.3)
    defv = float(r(np.array([defv]))[0])
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, dtype=np.float32)
    og = r(np.random.default_rng(18).uniform(-1, 1, want.shape))
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, dynamic_default=True, dtype=np.float32)
    for rows in (1, 0):
        try:
            _lib.set_tuning("umma_rows", rows)
            out, ig, fg, dg = run_gpu(images, filters, defv, bp, og, (1, 1, 1), (1, 1, 1), True, torch.bfloat16)
        finally:
            _lib.set_tuning("umma_rows", 1)
        assert helpers.rel_err(out, want) <= 1e-2
        assert helpers.rel_err(ig, ig_w) <= 1e-2
        assert helpers.rel_err(fg, fg_w) <= 2e-3
    assert _lib.lib().chop_umma_timeouts() == 0


TILE_CASES = [  # B, H, W, D, Cin, Cout, ksize, strides, dilations, virtual depth
    (1, 7, 9, 9, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), 20),
    (2, 6, 8, 5, 8, 16, (3, 3, 3), (2, 2, 2), (1, 1, 1), 14),
    (1, 8, 7, 6, 16, 8, (3, 3, 3), (2, 2, 1), (1, 1, 1), 14),
    (1, 6, 6, 7, 32, 16, (3, 3, 3), (1, 1, 1), (2, 2, 2), 18),
    (1, 5, 6, 4, 16, 32, (5, 3, 3), (1, 1, 1), (1, 1, 1), 12),
    (1, 6, 5, 3, 32, 32, (2, 2, 1), (2, 2, 1), (1, 1, 1), 10),
    (1, 5, 5, 1, 8, 8, (1, 1, 1), (1, 1, 1), (1, 1, 1), 6),
]


@pytest.mark.parametrize("case", TILE_CASES)
def test_float32_register_tiled_kernels(case):
    """float32 with 8/16/32 channels runs the register-tiled kernels (forward, image gradient); against the oracle and
    against the one-thread-per-element kernels on the same inputs."""
    from custom_helper_op_b200 import _lib
    B, H, W, D, Cin, Cout, ks, st, dl, vd = case
    images, filters, defv, bp, _ = make_case(19, B, H, W, D, Cin, Cout, ks, vd, np.float32)
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, st, dl, np.float32)
    og = np.random.default_rng(20).uniform(-1, 1, want.shape).astype(np.float32)
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, st, dl, True, np.float32)
    res = {}
    for tile in (1, 0):
        try:
            _lib.set_tuning("tile", tile)
            res[tile] = run_gpu(images, filters, defv, bp, og, st, dl, True, torch.float32)
        finally:
            _lib.set_tuning("tile", 1)
        out, ig, fg, dg = res[tile]
        assert helpers.rel_err(out, want) <= 1e-5
        assert helpers.rel_err(ig, ig_w) <= 1e-5
        assert helpers.rel_err(fg, fg_w) <= 1e-5
        assert abs(float(dg) - float(dg_w)) <= 1e-5 * max(1.0, abs(float(dg_w)))
    assert helpers.rel_err(res[1][0], res[0][0]) <= 1e-6 and helpers.rel_err(res[1][1], res[0][1]) <= 1e-6


@pytest.mark.parametrize("case", TILE_CASES[1:])
def test_bfloat16_register_tiled_kernels(case):
    """bf16 storage where the tensor-core kernels do not apply (8 channels, dilation, other filter sizes): the
    register-tiled kernels with float32 accumulation against the oracle on the bf16-rounded inputs."""
    from custom_helper_op_b200 import _lib
    B, H, W, D, Cin, Cout, ks, st, dl, vd = case
    images, filters, defv, bp, _ = make_case(21, B, H, W, D, Cin, Cout, ks, vd, np.float32)
    r = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    images, filters = r(images - 0.5), r(filters * 0.3)
    defv = float(r(np.array([defv]))[0])
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, st, dl, np.float32)
    og = r(np.random.default_rng(22).uniform(-1, 1, want.shape))
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, st, dl, True, np.float32)
    try:
        _lib.set_tuning("umma", 0)     # the (16|32)-channel 3x3x3 cases would otherwise take the tensor-core path
        out, ig, fg, dg = run_gpu(images, filters, defv, bp, og, st, dl, True, torch.bfloat16)
    finally:
        _lib.set_tuning("umma", 1)
    assert helpers.rel_err(out, want) <= 1e-2
    assert helpers.rel_err(ig, ig_w) <= 1e-2
    assert helpers.rel_err(fg, fg_w) <= 2e-3
    assert abs(float(dg) - float(dg_w)) <= 2e-3 * max(1.0, abs(float(dg_w)))


def test_autograd_wrapper():
    images, filters, defv, bp, _ = make_case(11, 1, 6, 7, 5, 4, 3, (3, 3, 3), 12, np.float32)
    want = oracle.sparse_conv3d_fwd(images, filters, defv, bp, dtype=np.float32)
    og = np.random.default_rng(12).uniform(-1, 1, want.shape).astype(np.float32)
    ig_w, fg_w, dg_w = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, dynamic_default=True, dtype=np.float32)
    dev = "cuda:0"
    ti = torch.from_numpy(images).to(dev).requires_grad_()
    tf = torch.from_numpy(filters).to(dev).requires_grad_()
    td = torch.tensor(float(defv), device=dev, requires_grad=True)
    out = ops.sparse_conv3d_fast(ti, tf, td, torch.from_numpy(bp).to(dev), dynamic_default=True)
    (out * torch.from_numpy(og).to(dev)).sum().backward()
    assert helpers.rel_err(out.detach().cpu().numpy(), want) <= 1e-5
    assert helpers.rel_err(ti.grad.cpu().numpy(), ig_w) <= 1e-5
    assert helpers.rel_err(tf.grad.cpu().numpy(), fg_w) <= 1e-5
    assert abs(float(td.grad) - float(dg_w)) <= 1e-4 * max(1.0, abs(float(dg_w)))
    with pytest.raises(ValueError):
        ops.sparse_conv3d_fast(ti.cpu(), tf.cpu(), 0.0, torch.from_numpy(bp))


def test_a_give_up_reaches_the_host_without_a_synchronising_poll():
    """The bookkeeping a tensor-core kernel performs when a bounded wait runs out, exercised without any wait: a
    one-thread kernel bumps the device counter and its pinned host mirror (test knob "note_timeout").  The host sees
    the count through chop_umma_watch() - a plain read of host memory - and the bf16 wrappers refuse to run until
    the counters are cleared."""
    from custom_helper_op_b200 import _lib
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops
    L = _lib.lib()
    assert L.chop_umma_watch() == 0 and L.chop_umma_timeouts() == 0
    images, filters, defv, bp, _ = make_case(31, 1, 6, 7, 9, 16, 16, (3, 3, 3), 24, np.float32)
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to("cuda:0").to(dt)
    args = (t(images, torch.bfloat16), t(filters, torch.bfloat16), float(defv), t(bp, torch.int32))
    ops.sparse_conv3d_forward(*args)
    try:
        _lib.set_tuning("note_timeout", 1)
        torch.cuda.synchronize()
        assert L.chop_umma_watch() == 1 and L.chop_umma_timeouts() == 1
        with pytest.raises(RuntimeError, match="timed out"):
            ops.sparse_conv3d_forward(*args)
        ops.sparse_conv3d_forward(args[0].float(), args[1].float(), args[2], args[3])   # float32: no tensor-core kernel, no check
    finally:
        _lib.set_tuning("note_timeout", 0)
    assert L.chop_umma_watch() == 0 and L.chop_umma_timeouts() == 0
    ops.sparse_conv3d_forward(*args)
