"""The allocation-free gradient entry point of the manifold convolution.

chop_sparse_conv3d_bwd_noalloc keeps its scratch (partial filter gradients) in a fixed array inside the
library, for callers that cannot hand over a workspace or call the CUDA allocator where the gradient
runs - a host whose device memory belongs to a framework pool, or a loop with a fixed memory budget.
This test drives it through the C ABI with ctypes and compares it with chop_sparse_conv3d_bwd (caller
workspace) on two consecutive calls: the shared array keeps the previous call's contents, so the second
call checks that nothing stale leaks into the result.  (Collected last on purpose: a run that stops at
the first failure has then already exercised everything else.)
"""
import ctypes

import numpy as np
import pytest
import torch

from custom_helper_op_b200 import _lib
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers
from tests.test_oracle_sparse import make_case

pytestmark = pytest.mark.gpu


def _call_noalloc(images, filters, defv, bp, og, dynamic_default):
    d, _ = ops._sc_desc(images, filters, (1, 1, 1), (1, 1, 1), dynamic_default)
    wdt = torch.float32 if images.dtype == torch.bfloat16 else images.dtype   # gradients of bf16 filters are float32
    ig = torch.empty_like(images)
    fg = torch.empty(filters.shape, dtype=wdt, device=images.device)
    dg = torch.empty((), dtype=wdt, device=images.device)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = _lib.lib().chop_sparse_conv3d_bwd_noalloc(ctypes.byref(d), p(images), p(filters), p(defv), p(bp), p(og), p(ig),
                                                   p(fg), p(dg), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, _lib.status_string(st)
    return ig, fg, dg


def test_noalloc_gradient_matches_workspace_gradient_twice_in_a_row():
    dev = "cuda:0"
    for seed, shape in ((21, (2, 10, 12, 9, 16, 16)), (22, (1, 7, 9, 5, 8, 4))):  # second problem is smaller: stale tail
        B, H, W, D, Cin, Cout = shape
        images, filters, defv, bp, _ = make_case(seed, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 6, np.float32)
        t_img = torch.from_numpy(images).to(dev)
        t_flt = torch.from_numpy(filters).to(dev)
        t_def = torch.tensor(float(defv), device=dev)
        t_bp = torch.from_numpy(bp).to(dev)
        og = torch.from_numpy(np.random.default_rng(seed).uniform(-1, 1, (B, H, W, D, Cout)).astype(np.float32)).to(dev)
        ig_w, fg_w, dg_w = ops.sparse_conv3d_backward(t_img, t_flt, t_def, t_bp, og, dynamic_default=True)
        for _ in range(2):
            ig, fg, dg = _call_noalloc(t_img, t_flt, t_def, t_bp, og, True)
            torch.cuda.synchronize()
            # same kernels, different number of partial slabs -> different summation order: float tolerance
            assert helpers.rel_err(ig.cpu().numpy(), ig_w.cpu().numpy()) <= 1e-5
            assert helpers.rel_err(fg.cpu().numpy(), fg_w.cpu().numpy()) <= 1e-5
            assert abs(float(dg) - float(dg_w)) <= 1e-4 * max(1.0, abs(float(dg_w)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float64"])
def test_noalloc_with_the_slab_count_cut_to_the_builtin_scratch(dtype):
    """81 920 voxels, 16 -> 16 channels: the workspace entry point uses 160 partial slabs of 27.6 KB (twice that in
    float64), more than the 4 MiB array holds, so the allocation-free call runs its filter-gradient kernels
    (tensor cores for bfloat16, register-tiled otherwise) on a SMALLER grid than any other test and reads its slabs
    from the built-in array.  Two calls in a row against the workspace entry point."""
    dev = "cuda:0"
    tdt = getattr(torch, dtype)
    B, H, W, D, Cin, Cout = 1, 64, 80, 16, 16, 16
    images, filters, defv, bp, _ = make_case(23, B, H, W, D, Cin, Cout, (3, 3, 3), 2 * D + 6, np.float64)
    t_img = torch.from_numpy(images).to(dev).to(tdt)
    t_flt = torch.from_numpy(filters).to(dev).to(tdt)
    t_def = torch.tensor(float(defv), device=dev, dtype=tdt)
    t_bp = torch.from_numpy(bp).to(dev)
    og = torch.from_numpy(np.random.default_rng(23).uniform(-1, 1, (B, H, W, D, Cout))).to(dev).to(tdt)
    d, _ = ops._sc_desc(t_img, t_flt, (1, 1, 1), (1, 1, 1), True)
    slab = (27 * Cin * Cout + 1) * (8 if dtype == "float64" else 4)
    assert _lib.lib().chop_sparse_conv3d_bwd_workspace_size(ctypes.byref(d)) // slab > (4 << 20) // slab  # the cut applies
    before = _lib.lib().chop_umma_timeouts()
    ig_w, fg_w, dg_w = ops.sparse_conv3d_backward(t_img, t_flt, t_def, t_bp, og, dynamic_default=True)
    tol = {"float32": 1e-5, "bfloat16": 2e-3, "float64": 1e-12}[dtype]
    for _ in range(2):
        ig, fg, dg = _call_noalloc(t_img, t_flt, t_def, t_bp, og, True)
        torch.cuda.synchronize()
        # the image gradient does not use the scratch: same kernel, same result
        assert torch.equal(ig, ig_w)
        assert helpers.rel_err(fg.double().cpu().numpy(), fg_w.double().cpu().numpy()) <= tol
        assert abs(float(dg) - float(dg_w)) <= max(tol, 1e-4) * max(1.0, abs(float(dg_w)))
    assert _lib.lib().chop_umma_timeouts() == before


def test_noalloc_rejects_a_slab_larger_than_the_builtin_scratch():
    dev = "cuda:0"
    # 3x3x3 x 32 x 1300 float32 accumulators = 4.49 MB per slab > 4 MiB
    images = torch.zeros((1, 3, 3, 3, 32), device=dev)
    filters = torch.zeros((3, 3, 3, 32, 1300), device=dev)
    d, _ = ops._sc_desc(images, filters, (1, 1, 1), (1, 1, 1), False)
    x = ctypes.c_void_p(images.data_ptr())
    st = _lib.lib().chop_sparse_conv3d_bwd_noalloc(ctypes.byref(d), x, x, x, x, x, x, x, x, None)
    assert st == -6 and "workspace" in _lib.status_string(st)
