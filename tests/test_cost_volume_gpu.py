"""Parity of the CUDA cost-volume kernels (called through the C ABI) with the CPU oracle.

Tolerances (float32): validity mask and MIN arg-indices bit-exact; cost bit-exact in strict mode and
within 1e-5 (scale-relative) in the default fused mode; gradients within 1e-4 (the sums are
accumulated in a different order and through atomics).  float64: 1e-12 / 1e-10.
"""
import numpy as np
import pytest
import torch

from custom_helper_op_b200 import _lib
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers

pytestmark = pytest.mark.gpu

TOL = {np.float32: (1e-5, 1e-4), np.float64: (1e-12, 1e-10)}


def run_gpu(kind, c, reduce, groups, half_centor, cost_grad, strict=False, bf16=False, mask=None):
    dev = "cuda:0"
    tt = lambda a, feat=False: None if a is None else (
        torch.from_numpy(a).to(dev).to(torch.bfloat16) if (feat and bf16) else torch.from_numpy(a).to(dev))
    ref, src = tt(c["ref"], True), tt(c["src"], True)
    depth, offs, Rs, Ts = tt(c["depth"]), tt(c["offsets"]), tt(c["Rs"]), tt(c["Ts"])
    cost, m = ops.cost_forward(kind, ref, src, depth, offs, Rs, Ts, reduce, groups, half_centor, strict=strict)
    use_mask = m if mask is None else torch.from_numpy(mask).to(dev)
    rg, sg, dg = ops.cost_backward(kind, ref, src, depth, offs, Rs, Ts, tt(cost_grad), use_mask, reduce, groups,
                                   half_centor)
    torch.cuda.synchronize()
    return dict(cost=cost.cpu().numpy(), mask=m.cpu().numpy(), ref_grad=rg.cpu().numpy(),
                src_grad=sg.cpu().numpy(), depth_grad=dg.cpu().numpy())


def check(got, want, dtype, exact_cost):
    ftol, gtol = TOL[dtype]
    assert helpers.bits_equal(got["mask"].reshape(want["mask"].shape), want["mask"]), "mask differs"
    gc = got["cost"].reshape(want["cost"].shape)
    if exact_cost:
        assert helpers.bits_equal(gc, want["cost"]), "strict cost differs"
    else:
        assert helpers.rel_err(gc, want["cost"]) <= ftol
    for k in ("ref_grad", "src_grad", "depth_grad"):
        assert helpers.rel_err(got[k].reshape(want[k].shape), want[k]) <= gtol, k


@pytest.mark.parametrize("name", helpers.golden_names())
def test_golden_fixtures(name):
    kind, reduce, groups, hc, ins, gold = helpers.load_golden(name)
    dtype = ins["ref"].dtype.type
    for strict in (False, True):
        got = run_gpu(kind, ins, reduce, groups, hc, gold["cost_grad"], strict=strict)
        check(got, gold, dtype, exact_cost=strict or reduce == "MIN")


SHAPES = [  # B, N, H, W, C, D   (ragged: odd sizes, C not a multiple of the vector width, D < / > lanes)
    (1, 1, 12, 16, 3, 5), (2, 2, 12, 18, 5, 10), (2, 3, 12, 16, 32, 6), (1, 2, 9, 11, 8, 33),
    (1, 4, 7, 13, 16, 3), (1, 5, 10, 10, 4, 9), (1, 2, 6, 8, 64, 4), (1, 6, 8, 9, 12, 7),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
@pytest.mark.parametrize("camera", ["identity", "shift", "rot_z", "rot_y", "random"])
def test_cost_volume_v1(shape, reduce, camera):
    B, N, H, W, C, D = shape
    c = helpers.make_case(1, 100 + C + D, B, N, H, W, C, D, camera, np.float32)
    want = helpers.oracle_fwd_bwd(1, c, reduce, 1, True, np.float32)
    for strict in (False, True):
        got = run_gpu(1, c, reduce, 1, True, want["cost_grad"], strict=strict)
        check(got, want, np.float32, exact_cost=strict or reduce == "MIN")


@pytest.mark.parametrize("cgs", [(9, 3), (8, 8), (8, 2), (8, 4), (32, 8), (32, 16), (32, 32), (16, 1), (16, 4), (16, 8), (16, 16),
                                 (12, 3), (6, 2), (64, 8), (24, 2)])
@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
def test_cost_volume_v2(cgs, reduce):
    C, G = cgs
    c = helpers.make_case(2, 200 + C, 2, 3, 10, 14, C, 7, "random", np.float32)
    want = helpers.oracle_fwd_bwd(2, c, reduce, G, True, np.float32)
    for strict in (False, True):
        got = run_gpu(2, c, reduce, G, True, want["cost_grad"], strict=strict)
        check(got, want, np.float32, exact_cost=strict or reduce == "MIN")


@pytest.mark.parametrize("C", [3, 8, 16, 20, 32, 64])
@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
def test_cost_aggregate(C, reduce):
    c = helpers.make_case(3, 300 + C, 2, 3, 10, 14, C, 6, "random", np.float32)
    want = helpers.oracle_fwd_bwd(3, c, reduce, 1, True, np.float32)
    for strict in (False, True):
        got = run_gpu(3, c, reduce, 1, True, want["cost_grad"], strict=strict)
        check(got, want, np.float32, exact_cost=strict or reduce == "MIN")


@pytest.mark.parametrize("kind", [1, 2, 3])
@pytest.mark.parametrize("C", [5, 8])
def test_float64(kind, C):
    groups = {5: 1, 8: 4}[C] if kind == 2 else 1
    c = helpers.make_case(kind, 400 + C, 1, 2, 10, 12, C, 6, "random", np.float64)
    want = helpers.oracle_fwd_bwd(kind, c, "MEAN", groups, True, np.float64)
    got = run_gpu(kind, c, "MEAN", groups, True, want["cost_grad"], strict=True)
    check(got, want, np.float64, exact_cost=True)


def test_no_half_centor():
    c = helpers.make_case(1, 17, 1, 2, 10, 12, 8, 6, "random", np.float32)
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, False, np.float32)
    got = run_gpu(1, c, "MEAN", 1, False, want["cost_grad"], strict=True)
    check(got, want, np.float32, exact_cost=True)


@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
@pytest.mark.parametrize("kind,C,G", [(1, 32, 1), (1, 8, 1), (1, 64, 1), (2, 32, 8), (2, 16, 8), (2, 8, 8), (3, 32, 1), (3, 16, 1)])
def test_bfloat16_features(kind, C, G, reduce):
    """bf16 features are an extension; the oracle is the float32 reference arithmetic on the
    bf16-rounded features."""
    c = helpers.make_case(kind, 500 + C, 1, 3, 10, 12, C, 6, "random", np.float32)
    for k in ("ref", "src"):
        c[k] = torch.from_numpy(c[k]).to(torch.bfloat16).to(torch.float32).numpy()
    want = helpers.oracle_fwd_bwd(kind, c, reduce, G, True, np.float32)
    got = run_gpu(kind, c, reduce, G, True, want["cost_grad"], strict=True, bf16=True)
    check(got, want, np.float32, exact_cost=True)
    # compile-time-C kernels (MEAN forward and backward, MIN backward)
    got = run_gpu(kind, c, reduce, G, True, want["cost_grad"], strict=False, bf16=True)
    check(got, want, np.float32, exact_cost=reduce == "MIN")


def test_depth_range_calls_compose():
    """Splitting a batch item by depth range (how work is sharded across GPUs) reproduces the
    single-call result: forward slices are disjoint, gradients add up."""
    c = helpers.make_case(1, 23, 1, 2, 12, 16, 8, 20, "random", np.float32)
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32)
    dev = "cuda:0"
    t = {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in c.items()}
    cg = torch.from_numpy(want["cost_grad"]).to(dev)
    cost = torch.zeros(want["cost"].shape, device=dev)
    mask = torch.zeros(want["mask"].shape, dtype=torch.int32, device=dev)
    grads = None
    for d0, d1 in ((0, 7), (7, 8), (8, 20)):
        ops.cost_forward(1, t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"], strict=True,
                         d_range=(d0, d1), out=(cost, mask))
        if grads is None:
            grads = ops.cost_backward(1, t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"], cg,
                                      torch.from_numpy(want["mask"]).to(dev), d_range=(d0, d1))
        else:
            ops.cost_backward(1, t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"], cg,
                              torch.from_numpy(want["mask"]).to(dev), d_range=(d0, d1), accumulate_into=grads)
    got = dict(cost=cost.cpu().numpy(), mask=mask.cpu().numpy(), ref_grad=grads[0].cpu().numpy(),
               src_grad=grads[1].cpu().numpy(), depth_grad=grads[2].cpu().numpy())
    check(got, want, np.float32, exact_cost=True)


@pytest.mark.parametrize("chunk", [8, 16, 64])
@pytest.mark.parametrize("views", [1, 2, 3, 4])
def test_tuning_knobs_do_not_change_results(chunk, views):
    c = helpers.make_case(1, 29, 1, 5, 10, 12, 32, 40, "random", np.float32)
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32)
    try:
        _lib.set_tuning("fwd_chunk", chunk)
        _lib.set_tuning("bwd_chunk", chunk)
        _lib.set_tuning("bwd_views", views)
        got = run_gpu(1, c, "MEAN", 1, True, want["cost_grad"], strict=True)
    finally:
        for k in ("fwd_chunk", "bwd_chunk", "bwd_views"):
            _lib.set_tuning(k, 0)
    check(got, want, np.float32, exact_cost=True)


@pytest.mark.parametrize("C", [8, 16, 32, 64])
@pytest.mark.parametrize("N", [1, 2, 3, 5])
def test_generic_and_tuned_kernels_agree_with_oracle(C, N):
    """CostVolume MEAN has compile-time-C kernels for common channel counts; the generic kernels must
    stay correct for the same inputs (knob tuned=0), including ragged pixel counts and depth tails."""
    c = helpers.make_case(1, 600 + C + N, 1, N, 9, 13, C, 21, "random", np.float32)
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32)
    for tuned in (1, 0):
        try:
            _lib.set_tuning("tuned", tuned)
            got = run_gpu(1, c, "MEAN", 1, True, want["cost_grad"], strict=False)
        finally:
            _lib.set_tuning("tuned", 1)
        check(got, want, np.float32, exact_cost=False)


def test_autograd_wrapper_matches_raw_ops():
    c = helpers.make_case(1, 41, 1, 2, 10, 12, 8, 6, "random", np.float32)
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32)
    dev = "cuda:0"
    ref = torch.from_numpy(c["ref"]).to(dev).requires_grad_()
    src = torch.from_numpy(c["src"]).to(dev).requires_grad_()
    base = torch.from_numpy(c["depth"]).to(dev).requires_grad_()
    cost, mask = ops.cost_volume(ref, src, base, c["offsets"], c["Rs"], c["Ts"])
    assert not mask.requires_grad
    (cost * torch.from_numpy(want["cost_grad"]).to(dev)).sum().backward()
    assert helpers.rel_err(ref.grad.cpu().numpy(), want["ref_grad"]) <= 1e-4
    assert helpers.rel_err(src.grad.cpu().numpy(), want["src_grad"]) <= 1e-4
    assert helpers.rel_err(base.grad.cpu().numpy(), want["depth_grad"]) <= 1e-4


def test_errors_are_loud():
    c = helpers.make_case(1, 43, 1, 2, 10, 12, 8, 6, "random", np.float32)
    t = {k: torch.from_numpy(v) for k, v in c.items()}
    with pytest.raises(ValueError):   # CPU tensors: there is no CPU kernel
        ops.cost_volume(t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"])
    g = {k: v.cuda() for k, v in t.items()}
    with pytest.raises(ValueError):
        ops.cost_volume(g["ref"], g["src"], g["depth"], g["offsets"], g["Rs"], g["Ts"], reduce_method="MAX")
    with pytest.raises(ValueError):
        ops.cost_volume(g["ref"], g["src"][:, :, :-1], g["depth"], g["offsets"], g["Rs"], g["Ts"])


@pytest.mark.parametrize("name", ["c0_cpu", "c1_mvsnet"])
def test_benchmark_configs_scaled(name):
    """The benchmark workloads at reduced image size, against the oracle."""
    from custom_helper_op_b200 import synth
    w = synth.make(name, scale=0.25)
    c = dict(ref=w["ref"], src=w["src"], depth=w["base_plane"], offsets=w["offsets"], Rs=w["Rs"], Ts=w["Ts"])
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32, cost_grad=w["cost_grad"])
    assert (want["mask"] > 0).mean() > 0.5
    got = run_gpu(1, c, "MEAN", 1, True, w["cost_grad"], strict=True)
    check(got, want, np.float32, exact_cost=True)
    got = run_gpu(1, c, "MEAN", 1, True, w["cost_grad"], strict=False)
    check(got, want, np.float32, exact_cost=False)


def test_host_pipeline_matches_device_ops():
    """The host-buffer pipeline (depth chunks on three streams) returns what one device-resident call returns."""
    from custom_helper_op_b200.host import HostPipeline
    c = helpers.make_case(1, 77, 2, 2, 10, 12, 8, 21, "random", np.float32)
    want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32)
    B, N, H, W, C, D = 2, 2, 10, 12, 8, 21
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    host = dict(ref=pin(c["ref"]), src=pin(c["src"]), base_plane=pin(c["depth"]), offsets=pin(c["offsets"]), Rs=pin(c["Rs"]),
                Ts=pin(c["Ts"]))
    out = dict(cost=torch.empty((B, H, W, D, C)).pin_memory(), mask=torch.empty((B, H, W, D, 1), dtype=torch.int32).pin_memory(),
               ref_grad=torch.empty((B, H, W, C)).pin_memory(), src_grad=torch.empty((B, N, H, W, C)).pin_memory(),
               base_plane_grad=torch.empty((B, H, W, 1)).pin_memory())
    pipe = HostPipeline(B, N, H, W, C, D, "cuda:0", nchunks=4)
    for _ in range(2):   # the second run reuses every buffer
        pipe.run(host, pin(want["cost_grad"]), out)
        got = dict(cost=out["cost"].numpy(), mask=out["mask"].numpy(), ref_grad=out["ref_grad"].numpy(),
                   src_grad=out["src_grad"].numpy(), depth_grad=out["base_plane_grad"].numpy())
        check(got, want, np.float32, exact_cost=False)


EDGE = [  # B, N, H, W, C, D : single plane, tiny images, many views, batch of odd sizes, wide channel counts
    (1, 1, 2, 2, 4, 1), (1, 9, 6, 7, 32, 5), (3, 2, 5, 3, 8, 17), (1, 2, 4, 4, 128, 3), (2, 11, 4, 5, 16, 2), (1, 3, 3, 50, 1, 9),
]


@pytest.mark.parametrize("shape", EDGE)
@pytest.mark.parametrize("kind", [1, 2, 3])
def test_edge_shapes(shape, kind):
    B, N, H, W, C, D = shape
    groups = (C // 4 if C % 4 == 0 else 1) if kind == 2 else 1
    c = helpers.make_case(kind, 900 + C + D, B, N, H, W, C, D, "random", np.float32)
    for reduce in ("MEAN", "MIN"):
        want = helpers.oracle_fwd_bwd(kind, c, reduce, groups, True, np.float32)
        got = run_gpu(kind, c, reduce, groups, True, want["cost_grad"], strict=True)
        check(got, want, np.float32, exact_cost=True)
        if reduce == "MEAN":
            got = run_gpu(kind, c, reduce, groups, True, want["cost_grad"], strict=False)
            check(got, want, np.float32, exact_cost=False)


def test_views_that_see_nothing():
    """A camera looking away (z <= 0 everywhere) and one translated out of the image: no valid sample, the MEAN
    cost stays 0 with mask 0, the MIN cost stays at the largest float with index -1, all gradients are zero."""
    c = helpers.make_case(1, 31, 1, 2, 6, 8, 8, 5, "identity", np.float32)
    c["Rs"][:, 0] = -np.eye(3, dtype=np.float32)      # z = -depth
    c["Ts"][:, 1] = np.array([1e6, 1e6, 0], np.float32)
    for reduce in ("MEAN", "MIN"):
        want = helpers.oracle_fwd_bwd(1, c, reduce, 1, True, np.float32)
        assert (want["mask"] <= 0).all()
        got = run_gpu(1, c, reduce, 1, True, want["cost_grad"], strict=True)
        check(got, want, np.float32, exact_cost=True)
        got = run_gpu(1, c, reduce, 1, True, want["cost_grad"], strict=False)
        assert helpers.bits_equal(got["mask"].reshape(want["mask"].shape), want["mask"])
        assert np.array_equal(got["cost"].reshape(want["cost"].shape), want["cost"])
        assert not got["ref_grad"].any() and not got["src_grad"].any() and not got["depth_grad"].any()


# ---- CostVolumeV3 -------------------------------------------------------------------------------------
@pytest.mark.parametrize("cgs", [(9, 3), (8, 8), (8, 2), (8, 4), (32, 8), (32, 4), (16, 2), (12, 3), (6, 1), (7, 1), (5, 5),
                                 (24, 3), (64, 8), (40, 5), (32, 32)])
@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
def test_cost_volume_v3(cgs, reduce):
    """Cost, validity count and the MIN winner (view, reference group, source group) are bit-exact."""
    C, G = cgs
    c = helpers.make_case(4, 600 + C, 2, 3, 10, 14, C, 7, "random", np.float32)
    want = helpers.oracle_fwd_bwd(4, c, reduce, G, True, np.float32)
    got = run_gpu(4, c, reduce, G, True, want["cost_grad"])
    check(got, want, np.float32, exact_cost=True)


@pytest.mark.parametrize("camera", ["identity", "shift", "rot_z", "rot_y", "random"])
@pytest.mark.parametrize("shape", [(1, 1, 12, 16, 6, 5, 3), (2, 2, 9, 11, 8, 33, 4), (1, 5, 7, 13, 16, 3, 2)])
def test_cost_volume_v3_cameras_and_ragged_shapes(camera, shape):
    B, N, H, W, C, D, G = shape
    c = helpers.make_case(4, 620 + D, B, N, H, W, C, D, camera, np.float32)
    for reduce in ("MEAN", "MIN"):
        want = helpers.oracle_fwd_bwd(4, c, reduce, G, True, np.float32)
        got = run_gpu(4, c, reduce, G, True, want["cost_grad"])
        check(got, want, np.float32, exact_cost=True)


def test_cost_volume_v3_signed_features_and_float64():
    """Zero-mean features: with one group about half of the views have no dot product above the start value
    (the smallest positive normal), which then is that view's cost and carries no gradient."""
    for dtype in (np.float32, np.float64):
        c = helpers.make_case(4, 640, 1, 3, 10, 12, 8, 6, "random", dtype)
        c["ref"] = (c["ref"] - 5).astype(dtype)
        c["src"] = (c["src"] - 5).astype(dtype)
        for G in (1, 4):
            for reduce in ("MEAN", "MIN"):
                want = helpers.oracle_fwd_bwd(4, c, reduce, G, True, dtype)
                got = run_gpu(4, c, reduce, G, True, want["cost_grad"])
                check(got, want, dtype, exact_cost=True)


def test_cost_volume_v3_bfloat16_depth_range_and_autograd():
    c = helpers.make_case(4, 660, 1, 3, 10, 12, 16, 12, "random", np.float32)
    for k in ("ref", "src"):
        c[k] = torch.from_numpy(c[k]).to(torch.bfloat16).to(torch.float32).numpy()
    want = helpers.oracle_fwd_bwd(4, c, "MEAN", 4, True, np.float32)
    got = run_gpu(4, c, "MEAN", 4, True, want["cost_grad"], bf16=True)
    check(got, want, np.float32, exact_cost=True)
    # two depth ranges compose to the full call
    dev = "cuda:0"
    t = {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in c.items()}
    cost, mask = ops.cost_forward(4, t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"], "MEAN", 4,
                                  d_range=(0, 5))
    ops.cost_forward(4, t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"], "MEAN", 4, d_range=(5, 12),
                     out=(cost, mask))
    assert helpers.bits_equal(cost.cpu().numpy(), want["cost"]) and helpers.bits_equal(mask.cpu().numpy(), want["mask"])
    # the public function under autograd
    ref = t["ref"].clone().requires_grad_()
    src = t["src"].clone().requires_grad_()
    base = t["depth"].clone().requires_grad_()
    cost, mask = ops.cost_volume_v3(ref, src, base, t["offsets"], t["Rs"], t["Ts"], "MEAN", 4)
    (cost * torch.from_numpy(want["cost_grad"]).to(dev)).sum().backward()
    assert helpers.rel_err(ref.grad.cpu().numpy(), want["ref_grad"]) <= 1e-4
    assert helpers.rel_err(src.grad.cpu().numpy(), want["src_grad"]) <= 1e-4
    assert helpers.rel_err(base.grad.cpu().numpy(), want["depth_grad"]) <= 1e-4
    with pytest.raises(ValueError):   # more than 8 channels per group
        ops.cost_volume_v3(ref, src, base, t["offsets"], t["Rs"], t["Ts"], "MEAN", 1)


@pytest.mark.parametrize("N", [1, 2, 3, 6])
@pytest.mark.parametrize("C", [8, 16, 32])
@pytest.mark.parametrize("bf16", [False, True])
def test_packed_forward_kernels(N, C, bf16):
    """The MEAN forward on packed pairs: the plane-major kernel (one or two views) and the view-major one (more),
    float32 and bfloat16 features, an odd pixel count, a depth count that is not a multiple of the planes per block,
    a camera that moves the footprint on most planes ("rot_y") and one that leaves it alone ("identity"), the whole
    range and two depth-range calls that cut a block of planes; mask bit-exact, cost within the scale-relative AND
    the element-wise tolerance; against the previous scalar kernel as well (knob `packed`)."""
    B, H, W, D = 2, 7, 9, 21
    dev = "cuda:0"
    for camera in ("rot_y", "identity", "random"):
        c = helpers.make_case(1, 300 + 7 * N + C, B, N, H, W, C, D, camera, np.float32)
        if bf16:
            for k in ("ref", "src"):
                c[k] = torch.from_numpy(c[k]).to(torch.bfloat16).float().numpy()
        want = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32)
        t = {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in c.items()}
        if bf16:
            t["ref"], t["src"] = t["ref"].to(torch.bfloat16), t["src"].to(torch.bfloat16)
        a = (t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"])
        cost, mask = ops.cost_forward(1, *a)
        assert helpers.bits_equal(mask.cpu().numpy(), want["mask"])
        assert helpers.rel_err(cost.cpu().numpy(), want["cost"]) <= 1e-5
        assert helpers.elementwise_excess(cost.cpu().numpy(), want["cost"], 1e-5) <= 1.0
        cost_r = torch.full_like(cost, -1.0)
        mask_r = torch.full_like(mask, -7)
        for d0, d1 in ((0, 5), (5, D)):
            ops.cost_forward(1, *a, d_range=(d0, d1), out=(cost_r, mask_r))
        assert torch.equal(cost_r, cost) and torch.equal(mask_r, mask)
        try:
            _lib.set_tuning("packed", 0)
            cost_s, mask_s = ops.cost_forward(1, *a)
        finally:
            _lib.set_tuning("packed", 1)
        assert torch.equal(mask_s, mask)
        assert float((cost_s - cost).abs().max()) <= 1e-5 * float(cost_s.abs().max())


@pytest.mark.parametrize("N", [1, 2, 3])
@pytest.mark.parametrize("C", [8, 16, 32])
@pytest.mark.parametrize("bf16", [False, True])
def test_packed_cost_aggregate_forward(N, C, bf16):
    """CostAggregate MEAN on the plane-major packed kernel (one or two source views; three take the scalar kernel):
    mask bit-exact, cost within the MEAN tolerances, depth-range calls that cut a block of planes, and the scalar
    kernel on the same inputs (knob `packed`)."""
    B, H, W, D = 2, 7, 9, 21
    dev = "cuda:0"
    for camera in ("rot_y", "identity", "random"):
        c = helpers.make_case(1, 400 + 7 * N + C, B, N, H, W, C, D, camera, np.float32)
        if bf16:
            for k in ("ref", "src"):
                c[k] = torch.from_numpy(c[k]).to(torch.bfloat16).float().numpy()
        want = helpers.oracle_fwd_bwd(3, c, "MEAN", 1, True, np.float32)
        t = {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in c.items()}
        if bf16:
            t["ref"], t["src"] = t["ref"].to(torch.bfloat16), t["src"].to(torch.bfloat16)
        a = (t["ref"], t["src"], t["depth"], t["offsets"], t["Rs"], t["Ts"])
        cost, mask = ops.cost_forward(3, *a)
        assert helpers.bits_equal(mask.cpu().numpy(), want["mask"])
        assert helpers.rel_err(cost.cpu().numpy(), want["cost"]) <= 1e-5
        assert helpers.elementwise_excess(cost.cpu().numpy(), want["cost"], 1e-5) <= 1.0
        cost_r = torch.full_like(cost, -1.0)
        mask_r = torch.full_like(mask, -7)
        for d0, d1 in ((0, 5), (5, D)):
            ops.cost_forward(3, *a, d_range=(d0, d1), out=(cost_r, mask_r))
        assert torch.equal(cost_r, cost) and torch.equal(mask_r, mask)
        try:
            _lib.set_tuning("packed", 0)
            cost_s, mask_s = ops.cost_forward(3, *a)
        finally:
            _lib.set_tuning("packed", 1)
        assert torch.equal(mask_s, mask)
        assert float((cost_s - cost).abs().max()) <= 1e-5 * float(cost_s.abs().max())


@pytest.mark.parametrize("seed", range(24))
def test_random_small_configurations(seed):
    """Seeded random draws over the dispatch boundaries: channel counts with and without a compile-time kernel, one
    to five source views (plane-major / view-major packed forward, generic kernels), depth counts around the planes
    per block and the chunk lengths the host picks for small problems, odd image sizes, every kind and reduction,
    default and strict arithmetic."""
    rng = np.random.default_rng(9000 + seed)
    kind = int(rng.choice([1, 1, 2, 3]))
    C = int(rng.choice([3, 4, 6, 8, 8, 12, 16, 16, 20, 32, 32, 40, 64]))
    groups = 1
    if kind == 2:
        divs = [g for g in (1, 2, 4, 8, 16, 32) if C % g == 0]
        groups = int(rng.choice(divs))
    N = int(rng.integers(1, 6))
    B = int(rng.integers(1, 3))
    H, W = int(rng.integers(3, 14)), int(rng.integers(3, 20))
    D = int(rng.choice([1, 2, 3, 5, 8, 9, 16, 17, 31, 32, 33, 48, 50]))
    reduce = str(rng.choice(["MEAN", "MIN"]))
    camera = str(rng.choice(["identity", "shift", "rot_z", "rot_y", "random"]))
    c = helpers.make_case(kind, 9100 + seed, B, N, H, W, C, D, camera, np.float32)
    want = helpers.oracle_fwd_bwd(kind, c, reduce, groups, True, np.float32)
    for strict in (False, True):
        got = run_gpu(kind, c, reduce, groups, True, want["cost_grad"], strict=strict)
        check(got, want, np.float32, exact_cost=strict or reduce == "MIN")
