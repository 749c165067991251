"""CPU tests of the oracle itself (no GPU): the plain-C restatement against the golden fixtures
minted from the reference's kernel bodies, against those bodies directly where the compiled library
is present, and against finite differences."""
import numpy as np
import pytest

import oracle
from tests import helpers


@pytest.mark.parametrize("name", helpers.golden_names())
def test_port_matches_golden_bit_for_bit(name):
    kind, reduce, groups, hc, ins, gold = helpers.load_golden(name)
    dtype = ins["ref"].dtype
    cost, mask = oracle.cost_fwd(kind, ins["ref"], ins["src"], ins["depth"], ins["offsets"], ins["Rs"], ins["Ts"],
                                 reduce, groups, hc, dtype, "port", nthreads=1)
    assert helpers.bits_equal(mask, gold["mask"])
    assert helpers.bits_equal(cost, gold["cost"])
    rg, sg, dg = oracle.cost_bwd(kind, ins["ref"], ins["src"], ins["depth"], ins["offsets"], ins["Rs"], ins["Ts"],
                                 gold["cost_grad"], gold["mask"], reduce, groups, hc, dtype, "port")
    assert helpers.bits_equal(rg, gold["ref_grad"])
    assert helpers.bits_equal(sg, gold["src_grad"])
    assert helpers.bits_equal(dg, gold["depth_grad"])


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("kind", [1, 2, 3, 4])
@pytest.mark.parametrize("reduce", ["MEAN", "MIN"])
@pytest.mark.parametrize("camera", ["identity", "shift", "rot_z", "rot_y", "random"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_port_matches_reference_kernels(kind, reduce, camera, dtype):
    groups = 3 if kind in (2, 4) else 1
    c = helpers.make_case(kind, 11, 2, 3, 12, 18, 9 if kind in (2, 4) else 5, 7, camera, dtype)
    a = helpers.oracle_fwd_bwd(kind, c, reduce, groups, True, dtype, impl="port")
    b = helpers.oracle_fwd_bwd(kind, c, reduce, groups, True, dtype, impl="ref")
    for k in ("mask", "cost", "ref_grad", "src_grad", "depth_grad"):
        assert helpers.bits_equal(a[k], b[k]), k


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (needs the reference checkout)")
def test_reference_threads_agree():
    """The multi-threaded sweep of the reference kernels (used as the timed CPU baseline) computes the
    same forward bits and the same gradients up to summation order."""
    c = helpers.make_case(1, 3, 1, 2, 16, 20, 8, 12, "random", np.float32)
    a = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32, impl="ref")
    cost, mask = oracle.cost_fwd(1, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], "MEAN", 1, True,
                                 np.float32, "ref", nthreads=4)
    assert helpers.bits_equal(cost, a["cost"]) and helpers.bits_equal(mask, a["mask"])
    g = oracle.cost_bwd(1, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], a["cost_grad"], mask,
                        "MEAN", 1, True, np.float32, "ref", nthreads=4)
    for x, k in zip(g, ("ref_grad", "src_grad", "depth_grad")):
        assert helpers.rel_err(x, a[k]) < 1e-5


@pytest.mark.parametrize("kind", [1, 2, 3, 4])
def test_float32_tracks_float64(kind):
    groups = 2 if kind in (2, 4) else 1
    c64 = helpers.make_case(kind, 21, 1, 2, 12, 16, 8, 6, "random", np.float64)
    c32 = {k: (None if v is None else v.astype(np.float32)) for k, v in c64.items()}
    # evaluate the double oracle on the float32-rounded inputs so only the arithmetic differs
    c64r = {k: (None if v is None else v.astype(np.float64)) for k, v in c32.items()}
    a = helpers.oracle_fwd_bwd(kind, c32, "MEAN", groups, True, np.float32)
    b = helpers.oracle_fwd_bwd(kind, c64r, "MEAN", groups, True, np.float64, cost_grad=a["cost_grad"].astype(np.float64))
    same = a["mask"] == b["mask"]
    assert same.mean() > 0.995          # only voxels within rounding of a validity boundary may differ
    sel = np.broadcast_to(same, a["cost"].shape)
    assert helpers.rel_err(a["cost"][sel], b["cost"][sel]) < 1e-5


def _loss(kind, c, groups, dtype, w):
    cost, mask = oracle.cost_fwd(kind, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], "MEAN", groups,
                                 True, dtype)
    return float((cost * w).sum()), mask


@pytest.mark.parametrize("kind", [1, 2, 3, 4])
def test_gradient_is_the_derivative(kind):
    """The reference validates its gradient op against a numeric Jacobian in float64
    (cost_volume_op_test.py:422-463); same check for the oracle with central differences."""
    groups = 2 if kind in (2, 4) else 1
    c = helpers.make_case(kind, 31, 1, 2, 8, 10, 4, 4, "shift", np.float64)
    rng = np.random.default_rng(1)
    cost0, mask0 = oracle.cost_fwd(kind, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], "MEAN",
                                   groups, True, np.float64)
    w = rng.standard_normal(cost0.shape)
    rg, sg, dg = oracle.cost_bwd(kind, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], w, mask0,
                                 "MEAN", groups, True, np.float64)
    eps = 1e-6
    for key, grad in (("ref", rg), ("src", sg), ("depth", dg)):
        flat = c[key].reshape(-1)
        for idx in rng.choice(flat.size, size=12, replace=False):
            old = flat[idx]
            flat[idx] = old + eps
            lp, mp = _loss(kind, c, groups, np.float64, w)
            flat[idx] = old - eps
            lm, mm = _loss(kind, c, groups, np.float64, w)
            flat[idx] = old
            if not (np.array_equal(mp, mask0) and np.array_equal(mm, mask0)):
                continue  # the perturbation moved a sample across a validity boundary
            num = (lp - lm) / (2 * eps)
            assert abs(num - grad.reshape(-1)[idx]) <= 5e-5 * max(1.0, abs(num)), (key, idx, num, grad.reshape(-1)[idx])
