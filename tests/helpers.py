"""Shared helpers of the parity tests."""
import glob
import os

import numpy as np

import oracle
from custom_helper_op_b200 import synth

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_names():
    """The cost-volume fixtures (v1_*, v2_*, v3_*, agg_*)."""
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz"))
                  if not os.path.basename(p).startswith("pad_"))


def pad_golden_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "pad_*.npz")))


def golden_meta(name):
    kind = {"v1": 1, "v2": 2, "agg": 3, "v3": 4}[name.split("_")[0]]
    reduce = name.split("_")[1].upper()
    return kind, reduce


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    ins = {k[3:]: z[k] for k in z.files if k.startswith("in_")}
    outs = {k[4:]: z[k] for k in z.files if k.startswith("out_")}
    ins.setdefault("offsets", None)
    kind, reduce = golden_meta(name)
    # groups / half_centor are encoded by the generator's case table
    from tests.golden.make_golden import CASES
    groups, half_centor = CASES[name][10], CASES[name][11]
    return kind, reduce, groups, half_centor, ins, outs


def make_case(kind, seed, B, N, H, W, C, D, camera="random", dtype=np.float32):
    """Reference-test style inputs for any kind: returns dict(ref, src, depth, offsets, Rs, Ts)."""
    t = synth.test_case(seed, B, N, H, W, C, D, camera=camera, dtype=np.float64)
    if kind == 2:
        depth = t["base_plane"] + t["offsets"][:, None, None, :]
        offsets = None
    else:
        depth, offsets = t["base_plane"], t["offsets"]
    cast = lambda a: None if a is None else a.astype(dtype)
    return dict(ref=cast(t["ref"]), src=cast(t["src"]), depth=cast(depth), offsets=cast(offsets),
                Rs=cast(t["Rs"]), Ts=cast(t["Ts"]))


def oracle_fwd_bwd(kind, c, reduce, groups, half_centor, dtype, cost_grad=None, seed=5, impl="port"):
    cost, mask = oracle.cost_fwd(kind, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], reduce,
                                 groups, half_centor, dtype, impl)
    if cost_grad is None:
        cost_grad = np.random.default_rng(seed).standard_normal(cost.shape).astype(dtype)
    rg, sg, dg = oracle.cost_bwd(kind, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], cost_grad,
                                 mask, reduce, groups, half_centor, dtype, impl)
    return dict(cost=cost, mask=mask, cost_grad=cost_grad, ref_grad=rg, src_grad=sg, depth_grad=dg)


def bits_equal(a, b):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def rel_err(a, b):
    """max |a-b| / max |b| - the scale-relative error used for the float tolerances."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.abs(b).max()
    return float(np.abs(a - b).max() / den) if den > 0 else float(np.abs(a - b).max())


def elementwise_excess(got, want, rtol, atol_rel=1e-6):
    """Element-wise closeness in the sense of the reference tests' assertAllClose(rtol=..) on a float32
    tensor (cost_volume_op_test.py:197-209): returns max over elements of |got-want| / (rtol*|want| + atol),
    where atol = atol_rel * max|want| plays the part of assertAllClose's default absolute tolerance (1e-6)
    on tensors of order one.  A value <= 1 passes."""
    g = np.asarray(got, np.float64).reshape(-1)
    w = np.asarray(want, np.float64).reshape(g.shape)
    atol = atol_rel * float(np.abs(w).max()) if w.size else 0.0
    bound = rtol * np.abs(w) + atol
    bound[bound == 0] = np.finfo(np.float64).tiny
    return float((np.abs(g - w) / bound).max()) if g.size else 0.0


def worst_relative(got, want, floor_rel=1e-3):
    """Largest |got-want|/|want| over the elements with |want| >= floor_rel * max|want| (reported, not asserted)."""
    g = np.asarray(got, np.float64).reshape(-1)
    w = np.asarray(want, np.float64).reshape(g.shape)
    keep = np.abs(w) >= floor_rel * np.abs(w).max()
    return float((np.abs(g - w)[keep] / np.abs(w)[keep]).max()) if keep.any() else 0.0
