#!/usr/bin/env python3
"""Mint the golden fixtures under tests/golden/ from the reference's own kernel bodies.

Needs oracle/_ref/libchop_ref.so (python oracle/build_ref.py, which needs the reference checkout);
the fixtures it writes are what pins the CPU oracle - and through it the CUDA kernels - wherever
the reference is not available.  Inputs follow the reference's unit tests (uniform features in
[0,10), base depth in [20,30), offsets in [-2,2), its four camera set-ups plus small random
cameras); gradients are produced single-threaded so the sums are reproducible.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from custom_helper_op_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (kind, reduce, dtype, camera, B, N, H, W, C, D, groups, half_centor)
CASES = {
    "v1_mean_f32_random": (1, "MEAN", "float32", "random", 2, 2, 12, 16, 8, 9, 1, True),
    "v1_mean_f32_shift": (1, "MEAN", "float32", "shift", 1, 3, 12, 18, 5, 6, 1, True),
    "v1_min_f32_random": (1, "MIN", "float32", "random", 1, 3, 12, 16, 4, 7, 1, True),
    "v1_mean_f64_roty": (1, "MEAN", "float64", "rot_y", 2, 2, 12, 16, 3, 5, 1, True),
    "v1_mean_f32_nohalf": (1, "MEAN", "float32", "random", 1, 2, 10, 14, 8, 8, 1, False),
    "v2_mean_f32_random": (2, "MEAN", "float32", "random", 2, 2, 12, 16, 9, 6, 3, True),
    "v2_min_f32_random": (2, "MIN", "float32", "random", 1, 3, 12, 16, 8, 5, 4, True),
    "v2_mean_f64_shift": (2, "MEAN", "float64", "shift", 1, 2, 12, 16, 8, 6, 2, True),
    "agg_mean_f32_random": (3, "MEAN", "float32", "random", 1, 2, 12, 16, 8, 6, 1, True),
    "agg_min_f32_random": (3, "MIN", "float32", "random", 1, 3, 12, 16, 5, 6, 1, True),
    "v3_mean_f32_random": (4, "MEAN", "float32", "random", 1, 2, 12, 16, 8, 6, 4, True),
    "v3_min_f32_shift": (4, "MIN", "float32", "shift", 1, 3, 12, 16, 6, 5, 2, True),
}

# SparsePad fixtures: name: (B, coarse h, w, d, C, strides).  The gradient fixture keeps the row/column
# strides at 1, where the reference kernel reads the pixel it means to.
PAD_CASES = {
    "pad_f32_s223": (2, 5, 6, 4, 3, (2, 2, 3)),
    "pad_f32_s112": (1, 6, 7, 5, 2, (1, 1, 2)),
}


def build_pad_case(name):
    B, h, w, d, C, st = PAD_CASES[name]
    rng = np.random.default_rng(2000 + sorted(PAD_CASES).index(name))
    images = rng.standard_normal((B, h, w, d, C)).astype(np.float32)
    base_plane = rng.integers(0, 10, (B, h * st[0], w * st[1], 1)).astype(np.int32)
    out_grad = rng.standard_normal((B, h * st[0], w * st[1], d * st[2], C)).astype(np.float32)
    return images, base_plane, out_grad, st


def build_case(name):
    kind, red, dt, cam, B, N, H, W, C, D, groups, hc = CASES[name]
    dtype = np.dtype(dt)
    seed = 1000 + sorted(CASES).index(name)
    t = synth.test_case(seed, B, N, H, W, C, D, camera=cam, dtype=dtype)
    if kind == 2:
        depth = (t["base_plane"] + t["offsets"][:, None, None, :]).astype(dtype)
        offsets = None
    else:
        depth, offsets = t["base_plane"], t["offsets"]
    return dict(kind=kind, reduce=red, dtype=dtype, groups=groups, half_centor=hc, ref=t["ref"], src=t["src"],
                depth=depth, offsets=offsets, Rs=t["Rs"], Ts=t["Ts"], seed=seed)


def run_case(c, impl):
    cost, mask = oracle.cost_fwd(c["kind"], c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"],
                                 c["reduce"], c["groups"], c["half_centor"], c["dtype"], impl, nthreads=1)
    rng = np.random.default_rng(c["seed"] + 77)
    cost_grad = rng.standard_normal(cost.shape).astype(c["dtype"])
    rg, sg, dg = oracle.cost_bwd(c["kind"], c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"],
                                 cost_grad, mask, c["reduce"], c["groups"], c["half_centor"], c["dtype"], impl,
                                 nthreads=1)
    return dict(cost=cost, mask=mask, cost_grad=cost_grad, ref_grad=rg, src_grad=sg, depth_grad=dg)


def main():
    if not oracle.have_ref():
        sys.exit("oracle/_ref/libchop_ref.so missing: run python oracle/build_ref.py first")
    for name in sorted(CASES):
        c = build_case(name)
        out = run_case(c, "ref")
        arrays = {("in_" + k): v for k, v in c.items() if isinstance(v, np.ndarray)}
        arrays.update({("out_" + k): v for k, v in out.items()})
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print("%-24s %7d bytes  valid voxels %.2f" % (name, os.path.getsize(path),
              float((out["mask"][..., :1] > (-1 if c["reduce"] == "MIN" else 0)).mean())))
    for name in sorted(PAD_CASES):
        images, base_plane, out_grad, st = build_pad_case(name)
        arrays = dict(in_images=images, in_base_plane=base_plane, in_out_grad=out_grad, in_strides=np.array(st),
                      out_output=oracle.sparse_pad_fwd(images, base_plane, st, impl="ref"))
        if st[0] == 1 and st[1] == 1:
            arrays["out_images_grad"] = oracle.sparse_pad_bwd(images, base_plane, out_grad, st, impl="ref")
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print("%-24s %7d bytes" % (name, os.path.getsize(path)))


if __name__ == "__main__":
    main()
