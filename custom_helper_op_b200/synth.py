"""Seeded synthetic inputs for the cost-volume path (numpy only; shared by tests and the benchmark).

The shapes and value distributions stand in for multi-view-stereo data (DTU / BlendedMVS style:
512x640 and 1184x1600 images at quarter resolution, depth range [425, 935]); no dataset is needed.

Draw order for every workload: ref, src, cameras, depth, upstream gradient.
"""
import numpy as np


def random_cameras(rng, B, N, H, W, max_angle_deg=5.0, t_range=(50.0, 100.0)):
    """Pinhole intrinsics K = [[0.8W,0,W/2],[0,0.8W,H/2],[0,0,1]] for all views; each source view is
    rotated by at most ``max_angle_deg`` about a random axis and translated by ``t_range`` mostly
    in x/y.  Returns the op inputs Rs = K R K^-1 [B,N,3,3] and Ts = K t [B,N,3] (float64), built the
    way the reference's tests combine projections
    (custom_helper_op/python/ops/op_tests/cost_volume_op_test.py:115-134)."""
    K = np.array([[0.8 * W, 0, W / 2.0], [0, 0.8 * W, H / 2.0], [0, 0, 1.0]])
    Kinv = np.linalg.inv(K)
    Rs = np.empty((B, N, 3, 3))
    Ts = np.empty((B, N, 3))
    for b in range(B):
        for n in range(N):
            axis = rng.normal(size=3)
            axis /= np.linalg.norm(axis)
            ang = np.deg2rad(rng.uniform(0.0, max_angle_deg))
            Kx = np.array([[0, -axis[2], axis[1]], [axis[2], 0, -axis[0]], [-axis[1], axis[0], 0]])
            R = np.eye(3) + np.sin(ang) * Kx + (1 - np.cos(ang)) * (Kx @ Kx)
            direction = rng.normal(size=3) * np.array([1.0, 1.0, 0.1])
            direction /= np.linalg.norm(direction)
            t = direction * rng.uniform(*t_range)
            Rs[b, n] = K @ R @ Kinv
            Ts[b, n] = K @ t
    return Rs, Ts


def smooth_depth_map(rng, B, H, W, centre=700.0, amp=200.0):
    """centre + sum of 4 random low-frequency sinusoids with total amplitude <= amp."""
    ys, xs = np.meshgrid(np.arange(H) / H, np.arange(W) / W, indexing="ij")
    out = np.full((B, H, W), centre)
    for b in range(B):
        a = rng.uniform(0.2, 1.0, size=4)
        a = a / a.sum() * amp
        for k in range(4):
            f, g = rng.uniform(0.5, 2.0, size=2)
            phi = rng.uniform(0, 2 * np.pi)
            out[b] += a[k] * np.sin(2 * np.pi * (f * xs + g * ys) + phi)
    return out


def plane_sweep(seed, B, V, C, H, W, D, depth_range=(425.0, 935.0), inverse_depth=False,
                dtype=np.float32, with_grad=True):
    """CostVolume workload with fronto-parallel planes: base_plane = depth_range[0] (or 0 for
    inverse-depth spacing) and per-batch offsets."""
    rng = np.random.default_rng(seed)
    N = V - 1
    ref = rng.standard_normal((B, H, W, C)).astype(dtype)
    src = rng.standard_normal((B, N, H, W, C)).astype(dtype)
    Rs, Ts = random_cameras(rng, B, N, H, W)
    lo, hi = depth_range
    if inverse_depth:
        base = np.zeros((B, H, W, 1))
        offs = 1.0 / np.linspace(1.0 / lo, 1.0 / hi, D)
    else:
        base = np.full((B, H, W, 1), lo)
        offs = np.arange(D) * (hi - lo) / max(D - 1, 1)
    offsets = np.tile(offs[None, :], (B, 1))
    out = dict(ref=ref, src=src, base_plane=base.astype(dtype), offsets=offsets.astype(dtype),
               Rs=Rs.astype(dtype), Ts=Ts.astype(dtype))
    if with_grad:
        out["cost_grad"] = rng.standard_normal((B, H, W, D, C)).astype(dtype)
    return out


def cascade_stage(seed, B, V, C, H, W, D, spacing, groups, dtype=np.float32, with_grad=True):
    """CostVolumeV2 workload: per-pixel hypotheses centred on a smooth random depth map."""
    rng = np.random.default_rng(seed)
    N = V - 1
    ref = rng.standard_normal((B, H, W, C)).astype(dtype)
    src = rng.standard_normal((B, N, H, W, C)).astype(dtype)
    Rs, Ts = random_cameras(rng, B, N, H, W)
    centre = smooth_depth_map(rng, B, H, W)
    grid = centre[..., None] + (np.arange(D) - D / 2.0)[None, None, None, :] * spacing
    out = dict(ref=ref, src=src, depth_grid=grid.astype(dtype), Rs=Rs.astype(dtype), Ts=Ts.astype(dtype),
               groups=groups)
    if with_grad:
        out["cost_grad"] = rng.standard_normal((B, H, W, D, groups)).astype(dtype)
    return out


def test_case(seed, B, N, H, W, C, D, camera="random", dtype=np.float64):
    """Small inputs in the style of the reference's unit tests
    (cost_volume_op_test.py:180-185): features U(0,10), base depth U(20,30), offsets U(-2,2), and one
    of its four camera set-ups: identity / shift T=(3,3,3) / 90 degrees about z / 22.5 degrees about y
    (:187-248), or small random rotations + translations."""
    rng = np.random.default_rng(seed)
    ref = rng.uniform(0, 10, (B, H, W, C))
    src = rng.uniform(0, 10, (B, N, H, W, C))
    base = (rng.uniform(0, 1, (B, H, W, 1)) + 2) * 10
    offsets = rng.uniform(0, 1, (B, D)) * 4 - 2
    Rs = np.tile(np.eye(3)[None, None], (B, N, 1, 1))
    Ts = np.zeros((B, N, 3))

    def rot(axis, ang):
        axis = np.asarray(axis, float)
        Kx = np.array([[0, -axis[2], axis[1]], [axis[2], 0, -axis[0]], [-axis[1], axis[0], 0]])
        return np.eye(3) + np.sin(ang) * Kx + (1 - np.cos(ang)) * (Kx @ Kx)

    if camera == "shift":
        Ts[:] = 3.0
    elif camera == "rot_z":
        Ts[:] = 3.0
        Rs[:] = rot([0, 0, 1], np.pi / 2)
    elif camera == "rot_y":
        Ts[:] = 3.0
        Rs[:] = rot([0, 1, 0], np.pi / 8)
    elif camera == "random":
        for b in range(B):
            for n in range(N):
                ax = rng.normal(size=3)
                ax /= np.linalg.norm(ax)
                Rs[b, n] = rot(ax, rng.uniform(0, 0.05))
                Ts[b, n] = rng.uniform(-3, 3, 3)
    elif camera != "identity":
        raise ValueError(camera)
    cast = lambda a: a.astype(dtype)
    return dict(ref=cast(ref), src=cast(src), base_plane=cast(base), offsets=cast(offsets), Rs=cast(Rs),
                Ts=cast(Ts))


def manifold_conv(seed, B=1, H=256, W=320, D=9, Cin=16, Cout=16, planes=64, with_grad=True):
    """Manifold-convolution workload: a band of D planes around a smooth coarse depth index.
    Activations and weights ~ N(0, 0.1^2), default_value 0; base_plane = clip(idx - D//2, 0, planes - D)."""
    rng = np.random.default_rng(seed)
    images = (rng.standard_normal((B, H, W, D, Cin)) * 0.1).astype(np.float32)
    filters = (rng.standard_normal((3, 3, 3, Cin, Cout)) * 0.1).astype(np.float32)
    centre = smooth_depth_map(rng, B, H, W)
    idx = np.rint((centre - 500.0) * (planes - 1) / 400.0)
    base_plane = np.clip(idx - D // 2, 0, planes - D).astype(np.int32)[..., None]
    out = dict(images=images, filters=filters, default_value=np.float32(0.0), base_plane=base_plane)
    if with_grad:
        out["out_grad"] = rng.standard_normal((B, H, W, D, Cout)).astype(np.float32)
    return out


# The benchmark / parity configurations.
CONFIGS = {
    # name: kind, kwargs
    "c0_cpu": dict(kind=1, B=1, V=3, C=8, H=64, W=80, D=32),
    "c1_mvsnet": dict(kind=1, B=1, V=3, C=32, H=128, W=160, D=192),
    "c2_stage1": dict(kind=2, B=1, V=5, C=32, H=288, W=384, D=48, spacing=8.0, groups=8),
    "c2_stage2": dict(kind=2, B=1, V=5, C=16, H=576, W=768, D=32, spacing=4.0, groups=8),
    "c2_stage3": dict(kind=2, B=1, V=5, C=8, H=1152, W=1536, D=8, spacing=1.0, groups=8),
    "c3_large": dict(kind=1, B=8, V=7, C=32, H=296, W=400, D=256, depth_range=(400.0, 1200.0),
                     inverse_depth=True),
}
CONFIG_SEEDS = {"c0_cpu": 20240, "c1_mvsnet": 20241, "c2_stage1": 20242, "c2_stage2": 20243,
                "c2_stage3": 20244, "c3_large": 20245}


def make(name, scale=1.0, dtype=np.float32, with_grad=True, **override):
    """Inputs of a named configuration; ``scale`` < 1 shrinks H and W (for CPU-sized parity runs)."""
    cfg = dict(CONFIGS[name])
    cfg.update(override)
    kind = cfg.pop("kind")
    cfg["H"] = max(4, int(round(cfg["H"] * scale)))
    cfg["W"] = max(4, int(round(cfg["W"] * scale)))
    seed = CONFIG_SEEDS[name]
    if kind == 1:
        return plane_sweep(seed, dtype=dtype, with_grad=with_grad, **cfg)
    return cascade_stage(seed, dtype=dtype, with_grad=with_grad, **cfg)
