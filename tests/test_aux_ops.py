"""FeatureAggregate, IndexInitializer and DecodePfm: CPU tests of the oracle (against the reference kernels compiled
for the host where present, and against first principles) and of the host-side PFM parser in the library; GPU parity
tests of the kernels through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers


def fa_case(seed, B, N, H, W, C, D, camera, dtype, src_hw=None):
    t = helpers.make_case(1, seed, B, N, H, W, C, D, camera, dtype)
    if src_hw is not None:   # source images of another size than the output grid
        rng = np.random.default_rng(seed + 1)
        t["src"] = rng.uniform(0, 10, (B, N, src_hw[0], src_hw[1], C)).astype(dtype)
    return t


# ---- oracle (CPU) -------------------------------------------------------------------------------------
@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("camera", ["identity", "shift", "rot_z", "rot_y", "random"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_feature_aggregate_port_matches_reference_kernels(camera, dtype):
    c = fa_case(81, 2, 3, 10, 12, 5, 6, camera, dtype, src_hw=(12, 9) if camera == "random" else None)
    a = oracle.feature_aggregate_fwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], True, dtype, "port")
    b = oracle.feature_aggregate_fwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], True, dtype, "ref")
    assert helpers.bits_equal(a[0], b[0]) and helpers.bits_equal(a[1], b[1])
    g = np.random.default_rng(82).standard_normal(a[0].shape).astype(dtype)
    ga = oracle.feature_aggregate_bwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], g, a[1], True, dtype, "port")
    gb = oracle.feature_aggregate_bwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], g, a[1], True, dtype, "ref")
    assert helpers.bits_equal(ga[0], gb[0]) and helpers.bits_equal(ga[1], gb[1])


def test_feature_aggregate_is_the_sample_the_cost_volume_uses():
    """mean over the seen views of (mapped - ref)^2 is the CostVolume MEAN cost; the mask sums to its view count."""
    c = helpers.make_case(1, 83, 1, 3, 10, 12, 4, 5, "random", np.float64)
    mapped, mask = oracle.feature_aggregate_fwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], True, np.float64)
    cost, used = oracle.cost_fwd(1, c["ref"], c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], "MEAN", 1, True, np.float64)
    assert np.array_equal(mask.sum(axis=4), used)
    sq = ((mapped - c["ref"][:, :, :, None, None, :]) ** 2 * mask).sum(axis=4)
    want = np.where(used > 0, sq / np.maximum(used, 1), 0.0)
    np.testing.assert_allclose(want, cost, rtol=1e-12, atol=1e-12)


def test_index_initializer_oracle():
    for H, W in ((5, 6), (1, 1), (1, 8), (8, 1), (37, 41)):     # the reference test's shapes, index_initializer_op_test.py:29-35
        for hc in (True, False):
            out = oracle.index_initializer(H, W, hc, np.float32)
            assert out.shape == (H, W, 3)
            for i in (0, H - 1):
                for j in (0, W - 1):
                    assert tuple(out[i, j]) == (j + 0.5 * hc, i + 0.5 * hc, 1.0)
            if oracle.have_ref():
                assert np.array_equal(out, oracle.index_initializer(H, W, hc, np.float32, "ref"))
                assert np.array_equal(oracle.index_initializer(H, W, hc, np.float64),
                                      oracle.index_initializer(H, W, hc, np.float64, "ref"))


PFM_IMG = (np.arange(12, dtype="<f4").reshape(3, 4) - 3.5) * 1.25
PFM_OK = b"Pf\n4 3\n-1.0\n" + PFM_IMG[::-1].tobytes()
PFM_BAD = [  # contents, fragment of the reference's message
    (b"P5\n4 3\n-1\n", "invalid format"),
    (b"Pf\n# c\n4 3\n-1.0\n" + PFM_IMG.tobytes(), "unable to parse width"),
    (b"Pf\n4 3\n1.0\n" + PFM_IMG.tobytes(), "mismatched endian"),
    (PFM_OK[:-1], "not enough data"),
    (b"PF\n4 3\n-1.0\n" + PFM_IMG.tobytes() * 3, "no implement"),
    (b"Pf", "no magic"), (b"Pf\n4", "no width"), (b"Pf\n4 3", "no height"), (b"Pf\n4 3 ", "no scaling_factor"),
    (b"Pf\n4 x\n-1.0\n", "unable to parse height"),
]


def test_decode_pfm_oracle_and_library_agree():
    """The library's host parser against the Python restatement of the reference parser: same image, same errors."""
    for contents in (PFM_OK, b"Pf 4\t3\r\n-0.5 " + PFM_IMG[::-1].tobytes() + b"trailing"):
        want = oracle.decode_pfm(contents)
        assert want.shape == (3, 4, 1) and np.array_equal(want[..., 0], PFM_IMG)
        got = ops.decode_pfm(contents)
        assert got.dtype == torch.float32 and np.array_equal(got.numpy(), want)
    for contents, frag in PFM_BAD:
        with pytest.raises(ValueError, match=frag):
            oracle.decode_pfm(contents)
        with pytest.raises(ValueError, match=frag):
            ops.decode_pfm(contents)


# ---- GPU ----------------------------------------------------------------------------------------------
DEV = "cuda:0"


def _t(a, tdtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return x if tdtype is None else x.to(tdtype)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 1, 12, 16, 3, 5), (2, 3, 9, 11, 8, 33), (1, 5, 7, 13, 16, 3), (1, 2, 6, 8, 64, 4),
                                   (1, 2, 8, 9, 12, 7), (1, 2, 8, 9, 128, 2)])
@pytest.mark.parametrize("camera", ["shift", "rot_y", "random"])
def test_feature_aggregate_gpu(shape, camera):
    """Forward bit-exact (unfused arithmetic in the reference's order), gradients within 1e-4."""
    B, N, H, W, C, D = shape
    c = fa_case(90 + C, B, N, H, W, C, D, camera, np.float32, src_hw=(H + 2, W - 1) if camera == "random" else None)
    want, mask = oracle.feature_aggregate_fwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"])
    g = np.random.default_rng(91).standard_normal(want.shape).astype(np.float32)
    sg_w, bg_w = oracle.feature_aggregate_bwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], g, mask)
    a = (_t(c["src"]), _t(c["depth"]), _t(c["offsets"]), _t(c["Rs"]), _t(c["Ts"]))
    got, m = ops.feature_aggregate_forward(*a)
    sg, bg = ops.feature_aggregate_backward(*a, _t(g), m)
    torch.cuda.synchronize()
    assert helpers.bits_equal(m.cpu().numpy(), mask)
    assert helpers.bits_equal(got.cpu().numpy(), want)
    assert helpers.rel_err(sg.cpu().numpy(), sg_w) <= 1e-4
    assert helpers.rel_err(bg.cpu().numpy(), bg_w) <= 1e-4


@pytest.mark.gpu
def test_feature_aggregate_float64_bfloat16_autograd():
    c = fa_case(95, 1, 2, 8, 10, 6, 5, "random", np.float64)
    want, mask = oracle.feature_aggregate_fwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], False, np.float64)
    g = np.random.default_rng(96).standard_normal(want.shape)
    sg_w, bg_w = oracle.feature_aggregate_bwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], g, mask, False, np.float64)
    src = _t(c["src"]).requires_grad_()
    base = _t(c["depth"]).requires_grad_()
    got, m = ops.feature_aggregate(src, base, _t(c["offsets"]), _t(c["Rs"]), _t(c["Ts"]), half_centor=False)
    (got * _t(g)).sum().backward()
    assert helpers.bits_equal(got.detach().cpu().numpy(), want) and helpers.bits_equal(m.cpu().numpy(), mask)
    assert helpers.rel_err(src.grad.cpu().numpy(), sg_w) <= 1e-10
    assert helpers.rel_err(base.grad.cpu().numpy(), bg_w) <= 1e-10
    # bfloat16 features: the float32 arithmetic on the rounded features
    c32 = {k: (None if v is None else v.astype(np.float32)) for k, v in c.items()}
    c32["src"] = torch.from_numpy(np.repeat(c32["src"], 2, axis=-1)[..., :8]).to(torch.bfloat16).float().numpy()
    want, mask = oracle.feature_aggregate_fwd(c32["src"], c32["depth"], c32["offsets"], c32["Rs"], c32["Ts"])
    got, m = ops.feature_aggregate_forward(_t(c32["src"], torch.bfloat16), _t(c32["depth"]), _t(c32["offsets"]),
                                           _t(c32["Rs"]), _t(c32["Ts"]))
    assert got.dtype == torch.float32 and helpers.bits_equal(got.cpu().numpy(), want)
    with pytest.raises(ValueError):
        ops.feature_aggregate_forward(src.detach().cpu(), base.detach().cpu(), c["offsets"], c["Rs"], c["Ts"])


@pytest.mark.gpu
def test_index_initializer_gpu():
    for shape in ((5, 6), (1, 1), (1, 8), (8, 1), (1000, 1000)):
        for hc in (True, False):
            for dt, ndt in ((torch.float32, np.float32), (torch.float64, np.float64)):
                out = ops.index_initializer((shape[0], shape[1], 3), hc, dt)
                assert np.array_equal(out.cpu().numpy(), oracle.index_initializer(shape[0], shape[1], hc, ndt))
    assert torch.equal(ops.IndexInitializer()((3, 4, 3)), ops.index_initializer((3, 4, 3)))
    with pytest.raises(ValueError):
        ops.index_initializer((3, 4, 2))


@pytest.mark.parametrize("w,h", [(2 ** 32, 2 ** 32), (2 ** 62, 4), (3, 2 ** 62), (2 ** 31, 2 ** 31)])
def test_decode_pfm_rejects_a_header_whose_size_product_overflows(w, h):
    """A crafted header whose width * height * 4 wraps around 64 bits must fail the "not enough data" check in the C
    ABI itself (a direct caller has no torch allocation in front of it), with or without an image buffer."""
    import ctypes
    from custom_helper_op_b200 import _lib
    contents = ("Pf\n%d %d\n-1.0\n" % (w, h)).encode() + b"\0" * 64
    hh, ww, cc = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    msg = ctypes.create_string_buffer(256)
    buf = (ctypes.c_float * 16)()
    for image, cap in ((None, 0), (ctypes.cast(buf, ctypes.c_void_p), 16)):
        st = _lib.lib().chop_decode_pfm(contents, len(contents), ctypes.byref(hh), ctypes.byref(ww), ctypes.byref(cc),
                                        image, cap, msg, 256)
        assert st == _lib.ERR_FORMAT and b"not enough data" in msg.value



@pytest.mark.gpu
@pytest.mark.parametrize("case", [(1, 2, 6, 9, 32, 20, np.float32), (1, 3, 5, 7, 64, 5, np.float64), (2, 1, 6, 5, 8, 9, np.float64),
                                   (1, 6, 5, 6, 32, 11, np.float32)])
def test_feature_aggregate_gradient_with_staged_upstream(case):
    """Channel counts where every lane carries a 16-byte slice: the gradient kernel copies the upstream tensor into
    shared memory one (block of planes, view) ahead (cp.async, two buffers).  Ragged last blocks, one to six views,
    float32 and float64 (three views of 64 double channels: the staging area starts at a rounded-up offset)."""
    B, N, H, W, C, D, dt = case
    c = fa_case(120 + C + N, B, N, H, W, C, D, "random", dt, src_hw=(H + 2, W + 1))
    want, mask = oracle.feature_aggregate_fwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], True, dt)
    g = np.random.default_rng(121).standard_normal(want.shape).astype(dt)
    sg_w, bg_w = oracle.feature_aggregate_bwd(c["src"], c["depth"], c["offsets"], c["Rs"], c["Ts"], g, mask, True, dt)
    a = (_t(c["src"]), _t(c["depth"]), _t(c["offsets"]), _t(c["Rs"]), _t(c["Ts"]))
    from custom_helper_op_b200 import _lib
    got, m = ops.feature_aggregate_forward(*a)
    assert helpers.bits_equal(m.cpu().numpy(), mask) and helpers.bits_equal(got.cpu().numpy(), want)
    tol = 1e-4 if dt == np.float32 else 1e-10
    for stage in (1, 0):   # the staged kernel, then the same shapes read plane by plane (knob "fa_stage")
        try:
            _lib.set_tuning("fa_stage", stage)
            sg, bg = ops.feature_aggregate_backward(*a, _t(g), m)
            torch.cuda.synchronize()
        finally:
            _lib.set_tuning("fa_stage", 1)
        assert helpers.rel_err(sg.cpu().numpy(), sg_w) <= tol
        assert helpers.rel_err(bg.cpu().numpy(), bg_w) <= tol
