"""CPU tests of the manifold-convolution oracle: against a dense convolution over the densified band
(the reference tests' own method, sparse_conv_fast_op_test.py:42-85), against torch autograd for the
gradients, and against the reference's older forward kernel compiled as host code."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle


def make_case(seed, B, H, W, D, Cin, Cout, ksize, virtual_depth, dtype=np.float64, margin=4):
    rng = np.random.default_rng(seed)
    full = rng.uniform(0, 1, (B, H, W, virtual_depth, Cin)).astype(dtype)
    filters = rng.uniform(-1, 1, (*ksize, Cin, Cout)).astype(dtype)
    # (the margin keeps the strided output band inside the dense volume the comparison builds)
    base_plane = rng.integers(0, virtual_depth - D + 1 - margin, (B, H, W, 1)).astype(np.int32)
    default_value = dtype(rng.uniform(0, 1))
    idx = base_plane + np.arange(D, dtype=np.int32)[None, None, None, :]
    images = np.take_along_axis(full, idx[..., None], axis=3)
    return images, filters, default_value, base_plane, idx


def dense_reference(images, filters, default_value, base_plane, idx, strides, dilations, virtual_depth, out_grad=None):
    """Scatter the band into a dense volume filled with default_value, pad with default_value, run a
    VALID dense conv3d, gather the output band back.  Returns output (and gradients via autograd)."""
    B, H, W, D, Cin = images.shape
    fh, fw, fd, _, Cout = filters.shape
    t_img = torch.tensor(images, requires_grad=True)
    t_flt = torch.tensor(filters, requires_grad=True)
    t_def = torch.tensor(default_value, requires_grad=True)
    t_idx = torch.tensor(idx.astype(np.int64))
    dense = t_def.expand(B, H, W, virtual_depth, Cin).clone()
    dense = dense.scatter(3, t_idx[..., None].expand(-1, -1, -1, -1, Cin), t_img)
    full_in = np.array([H, W, virtual_depth])
    st, dl, ks = np.array(strides), np.array(dilations), np.array([fh, fw, fd])
    full_out = (full_in + st - 1) // st
    partial = (full_out - 1) * st + 1 - full_in
    pad_l = ks // 2 * dl
    pad_r = np.maximum((ks - 1) * dl - pad_l + partial, 0)
    x = dense.permute(0, 4, 1, 2, 3)  # N C H W D
    # F.pad pads last dim first: (D_l, D_r, W_l, W_r, H_l, H_r); constant must be a python number, so pad by
    # subtracting the default, zero-padding, adding it back
    x = F.pad(x - t_def, (int(pad_l[2]), int(pad_r[2]), int(pad_l[1]), int(pad_r[1]), int(pad_l[0]), int(pad_r[0]))) + t_def
    w = t_flt.permute(4, 3, 0, 1, 2)  # Cout Cin fh fw fd
    y = F.conv3d(x, w, stride=tuple(int(s) for s in strides), dilation=tuple(int(d) for d in dilations))
    y = y.permute(0, 2, 3, 4, 1)  # B oH oW oDfull Cout
    sbp = torch.tensor(base_plane[:, ::strides[0], ::strides[1], :].astype(np.int64))
    sbp = (sbp + strides[2] - 1) // strides[2]
    oD = (D + strides[2] - 1) // strides[2]
    gidx = sbp + torch.arange(oD)[None, None, None, :]
    out = torch.gather(y, 3, gidx[..., None].expand(-1, -1, -1, -1, Cout))
    if out_grad is None:
        return out.detach().numpy()
    (out * torch.tensor(out_grad)).sum().backward()
    return out.detach().numpy(), t_img.grad.numpy(), t_flt.grad.numpy(), t_def.grad.numpy()


CASES = [  # B, H, W, D, Cin, Cout, ksize, strides, dilations, virtual depth
    (1, 6, 5, 4, 3, 2, (3, 3, 3), (1, 1, 1), (1, 1, 1), 9),
    (2, 7, 8, 5, 4, 4, (3, 3, 3), (1, 1, 1), (1, 1, 1), 12),
    (1, 8, 13, 6, 3, 4, (3, 3, 3), (2, 2, 2), (1, 1, 1), 15),
    (2, 6, 6, 5, 2, 1, (5, 3, 3), (2, 2, 2), (2, 2, 2), 12),
    (1, 6, 7, 4, 2, 3, (2, 2, 1), (2, 2, 1), (1, 1, 1), 10),
    (1, 5, 5, 9, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), 20),
]


@pytest.mark.parametrize("case", CASES)
def test_forward_and_gradients_match_dense_convolution(case):
    B, H, W, D, Cin, Cout, ks, st, dl, vd = case
    images, filters, defv, bp, idx = make_case(3, B, H, W, D, Cin, Cout, ks, vd)
    out = oracle.sparse_conv3d_fwd(images, filters, defv, bp, st, dl, np.float64)
    rng = np.random.default_rng(4)
    og = rng.uniform(-1, 1, out.shape)
    want, ig_w, fg_w, dg_w = dense_reference(images, filters, defv, bp, idx, st, dl, vd, og)
    np.testing.assert_allclose(out, want, rtol=1e-10, atol=1e-12)
    ig, fg, dg = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, st, dl, True, np.float64)
    np.testing.assert_allclose(ig, ig_w, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(fg, fg_w, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(dg, dg_w, rtol=1e-10, atol=1e-12)
    # without dynamic_default the default gradient stays zero (sparse_conv3d_fast_op.cc:269)
    _, _, dg0 = oracle.sparse_conv3d_bwd(images, filters, defv, bp, og, st, dl, False, np.float64)
    assert dg0 == 0


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_forward_matches_reference_thread_per_voxel_kernel(case, dtype):
    B, H, W, D, Cin, Cout, ks, st, dl, vd = case
    images, filters, defv, bp, idx = make_case(5, B, H, W, D, Cin, Cout, ks, vd, dtype)
    a = oracle.sparse_conv3d_fwd(images, filters, defv, bp, st, dl, dtype, "port")
    b = oracle.sparse_conv3d_fwd(images, filters, defv, bp, st, dl, dtype, "ref")
    np.testing.assert_allclose(a, b, rtol=1e-5 if dtype == np.float32 else 1e-12, atol=1e-5 if dtype == np.float32 else 1e-12)


# ---- transposed convolution ---------------------------------------------------------------------------
def make_transpose_case(seed, B, H, W, D, Cin, Cout, ksize, strides, max_bp=6, dtype=np.float64, default=None):
    """Fine grid (H,W,D) with base_plane in [0,max_bp); coarse input of the transposed op with Cout channels."""
    rng = np.random.default_rng(seed)
    coarse = tuple((n + s - 1) // s for n, s in zip((H, W, D), strides))
    images = rng.uniform(-1, 1, (B, *coarse, Cout)).astype(dtype)
    filters = rng.uniform(-1, 1, (*ksize, Cin, Cout)).astype(dtype)
    base_plane = rng.integers(0, max_bp, (B, H, W, 1)).astype(np.int32)
    defv = dtype(rng.uniform(0.2, 1)) if default is None else dtype(default)
    return images, filters, defv, base_plane


def dense_transpose_reference(images, filters, defv, base_plane, out_size, strides, dilations, out_grad=None):
    """What the gather-form transposed op computes, densely: put every coarse voxel at its fine position
    (row r*sr, column c*sc, absolute depth (ceil(bp/sd) + d)*sd) in a fine-resolution volume filled with
    default_value, pad with default_value, correlate at stride 1 with the spatially flipped filter (Cout in,
    Cin out) and read the fine band back."""
    B, oH, oW, oD, Cout = images.shape
    H, W, D = out_size
    fh, fw, fd, Cin, _ = filters.shape
    sr, sc, sd = strides
    vd = int(base_plane.max()) + D + sd * 2 + 2
    t_img = torch.tensor(images, requires_grad=True)
    t_flt = torch.tensor(filters, requires_grad=True)
    t_def = torch.tensor(defv)
    bp = torch.tensor(base_plane[..., 0].astype(np.int64))
    # linear index of every coarse voxel inside the dense fine volume [B,H,W,vd]
    cbp = (bp[:, ::sr, ::sc] + sd - 1) // sd                                    # [B,oH,oW]
    depth = (cbp[..., None] + torch.arange(oD)[None, None, None, :]) * sd       # [B,oH,oW,oD]
    rows = (torch.arange(oH) * sr)[None, :, None, None].expand(B, oH, oW, oD)
    cols = (torch.arange(oW) * sc)[None, None, :, None].expand(B, oH, oW, oD)
    bb = torch.arange(B)[:, None, None, None].expand(B, oH, oW, oD)
    lin = ((bb * H + rows) * W + cols) * vd + depth
    assert int(depth.max()) < vd
    dense = t_def.expand(B * H * W * vd, Cout).clone()
    dense = dense.index_put((lin.reshape(-1),), t_img.reshape(-1, Cout))
    dense = dense.reshape(B, H, W, vd, Cout)
    ks, dl = np.array([fh, fw, fd]), np.array(dilations)
    pad_l = (ks - 1) * dl - ks // 2 * dl      # the right padding of the forward problem
    pad_r = ks // 2 * dl
    x = dense.permute(0, 4, 1, 2, 3)
    x = F.pad(x - t_def, (int(pad_l[2]), int(pad_r[2]), int(pad_l[1]), int(pad_r[1]), int(pad_l[0]), int(pad_r[0]))) + t_def
    w = torch.flip(t_flt, (0, 1, 2)).permute(3, 4, 0, 1, 2)                     # [Cin(out), Cout(in), fh, fw, fd]
    y = F.conv3d(x, w, dilation=tuple(int(d) for d in dilations)).permute(0, 2, 3, 4, 1)   # [B,H,W,vd,Cin]
    gidx = bp[..., None] + torch.arange(D)[None, None, None, :]
    out = torch.gather(y, 3, gidx[..., None].expand(-1, -1, -1, -1, Cin))
    if out_grad is None:
        return out.detach().numpy()
    (out * torch.tensor(out_grad)).sum().backward()
    return out.detach().numpy(), t_img.grad.numpy(), t_flt.grad.numpy()


TCASES = [  # B, H, W, D, Cin, Cout, ksize, strides, dilations
    (1, 5, 1, 1, 1, 1, (1, 1, 1), (1, 1, 1), (1, 1, 1)),
    (2, 6, 7, 5, 3, 4, (3, 3, 3), (1, 1, 1), (1, 1, 1)),
    (1, 8, 10, 6, 3, 2, (3, 3, 3), (2, 2, 2), (1, 1, 1)),
    (2, 7, 9, 8, 2, 3, (3, 3, 3), (2, 2, 1), (1, 1, 1)),
    (1, 6, 6, 6, 2, 2, (2, 2, 1), (2, 2, 2), (1, 1, 1)),
    (1, 8, 6, 6, 2, 1, (5, 3, 3), (2, 2, 2), (2, 2, 2)),
    (1, 9, 8, 7, 4, 4, (3, 3, 3), (3, 2, 2), (1, 1, 1)),
]


@pytest.mark.parametrize("case", TCASES)
@pytest.mark.parametrize("default", [0.0, None])
def test_transpose_matches_dense_convolution(case, default):
    B, H, W, D, Cin, Cout, ks, st, dl = case
    images, filters, defv, bp = make_transpose_case(11, B, H, W, D, Cin, Cout, ks, st, default=default)
    out = oracle.sparse_conv3d_transpose_fwd(images, filters, defv, bp, (H, W, D), st, dl, np.float64)
    og = np.random.default_rng(12).uniform(-1, 1, out.shape)
    want, ig_w, fg_w = dense_transpose_reference(images, filters, defv, bp, (H, W, D), st, dl, og)
    np.testing.assert_allclose(out, want, rtol=1e-10, atol=1e-12)
    ig, fg = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, st, dl, False, np.float64)
    np.testing.assert_allclose(ig, ig_w, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(fg, fg_w, rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("case", TCASES)
def test_transpose_is_the_adjoint_of_the_forward_convolution(case):
    """With default_value 0 the transposed op applied to Z is the image gradient of the forward op for the
    upstream gradient Z (both gather over the same taps)."""
    B, H, W, D, Cin, Cout, ks, st, dl = case
    images, filters, _, bp = make_transpose_case(13, B, H, W, D, Cin, Cout, ks, st, default=0.0)
    out = oracle.sparse_conv3d_transpose_fwd(images, filters, 0.0, bp, (H, W, D), st, dl, np.float64)
    x = np.zeros((B, H, W, D, Cin))
    ig, _, _ = oracle.sparse_conv3d_bwd(x, filters, 0.0, bp, images, st, dl, False, np.float64)
    assert np.array_equal(out, ig)


@pytest.mark.parametrize("case", TCASES[1:4])
def test_transpose_gradient_reference_buffers(case):
    """What the reference's grad op writes, against the derivatives: its filter-gradient buffer holds the
    channel axes in the order [Cout, Cin]; its image gradient adds default_value at padded taps and so
    agrees with the derivative when default_value is 0."""
    B, H, W, D, Cin, Cout, ks, st, dl = case
    images, filters, defv, bp = make_transpose_case(14, B, H, W, D, Cin, Cout, ks, st)
    og = np.random.default_rng(15).uniform(-1, 1, (B, H, W, D, Cin))
    ig, fg = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, st, dl, False, np.float64)
    ig_q, fg_q = oracle.sparse_conv3d_transpose_bwd(images, filters, defv, bp, (H, W, D), og, st, dl, True, np.float64)
    assert np.array_equal(fg_q.reshape(*ks, Cout, Cin).transpose(0, 1, 2, 4, 3), fg)
    assert not np.allclose(ig_q, ig)
    ig0, _ = oracle.sparse_conv3d_transpose_bwd(images, filters, 0.0, bp, (H, W, D), og, st, dl, False, np.float64)
    ig0_q, _ = oracle.sparse_conv3d_transpose_bwd(images, filters, 0.0, bp, (H, W, D), og, st, dl, True, np.float64)
    assert np.array_equal(ig0, ig0_q) and np.array_equal(ig0, ig)


# ---- SparsePad ----------------------------------------------------------------------------------------
PAD_CASES = [  # B, coarse h, w, d, C, strides
    (1, 7, 9, 4, 5, (2, 2, 2)),
    (2, 12, 16, 20, 3, (1, 1, 1)),
    (1, 10, 9, 3, 6, (3, 3, 2)),
    (1, 6, 5, 5, 4, (5, 4, 3)),
    (2, 6, 7, 5, 2, (1, 1, 3)),
]


def make_pad_case(seed, B, h, w, d, C, st, dtype):
    rng = np.random.default_rng(seed)
    images = rng.standard_normal((B, h, w, d, C)).astype(dtype)
    base_plane = rng.integers(0, 10, (B, h * st[0], w * st[1], 1)).astype(np.int32)
    out_grad = rng.standard_normal((B, h * st[0], w * st[1], d * st[2], C)).astype(dtype)
    return images, base_plane, out_grad


@pytest.mark.parametrize("case", PAD_CASES)
def test_pad_places_every_coarse_voxel_once(case):
    """The property the reference's test checks (sparse_pad_op_test.py:33-41): a fine voxel holds a coarse
    value iff its row, column and absolute depth are multiples of the strides, else zero; plus adjointness of
    the gradient."""
    B, h, w, d, C, st = case
    images, bp, og = make_pad_case(21, B, h, w, d, C, st, np.float64)
    out = oracle.sparse_pad_fwd(images, bp, st, np.float64)
    H, W, D = h * st[0], w * st[1], d * st[2]
    rr, cc, dd = np.meshgrid(np.arange(H), np.arange(W), np.arange(D), indexing="ij")
    aligned = ((rr % st[0]) == 0) & ((cc % st[1]) == 0) & (((dd[None] + bp) % st[2]) == 0)
    assert np.all(out[~aligned] == 0)
    assert aligned.sum() == B * h * w * d
    assert np.array_equal(np.sort(out[aligned].ravel()), np.sort(images.ravel()))
    ig = oracle.sparse_pad_bwd(images, bp, og, st, False, np.float64)
    np.testing.assert_allclose((out * og).sum(), (images * ig).sum(), rtol=1e-12)


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("case", PAD_CASES)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_pad_matches_reference_kernels(case, dtype):
    B, h, w, d, C, st = case
    images, bp, og = make_pad_case(22, B, h, w, d, C, st, dtype)
    assert np.array_equal(oracle.sparse_pad_fwd(images, bp, st, dtype, "port"),
                          oracle.sparse_pad_fwd(images, bp, st, dtype, "ref"))
    ref_g = oracle.sparse_pad_bwd(images, bp, og, st, dtype=dtype, impl="ref")
    assert np.array_equal(oracle.sparse_pad_bwd(images, bp, og, st, True, dtype, "port"), ref_g)
    if st[0] == 1 and st[1] == 1:
        assert np.array_equal(oracle.sparse_pad_bwd(images, bp, og, st, False, dtype, "port"), ref_g)


def test_pad_matches_golden():
    from tests import helpers
    names = helpers.pad_golden_names()
    assert names
    for name in names:
        z = np.load(f"{helpers.GOLDEN_DIR}/{name}.npz")
        st = tuple(int(s) for s in z["in_strides"])
        assert np.array_equal(oracle.sparse_pad_fwd(z["in_images"], z["in_base_plane"], st), z["out_output"])
        if "out_images_grad" in z.files:
            assert np.array_equal(oracle.sparse_pad_bwd(z["in_images"], z["in_base_plane"], z["in_out_grad"], st),
                                  z["out_images_grad"])
