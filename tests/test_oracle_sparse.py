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
