"""Full-size runs of the benchmark configurations on the GPU, checked through properties that do not
need a full CPU oracle run: the oracle on a band of image rows (cost, mask, d(ref), d(base_plane) are
per pixel), bit-identical repeat runs of the forward pass, depth-range calls composing to the full
call, linearity of the gradient in the upstream gradient, and the channel-wise checksum
sum(d src) == -sum(d ref) that follows from the bilinear weights adding up to one."""
import numpy as np
import pytest
import torch

import oracle
from custom_helper_op_b200 import _lib, synth
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _band_check(w, cost, mask, rg, bg, cg, rows, item=0, args=None):
    """Oracle on image rows [0, rows) of one batch item against the full GPU result: cost, mask, d(ref) and
    d(base_plane) are per pixel.  Element-wise as well as scale-relative: |got - want| <= rtol*|want| + atol with
    atol = 1e-6 * max|want| (1e-5 * max for gradients, which are sums in atomic order), rtol 1e-5 forward and
    1e-4 gradients.  With `args` (the op's device inputs) the source-feature gradient is checked too: the oracle's
    gradient over the band is the partial d(src) of those pixels, and the GPU gradient with the upstream gradient
    zeroed everywhere else must reproduce the whole of it."""
    b = slice(item, item + 1)
    ref = np.ascontiguousarray(w["ref"][b, :rows])
    base = np.ascontiguousarray(w["base_plane"][b, :rows])
    c_o, m_o = oracle.cost_fwd(1, ref, w["src"][b], base, w["offsets"][b], w["Rs"][b], w["Ts"][b])
    assert helpers.bits_equal(mask[b, :rows].cpu().numpy(), m_o)
    c_g = cost[b, :rows].cpu().numpy()
    assert helpers.rel_err(c_g, c_o) <= 1e-5
    assert helpers.elementwise_excess(c_g, c_o, 1e-5) <= 1.0
    cg_band = cg[b, :rows].cpu().numpy()
    rg_o, sg_o, bg_o = oracle.cost_bwd(1, ref, w["src"][b], base, w["offsets"][b], w["Rs"][b], w["Ts"][b], cg_band, m_o)
    for got, want in ((rg[b, :rows], rg_o), (bg[b, :rows], bg_o)):
        got = got.cpu().numpy()
        assert helpers.rel_err(got, want) <= 1e-4
        assert helpers.elementwise_excess(got, want, 1e-4, 1e-5) <= 1.0
    if args is not None:
        cg_only = torch.zeros_like(cg)
        cg_only[b, :rows] = cg[b, :rows]
        rg2, sg2, bg2 = ops.cost_backward(1, *args, cg_only, mask)
        del cg_only
        sg_g = sg2[b].cpu().numpy()
        assert helpers.rel_err(sg_g, sg_o) <= 1e-4
        assert helpers.elementwise_excess(sg_g, sg_o, 1e-4, 1e-5) <= 1.0
        # nothing leaks to the other items' source gradients or to reference pixels outside the band
        for o in range(sg2.shape[0]):
            if o != item:
                assert float(sg2[o].abs().max()) == 0.0
        assert float(rg2[b, rows:].abs().max()) == 0.0
        assert helpers.rel_err(rg2[b, :rows].cpu().numpy(), rg_o) <= 1e-4


@pytest.mark.parametrize("name", ["c0_cpu", "c1_mvsnet"])
def test_cost_volume_full_size(name):
    w = synth.make(name, with_grad=False)
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    args = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
    cost, mask = ops.cost_forward(1, *args)
    cost2, mask2 = ops.cost_forward(1, *args)
    assert torch.equal(cost, cost2) and torch.equal(mask, mask2)            # the forward pass is deterministic
    assert float((mask > 0).float().mean()) > 0.9                           # the synthetic cameras see the volume
    # strict mode agrees with the fused mode to rounding
    cost_s, mask_s = ops.cost_forward(1, *args, strict=True)
    assert torch.equal(mask, mask_s)
    assert float((cost - cost_s).abs().max() / cost_s.abs().max()) <= 1e-5
    g = torch.Generator(device=DEV)
    g.manual_seed(5)
    g1 = torch.randn(cost.shape, device=DEV, generator=g)
    g2 = torch.randn(cost.shape, device=DEV, generator=g)
    r1 = ops.cost_backward(1, *args, g1, mask)
    r2 = ops.cost_backward(1, *args, g2, mask)
    r12 = ops.cost_backward(1, *args, 0.5 * g1 + g2, mask)
    for a, b, c in zip(r1, r2, r12):                                         # linear in the upstream gradient
        scale = float(c.abs().max())
        assert float((0.5 * a + b - c).abs().max()) <= 1e-4 * scale
    rg, sg, bg = r1
    # checksum: every sample spreads its gradient over four corners with weights that sum to one
    lhs = sg.double().sum(dim=(0, 1, 2, 3))
    rhs = -rg.double().sum(dim=(0, 1, 2))
    assert float((lhs - rhs).abs().max()) <= 1e-4 * float(rhs.abs().max())
    # depth-range calls compose
    D = t["offsets"].shape[1]
    cost_r = torch.zeros_like(cost)
    mask_r = torch.zeros_like(mask)
    acc = None
    for d0, d1 in ((0, D // 3), (D // 3, D // 3 + 5), (D // 3 + 5, D)):
        ops.cost_forward(1, *args, d_range=(d0, d1), out=(cost_r, mask_r))
        if acc is None:
            acc = ops.cost_backward(1, *args, g1, mask, d_range=(d0, d1))
        else:
            ops.cost_backward(1, *args, g1, mask, d_range=(d0, d1), accumulate_into=acc)
    assert torch.equal(cost_r, cost) and torch.equal(mask_r, mask)
    for a, b in zip(acc, r1):
        assert float((a - b).abs().max()) <= 1e-4 * float(b.abs().max())
    _band_check(w, cost, mask, rg, bg, g1, rows=3, args=args)


@pytest.mark.parametrize("kind", [1, 3])
def test_min_reduction_full_size(kind):
    """MIN (the reference layers' default) at the c1 size, CostVolume (1) and CostAggregate (3): the compile-time-C
    kernels against the generic kernels (two implementations of the same unfused arithmetic: cost and arg indices
    bit-identical, gradients to rounding), the oracle on a band of rows, and depth-range calls composing."""
    w = synth.make("c1_mvsnet", with_grad=False)
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    args = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
    cost, mask = ops.cost_forward(kind, *args, "MIN")
    g = torch.Generator(device=DEV)
    g.manual_seed(7)
    cg = torch.randn(cost.shape, device=DEV, generator=g)
    grads = ops.cost_backward(kind, *args, cg, mask, "MIN")
    try:
        _lib.set_tuning("tuned", 0)
        cost_g, mask_g = ops.cost_forward(kind, *args, "MIN")
        grads_g = ops.cost_backward(kind, *args, cg, mask, "MIN")
    finally:
        _lib.set_tuning("tuned", 1)
    assert torch.equal(mask, mask_g) and torch.equal(cost, cost_g)
    assert float((mask >= 0).float().mean()) > 0.9
    for a, b in zip(grads, grads_g):
        assert float((a - b).abs().max()) <= 1e-4 * float(b.abs().max())
    # oracle on the first rows of the image (cost, arg indices, d(ref), d(base_plane) are per pixel)
    rows = 2
    ref = np.ascontiguousarray(w["ref"][:1, :rows])
    base = np.ascontiguousarray(w["base_plane"][:1, :rows])
    c_o, m_o = oracle.cost_fwd(kind, ref, w["src"][:1], base, w["offsets"][:1], w["Rs"][:1], w["Ts"][:1], reduce_method="MIN")
    assert helpers.bits_equal(mask[:1, :rows].cpu().numpy(), m_o)
    assert helpers.bits_equal(cost[:1, :rows].cpu().numpy(), c_o)
    rg_o, _, bg_o = oracle.cost_bwd(kind, ref, w["src"][:1], base, w["offsets"][:1], w["Rs"][:1], w["Ts"][:1],
                                    cg[:1, :rows].cpu().numpy(), m_o, reduce_method="MIN")
    assert helpers.rel_err(grads[0][:1, :rows].cpu().numpy(), rg_o) <= 1e-4
    assert helpers.rel_err(grads[2][:1, :rows].cpu().numpy(), bg_o) <= 1e-4
    # depth-range calls compose
    D = t["offsets"].shape[1]
    cost_r = torch.zeros_like(cost)
    mask_r = torch.zeros_like(mask)
    acc = None
    for d0, d1 in ((0, 7), (7, D // 2 + 3), (D // 2 + 3, D)):
        ops.cost_forward(kind, *args, "MIN", d_range=(d0, d1), out=(cost_r, mask_r))
        if acc is None:
            acc = ops.cost_backward(kind, *args, cg, mask, "MIN", d_range=(d0, d1))
        else:
            ops.cost_backward(kind, *args, cg, mask, "MIN", d_range=(d0, d1), accumulate_into=acc)
    assert torch.equal(cost_r, cost) and torch.equal(mask_r, mask)
    for a, b in zip(acc, grads):
        assert float((a - b).abs().max()) <= 1e-4 * float(b.abs().max())


def test_large_item_bf16_features():
    """One batch item of the large multi-view configuration (V=7, 296x400, D=256, inverse-depth planes),
    bf16 features: band check against the float32 oracle on the bf16-rounded features."""
    w = synth.make("c3_large", with_grad=False, B=1)
    for k in ("ref", "src"):
        w[k] = torch.from_numpy(w[k]).to(torch.bfloat16).float().numpy()
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    args = (t["ref"].to(torch.bfloat16), t["src"].to(torch.bfloat16), t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
    cost, mask = ops.cost_forward(1, *args)
    g = torch.Generator(device=DEV)
    g.manual_seed(6)
    cg = torch.randn(cost.shape, device=DEV, generator=g)
    rg, sg, bg = ops.cost_backward(1, *args, cg, mask)
    lhs = sg.double().sum(dim=(0, 1, 2, 3))
    rhs = -rg.double().sum(dim=(0, 1, 2))
    assert float((lhs - rhs).abs().max()) <= 1e-4 * float(rhs.abs().max())
    _band_check(w, cost, mask, rg, bg, cg, rows=2, args=args)


def test_more_than_2_31_cost_elements():
    """Three items of the large configuration in ONE call (bf16 features): cost and cost_grad hold 2.91 G elements
    each, so the voxel offsets of the last item exceed 32 bits - where the reference switches to 64-bit indices
    (cost_volume_kernels_gpu.cu.cc:313,619).  Band check on the LAST item, forward and all three gradients."""
    B = 3
    w = synth.make("c3_large", with_grad=False, B=B)
    for k in ("ref", "src"):
        w[k] = torch.from_numpy(w[k]).to(torch.bfloat16).float().numpy()
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    args = (t["ref"].to(torch.bfloat16), t["src"].to(torch.bfloat16), t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
    cost, mask = ops.cost_forward(1, *args)
    assert cost.numel() > 2 ** 31
    rows = 2
    g = torch.Generator(device=DEV)
    g.manual_seed(8)
    cg = torch.zeros_like(cost)
    cg[B - 1, :rows] = torch.randn(cg[B - 1, :rows].shape, device=DEV, generator=g)
    rg, sg, bg = ops.cost_backward(1, *args, cg, mask)
    b = slice(B - 1, B)
    ref = np.ascontiguousarray(w["ref"][b, :rows])
    base = np.ascontiguousarray(w["base_plane"][b, :rows])
    c_o, m_o = oracle.cost_fwd(1, ref, w["src"][b], base, w["offsets"][b], w["Rs"][b], w["Ts"][b])
    assert helpers.bits_equal(mask[b, :rows].cpu().numpy(), m_o)
    c_g = cost[b, :rows].cpu().numpy()
    assert helpers.rel_err(c_g, c_o) <= 1e-5 and helpers.elementwise_excess(c_g, c_o, 1e-5) <= 1.0
    rg_o, sg_o, bg_o = oracle.cost_bwd(1, ref, w["src"][b], base, w["offsets"][b], w["Rs"][b], w["Ts"][b],
                                       cg[b, :rows].cpu().numpy(), m_o)
    for got, want in ((rg[b, :rows], rg_o), (sg[b], sg_o), (bg[b, :rows], bg_o)):
        got = got.cpu().numpy()
        assert helpers.rel_err(got, want) <= 1e-4
        assert helpers.elementwise_excess(got, want, 1e-4, 1e-5) <= 1.0
    assert float(sg[:B - 1].abs().max()) == 0.0 and float(rg[:B - 1].abs().max()) == 0.0
    # the first item of the same call against its own band (offsets below 2^31): same code path, small indices
    c_o0, m_o0 = oracle.cost_fwd(1, np.ascontiguousarray(w["ref"][:1, :rows]), w["src"][:1],
                                 np.ascontiguousarray(w["base_plane"][:1, :rows]), w["offsets"][:1], w["Rs"][:1], w["Ts"][:1])
    assert helpers.bits_equal(mask[:1, :rows].cpu().numpy(), m_o0)
    assert helpers.rel_err(cost[:1, :rows].cpu().numpy(), c_o0) <= 1e-5


@pytest.mark.parametrize("name", ["c2_stage1", "c2_stage2", "c2_stage3"])
def test_cascade_stage_v2(name):
    """CostVolumeV2 stages at full size (V=5, 8 groups, bf16 features): band check of cost, mask, d(ref) and the
    per-voxel depth-hypothesis gradient against the oracle; d(src) through the band-only upstream gradient."""
    w = synth.make(name, with_grad=False)
    G = w.pop("groups")
    for k in ("ref", "src"):
        w[k] = torch.from_numpy(w[k]).to(torch.bfloat16).float().numpy()
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    args = (t["ref"].to(torch.bfloat16), t["src"].to(torch.bfloat16), t["depth_grid"], None, t["Rs"], t["Ts"])
    cost, mask = ops.cost_forward(2, *args, groups=G)
    g = torch.Generator(device=DEV)
    g.manual_seed(7)
    cg = torch.randn(cost.shape, device=DEV, generator=g)
    rg, sg, dg = ops.cost_backward(2, *args, cg, mask, groups=G)
    rows = 2
    ref = np.ascontiguousarray(w["ref"][:1, :rows])
    grid = np.ascontiguousarray(w["depth_grid"][:1, :rows])
    c_o, m_o = oracle.cost_fwd(2, ref, w["src"][:1], grid, None, w["Rs"][:1], w["Ts"][:1], groups=G)
    assert helpers.bits_equal(mask[:1, :rows].cpu().numpy(), m_o)
    assert helpers.rel_err(cost[:1, :rows].cpu().numpy(), c_o) <= 1e-5
    rg_o, sg_o, dg_o = oracle.cost_bwd(2, ref, w["src"][:1], grid, None, w["Rs"][:1], w["Ts"][:1], cg[:1, :rows].cpu().numpy(), m_o,
                                       groups=G)
    assert helpers.rel_err(rg[:1, :rows].cpu().numpy(), rg_o) <= 1e-4
    assert helpers.rel_err(dg[:1, :rows].cpu().numpy(), dg_o) <= 1e-4
    assert helpers.elementwise_excess(cost[:1, :rows].cpu().numpy(), c_o, 1e-5) <= 1.0
    cg_only = torch.zeros_like(cg)
    cg_only[:1, :rows] = cg[:1, :rows]
    _, sg2, _ = ops.cost_backward(2, *args, cg_only, mask, groups=G)
    assert helpers.rel_err(sg2[:1].cpu().numpy(), sg_o) <= 1e-4
    assert helpers.elementwise_excess(sg2[:1].cpu().numpy(), sg_o, 1e-4, 1e-5) <= 1.0


def test_manifold_conv_full_size():
    """c4 (256x320 pixels, 9-plane band, 16 -> 16, bf16): tensor-core kernels against the generic kernels on the
    whole problem, and the forward pass against the oracle."""
    w = synth.manifold_conv(20246)
    r = lambda a: torch.from_numpy(a).to(torch.bfloat16)
    img, flt, og = r(w["images"]).to(DEV), r(w["filters"]).to(DEV), r(w["out_grad"]).to(DEV)
    bp = torch.from_numpy(w["base_plane"]).to(DEV)
    res = {}
    for umma in (1, 0):
        try:
            _lib.set_tuning("umma", umma)
            out = ops.sparse_conv3d_forward(img, flt, 0.0, bp)
            res[umma] = (out,) + ops.sparse_conv3d_backward(img, flt, 0.0, bp, og)
        finally:
            _lib.set_tuning("umma", 1)
    torch.cuda.synchronize()
    assert _lib.lib().chop_umma_timeouts() == 0
    for a, b in zip(res[1][:3], res[0][:3]):
        a, b = a.float(), b.float()
        assert float((a - b).abs().max()) <= 2.0 ** -7 * float(b.abs().max())
    want = oracle.sparse_conv3d_fwd(r(w["images"]).float().numpy(), r(w["filters"]).float().numpy(), 0.0, w["base_plane"])
    assert helpers.rel_err(res[1][0].float().cpu().numpy(), want) <= 1e-2


def test_feature_aggregate_and_v3_full_size():
    """c1 shapes.  FeatureAggregate: the mean over the seen views of (mapped - ref)^2 is the CostVolume cost and the mask
    sums to its view count; a band of rows against the oracle bit for bit; the gradient checksum sum(d src) = sum over
    seen samples of the upstream gradient.  CostVolumeV3: deterministic, MIN cost >= MEAN cost where every view sees the
    voxel, a band of rows against the oracle bit for bit (cost, mask and winner indices)."""
    w = synth.make("c1_mvsnet", with_grad=False)
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    args = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
    fa_args = args[1:]
    mapped, fmask = ops.feature_aggregate_forward(*fa_args)
    cost, used = ops.cost_forward(1, *args)
    assert torch.equal(fmask.sum(dim=4), used)
    sq = ((mapped - t["ref"][:, :, :, None, None, :]) ** 2 * fmask).sum(dim=4)
    want = torch.where(used > 0, sq / used.clamp(min=1), torch.zeros_like(sq))
    assert float((want - cost).abs().max() / cost.abs().max()) <= 1e-5
    rows = 3
    m_o, k_o = oracle.feature_aggregate_fwd(w["src"], np.ascontiguousarray(w["base_plane"][:, :rows]), w["offsets"], w["Rs"], w["Ts"])
    assert helpers.bits_equal(mapped[:, :rows].cpu().numpy(), m_o) and helpers.bits_equal(fmask[:, :rows].cpu().numpy(), k_o)
    g = torch.Generator(device=DEV)
    g.manual_seed(6)
    mg = torch.randn(mapped.shape, device=DEV, generator=g)
    sg, bg = ops.feature_aggregate_backward(*fa_args, mg, fmask)
    lhs = sg.double().sum(dim=(0, 2, 3))                                # [N, C]
    rhs = (mg.double() * fmask).sum(dim=(0, 1, 2, 3))                   # [N, C]
    assert float((lhs - rhs).abs().max()) <= 1e-4 * float(rhs.abs().max())
    del mapped, mg, sq, want
    torch.cuda.empty_cache()

    G = 8
    c_mean, m_mean = ops.cost_forward(4, *args, "MEAN", G)
    c_mean2, m_mean2 = ops.cost_forward(4, *args, "MEAN", G)
    assert torch.equal(c_mean, c_mean2) and torch.equal(m_mean, m_mean2)
    assert torch.equal(m_mean, used)                                     # the same validity count as CostVolume
    c_min, m_min = ops.cost_forward(4, *args, "MIN", G)
    full = (used == t["src"].shape[1]).squeeze(-1)
    assert bool((c_min.squeeze(-1)[full] >= c_mean.squeeze(-1)[full]).all())
    ref_b = np.ascontiguousarray(w["ref"][:, :rows])
    base_b = np.ascontiguousarray(w["base_plane"][:, :rows])
    for red, c_gpu, m_gpu in (("MEAN", c_mean, m_mean), ("MIN", c_min, m_min)):
        c_o, m_o = oracle.cost_fwd(4, ref_b, w["src"], base_b, w["offsets"], w["Rs"], w["Ts"], red, G)
        assert helpers.bits_equal(m_gpu[:, :rows].cpu().numpy(), m_o)
        assert helpers.bits_equal(c_gpu[:, :rows].cpu().numpy(), c_o)
    cg = torch.randn(c_mean.shape, device=DEV, generator=g)
    rg, sg3, bg3 = ops.cost_backward(4, *args, cg, m_mean, "MEAN", G)
    rg_o, _, bg_o = oracle.cost_bwd(4, ref_b, w["src"], base_b, w["offsets"], w["Rs"], w["Ts"], cg[:, :rows].cpu().numpy(),
                                    m_mean[:, :rows].cpu().numpy(), "MEAN", G)
    assert helpers.rel_err(rg[:, :rows].cpu().numpy(), rg_o) <= 1e-4
    assert helpers.rel_err(bg3[:, :rows].cpu().numpy(), bg_o) <= 1e-4


def test_up_down_convolution_full_size():
    """c4 band, bf16, strides (2,2,2) on the tensor cores.  The transposed convolution is the adjoint of the strided one
    (default_value 0): <conv(x), z> = <x, convT(z)>; both gradients of a pair agree with that; SparsePad followed by its
    gradient is the identity; tensor-core and generic kernels agree."""
    w = synth.manifold_conv(20247)
    bf = torch.bfloat16
    x = torch.from_numpy(w["images"]).to(DEV).to(bf)
    flt = torch.from_numpy(w["filters"]).to(DEV).to(bf)
    bp = torch.from_numpy(w["base_plane"]).to(DEV)
    B, H, W, D, C = x.shape
    st = (2, 2, 2)
    y = ops.sparse_conv3d_forward(x, flt, 0.0, bp, st)
    g = torch.Generator(device=DEV)
    g.manual_seed(7)
    z = (torch.randn(y.shape, device=DEV, generator=g) * 0.1).to(bf)
    xt = ops.sparse_conv3d_transpose_forward(z, flt, 0.0, bp, (H, W, D), st)
    assert _lib.lib().chop_umma_timeouts() == 0
    lhs = float((y.double() * z.double()).sum())
    rhs = float((x.double() * xt.double()).sum())
    scale = float((y.double().abs() * z.double().abs()).sum())
    assert abs(lhs - rhs) <= 2e-3 * scale                                 # bf16-rounded outputs on both sides
    # the image gradient of the strided convolution IS the transposed convolution of the upstream gradient
    ig, fg, _ = ops.sparse_conv3d_backward(x, flt, 0.0, bp, z, st)
    assert torch.equal(ig, xt)
    # and the two filter gradients of the pair agree: d<conv(x), z>/dW = d<x, convT(z)>/dW
    _, fg_t = ops.sparse_conv3d_transpose_backward(z, flt, 0.0, bp, (H, W, D), x, st)
    assert float((fg - fg_t).abs().max()) <= 2e-3 * float(fg.abs().max())
    try:
        _lib.set_tuning("umma", 0)
        xt_g = ops.sparse_conv3d_transpose_forward(z, flt, 0.0, bp, (H, W, D), st)
        _, fg_g = ops.sparse_conv3d_transpose_backward(z, flt, 0.0, bp, (H, W, D), x, st)
    finally:
        _lib.set_tuning("umma", 1)
    assert float((xt.float() - xt_g.float()).abs().max()) <= 2.0 ** -7 * float(xt_g.float().abs().max())
    assert float((fg_t - fg_g).abs().max()) <= 2e-3 * float(fg_g.abs().max())
    pbp = bp[:, :y.shape[1] * 2, :y.shape[2] * 2].contiguous()
    padded = ops.sparse_pad_forward(y, pbp, st)
    assert torch.equal(ops.sparse_pad_backward(y, pbp, padded, st), y)
    assert int((padded != 0).sum()) == int((y != 0).sum())
