"""The entry points only enqueue work on the caller's stream: they do not synchronise, allocate or copy from the
host, so a forward + gradient step can be captured in a CUDA graph and replayed on new input values.  (What a
framework that replays captured steps relies on; also the way to run a launch-latency-sized problem.)"""
import numpy as np
import pytest
import torch

from custom_helper_op_b200 import synth
from custom_helper_op_b200.python.ops import custom_helper_ops as ops
from tests import helpers
from tests.test_oracle_sparse import make_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _capture(step):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):      # first calls outside the capture: per-kernel shared-memory grants and the like
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    return graph


@pytest.mark.parametrize("kind,reduce", [(1, "MEAN"), (1, "MIN"), (3, "MIN"), (2, "MEAN")])
def test_cost_volume_step_replays_from_a_graph(kind, reduce):
    w = synth.make("c0_cpu", with_grad=False)
    t = {k: torch.from_numpy(v).to(DEV) for k, v in w.items()}
    if kind == 2:   # CostVolumeV2: a depth hypothesis per voxel
        depth = (t["base_plane"] + t["offsets"][:, None, None, :]).contiguous()
        a = (t["ref"], t["src"], depth, None, t["Rs"], t["Ts"])
        extra = (reduce, 4)
    else:
        a = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
        extra = (reduce,)
    cost, mask = ops.cost_forward(kind, *a, *extra)
    cg = torch.randn_like(cost)
    grads = ops.cost_backward(kind, *a, cg, mask, *extra)

    def step():
        ops.cost_forward(kind, *a, *extra, out=(cost, mask))
        ops.cost_backward(kind, *a, cg, mask, *extra, zero_into=grads)

    graph = _capture(step)
    t["ref"].copy_(torch.randn_like(t["ref"]))       # new values in the same buffers
    cg.copy_(torch.randn_like(cg))
    graph.replay()
    torch.cuda.synchronize()
    got = [cost.clone(), mask.clone()] + [x.clone() for x in grads]
    step()
    torch.cuda.synchronize()
    assert torch.equal(got[0], cost) and torch.equal(got[1], mask)
    for x, y in zip(got[2:], grads):                 # float atomics: order differs between runs
        assert helpers.rel_err(x.cpu().numpy(), y.cpu().numpy()) <= 1e-5


def test_manifold_convolution_step_replays_from_a_graph():
    images, filters, defv, bp, _ = make_case(41, 1, 12, 14, 9, 16, 16, (3, 3, 3), 24, np.float32)
    img = torch.from_numpy(images).to(DEV).to(torch.bfloat16)
    flt = torch.from_numpy(filters * 0.3).to(DEV).to(torch.bfloat16)
    dv = torch.tensor(float(defv), device=DEV, dtype=torch.bfloat16)
    bpt = torch.from_numpy(bp).to(DEV)
    og = torch.randn((1, 12, 14, 9, 16), device=DEV).to(torch.bfloat16)
    res = {}

    def step():
        res["out"] = ops.sparse_conv3d_forward(img, flt, dv, bpt)
        res["grads"] = ops.sparse_conv3d_backward(img, flt, dv, bpt, og, dynamic_default=True)

    graph = _capture(step)
    img.copy_(torch.randn_like(img.float()).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    got = [res["out"].clone()] + [x.clone() for x in res["grads"]]
    want_out = ops.sparse_conv3d_forward(img, flt, dv, bpt)
    want_grads = ops.sparse_conv3d_backward(img, flt, dv, bpt, og, dynamic_default=True)
    torch.cuda.synchronize()
    assert torch.equal(got[0], want_out)
    for x, y in zip(got[1:], want_grads):
        assert helpers.rel_err(x.float().cpu().numpy(), y.float().cpu().numpy()) <= 1e-6
