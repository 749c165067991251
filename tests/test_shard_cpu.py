"""Host-side logic of multi-GPU sharding, on CPU: the partition, and a world_size-2 gloo run in which
two ranks split one item's depth range, compute their slices (with the CPU oracle standing in for the
CUDA ops) and all-reduce the packed partial gradients - the result must equal the unsharded one."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from custom_helper_op_b200 import shard


def test_partition_covers_everything_exactly_once():
    for batch, depth, world in [(8, 256, 8), (8, 256, 2), (8, 256, 4), (1, 192, 8), (2, 48, 8), (3, 10, 8), (1, 3, 8), (5, 7, 3)]:
        plan = shard.partition(batch, depth, world)
        assert len(plan) == world
        cover = np.zeros((batch, depth), int)
        for r, shards in enumerate(plan):
            for s in shards:
                assert r in s.group_ranks
                cover[s.item, s.d_begin:s.d_end] += 1
        assert (cover == 1).all(), (batch, depth, world)
        if world <= batch:
            assert all(len(s.group_ranks) == 1 for shards in plan for s in shards)   # pure batch sharding: no exchange
            sizes = [len(shards) for shards in plan]
            assert max(sizes) - min(sizes) <= 1
        else:
            for shards in plan:
                assert len(shards) == 1
            for b in range(batch):
                widths = [s.d_end - s.d_begin for shards in plan for s in shards if s.item == b]
                assert max(widths) - min(w for w in widths if w > 0 or depth < len(widths)) <= 1


def test_pack_layout():
    offs, total = shard.pack_layout([(1, 4, 5, 3), (1, 2, 4, 5, 3), (1, 4, 5, 1)])
    assert offs == [(0, 60), (60, 120), (180, 20)] and total == 200


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, batch, tmp):
    import oracle
    from tests import helpers
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D = 10
        items, full = {}, {}
        for b in range(batch):
            c = helpers.make_case(1, 50 + b, 1, 2, 8, 10, 4, D, "random", np.float32)
            items[b] = {k: (None if v is None else torch.from_numpy(v)) for k, v in
                        dict(ref=c["ref"], src=c["src"], base_plane=c["depth"], offsets=c["offsets"], Rs=c["Rs"], Ts=c["Ts"]).items()}
            full[b] = helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32, seed=70 + b)
        plan = shard.partition(batch, D, world)
        groups = shard.make_groups(plan)

        def fwd(inp, d0, d1):
            # the CPU stand-in computes a depth slice by slicing the offsets (depth = base_plane + offsets[d])
            cost, mask = oracle.cost_fwd(1, inp["ref"].numpy(), inp["src"].numpy(), inp["base_plane"].numpy(),
                                         inp["offsets"].numpy()[:, d0:d1], inp["Rs"].numpy(), inp["Ts"].numpy())
            fc = torch.zeros((1, 8, 10, D, 4))
            fm = torch.zeros((1, 8, 10, D, 1), dtype=torch.int32)
            fc[:, :, :, d0:d1] = torch.from_numpy(cost)
            fm[:, :, :, d0:d1] = torch.from_numpy(mask)
            return fc, fm

        def bwd(inp, cost_grad, mask, d0, d1, views):
            g = oracle.cost_bwd(1, inp["ref"].numpy(), inp["src"].numpy(), inp["base_plane"].numpy(),
                                inp["offsets"].numpy()[:, d0:d1], inp["Rs"].numpy(), inp["Ts"].numpy(),
                                cost_grad.numpy()[:, :, :, d0:d1], mask.numpy()[:, :, :, d0:d1])
            for v, x in zip(views, g):
                v.copy_(torch.from_numpy(x))       # the op writes its outputs (the CUDA op zero-fills them first)

        res = shard.sharded_forward_backward(rank, plan, groups, items, lambda b, cost: torch.from_numpy(full[b]["cost_grad"]),
                                             fwd, bwd, "cpu")
        ok = True
        for b, (cost, mask, rg, sg, bg) in res.items():
            sh = [s for s in plan[rank] if s.item == b][0]
            if sh.d_end > sh.d_begin:
                ok &= np.array_equal(cost.numpy()[:, :, :, sh.d_begin:sh.d_end], full[b]["cost"][:, :, :, sh.d_begin:sh.d_end])
                ok &= np.array_equal(mask.numpy()[:, :, :, sh.d_begin:sh.d_end], full[b]["mask"][:, :, :, sh.d_begin:sh.d_end])
            for got, key in ((rg, "ref_grad"), (sg, "src_grad"), (bg, "depth_grad")):
                ok &= helpers.rel_err(got.numpy(), full[b][key]) < 1e-5
        open(os.path.join(tmp, "rank%d.ok" % rank), "w").write("1" if ok else "0")
    finally:
        dist.destroy_process_group()


def _pipeline_worker(rank, world, port, tmp):
    """Three consecutive steps of one depth-split item through PipelinedReducer: every step's reduced gradients
    equal the unsharded ones although step k's all-reduce is only joined after step k+1 has been issued."""
    import oracle
    from tests import helpers
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D = 10
        c = helpers.make_case(1, 61, 1, 2, 8, 10, 4, D, "random", np.float32)
        steps = [helpers.oracle_fwd_bwd(1, c, "MEAN", 1, True, np.float32, seed=80 + k) for k in range(3)]
        mine = shard.partition(1, D, world)[rank][0]
        d0, d1 = mine.d_begin, mine.d_end
        pipe = shard.PipelinedReducer([c["ref"].shape, c["src"].shape, c["depth"].shape], torch.float32, "cpu", dist.group.WORLD)
        slots = []
        for k in range(3):
            views = pipe.next_views()
            g = oracle.cost_bwd(1, c["ref"], c["src"], c["depth"], c["offsets"][:, d0:d1], c["Rs"], c["Ts"],
                                steps[k]["cost_grad"][:, :, :, d0:d1], steps[k]["mask"][:, :, :, d0:d1])
            for v, x in zip(views, g):
                v.copy_(torch.from_numpy(x))
            slots.append(pipe.reduce_async())
            if k >= 1:   # read step k-1 only now: its collective overlapped this step's work
                got = [t.clone() for t in pipe.result(slots[k - 1])]
                slots[k - 1] = got
        slots[2] = [t.clone() for t in pipe.result(slots[2])]
        pipe.finish()
        ok = True
        for k in range(3):
            for got, key in zip(slots[k], ("ref_grad", "src_grad", "depth_grad")):
                ok &= helpers.rel_err(got.numpy(), steps[k][key]) < 1e-5
        open(os.path.join(tmp, "rank%d.ok" % rank), "w").write("1" if ok else "0")
    finally:
        dist.destroy_process_group()


def test_pipelined_reducer_over_gloo(tmp_path):
    port = _free_port()
    mp.spawn(_pipeline_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [open(tmp_path / ("rank%d.ok" % r)).read() for r in range(2)] == ["1", "1"]


@pytest.mark.parametrize("batch", [1, 2])
def test_two_ranks_over_gloo(tmp_path, batch):
    """batch=1: both ranks split the item's depth range and all-reduce; batch=2: one item each, no exchange."""
    port = _free_port()
    mp.spawn(_worker, args=(2, port, batch, str(tmp_path)), nprocs=2, join=True)
    assert [open(tmp_path / ("rank%d.ok" % r)).read() for r in range(2)] == ["1", "1"]
