"""Sharding of the cost-volume path over the GPUs of one box (one process per GPU).

Forward voxels are independent and the gradients combine by summation, so the work splits
  * by batch item first - no exchange at all: features, cameras and gradients are per item;
  * by contiguous depth ranges inside an item when there are more ranks than items - the forward slices
    are disjoint, and the partial d(ref), d(src), d(base_plane) of the ranks that share an item are
    summed with ONE all-reduce over a packed buffer [ref_grad | src_grad | base_plane_grad].
    (CostVolumeV2's depth_grid gradient is per voxel, hence disjoint: it is not reduced.)
The reference has no multi-GPU code; this module is the host logic around the depth-range fields of
chop_cv_desc.  It is backend-agnostic: `compute_fwd` / `compute_bwd` are callables, by default the CUDA
ops; the CPU tests plug in other callables and run the same partition / packing / collective over gloo.
"""
from dataclasses import dataclass
from typing import List, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    item: int                 # batch item
    d_begin: int
    d_end: int
    group_ranks: Tuple[int, ...]  # ranks that share this item (length 1: nothing to reduce)


def partition(batch: int, depth: int, world: int) -> List[List[Shard]]:
    """Shards of every rank.  world <= batch: items are dealt out contiguously, whole depth range each.
    world > batch: the ranks are split into `batch` contiguous groups as evenly as possible and each
    group cuts its item's depth range into near-equal contiguous pieces."""
    if batch < 1 or depth < 1 or world < 1:
        raise ValueError("batch, depth and world must be positive")
    out: List[List[Shard]] = [[] for _ in range(world)]
    if world <= batch:
        per, extra = divmod(batch, world)
        b = 0
        for r in range(world):
            n = per + (1 if r < extra else 0)
            for _ in range(n):
                out[r].append(Shard(b, 0, depth, (r,)))
                b += 1
        return out
    per, extra = divmod(world, batch)
    r0 = 0
    for b in range(batch):
        n = per + (1 if b < extra else 0)
        ranks = tuple(range(r0, r0 + n))
        n_eff = min(n, depth)  # never more pieces than planes; surplus ranks get an empty range
        base, rem = divmod(depth, n_eff)
        d = 0
        for i, r in enumerate(ranks):
            if i < n_eff:
                size = base + (1 if i < rem else 0)
                out[r].append(Shard(b, d, d + size, ranks))
                d += size
            else:
                out[r].append(Shard(b, depth, depth, ranks))
        r0 += n
    return out


def pack_layout(shapes):
    """Offsets of tensors of the given shapes inside one flat buffer."""
    offs, total = [], 0
    for s in shapes:
        n = 1
        for x in s:
            n *= int(x)
        offs.append((total, n))
        total += n
    return offs, total


class GradReducer:
    """Packed gradient buffer of one batch item + the all-reduce over the ranks sharing that item.
    The buffer starts uninitialised (`zero=False`): the gradient op zero-fills the three views it is given."""

    def __init__(self, shapes, dtype, device, group=None, zero=False):
        self.shapes = [tuple(int(x) for x in s) for s in shapes]
        offs, total = pack_layout(self.shapes)
        self.flat = (torch.zeros if zero else torch.empty)(total, dtype=dtype, device=device)
        self.views = [self.flat[o:o + n].view(s) for (o, n), s in zip(offs, self.shapes)]
        self.group = group
        self.work = None

    def zero_(self):
        self.flat.zero_()

    def all_reduce(self):
        if self.group is not None:
            dist.all_reduce(self.flat, group=self.group)
        return self.views

    def all_reduce_async(self):
        """Issue the all-reduce without making the caller's stream wait for it: the collective runs on the
        backend's own stream (after the work already enqueued on the current stream) and what the caller
        launches next - the following step's forward - overlaps it.  `wait()` joins it."""
        if self.group is not None:
            self.work = dist.all_reduce(self.flat, group=self.group, async_op=True)

    def wait(self):
        if self.work is not None:
            self.work.wait()
            self.work = None
        return self.views


class PipelinedReducer:
    """Two packed buffers used in turn by consecutive steps of a depth-sharded item.  Step k's backward
    writes its partial gradients into buffer k % 2 and `reduce_async()` starts their all-reduce; the compute
    stream goes straight on with step k+1's forward and backward (other buffer).  A buffer is joined just
    before it is written again (`next_views`) or read (`result`, `finish`), so at most one collective is in
    flight behind the compute stream and its latency hides behind the next step's kernels."""

    def __init__(self, shapes, dtype, device, group):
        self.slots = [GradReducer(shapes, dtype, device, group), GradReducer(shapes, dtype, device, group)]
        self.k = 0

    def next_views(self):
        slot = self.slots[self.k % 2]
        slot.wait()
        return slot.views

    def reduce_async(self):
        slot = self.slots[self.k % 2]
        slot.all_reduce_async()
        self.k += 1
        return slot

    def result(self, slot):
        """The summed gradients of the step whose reduce_async() returned `slot`."""
        return slot.wait()

    def finish(self):
        for s in self.slots:
            s.wait()


def make_groups(plan: List[List[Shard]]):
    """One process group per set of ranks sharing an item (every rank must call this, in the same
    order, as torch.distributed requires).  Returns {ranks tuple: group or None}."""
    groups = {}
    seen = []
    for shards in plan:
        for s in shards:
            if s.group_ranks not in seen:
                seen.append(s.group_ranks)
    for ranks in seen:
        groups[ranks] = dist.new_group(list(ranks)) if len(ranks) > 1 else None
    return groups


def sharded_forward_backward(rank, plan, groups, inputs, cost_grad_fn, compute_fwd, compute_bwd, device):
    """Run this rank's shards.  `inputs[b]` holds item b's tensors (ref [1,H,W,C], src [1,N,H,W,C],
    base_plane, offsets, Rs, Ts); `cost_grad_fn(b, cost)` supplies the upstream gradient for the planes
    this rank computed (a [1,H,W,D,C] tensor, only [d_begin,d_end) is read).
    compute_fwd(inp, d0, d1) -> (cost, mask) full-extent tensors with planes [d0,d1) filled;
    compute_bwd(inp, cost_grad, mask, d0, d1, (ref_grad, src_grad, base_grad)) WRITES the partial gradients
    of planes [d0,d1) into the three views (they arrive uninitialised: the CUDA op zero-fills its outputs).
    The all-reduces are issued asynchronously and joined after the last shard has been launched.
    Returns {item: (cost, mask, ref_grad, src_grad, base_plane_grad)}; the gradients are complete (summed
    over the item's ranks) on every rank of the item's group."""
    pending = []
    for sh in plan[rank]:
        inp = inputs[sh.item]
        empty = sh.d_end <= sh.d_begin          # more ranks than planes: this rank contributes zeros
        red = GradReducer([inp["ref"].shape, inp["src"].shape, inp["base_plane"].shape], inp["base_plane"].dtype, device,
                          groups.get(sh.group_ranks), zero=empty)
        cost = mask = None
        if not empty:
            cost, mask = compute_fwd(inp, sh.d_begin, sh.d_end)
            compute_bwd(inp, cost_grad_fn(sh.item, cost), mask, sh.d_begin, sh.d_end, tuple(red.views))
        red.all_reduce_async()
        pending.append((sh.item, cost, mask, red))
    results = {}
    for item, cost, mask, red in pending:
        rg, sg, bg = red.wait()
        results[item] = (cost, mask, rg, sg, bg)
    return results


def cuda_compute_fns(half_centor=True, buffers=None):
    """compute_fwd / compute_bwd over the CUDA ops for sharded_forward_backward.  With `buffers` = (cost, mask)
    preallocated full-extent tensors they are reused for every shard (one item at a time fits a GPU even when
    a batch of them does not)."""
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops

    def fwd(inp, d0, d1):
        return ops.cost_forward(1, inp["ref"], inp["src"], inp["base_plane"], inp["offsets"], inp["Rs"], inp["Ts"],
                                half_centor=half_centor, d_range=(d0, d1), out=buffers)

    def bwd(inp, cost_grad, mask, d0, d1, views):
        ops.cost_backward(1, inp["ref"], inp["src"], inp["base_plane"], inp["offsets"], inp["Rs"], inp["Ts"], cost_grad, mask,
                          half_centor=half_centor, d_range=(d0, d1), zero_into=views)

    return fwd, bwd
