"""CostVolume forward + backward for callers whose tensors live in HOST memory.

The op's two big tensors - cost (output of the forward) and cost_grad (input of the backward) - are
D*C floats per pixel, far larger than everything else, and each depth plane of them is independent.
HostPipeline therefore cuts the depth range into chunks and runs three CUDA streams:
    copy-in : features / cameras / depths once, then cost_grad chunk by chunk   (host -> device)
    compute : forward(chunk k), backward(chunk k, accumulating)                  (C ABI, depth-range calls)
    copy-out: cost chunk k as soon as its forward is done; mask and the three gradients at the end
so the PCIe traffic in both directions overlaps with the kernels and with each other.  Device buffers are
allocated once in the constructor; `run` allocates nothing.  Host tensors must be pinned.
"""
import ctypes

import torch

from custom_helper_op_b200 import _lib
from custom_helper_op_b200.python.ops import custom_helper_ops as ops


class HostPipeline:
    def __init__(self, B, N, H, W, C, D, device, nchunks=4, half_centor=True):
        self.dims = (B, N, H, W, C, D)
        self.dev = torch.device(device)
        self.half_centor = half_centor
        nchunks = max(1, min(nchunks, D))
        per = (D + nchunks - 1) // nchunks
        self.chunks = [(d0, min(D, d0 + per)) for d0 in range(0, D, per)]
        f32 = dict(dtype=torch.float32, device=self.dev)
        self.d = dict(ref=torch.empty((B, H, W, C), **f32), src=torch.empty((B, N, H, W, C), **f32),
                      base_plane=torch.empty((B, H, W, 1), **f32), offsets=torch.empty((B, D), **f32),
                      Rs=torch.empty((B, N, 3, 3), **f32), Ts=torch.empty((B, N, 3), **f32))
        self.cost = torch.empty((B, H, W, D, C), **f32)
        self.mask = torch.empty((B, H, W, D, 1), dtype=torch.int32, device=self.dev)
        self.cost_grad = torch.empty((B, H, W, D, C), **f32)
        self.grads = (torch.empty((B, H, W, C), **f32), torch.empty((B, N, H, W, C), **f32),
                      torch.empty((B, H, W, 1), **f32))
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        self.ev_in = torch.cuda.Event()
        self.ev_cg = [torch.cuda.Event() for _ in self.chunks]
        self.ev_fwd = [torch.cuda.Event() for _ in self.chunks]
        self.ev_bwd = torch.cuda.Event()
        self.h2d_bytes = sum(t.numel() * 4 for t in self.d.values()) + self.cost_grad.numel() * 4
        self.d2h_bytes = (self.cost.numel() + self.mask.numel() + sum(g.numel() for g in self.grads)) * 4

    def _copy_depth_range(self, dst, src, d0, d1, stream):
        B, N, H, W, C, D = self.dims
        row = D * C * 4
        off = d0 * C * 4
        st = _lib.lib().chop_copy_2d_async(ctypes.c_void_p(dst.data_ptr() + off), row, ctypes.c_void_p(src.data_ptr() + off), row,
                                           (d1 - d0) * C * 4, B * H * W, ctypes.c_void_p(stream.cuda_stream))
        _lib.check(st, "chop_copy_2d_async")

    def run(self, host_in, host_cost_grad, host_out):
        """host_in: dict of pinned tensors (ref, src, base_plane, offsets, Rs, Ts); host_cost_grad: pinned
        [B,H,W,D,C]; host_out: dict of pinned tensors cost, mask, ref_grad, src_grad, base_plane_grad.
        Returns after everything has landed in host_out."""
        for t in list(host_in.values()) + [host_cost_grad] + list(host_out.values()):
            if not t.is_pinned():
                raise ValueError("HostPipeline needs pinned host tensors")
        d = self.d
        with torch.cuda.stream(self.s_in):
            for k, t in d.items():
                t.copy_(host_in[k], non_blocking=True)
            self.ev_in.record(self.s_in)
            for i, (d0, d1) in enumerate(self.chunks):
                self._copy_depth_range(self.cost_grad, host_cost_grad, d0, d1, self.s_in)
                self.ev_cg[i].record(self.s_in)
        with torch.cuda.stream(self.s_cmp):
            self.s_cmp.wait_event(self.ev_in)
            for i, (d0, d1) in enumerate(self.chunks):
                ops.cost_forward(1, d["ref"], d["src"], d["base_plane"], d["offsets"], d["Rs"], d["Ts"],
                                 half_centor=self.half_centor, d_range=(d0, d1), out=(self.cost, self.mask))
                self.ev_fwd[i].record(self.s_cmp)
                self.s_cmp.wait_event(self.ev_cg[i])
                if i == 0:   # the first depth-range call zero-fills the gradient buffers, the others add
                    ops.cost_backward(1, d["ref"], d["src"], d["base_plane"], d["offsets"], d["Rs"], d["Ts"], self.cost_grad,
                                      self.mask, half_centor=self.half_centor, d_range=(d0, d1), zero_into=self.grads)
                else:
                    ops.cost_backward(1, d["ref"], d["src"], d["base_plane"], d["offsets"], d["Rs"], d["Ts"], self.cost_grad,
                                      self.mask, half_centor=self.half_centor, d_range=(d0, d1), accumulate_into=self.grads)
            self.ev_bwd.record(self.s_cmp)
        with torch.cuda.stream(self.s_out):
            for i, (d0, d1) in enumerate(self.chunks):
                self.s_out.wait_event(self.ev_fwd[i])
                self._copy_depth_range(host_out["cost"], self.cost, d0, d1, self.s_out)
            host_out["mask"].copy_(self.mask, non_blocking=True)
            self.s_out.wait_event(self.ev_bwd)
            host_out["ref_grad"].copy_(self.grads[0], non_blocking=True)
            host_out["src_grad"].copy_(self.grads[1], non_blocking=True)
            host_out["base_plane_grad"].copy_(self.grads[2], non_blocking=True)
        self.s_out.synchronize()
        self.s_cmp.synchronize()
        self.s_in.synchronize()
