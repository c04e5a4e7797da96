"""Megatron-style tensor-parallel SwiGLU MLP forward: one process per GPU.

Rank r keeps rows [lo, hi) of W_gate / W_up (column-parallel: it owns h[:, lo:hi], no
communication) and columns [lo, hi) of W_down (row-parallel), so it produces a full-shape
partial out_r [M, d]; the MLP output is the sum over ranks.  The reference has no multi-GPU
code at all; this is the layout BASELINE's 70B and ragged configurations prescribe.

Numerics: partial sums leave the down GEMM in fp32, are summed in fp32 by the collective,
and are rounded to bf16 once at the end, which keeps the relative Frobenius error at the
single-GPU level (bf16 partials with bf16 accumulation would sit at 4.4e-3, next to the 5e-3
limit).

Overlap: rows of x are independent, so M is cut into slabs; the all-reduce (or
reduce-scatter + all-gather) of slab i runs on a communication stream while the GEMMs of
slab i+1 run on the compute stream.

`torch.distributed` is plumbing here (NCCL communicator, streams); the GEMMs and the final
rounding are libfswiglu kernels.  The class takes the local compute and rounding steps as
callables so that the host-side logic (sharding, slab schedule, collective, rounding) can be
exercised with CPU ranks over gloo.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import pack


def _cuda_local_partial(x, w_gate, w_up, w_down, out_f32, workspace):
    from . import ops

    ops.fused_swiglu_mlp_bf16(x, w_gate, w_up, w_down, out_dtype=torch.float32, workspace=workspace, out=out_f32)


def _cuda_round(src_f32, dst_bf16):
    import ctypes

    from . import capi

    with torch.cuda.device(src_f32.device):
        rc = capi.lib.fswiglu_cast_f32_to_bf16(ctypes.c_void_p(src_f32.data_ptr()), ctypes.c_void_p(dst_bf16.data_ptr()),
                                               src_f32.numel(),
                                               ctypes.c_void_p(torch.cuda.current_stream(src_f32.device).cuda_stream))
    capi.check(rc, "fswiglu_cast_f32_to_bf16")


class TensorParallelSwiGLU:
    """Rank-local shard of the MLP plus the collective that completes the forward.

    mode "allreduce": fp32 all-reduce of each slab, then one rounding to bf16.
    mode "rs_ag":     fp32 reduce-scatter over rows, rounding of the local rows, bf16 all-gather
                      (a quarter less wire traffic than the fp32 all-reduce).
    """

    def __init__(self, w_gate_shard: torch.Tensor, w_up_shard: torch.Tensor, w_down_shard: torch.Tensor,
                 group: Optional[dist.ProcessGroup] = None, n_slabs: int = 4, mode: str = "allreduce",
                 local_partial: Callable = _cuda_local_partial, round_fn: Callable = _cuda_round):
        if mode not in ("allreduce", "rs_ag"):
            raise ValueError("mode must be 'allreduce' or 'rs_ag'")
        self.w_gate, self.w_up, self.w_down = w_gate_shard, w_up_shard, w_down_shard
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_slabs = max(1, n_slabs)
        self.mode = mode
        self.local_partial = local_partial
        self.round_fn = round_fn
        self.device = w_gate_shard.device
        self.F_local, self.d = w_gate_shard.shape
        self._bufs = {}
        self._cuda = self.device.type == "cuda"
        self._comm_stream = torch.cuda.Stream(device=self.device) if self._cuda else None

    @classmethod
    def from_full(cls, w_gate, w_up, w_down, device, group=None, **kw):
        """Cut this rank's shard out of full (CPU) weights and move it to `device`."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        g, u, dn = pack.shard_mlp_weights(w_gate, w_up, w_down, world, rank)
        return cls(g.to(device), u.to(device), dn.to(device), group=group, **kw)

    # slab r0:r1 boundaries; with rs_ag every slab must split evenly over the ranks
    def slab_bounds(self, M: int):
        n = min(self.n_slabs, max(1, M))
        quantum = self.world * 8 if self.mode == "rs_ag" else 1
        per = (M + n - 1) // n
        per = (per + quantum - 1) // quantum * quantum
        bounds = []
        r0 = 0
        while r0 < M:
            r1 = min(M, r0 + per)
            bounds.append((r0, r1))
            r0 = r1
        return bounds

    def _buffers(self, M: int):
        key = M
        if key not in self._bufs:
            dev = self.device
            Mp = M
            if self.mode == "rs_ag":
                q = self.world
                Mp = sum(((r1 - r0 + q - 1) // q * q) for r0, r1 in self.slab_bounds(M))
            partial = torch.empty((Mp, self.d), dtype=torch.float32, device=dev)
            out = torch.empty((Mp, self.d), dtype=torch.bfloat16, device=dev)
            ws = None
            if self._cuda:
                from . import ops

                per = max(r1 - r0 for r0, r1 in self.slab_bounds(M))
                ws = ops.mlp_workspace(per, self.d, self.F_local, dev)
            self._bufs = {key: (partial, out, ws)}
        return self._bufs[key]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [M, d] replicated on every rank -> out [M, d] bf16, identical on every rank."""
        M = x.size(0)
        if M == 0:
            return torch.empty((0, self.d), dtype=torch.bfloat16, device=self.device)
        partial, out, ws = self._buffers(M)
        bounds = self.slab_bounds(M)
        compute = torch.cuda.current_stream(self.device) if self._cuda else None
        off = 0  # row offset in the (possibly padded) partial / out buffers
        for (r0, r1) in bounds:
            rows = r1 - r0
            if self.mode == "rs_ag":
                rows_p = (rows + self.world - 1) // self.world * self.world
            else:
                rows_p = rows
            p_slab = partial[off:off + rows_p]
            o_slab = out[off:off + rows_p]
            if rows_p != rows:
                p_slab[rows:].zero_()
            self.local_partial(x[r0:r1], self.w_gate, self.w_up, self.w_down, p_slab[:rows], ws)
            if self._cuda:
                ev = torch.cuda.Event()
                ev.record(compute)
                self._comm_stream.wait_event(ev)
                ctx = torch.cuda.stream(self._comm_stream)
            else:
                ctx = _NullCtx()
            with ctx:
                if self.world == 1:
                    self.round_fn(p_slab, o_slab)
                elif self.mode == "allreduce":
                    dist.all_reduce(p_slab, op=dist.ReduceOp.SUM, group=self.group)
                    self.round_fn(p_slab, o_slab)
                else:
                    per = rows_p // self.world
                    mine = p_slab[self.rank * per:(self.rank + 1) * per]
                    red = torch.empty_like(mine)
                    dist.reduce_scatter_tensor(red, p_slab, op=dist.ReduceOp.SUM, group=self.group)
                    mine_bf16 = torch.empty((per, self.d), dtype=torch.bfloat16, device=self.device)
                    self.round_fn(red, mine_bf16)
                    dist.all_gather_into_tensor(o_slab, mine_bf16, group=self.group)
            off += rows_p
        if self._cuda:
            compute.wait_stream(self._comm_stream)
        if self.mode == "rs_ag" and out.size(0) != M:
            # drop the per-slab padding rows
            pieces, off = [], 0
            for (r0, r1) in bounds:
                rows = r1 - r0
                rows_p = (rows + self.world - 1) // self.world * self.world
                pieces.append(out[off:off + rows])
                off += rows_p
            return torch.cat(pieces, dim=0)
        return out[:M]


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
