"""Megatron-style tensor-parallel SwiGLU MLP forward: one process per GPU.

Rank r keeps rows [lo, hi) of W_gate / W_up (column-parallel: it owns h[:, lo:hi], no
communication) and columns [lo, hi) of W_down (row-parallel), so it produces a full-shape
partial out_r [M, d]; the MLP output is the sum over ranks.  The reference has no multi-GPU
code at all; this is the layout the 70B-shape and ragged-batch benchmark configurations prescribe.

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

import os
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import pack


def _cuda_local_partial(x, w_gate, w_up, w_down, out_partial, workspace):
    from . import ops

    ops.fused_swiglu_mlp_bf16(x, w_gate, w_up, w_down, out_dtype=out_partial.dtype, workspace=workspace,
                              out=out_partial)


def _cuda_round(src_f32, dst_bf16):
    import ctypes

    from . import capi

    with torch.cuda.device(src_f32.device):
        rc = capi.lib.fswiglu_cast_f32_to_bf16(ctypes.c_void_p(src_f32.data_ptr()), ctypes.c_void_p(dst_bf16.data_ptr()),
                                               src_f32.numel(),
                                               ctypes.c_void_p(torch.cuda.current_stream(src_f32.device).cuda_stream))
    capi.check(rc, "fswiglu_cast_f32_to_bf16")


# ------------------------------------------------------------------------------------------------
# Slab planner for the "push" mode.  Measured on 8 x B200 at the 70B shape, equal slabs lose time twice:
# every slab's GEMMs end with a partly filled wave of the persistent schedule, and every slab boundary
# costs launch gaps.  One large slab followed by a small one ([7168, 1024] rows) was 5 % faster than four
# equal slabs: the large slab's reduction hides behind the small slab's GEMMs and only the small slab's
# reduction is exposed.  The planner below picks the slab heights from a cost model of exactly these
# effects (the GEMM tile model of pick_tile_n in csrc/api.cu + a compute/communication timeline).
# ------------------------------------------------------------------------------------------------
_UNIT_US = 1.375e-3       # one 128-byte operand row of one k-block, per CTA (measured: ~93 GB/s per SM)
_LAUNCH_US = 8.0          # launch gaps of a slab's two GEMMs
_BARRIER_US = 15.0        # cross-rank barrier before a slab's reduction
_NVLINK_BYTES_PER_US = 6.0e5


def _gemm_cost_units(m_tiles: int, n_out: int, max_tile: int, mma_per_col: int, ctas: int) -> float:
    best = float("inf")
    t = max_tile
    while t >= 32 // mma_per_col:
        waves = -(-(-(-n_out // t) * m_tiles) // ctas)
        cost = waves * (128 + t * mma_per_col)
        if cost < best * 0.97:
            best = cost
        t -= 16
    return best


def _slab_compute_us(rows: int, d: int, F_local: int, ctas: int) -> float:
    m_tiles = -(-rows // 128)
    gate_up = _gemm_cost_units(m_tiles, F_local, 128, 2, ctas) * -(-d // 64)
    down = _gemm_cost_units(m_tiles, d, 256, 1, ctas) * -(-F_local // 64)
    return (gate_up + down) * _UNIT_US + _LAUNCH_US


def _timeline_us(rows_list, d, F_local, world, ctas) -> float:
    compute_end = comm_end = 0.0
    for rows in rows_list:
        compute_end += _slab_compute_us(rows, d, F_local, ctas)
        out_bytes = rows / world * d * 2 * (world - 1)
        comm_end = max(compute_end, comm_end) + _BARRIER_US + out_bytes / _NVLINK_BYTES_PER_US
    return comm_end


def plan_slabs(M: int, d: int, F_local: int, world: int, ctas: int) -> list:
    """Slab heights (rows) for the push mode: all but the last a multiple of 256 (the row count of a two-SM
    tile, hence also of 8 * world)."""
    if M <= 1024 or world == 1:
        return [M]
    best_rows, best_t = [M], _timeline_us([M], d, F_local, world, ctas)
    for R in range(256, M, 256):
        n = -(-M // R)
        if n > 8:
            continue
        rows = [R] * (n - 1) + [M - R * (n - 1)]
        t = _timeline_us(rows, d, F_local, world, ctas)
        if t < best_t:
            best_rows, best_t = rows, t
    return best_rows


_PCIE_BYTES_PER_US = 5.0e4   # host link per GPU and direction (measured: about 53 GB/s)


def _host_timeline_us(rows_list, d, F_local, world, ctas) -> float:
    """Step time when every slab's rows come from and go back to host memory, 1/world of them per rank, on copy
    streams beside the GEMMs: in-copies queue one behind the other, a slab computes once its rows are in, a
    rank's finished rows leave after the slab's reduction."""
    in_end = compute_end = comm_end = out_end = 0.0
    for rows in rows_list:
        io = rows / world * d * 2 / _PCIE_BYTES_PER_US
        in_end += io + rows / world * d * 2 * (world - 1) / _NVLINK_BYTES_PER_US + _BARRIER_US
        compute_end = max(compute_end, in_end) + _slab_compute_us(rows, d, F_local, ctas)
        out_bytes = rows / world * d * 2 * (world - 1)
        comm_end = max(compute_end, comm_end) + _BARRIER_US + out_bytes / _NVLINK_BYTES_PER_US
        out_end = max(comm_end, out_end) + io
    return out_end


def plan_host_slabs(M: int, d: int, F_local: int, world: int, ctas: int) -> list:
    """Slab heights for the host-buffer step of the push mode: as plan_slabs, but the first slab's copy in and
    the last slab's copy out are exposed, so more and more equal slabs win than in the device-resident step."""
    if M <= 1024 or world == 1:
        return [M]
    best_rows, best_t = [M], _host_timeline_us([M], d, F_local, world, ctas)
    for R in range(256, M, 256):
        n = -(-M // R)
        if n > 8:
            continue
        rows = [R] * (n - 1) + [M - R * (n - 1)]
        t = _host_timeline_us(rows, d, F_local, world, ctas)
        if t < best_t:
            best_rows, best_t = rows, t
    return best_rows


class TensorParallelSwiGLU:
    """Rank-local shard of the MLP plus the collective that completes the forward.

    mode "allreduce": fp32 all-reduce of each slab, then one rounding to bf16.
    mode "rs_ag":     fp32 reduce-scatter over rows, rounding of the local rows, bf16 all-gather
                      (a quarter less wire traffic than the fp32 all-reduce).
    mode "push":      no NCCL on the data path.  The down-GEMM epilogue stores each bf16 partial row
                      straight into its owner rank's receive buffer (peer memory over NVLink, tile by
                      tile while the GEMM runs); after a cross-rank barrier every rank sums the copies
                      of its rows in fp32, rounds once and stores the result into all ranks' outputs.
                      bf16 on the wire, fp32 accumulation, one rounding; buffers are symmetric memory.
    """

    def __init__(self, w_gate_shard: torch.Tensor, w_up_shard: torch.Tensor, w_down_shard: torch.Tensor,
                 group: Optional[dist.ProcessGroup] = None, n_slabs: int = 0, mode: str = "push",
                 local_partial: Callable = _cuda_local_partial, round_fn: Callable = _cuda_round,
                 comm_sms: int = 0, wire_dtype: torch.dtype = torch.float32, reduce_ctas: int = 0,
                 slab_rows: Optional[list] = None):
        if mode not in ("allreduce", "rs_ag", "push"):
            raise ValueError("mode must be 'allreduce', 'rs_ag' or 'push'")
        if wire_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("wire_dtype must be float32 or bfloat16")
        self.wire_dtype = wire_dtype
        self.w_gate, self.w_up, self.w_down = w_gate_shard, w_up_shard, w_down_shard
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_slabs_auto = n_slabs <= 0   # push mode: slab heights from plan_slabs()
        self.n_slabs = max(1, n_slabs) if n_slabs > 0 else 4
        self._gemm_ctas = 148  # replaced by the device's SM count below when there is a device
        self._prev_max_ctas = None
        self.mode = mode
        self.local_partial = local_partial
        self.round_fn = round_fn
        self.device = w_gate_shard.device
        self.F_local, self.d = w_gate_shard.shape
        self._bufs = {}
        self._scratch = None
        self._recv_hdl = self._out_hdl = self._recv_bases = self._out_bases = None
        self._cuda = self.device.type == "cuda"
        self._comm_stream = torch.cuda.Stream(device=self.device, priority=-1) if self._cuda else None
        # reduce + broadcast kernel (push mode): 128 CTAs of 128 threads, one beside each GEMM CTA on most SMs.
        # Measured on 8 GPUs at the 70B shape: 64 CTAs 1.360 ms per step (the reduction of the first slab
        # outlasts the second slab's GEMMs), 128 CTAs 1.264 ms.
        self._reduce_ctas = reduce_ctas if reduce_ctas > 0 else 128
        self._xin = None
        self._copy_streams = None
        self._bounds_cache = {}
        # explicit slab heights (rows), e.g. [3840, 3840, 512]; every slab but the last must be a
        # multiple of 8 * world.  None: n_slabs equal slabs.
        self.slab_rows = list(slab_rows) if slab_rows else None
        # optional callable(tag, slab, stream), push mode: called at "gateup_begin", "gateup_end", "down_end" (compute
        # stream), "barrier_end", "reduce_end" (communication stream) of every slab and at "final_barrier_end" (slab
        # -1); a benchmark records an event on `stream` there to time the phases
        self.trace = None
        if mode != "push" and comm_sms == 0:
            comm_sms = 16  # NCCL kernels cannot share an SM with a persistent GEMM CTA
        if self._cuda and self.world > 1 and comm_sms > 0:
            # leave `comm_sms` SMs to the collective kernels that run beside the GEMMs (the launcher
            # should cap NCCL to the same number, e.g. NCCL_MAX_CTAS), see fswiglu_set_max_ctas
            from . import capi

            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            self._gemm_ctas = max(1, sms - comm_sms)
            with torch.cuda.device(self.device):
                self._prev_max_ctas = capi.lib.fswiglu_set_max_ctas(self._gemm_ctas)
        elif self._cuda:
            self._gemm_ctas = torch.cuda.get_device_properties(self.device).multi_processor_count

    def close(self) -> None:
        """Give the SMs that were set aside for the collectives back to this device's GEMM kernels."""
        if self._prev_max_ctas is not None and self._prev_max_ctas >= 0:
            from . import capi

            with torch.cuda.device(self.device):
                capi.lib.fswiglu_set_max_ctas(self._prev_max_ctas)
        self._prev_max_ctas = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown: the library may be gone already)
            pass

    @classmethod
    def from_full(cls, w_gate, w_up, w_down, device, group=None, **kw):
        """Cut this rank's shard out of full (CPU) weights and move it to `device`."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        g, u, dn = pack.shard_mlp_weights(w_gate, w_up, w_down, world, rank)
        return cls(g.to(device), u.to(device), dn.to(device), group=group, **kw)

    # slab r0:r1 boundaries; with rs_ag every slab must split evenly over the ranks
    def slab_bounds(self, M: int, host: bool = False):
        """Row slabs of a step over M rows; host=True: of the host-buffer step (forward_from_host), whose
        planned slabs also weigh the exposed copies."""
        # planned once per batch size: the planner walks a cost model over candidate splits, which costs
        # milliseconds of host time at large M, and this is called on the critical path of every step
        key = (M, tuple(self.slab_rows or ()), self.n_slabs, self.mode, host)
        cached = self._bounds_cache.get(key)
        if cached is None:
            cached = self._bounds_cache[key] = self._plan_bounds(M, host)
        return list(cached)

    def _plan_bounds(self, M: int, host: bool):
        quantum = self.world * 8 if self.mode in ("rs_ag", "push") else 1
        if self.slab_rows and sum(self.slab_rows) == M and all(r > 0 for r in self.slab_rows) and \
                all(r % quantum == 0 for r in self.slab_rows[:-1]):
            bounds, r0 = [], 0
            for r in self.slab_rows:
                bounds.append((r0, r0 + r))
                r0 += r
            return bounds
        if self.mode == "push" and self.world > 1 and self.n_slabs_auto and 128 % quantum == 0:
            bounds, r0 = [], 0
            planner = plan_host_slabs if host else plan_slabs
            for r in planner(M, self.d, self.F_local, self.world, self._gemm_ctas):
                bounds.append((r0, r0 + r))
                r0 += r
            return bounds
        n = min(self.n_slabs, max(1, M))
        per = (M + n - 1) // n
        per = (per + quantum - 1) // quantum * quantum
        bounds = []
        r0 = 0
        while r0 < M:
            r1 = min(M, r0 + per)
            bounds.append((r0, r1))
            r0 = r1
        return bounds

    def _buffers(self, M: int, bounds):
        """Receive / output / workspace buffers of a step over these slabs (kept per slab plan: the symmetric
        buffers are laid out slab by slab, each padded to a multiple of the world size)."""
        key = (M, tuple(bounds))
        if key not in self._bufs:
            dev = self.device
            Mp = M
            if self.mode in ("rs_ag", "push"):
                q = self.world
                Mp = sum(((r1 - r0 + q - 1) // q * q) for r0, r1 in bounds)
            handles = None
            if self.mode == "push" and self.world > 1:
                import torch.distributed._symmetric_memory as symm_mem

                grp = self.group if self.group is not None else dist.group.WORLD
                partial = symm_mem.empty((Mp, self.d), dtype=torch.bfloat16, device=dev)  # receive buffer
                out = symm_mem.empty((Mp, self.d), dtype=torch.bfloat16, device=dev)
                recv_hdl, out_hdl = symm_mem.rendezvous(partial, grp), symm_mem.rendezvous(out, grp)
                # peer base addresses, read once: they are used for every launch of every step
                handles = (recv_hdl, out_hdl, [int(p) for p in recv_hdl.buffer_ptrs], [int(p) for p in out_hdl.buffer_ptrs])
            else:
                partial = torch.empty((Mp, self.d), dtype=self.wire_dtype, device=dev)
                out = torch.empty((Mp, self.d), dtype=torch.bfloat16, device=dev)
            ws = None
            if self._cuda:
                from . import ops

                per = max(r1 - r0 for r0, r1 in bounds)
                ws = ops.mlp_workspace(per, self.d, self.F_local, dev)
                if self._scratch is None:
                    self._scratch = ops.gemm_scratch(dev)
            if len(self._bufs) >= 4:  # a handful of batch sizes / plans at most
                self._bufs.pop(next(iter(self._bufs)))
            self._bufs[key] = (partial, out, ws, handles)
        partial, out, ws, handles = self._bufs[key]
        if handles is not None:
            self._recv_hdl, self._out_hdl, self._recv_bases, self._out_bases = handles
        return partial, out, ws

    def forward(self, x: torch.Tensor, slab_ready=None, slab_done=None, host_plan: bool = False) -> torch.Tensor:
        """x [M, d] replicated on every rank -> out [M, d] bf16, identical on every rank.

        push mode only: `slab_ready[i]` is an event the compute stream waits for before it touches the rows of
        slab i of x; `slab_done(i, out_rows)` is called, with the reduction stream current, once this rank's own
        rows of slab i (owned_rows) are final in `out_rows`.  forward_from_host uses both to overlap the host
        copies with the GEMMs."""
        M = x.size(0)
        if M == 0:
            return torch.empty((0, self.d), dtype=torch.bfloat16, device=self.device)
        bounds = self.slab_bounds(M, host_plan)
        partial, out, ws = self._buffers(M, bounds)
        if self.mode == "push" and self.world > 1:
            return self._forward_push(x, partial, out, ws, bounds, slab_ready, slab_done)
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
                bf16_wire = self.wire_dtype == torch.bfloat16
                if self.world == 1:
                    o_slab.copy_(p_slab) if bf16_wire else self.round_fn(p_slab, o_slab)
                elif self.mode == "allreduce":
                    dist.all_reduce(p_slab, op=dist.ReduceOp.SUM, group=self.group)
                    o_slab.copy_(p_slab) if bf16_wire else self.round_fn(p_slab, o_slab)
                else:
                    per = rows_p // self.world
                    mine = p_slab[self.rank * per:(self.rank + 1) * per]
                    red = torch.empty_like(mine)
                    dist.reduce_scatter_tensor(red, p_slab, op=dist.ReduceOp.SUM, group=self.group)
                    if bf16_wire:
                        mine_bf16 = red
                    else:
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


    def owned_rows(self, M: int):
        """The rows of the result this rank hands back in forward_from_host, as (first, end) ranges in order.
        push mode: the rows it reduces, slab by slab (rank r owns the r-th 1/world of every slab); otherwise
        the r-th 1/world of all rows."""
        world, rank = self.world, self.rank
        if world == 1 or self.mode != "push":
            per = (M + world - 1) // world
            return [(min(M, rank * per), min(M, (rank + 1) * per))]
        ranges = []
        for (r0, r1) in self.slab_bounds(M, host=True):
            rpo = ((r1 - r0) + world - 1) // world
            g0 = min(r1, r0 + rank * rpo)
            ranges.append((g0, min(r1, g0 + rpo)))
        return ranges

    def forward_from_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """End-to-end step with host buffers.  x_host [M, d] is the (pinned) host copy of the replicated
        input; out_host receives this rank's rows of the result, the ranges owned_rows(M) one after the other.

        Every rank copies only its own rows over PCIe and hands them to the peers over NVLink (copy engines
        writing into the peers' symmetric input buffers), so the host link carries M*d*2/world bytes per rank
        instead of M*d*2.  In push mode this goes slab by slab on a copy stream of its own: slab i+1 arrives
        while slab i is in the GEMMs, and this rank's rows of slab i go back to the host as soon as its
        reduction is done, while later slabs compute.  Returns when out_host is filled."""
        M = x_host.size(0)
        world, rank = self.world, self.rank
        owned = self.owned_rows(M)
        if sum(g1 - g0 for g0, g1 in owned) != out_host.size(0):
            raise RuntimeError("out_host must hold exactly the rows of owned_rows(M)")
        if world == 1 or self.mode != "push":
            (r0, r1), = owned
            x = x_host.to(self.device, non_blocking=True)
            out = self.forward(x)
            out_host.copy_(out[r0:r1], non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            return
        import torch.distributed._symmetric_memory as symm_mem

        if self._xin is None or self._xin[0].size(0) != M:
            grp = self.group if self.group is not None else dist.group.WORLD
            xin = symm_mem.empty((M, self.d), dtype=torch.bfloat16, device=self.device)
            hdl = symm_mem.rendezvous(xin, grp)
            peers = [hdl.get_buffer(p, (M, self.d), torch.bfloat16) for p in range(world)]
            self._xin = (xin, hdl, peers)
        xin, hdl, peers = self._xin
        if os.environ.get("FSWIGLU_TP_HOST_PIPELINE", "1") == "0":
            # the plain order, for comparison: everything in, all slabs, everything out
            for g0, g1 in owned:
                if g1 > g0:
                    xin[g0:g1].copy_(x_host[g0:g1], non_blocking=True)
                    for k in range(1, world):
                        peers[(rank + k) % world][g0:g1].copy_(xin[g0:g1], non_blocking=True)
            hdl.barrier(channel=14)
            out = self.forward(xin, host_plan=True)
            o = 0
            for g0, g1 in owned:
                out_host[o:o + g1 - g0].copy_(out[g0:g1], non_blocking=True)
                o += g1 - g0
            hdl.barrier(channel=15)
            torch.cuda.current_stream(self.device).synchronize()
            return
        if self._copy_streams is None:
            self._copy_streams = (torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device))
        h2d, d2h = self._copy_streams
        cur = torch.cuda.current_stream(self.device)
        h2d.wait_stream(cur)
        ready = []
        with torch.cuda.stream(h2d):
            for si, (g0, g1) in enumerate(owned):
                if g1 > g0:
                    xin[g0:g1].copy_(x_host[g0:g1], non_blocking=True)        # PCIe: own rows of this slab only
                    for k in range(1, world):                                 # NVLink: to every peer
                        peers[(rank + k) % world][g0:g1].copy_(xin[g0:g1], non_blocking=True)
                hdl.barrier(channel=si % 8)                                   # all ranks' rows of slab si are here
                ev = torch.cuda.Event()
                ev.record(h2d)
                ready.append(ev)
        out_off = [0]
        for g0, g1 in owned:
            out_off.append(out_off[-1] + (g1 - g0))

        def slab_done(si, out_rows):
            n = owned[si][1] - owned[si][0]
            if n <= 0:
                return
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            d2h.wait_event(ev)
            with torch.cuda.stream(d2h):
                out_host[out_off[si]:out_off[si] + n].copy_(out_rows[:n], non_blocking=True)

        self.forward(xin, slab_ready=ready, slab_done=slab_done, host_plan=True)
        hdl.barrier(channel=15)                                       # nobody overwrites xin while it is read
        cur.wait_stream(d2h)
        cur.synchronize()

    def _forward_push(self, x, recv, out, ws, bounds, slab_ready=None, slab_done=None):
        """Reduce-scatter inside the down-GEMM epilogue (peer stores), then reduce + broadcast."""
        import ctypes

        from . import capi

        M = x.size(0)
        lib, world, rank, d, Fl = capi.lib, self.world, self.rank, self.d, self.F_local
        compute = torch.cuda.current_stream(self.device)
        comm = self._comm_stream
        recv_bases, out_bases = self._recv_bases, self._out_bases
        PtrArr = ctypes.c_void_p * world
        vp = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        off = 0
        with torch.cuda.device(self.device):
            for si, (r0, r1) in enumerate(bounds):
                rows = r1 - r0
                rows_p = (rows + world - 1) // world * world
                rpo = rows_p // world
                xs = x[r0:r1]
                h = ws[: rows * Fl * 2].view(torch.bfloat16).view(rows, Fl)
                sp = ctypes.c_void_p(compute.cuda_stream)
                if slab_ready is not None:
                    compute.wait_event(slab_ready[si])
                if self.trace is not None:
                    self.trace("gateup_begin", si, compute)
                rc = lib.fswiglu_gateup_bf16_ex(vp(xs), xs.stride(0), vp(self.w_gate), self.w_gate.stride(0),
                                                vp(self.w_up), vp(h), Fl, rows, Fl, d, 0, None, vp(self._scratch),
                                                self._scratch.numel(), sp)
                capi.check(rc, "fswiglu_gateup_bf16")
                if self.trace is not None:
                    self.trace("gateup_end", si, compute)
                slab_bytes = off * d * 2
                recv_ptrs = PtrArr(*[b + slab_bytes for b in recv_bases])
                rc = lib.fswiglu_down_scatter_bf16(vp(h), Fl, vp(self.w_down), self.w_down.stride(0), recv_ptrs, world,
                                                   rank, rpo, rows, d, Fl, vp(self._scratch), self._scratch.numel(),
                                                   sp)
                capi.check(rc, "fswiglu_down_scatter_bf16")
                if self.trace is not None:
                    self.trace("down_end", si, compute)
                ev = torch.cuda.Event()
                ev.record(compute)
                comm.wait_event(ev)
                with torch.cuda.stream(comm):
                    self._recv_hdl.barrier(channel=si % 4)  # every rank's partial rows of this slab have landed
                    if self.trace is not None:
                        self.trace("barrier_end", si, comm)
                    out_ptrs = PtrArr(*[b + (off + rank * rpo) * d * 2 for b in out_bases])
                    rc = lib.fswiglu_reduce_bcast_bf16(ctypes.c_void_p(recv_bases[rank] + slab_bytes), out_ptrs, world,
                                                       rpo, d, self._reduce_ctas, ctypes.c_void_p(comm.cuda_stream))
                    capi.check(rc, "fswiglu_reduce_bcast_bf16")
                    if self.trace is not None:
                        self.trace("reduce_end", si, comm)
                    if slab_done is not None:
                        slab_done(si, out[off + rank * rpo:off + (rank + 1) * rpo])
                off += rows_p
            with torch.cuda.stream(comm):
                self._out_hdl.barrier(channel=0)  # every rank's result rows have landed everywhere
                if self.trace is not None:
                    self.trace("final_barrier_end", -1, comm)
            compute.wait_stream(comm)
        if out.size(0) != M:
            pieces, off = [], 0
            for (r0, r1) in bounds:
                rows = r1 - r0
                pieces.append(out[off:off + rows])
                off += (rows + world - 1) // world * world
            return torch.cat(pieces, dim=0)
        return out[:M]


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
