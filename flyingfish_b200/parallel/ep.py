"""Expert-parallel communicator: every rank owns ``E / world`` experts and its own token rows
(attention is data-parallel), token rows travel to the experts' owners and results come back.

CUDA path (``csrc/moe_ep.cu``): rows are scattered straight into the owners' expert input buffers
with peer stores issued by the dispatch kernel, the owners run the grouped tcgen05 GEMMs on what
arrived, and the combine kernel reads the expert outputs directly out of the owners' memory --
no NCCL all-to-all on the hot path, no host involvement. CPU path (gloo): the same semantics
written with collectives, used by the host-side tests and as the library-call baseline.

The reference's closest feature is its 2-GPU "peer compute" expert residency, which moves one
layer's packet through pinned host memory (src/backend/cuda/engine_moe.rs:1643-1830).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_longlong, c_ulonglong

import torch
import torch.distributed as dist

from .. import ops
from ..ops import lib as oplib
from ..ops import moe_ops, ref


class EpArenaHost(ctypes.Structure):
    _fields_ = [("ptrs", c_ulonglong * 8), ("rank", c_int), ("world", c_int), ("E", c_int), ("E_local", c_int),
                ("hidden", c_int), ("capacity", c_int), ("off_flags", c_longlong), ("off_counts", c_longlong),
                ("off_x", c_longlong), ("off_y", c_longlong)]


# FP8-resident experts: ship rows as packed E4M3 records (FLYINGFISH_EP_FP8_DISPATCH=0: BF16 rows, quantised on arrival)
FP8_DISPATCH = os.environ.get("FLYINGFISH_EP_FP8_DISPATCH", "1") != "0"


class EPComm:
    def __init__(self, group: dist.ProcessGroup, device: torch.device | str, num_experts: int, hidden: int,
                 max_rows: int = 0, top_k: int = 1, inter: int = 0):
        self.group = group
        self.device = torch.device(device)
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        assert num_experts % self.size == 0, "experts must divide evenly over the expert-parallel ranks"
        self.E, self.El, self.hidden = num_experts, num_experts // self.size, hidden
        self.stats = {"fused_calls": 0, "baseline_calls": 0}
        self.provider = None          # experts.provider.TieredExpertProvider when this rank tiers its own experts
        self.arena = None
        self.max_rows = max_rows      # most local rows one layer call may dispatch (the engine caps its prefill chunk by it)
        if self.device.type == "cuda" and self.size > 1:
            self._setup_arena(max_rows, top_k)

    # -- symmetric buffers -----------------------------------------------------------------------
    def _setup_arena(self, max_rows: int, top_k: int) -> None:
        import torch.distributed._symmetric_memory as symm
        lib = oplib.kernels()
        lib.ff_ep_arena_layout.restype = c_longlong
        # Real routers are skewed, so the receive buffers are sized for the worst case -- every rank sends all of its
        # assignments to this owner -- whenever that fits the byte budget (FF_EP_ARENA_MAX_GIB, default 4 GiB for the
        # two row buffers; decode batches and the benchmark prefill chunks do). Only beyond it the budget falls back
        # to a multiple of the balanced share (FF_EP_CAPACITY_FACTOR, default 2x); a layer call is then run in several
        # passes over slices of the local rows, each small enough that even its worst case fits (``rows_fit``), so a
        # skewed router costs extra passes instead of an overflow.
        import os
        budget = float(os.environ.get("FF_EP_ARENA_MAX_GIB", "4")) * (1 << 30)
        factor = float(os.environ.get("FF_EP_CAPACITY_FACTOR", "2"))
        balanced = max_rows * top_k
        worst = self.size * balanced
        fit = int(budget // (2 * self.hidden * 2))
        cap = max(256, min(worst, max(int(factor * balanced), fit)) + 16 * self.El)
        cap = (cap + 15) // 16 * 16
        self.capacity_is_worst_case = cap >= worst + 16 * self.El
        self.rows_fit = max(1, (cap - 16 * self.El) // (self.size * top_k))
        self.passes = 1 if self.capacity_is_worst_case else -(-max_rows // self.rows_fit)
        offs = [c_longlong(0) for _ in range(4)]
        total = lib.ff_ep_arena_layout(self.size, self.E, self.hidden, cap, *[ctypes.byref(o) for o in offs])
        self.buf = symm.empty(int(total), dtype=torch.uint8, device=self.device)
        self.handle = symm.rendezvous(self.buf, self.group)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        h = EpArenaHost()
        for i in range(8):
            h.ptrs[i] = ptrs[i] if i < len(ptrs) else 0
        h.rank, h.world, h.E, h.E_local, h.hidden, h.capacity = self.rank, self.size, self.E, self.El, self.hidden, cap
        h.off_flags, h.off_counts, h.off_x, h.off_y = (o.value for o in offs)
        self.arena = h
        self.capacity = cap
        self.recv_x = self.buf[h.off_x: h.off_x + cap * self.hidden * 2].view(torch.bfloat16).view(cap, self.hidden)
        self.out_y = self.buf[h.off_y: h.off_y + cap * self.hidden * 2].view(torch.bfloat16).view(cap, self.hidden)
        self.scratch = torch.zeros(2 * self.E + 2 * self.El + 1, dtype=torch.int32, device=self.device)

    # -- one MoE layer ---------------------------------------------------------------------------
    def dispatch_ffn_combine(self, x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, lw, mode: int,
                             layer: int = -1) -> torch.Tensor:
        """Routed-expert output for the local rows ``x`` (shared expert not included). ``layer``: the model's layer
        number, needed when this rank serves its experts from tiers."""
        if self.arena is not None and x.is_cuda:
            if self.passes == 1:
                return self._fused(x, weights, ids, lw, mode, layer)
            # every rank runs the same number of passes (the phases are collective); a rank whose rows are used up
            # sends one zero-weight row so that its kernels still take part
            if x.shape[0] > self.passes * self.rows_fit:
                raise ValueError(f"expert-parallel call of {x.shape[0]} rows exceeds max_rows={self.max_rows}")
            out = torch.empty_like(x)
            for p in range(self.passes):
                lo, hi = p * self.rows_fit, min((p + 1) * self.rows_fit, x.shape[0])
                if hi > lo:
                    out[lo:hi] = self._fused(x[lo:hi], weights[lo:hi], ids[lo:hi], lw, mode, layer)
                else:
                    self._fused(torch.zeros_like(x[:1]), torch.zeros_like(weights[:1]), torch.zeros_like(ids[:1]), lw, mode, layer)
            self.stats["multi_pass_calls"] = self.stats.get("multi_pass_calls", 0) + 1
            return out
        if self.provider is not None:
            raise RuntimeError("tiered experts under expert parallelism need the CUDA peer-memory path")
        return self._baseline(x, weights, ids, lw, mode)

    def _fused(self, x, weights, ids, lw, mode, layer: int = -1):
        if self.provider is None and not isinstance(lw.experts_gu, torch.Tensor) and self.fp8_dispatch_ok():
            # FP8-resident experts: rows are quantised 1x128 HERE and travel as packed records [codes | scales]
            # (hidden + hidden / 32 bytes instead of 2 * hidden): the owners' W8A8 GEMMs read the records in place
            pos = self.dispatch_fp8(x, ids)
            self.experts_fp8_packed(lw)
            out = self.combine(pos, ids, weights, x.shape[0])
            self.stats["fused_calls"] += 1
            self.stats["fp8_dispatch_calls"] = self.stats.get("fp8_dispatch_calls", 0) + 1
            return out
        pos = self.dispatch(x, ids)
        if self.provider is not None:
            self.provider.ep_experts(layer, self.recv_x, self._seg_off, self._counts, self.capacity, self.out_y,
                                     expected_rows=self._rows_per_expert * self.El)
        else:
            self.experts(lw)
        out = self.combine(pos, ids, weights, x.shape[0])
        self.stats["fused_calls"] += 1
        return out

    # The three phases of the fused path (also timed one by one by ``utils/epbench.py``). Every rank must call
    # all three, in this order, once per layer call: the kernels wait (bounded) on one another's flags.
    def dispatch(self, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Scatters the local rows into the owners' expert input buffers; returns ``pos`` [rows * top_k]."""
        lib = oplib.kernels()
        rows, top_k = ids.shape
        E, El = self.E, self.El
        counts_s, cursors = self.scratch[:E], self.scratch[E: 2 * E]
        self._seg_off, self._counts = self.scratch[2 * E: 2 * E + El + 1], self.scratch[2 * E + El + 1:]
        pos = torch.empty(rows * top_k, dtype=torch.int32, device=x.device)
        self._rows_per_expert = rows * top_k / El        # expected segment length when every rank sends as many rows
        x = x.contiguous(); ids = ids.contiguous()
        rc = lib.ff_ep_dispatch(ctypes.byref(self.arena), oplib.ptr(x), oplib.ptr(ids), rows, top_k, x.stride(0),
                                oplib.ptr(counts_s), oplib.ptr(cursors), oplib.ptr(pos), oplib.ptr(self._seg_off),
                                oplib.ptr(self._counts), oplib.ptr(oplib.status_tensor(x.device)), oplib.stream_ptr())
        oplib.check(rc, "ff_ep_dispatch")
        ops._count(3)
        return pos

    def fp8_dispatch_ok(self) -> bool:
        rec = self.hidden + self.hidden // 32
        return FP8_DISPATCH and self.hidden % 128 == 0 and rec % 16 == 0

    def dispatch_fp8(self, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Quantise the local rows (E4M3, one scale per 128) into packed records and scatter them to the owners."""
        lib = oplib.kernels()
        rows, top_k = ids.shape
        E, El, h = self.E, self.El, self.hidden
        rec = h + h // 32
        counts_s, cursors = self.scratch[:E], self.scratch[E: 2 * E]
        self._seg_off, self._counts = self.scratch[2 * E: 2 * E + El + 1], self.scratch[2 * E + El + 1:]
        pos = torch.empty(rows * top_k, dtype=torch.int32, device=x.device)
        self._rows_per_expert = rows * top_k / El
        x = x.contiguous(); ids = ids.contiguous()
        packed = torch.empty(rows, rec, dtype=torch.uint8, device=x.device)
        rc = lib.ff_quant_fp8_1x128_strided(oplib.ptr(x), oplib.ptr(packed), ctypes.c_void_p(packed.data_ptr() + h), rows, h,
                                            x.stride(0), ctypes.c_longlong(rec), ctypes.c_longlong(rec // 4),
                                            oplib.stream_ptr())
        oplib.check(rc, "ff_quant_fp8_1x128_strided")
        rc = lib.ff_ep_dispatch_bytes(ctypes.byref(self.arena), oplib.ptr(packed), oplib.ptr(ids), rows, top_k, rec, rec,
                                      oplib.ptr(counts_s), oplib.ptr(cursors), oplib.ptr(pos), oplib.ptr(self._seg_off),
                                      oplib.ptr(self._counts), oplib.ptr(oplib.status_tensor(x.device)), oplib.stream_ptr())
        oplib.check(rc, "ff_ep_dispatch_bytes")
        ops._count(4)
        return pos

    def experts_fp8_packed(self, lw) -> None:
        """W8A8 grouped GEMMs of this rank's experts over the packed records in the receive buffer."""
        from ..ops import quant_ops
        lib = oplib.kernels()
        h = self.hidden
        rec = h + h // 32
        base = self.recv_x.data_ptr()
        gu = lw.experts_gu
        el, nw, _ = gu.codes.shape
        mid = torch.empty(self.capacity, nw // 2, dtype=torch.bfloat16, device=self.recv_x.device)
        rc = lib.ff_gemm_fp8_strided(ctypes.c_void_p(base), ctypes.c_void_p(base + h), ctypes.c_longlong(rec), rec // 4,
                                     oplib.ptr(gu.codes), oplib.ptr(gu.scale), oplib.ptr(mid), oplib.ptr(self._seg_off),
                                     oplib.ptr(self._counts), el, self.capacity, nw, h, nw // 2, 1,
                                     oplib.ptr(oplib.status_tensor(mid.device)), oplib.stream_ptr())
        oplib.check(rc, "ff_gemm_fp8_strided")
        ops._count()
        hq, hs = quant_ops.quant_fp8_act(mid)
        quant_ops.grouped_gemm_fp8(hq, hs, lw.experts_down.codes, lw.experts_down.scale, self._seg_off, self._counts,
                                   self.capacity, epi=0, out=self.out_y)

    def experts(self, lw) -> None:
        """Grouped gate/up (+SwiGLU) and down GEMMs of this rank's experts over the received rows."""
        from ..ops import moe_cuda
        lib = oplib.kernels()
        if not isinstance(lw.experts_gu, torch.Tensor):
            # FP8-resident experts: the received BF16 rows are quantised 1x128 on arrival and both grouped GEMMs
            # run W8A8; the down projection writes into the symmetric output buffer the peers read from
            from ..ops import quant_ops
            xq, xs = quant_ops.quant_fp8_act(self.recv_x)
            h = quant_ops.grouped_gemm_fp8(xq, xs, lw.experts_gu.codes, lw.experts_gu.scale, self._seg_off, self._counts,
                                           self.capacity, epi=1)
            hq, hs = quant_ops.quant_fp8_act(h)
            quant_ops.grouped_gemm_fp8(hq, hs, lw.experts_down.codes, lw.experts_down.scale, self._seg_off, self._counts,
                                       self.capacity, epi=0, out=self.out_y)
            return
        wgu = moe_cuda._gu_interleaved(lw.experts_gu)
        h = moe_cuda.grouped_gemm(self.recv_x, wgu, self._seg_off, self._counts, self.capacity, epi=1,
                                  rows_per_expert=self._rows_per_expert)
        # the down projection writes into the symmetric output buffer the peers read from
        fn = lib.ff_moe_grouped_gemm_tiled if self._rows_per_expert >= moe_cuda.TILED_MIN_ROWS else lib.ff_moe_grouped_gemm
        rc = fn(oplib.ptr(h), oplib.ptr(lw.experts_down), oplib.ptr(self.out_y),
                                     oplib.ptr(self._seg_off), oplib.ptr(self._counts), self.El, self.hidden, h.shape[1],
                                     self.capacity, self.hidden, 0, oplib.ptr(oplib.status_tensor(h.device)),
                                     oplib.stream_ptr())
        oplib.check(rc, "ff_moe_grouped_gemm(down)")
        ops._count(1)

    def combine(self, pos: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, rows: int) -> torch.Tensor:
        """Weighted sum, in ascending expert id, of the expert outputs read out of the owners' memory."""
        lib = oplib.kernels()
        out = torch.empty(rows, self.hidden, dtype=torch.bfloat16, device=pos.device)
        ids = ids.contiguous(); weights = weights.contiguous()
        rc = lib.ff_ep_combine(ctypes.byref(self.arena), oplib.ptr(pos), oplib.ptr(ids), oplib.ptr(weights),
                               oplib.ptr(out), rows, ids.shape[1], oplib.ptr(oplib.status_tensor(pos.device)),
                               oplib.stream_ptr())
        oplib.check(rc, "ff_ep_combine")
        ops._count(1)
        return out

    def _baseline(self, x, weights, ids, lw, mode):
        """Collective formulation (gloo / NCCL): gather rows, every rank computes the contributions of
        its experts, contributions are summed across ranks (exactly one rank is non-zero per
        entry), each rank reduces its own rows in ascending expert id."""
        rows, k = ids.shape
        n_rows = torch.tensor([rows], dtype=torch.int64, device=x.device)
        all_n = [torch.zeros_like(n_rows) for _ in range(self.size)]
        dist.all_gather(all_n, n_rows, group=self.group)
        counts = [int(t.item()) for t in all_n]
        mx = max(counts)

        def gather(t, pad_val=0):
            pad = torch.full((mx,) + t.shape[1:], pad_val, dtype=t.dtype, device=t.device)
            pad[: t.shape[0]] = t
            out = [torch.empty_like(pad) for _ in range(self.size)]
            dist.all_gather(out, pad, group=self.group)
            return torch.cat([o[:c] for o, c in zip(out, counts)], 0)

        xf = x.to(torch.float32) if x.dtype == torch.bfloat16 and not x.is_cuda else x
        ax = gather(xf).to(x.dtype)
        aid = gather(ids)
        aw = gather(weights)
        total = ax.shape[0]
        e0 = self.rank * self.El
        contrib = torch.zeros(total, k, self.hidden, dtype=torch.float32, device=x.device)
        for le in range(self.El):
            r, c = torch.nonzero(aid == e0 + le, as_tuple=True)
            if r.numel() == 0:
                continue
            if not isinstance(lw.experts_gu, torch.Tensor):
                from ..ops import quant_ops
                gu = ops.linear(ax[r].contiguous(), lw.experts_gu.expert(le))
                if lw.experts_gu.interleaved:
                    gu = quant_ops._deinterleave_cols(gu)
                y = ops.linear(ops.silu_mul(gu, mode), lw.experts_down.expert(le))
            else:
                y = ref.expert_ffn(ax[r], lw.experts_gu[le], lw.experts_down[le], mode) if not x.is_cuda else \
                    ops.linear(ops.silu_mul(ops.linear(ax[r].contiguous(), lw.experts_gu[le]), mode), lw.experts_down[le])
            contrib[r, c] = y.to(torch.float32) * aw[r, c, None]
        dist.all_reduce(contrib, group=self.group)
        start = sum(counts[: self.rank])
        mine = contrib[start: start + rows]
        order = torch.argsort(ids.long(), dim=-1, stable=True)
        ordered = torch.gather(mine, 1, order[:, :, None].expand_as(mine))
        acc = torch.zeros(rows, self.hidden, dtype=torch.float32, device=x.device)
        for j in range(k):
            acc = acc + ordered[:, j]
        self.stats["baseline_calls"] += 1
        return acc.to(x.dtype)
