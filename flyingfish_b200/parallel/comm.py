"""Tensor-parallel communicator.

The reference has no distributed runtime at all (its only multi-GPU feature bounces one layer's
activations through pinned host memory, src/backend/cuda/engine_moe.rs:1643-1830, and forbids
direct peer access, src/backend/cuda/mod.rs:448-484). On an NVSwitch box every GPU can store
into every peer at full NVLink bandwidth, so this build does the opposite:

* plumbing (rendezvous, barriers, large collectives, baseline path): ``torch.distributed`` over
  NCCL (``gloo`` on CPU for the host-side tests);
* hot path: one arena of *symmetric memory* per rank, mapped into every peer, and hand-written
  kernels that push tiles / vectors into peers' arenas with plain stores and poll local flags
  (``csrc/comm.cuh``). ``row_linear`` runs the row-parallel projection and its all-reduce as ONE
  kernel (``ff_gemm_ar``) at decode sizes.

A start-up self-test writes a rank-specific pattern into every peer's arena and verifies what
arrived (the reference verifies its transport the same way, src/backend/cuda/mod.rs:487-664).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_longlong, c_ulonglong

import torch
import torch.distributed as dist

from .. import ops
from ..ops import lib as oplib
from ..utils.log import log_json

SLOT_BYTES = 4 << 20          # one source-rank slot: 256 rows x 8192 columns of BF16


class TransportError(RuntimeError):
    pass


class SymmArena:
    """Symmetric per-rank buffer with peer mappings (``torch.distributed._symmetric_memory``)."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, slot_bytes: int = SLOT_BYTES):
        import torch.distributed._symmetric_memory as symm
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        lib = oplib.kernels()
        lib.ff_arena_data_offset.restype = c_longlong
        self.data_off = int(lib.ff_arena_data_offset())
        self.slot_bytes = slot_bytes
        self.half_bytes = slot_bytes * self.world
        total = self.data_off + 2 * self.half_bytes
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buf, group)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.ptrs = (c_ulonglong * 8)(*(ptrs + [0] * (8 - len(ptrs))))
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def args(self) -> tuple:
        return (self.ptrs, self.rank, self.world, c_longlong(self.half_bytes), c_longlong(self.slot_bytes))

    def self_test(self, words: int = 1 << 16) -> None:
        """Every rank writes a pattern into its slot on every peer; every rank verifies all slots,
        then verifies that a planted single-word flip IS detected."""
        lib = oplib.kernels()
        s = oplib.stream_ptr()
        bad = torch.zeros(1, dtype=torch.int32, device=self.device)
        oplib.check(lib.ff_transport_fill(*self.args(), words, 0x5EED, s), "ff_transport_fill")
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        oplib.check(lib.ff_transport_verify(*self.args(), words, 0x5EED, oplib.ptr(bad), s), "ff_transport_verify")
        n_bad = int(bad.item())
        if n_bad:
            raise TransportError(f"rank {self.rank}: {n_bad} corrupted words in the peer transport self-test")
        # negative control: flip one word locally, the verifier must see exactly one mismatch
        off = self.data_off + ((self.rank + 1) % self.world) * self.slot_bytes + 4 * 123
        self.buf[off] ^= 0x40
        bad.zero_()
        oplib.check(lib.ff_transport_verify(*self.args(), words, 0x5EED, oplib.ptr(bad), s), "ff_transport_verify")
        if int(bad.item()) != 1:
            raise TransportError("transport self-test did not detect a planted corruption")
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        # leave the data area clean (flags/epoch untouched: they were not used)
        self.buf[self.data_off:].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)


class TPComm:
    """Tensor-parallel group: fused peer-memory kernels on CUDA, plain collectives on CPU."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, arena: SymmArena | None):
        self.group, self.device, self.arena = group, device, arena
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.fused = arena is not None
        self.stats = {"gemm_ar": 0, "oneshot_ar": 0, "nccl_ar": 0, "ag_gemm": 0, "gemm_rs": 0}
        self.tile_counters = torch.zeros(4096, dtype=torch.int32, device=device) if arena is not None else None
        # NVLS: when the arena has a multicast mapping the fused GEMM + all-reduce exchanges through the switch. Two
        # forms (FF_NVLS_ONESHOT): one-shot (default) -- every rank multicasts its partial tile and one flag with
        # multimem.st, then sums all slots locally: one flag round, one store per value instead of world-1; two-shot
        # (=0) -- partials stay local, the owner of a chunk sums them inside the switch (multimem.ld_reduce) and
        # multicasts the result: two flag rounds. Measured per projection at M 64 (o_proj / down) and per decode step of
        # the 8-B shape: 8 ranks: one-shot 35 / 38 us and 3.56 ms, two-shot 46 / 49 us and 4.13 ms, plain peer stores
        # 68 / 62 us and 4.97 ms (GEMM + NCCL all-reduce: 47-68 us); 2 ranks: one-shot 32 / 41 us = plain peer stores
        # 32 / 40 us, two-shot 44 / 54 us. FLYINGFISH_NVLS=auto (default): on from four ranks; 1 / 0 force it. Always
        # off with NCCL_NVLS_ENABLE=0 (tests in which a rank may leave run on plain peer stores: a rank that dies while
        # bound to a multicast object faults its peers).
        mode = os.environ.get("FLYINGFISH_NVLS", "auto")
        want = mode == "1" or (mode == "auto" and self.size >= 4)
        self.nvls = bool(arena is not None and arena.multicast_ptr and want
                         and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0")
        # Sequence-parallel prefill pair (all-gather -> GEMM, GEMM -> reduce-scatter): the one-kernel forms win at
        # two ranks (1.03-1.38 x the GEMM + NCCL collective) but at eight ranks, where 7/8 of every tile crosses
        # NVLink, their tile pushes reached a quarter of the link rate and NCCL's collectives around the same GEMM
        # were faster (944 us against 1235 us per layer of 8192 rows). FLYINGFISH_SP_FUSED=auto (default): one
        # kernel up to four ranks, GEMM + NCCL collective from eight; 1 / 0 force either.
        sp = os.environ.get("FLYINGFISH_SP_FUSED", "auto")
        self.sp_fused = sp == "1" or (sp == "auto" and self.size <= 4)

    @classmethod
    def create(cls, group: dist.ProcessGroup, device: torch.device | str, fused: bool = True,
               self_test: bool = True, slot_bytes: int = SLOT_BYTES) -> "TPComm":
        """``slot_bytes``: bytes one rank may deposit in a peer per collective; sequence-parallel
        prefill needs ``rows_per_rank * hidden * 2``."""
        device = torch.device(device)
        arena = None
        if device.type == "cuda" and fused and dist.get_world_size(group) > 1:
            arena = SymmArena(group, device, max(SLOT_BYTES, (slot_bytes + 255) // 256 * 256))
            if self_test:
                arena.self_test()
            log_json("cuda_peer_topology", verbose_only=True, rank=arena.rank, world=arena.world,
                     transport="symmetric_memory_p2p", multicast=bool(arena.multicast_ptr))
        return cls(group, device, arena)

    # -- collectives --------------------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        if self.fused and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0 \
                and x.numel() * 2 <= self.arena.slot_bytes:
            out = torch.empty_like(x)
            rc = oplib.kernels().ff_allreduce_oneshot(*self.arena.args(), oplib.ptr(x), oplib.ptr(out),
                                                      c_longlong(x.numel()), oplib.ptr(oplib.status_tensor(x.device)),
                                                      oplib.stream_ptr())
            oplib.check(rc, "ff_allreduce_oneshot")
            self.stats["oneshot_ar"] += 1
            ops._count()
            return out
        if x.dtype in (torch.bfloat16, torch.float16) and not x.is_cuda:
            y = x.to(torch.float32)                      # gloo has no 16-bit reductions on every build
            dist.all_reduce(y, group=self.group)
            return y.to(x.dtype)
        dist.all_reduce(x, group=self.group)
        self.stats["nccl_ar"] += 1
        return x

    def row_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Row-parallel projection: ``sum_r x_r @ w_r.T``. One fused kernel at decode sizes."""
        if self.size == 1:
            return ops.linear(x, w)
        m, n = x.shape[0], w.shape[0]
        if self.fused and x.is_cuda and isinstance(w, torch.Tensor) and m <= ops.SKINNY_MAX_M and n % 8 == 0 \
                and m * n * 2 <= self.arena.slot_bytes:
            lib = oplib.kernels()
            k = x.shape[1]
            sb, cb = c_longlong(0), c_longlong(0)
            grid = lib.ff_gemm_skinny_plan(m, n, k, ctypes.byref(sb), ctypes.byref(cb))
            ws = ops.workspace(x.device)
            scratch = ws.ensure("gemm_scratch", sb.value // 4) if sb.value > 0 else None
            out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
            rc = lib.ff_gemm_ar(*self.arena.args(), oplib.ptr(x), oplib.ptr(w), oplib.ptr(out), m, n, k, x.stride(0),
                                w.stride(0), n, grid, oplib.ptr(scratch), oplib.ptr(ws.gemm_counters),
                                ctypes.c_ulonglong(self.arena.multicast_ptr if self.nvls else 0),
                                oplib.ptr(oplib.status_tensor(x.device)), oplib.stream_ptr())
            oplib.check(rc, "ff_gemm_ar")
            self.stats["gemm_ar"] += 1
            ops._count()
            return out
        return self.all_reduce(ops.linear(x, w))

    # -- sequence-parallel prefill: fused all-gather -> GEMM and GEMM -> reduce-scatter ---------
    def sp_ok(self, rows: int, k: int, n: int) -> bool:
        """Can ``rows`` (total) be processed with the fused sequence-parallel kernels?"""
        if not self.fused or rows % (self.size * 128):
            return False
        rpr = rows // self.size
        return rpr * max(k, n) * 2 <= self.arena.slot_bytes

    def ag_linear(self, x_shard: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
        """Column-parallel projection of row-sharded activations: returns ``[rows_total, N_local]``
        (``N_local / 2`` with the fused SwiGLU epilogue) -- one kernel (``ff_ag_gemm``)."""
        rpr, k = x_shard.shape
        n = w.shape[0]
        m = rpr * self.size
        if not self.sp_fused:
            full = self.all_gather_rows(x_shard)
            self.stats["nccl_ag"] = self.stats.get("nccl_ag", 0) + 1
            return ops.linear_swiglu(full, w) if swiglu else ops.linear(full, w)
        out = torch.empty(m, n // 2 if swiglu else n, dtype=torch.bfloat16, device=x_shard.device)
        rc = oplib.kernels().ff_ag_gemm(*self.arena.args(), oplib.ptr(x_shard), oplib.ptr(w), oplib.ptr(out), m, n, k,
                                        x_shard.stride(0), w.stride(0), out.stride(0), 1 if swiglu else 0,
                                        oplib.ptr(self.tile_counters), oplib.ptr(oplib.status_tensor(x_shard.device)),
                                        oplib.stream_ptr())
        oplib.check(rc, "ff_ag_gemm")
        self.stats["ag_gemm"] += 1
        ops._count()
        return out

    def rs_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Row-parallel projection with the reduce-scatter fused in: returns this rank's
        ``[rows_total / world, N]`` rows of the summed output -- one kernel (``ff_gemm_rs``)."""
        m, k = x.shape
        n = w.shape[0]
        out = torch.empty(m // self.size, n, dtype=torch.bfloat16, device=x.device)
        if not self.sp_fused:
            dist.reduce_scatter_tensor(out, ops.linear(x, w), group=self.group)
            self.stats["nccl_rs"] = self.stats.get("nccl_rs", 0) + 1
            return out
        rc = oplib.kernels().ff_gemm_rs(*self.arena.args(), oplib.ptr(x), oplib.ptr(w), oplib.ptr(out), m, n, k,
                                        x.stride(0), w.stride(0), oplib.ptr(self.tile_counters),
                                        oplib.ptr(oplib.status_tensor(x.device)), oplib.stream_ptr())
        oplib.check(rc, "ff_gemm_rs")
        self.stats["gemm_rs"] += 1
        ops._count()
        return out

    def all_gather_rows(self, x_shard: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x_shard.shape[0] * self.size, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(out, x_shard.contiguous(), group=self.group)
        return out

    def all_gather_cat(self, x: torch.Tensor) -> torch.Tensor:
        """Concatenate equally-shaped shards along the last dim."""
        if self.size == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def argmax_merge(self, vals: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Merge vocabulary-parallel greedy candidates: (row max, global id) per rank -> global
        argmax with ties to the lower id."""
        rows = vals.numel()
        if self.fused and vals.is_cuda and rows * 8 <= self.arena.slot_bytes:
            pad = (rows + 3) // 4 * 4
            packed = torch.zeros(2 * pad, dtype=torch.int32, device=vals.device)
            packed[:rows] = vals.view(torch.int32)
            packed[pad: pad + rows] = ids
            gathered = torch.empty(self.size, 2 * pad, dtype=torch.int32, device=vals.device)
            lib = oplib.kernels()
            rc = lib.ff_allgather_push(*self.arena.args(), oplib.ptr(packed), oplib.ptr(gathered), packed.numel() * 4,
                                       oplib.ptr(oplib.status_tensor(vals.device)), oplib.stream_ptr())
            oplib.check(rc, "ff_allgather_push")
            all_vals = gathered[:, :rows].contiguous().view(torch.float32)
            all_ids = gathered[:, pad: pad + rows].contiguous()
            out = torch.empty(rows, dtype=torch.int32, device=vals.device)
            oplib.check(lib.ff_argmax_merge(oplib.ptr(all_vals), oplib.ptr(all_ids), oplib.ptr(out), self.size, rows,
                                            oplib.stream_ptr()), "ff_argmax_merge")
            ops._count(2)
            return out
        vs = [torch.empty_like(vals) for _ in range(self.size)]
        is_ = [torch.empty_like(ids) for _ in range(self.size)]
        dist.all_gather(vs, vals, group=self.group)
        dist.all_gather(is_, ids, group=self.group)
        v, i = torch.stack(vs), torch.stack(is_)
        best = v.max(0).values
        cand = torch.where(v == best[None], i, torch.full_like(i, 2 ** 31 - 1))
        return cand.min(0).values.to(torch.int32)

    def barrier(self) -> None:
        dist.barrier(self.group)
