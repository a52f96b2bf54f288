"""Row-flattened forward batches.

A forward pass processes ``rows`` token rows that belong to ``batch`` sequences. Prefill chunks
contribute ``q_len`` consecutive rows per sequence, decode contributes ``nq`` rows per sequence
(1 for plain decode, k+1 for speculative verification). All per-step metadata lives in ONE int32
buffer so a step needs a single host-to-device copy from pinned memory; the layout is fixed per
(batch capacity, row capacity, block-table width), which also makes it a stable input of a CUDA
graph. The reference's equivalent is the 32-byte ``SequenceMeta`` record and row work layout for
its single sequence (src/work_layout.rs:57-228).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class BatchLayout:
    """Offsets (in int32 elements) of each field inside the packed metadata buffer."""
    max_batch: int
    max_rows: int
    max_blocks: int
    max_groups: int = 0               # > 0: the sequences may have sealed 8-bit groups (kv_start + group table fields)

    def __post_init__(self) -> None:
        o = 0
        self.ids = o; o += self.max_rows
        self.positions = o; o += self.max_rows
        self.slots = o; o += self.max_rows
        self.q_start = o; o += self.max_batch
        self.q_lens = o; o += self.max_batch
        self.ctx_lens = o; o += self.max_batch
        self.n_logit = max(self.max_batch * 8, self.max_rows)   # verify rows / all-row logits
        self.logit_rows = o; o += self.n_logit
        self.block_table = o; o += self.max_batch * self.max_blocks
        self.tree_mask = o; o += 2 * self.max_rows        # int64 per row, stored as two int32
        self.row_start = o; o += self.max_batch + 1          # first row of every sequence, then the row count
        self.state_slots = o; o += self.max_batch            # per-sequence state slot (models with recurrent state)
        self.kv_start = o; o += self.max_batch if self.max_groups else 0
        self.groups = o; o += self.max_batch * self.max_groups
        self.total = o


class ForwardBatch:
    """Device view of a packed metadata buffer plus the host-side scalars the launchers need."""

    def __init__(self, layout: BatchLayout, device: torch.device | str, pinned: bool | None = None):
        self.layout = layout
        self.device = torch.device(device)
        pin = self.device.type == "cuda" if pinned is None else pinned
        self.host = torch.zeros(layout.total, dtype=torch.int32, pin_memory=pin)
        self.dev = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
        # host-side scalars of the current step
        self.batch = 0
        self.rows = 0
        self.nq = 1
        self.is_decode = True
        self.max_q_len = 1
        self.max_ctx = 0
        self.n_logit_rows = 0
        self.use_tree_mask = False
        self._bt_sig: list = []           # block list last written to each block-table row of the host buffer

    # -- device views (fixed addresses) ------------------------------------------------------
    def _v(self, off: int, n: int) -> torch.Tensor:
        return self.dev[off: off + n]

    @property
    def ids(self) -> torch.Tensor: return self._v(self.layout.ids, self.rows)
    @property
    def positions(self) -> torch.Tensor: return self._v(self.layout.positions, self.rows)
    @property
    def slots(self) -> torch.Tensor: return self._v(self.layout.slots, self.rows)
    @property
    def q_start(self) -> torch.Tensor: return self._v(self.layout.q_start, self.batch)
    @property
    def q_lens(self) -> torch.Tensor: return self._v(self.layout.q_lens, self.batch)
    @property
    def ctx_lens(self) -> torch.Tensor: return self._v(self.layout.ctx_lens, self.batch)
    @property
    def logit_rows(self) -> torch.Tensor: return self._v(self.layout.logit_rows, self.n_logit_rows)
    @property
    def block_table(self) -> torch.Tensor:
        L = self.layout
        return self.dev[L.block_table: L.block_table + L.max_batch * L.max_blocks].view(L.max_batch, L.max_blocks)[: self.batch]
    @property
    def row_start(self) -> torch.Tensor: return self._v(self.layout.row_start, self.batch + 1)
    @property
    def state_slots_dev(self) -> torch.Tensor: return self._v(self.layout.state_slots, self.batch)
    @property
    def kv_start(self) -> torch.Tensor | None:
        L = self.layout
        return self._v(L.kv_start, self.batch) if L.max_groups else None
    @property
    def group_table(self) -> torch.Tensor | None:
        L = self.layout
        if not L.max_groups:
            return None
        return self.dev[L.groups: L.groups + L.max_batch * L.max_groups].view(L.max_batch, L.max_groups)[: self.batch]
    @property
    def tree_mask(self) -> torch.Tensor | None:
        if not self.use_tree_mask:
            return None
        L = self.layout
        return self.dev[L.tree_mask: L.tree_mask + 2 * self.rows].view(torch.int64)

    # -- host fill -----------------------------------------------------------------------------
    def fill(self, *, ids, positions, slots, q_lens, ctx_lens, block_rows, logit_rows, is_decode: bool, nq: int = 1,
             tree_mask=None, kv_start=None, group_rows=None, state_slots=None) -> None:
        """Write one step's metadata into the pinned host buffer (lists of ints)."""
        L = self.layout
        h = self.host
        rows, batch = len(ids), len(q_lens)
        assert rows <= L.max_rows and batch <= L.max_batch, "batch exceeds the layout capacity"
        assert len(logit_rows) <= L.n_logit
        self.rows, self.batch, self.nq, self.is_decode = rows, batch, nq, is_decode
        h[L.ids: L.ids + rows] = torch.as_tensor(ids, dtype=torch.int32)
        h[L.positions: L.positions + rows] = torch.as_tensor(positions, dtype=torch.int32)
        h[L.slots: L.slots + rows] = torch.as_tensor(slots, dtype=torch.int32)
        ql = torch.as_tensor(q_lens, dtype=torch.int32)
        h[L.q_lens: L.q_lens + batch] = ql
        qs = torch.zeros(batch, dtype=torch.int32)
        if batch > 1:
            qs[1:] = torch.cumsum(ql, 0)[:-1].to(torch.int32)
        h[L.q_start: L.q_start + batch] = qs
        h[L.row_start: L.row_start + batch] = qs
        h[L.row_start + batch] = int(ql.sum()) if batch else 0
        if state_slots is not None:
            h[L.state_slots: L.state_slots + batch] = torch.as_tensor(state_slots, dtype=torch.int32)
            self.state_slots = list(state_slots)
        h[L.ctx_lens: L.ctx_lens + batch] = torch.as_tensor(ctx_lens, dtype=torch.int32)
        self.n_logit_rows = len(logit_rows)
        h[L.logit_rows: L.logit_rows + len(logit_rows)] = torch.as_tensor(logit_rows, dtype=torch.int32)
        bt = h[L.block_table: L.block_table + L.max_batch * L.max_blocks].view(L.max_batch, L.max_blocks)
        # a decode batch keeps the same sequences in the same rows for many steps and a block list changes only when
        # a sequence crosses a block boundary: rows whose list is unchanged are not rewritten (the pinned buffer
        # still holds them), which takes most of the host time out of a decode step
        sig = self._bt_sig
        for i, row in enumerate(block_rows):
            t = tuple(row)
            if i < len(sig) and sig[i] == t:
                continue
            n = len(t)
            assert n <= L.max_blocks
            if n:
                bt[i, :n] = torch.as_tensor(t, dtype=torch.int32)
            if i < len(sig):
                sig[i] = t
            else:
                sig.extend([None] * (i - len(sig)) + [t])
        if L.max_groups:
            ks = torch.zeros(batch, dtype=torch.int32)
            if kv_start is not None:
                ks[: len(kv_start)] = torch.as_tensor(kv_start, dtype=torch.int32)
            h[L.kv_start: L.kv_start + batch] = ks
            gt = h[L.groups: L.groups + L.max_batch * L.max_groups].view(L.max_batch, L.max_groups)
            for i, row in enumerate(group_rows or []):
                if row:
                    assert len(row) <= L.max_groups
                    gt[i, : len(row)] = torch.as_tensor(row, dtype=torch.int32)
        self.max_q_len = int(max(q_lens)) if batch else 0
        self.max_ctx = int(max(ctx_lens)) if batch else 0
        self.use_tree_mask = tree_mask is not None
        if tree_mask is not None:
            # bit 63 may be set: store the two's complement value
            tm = torch.as_tensor([m - (1 << 64) if m >= (1 << 63) else m for m in tree_mask], dtype=torch.int64)
            h[L.tree_mask: L.tree_mask + 2 * rows].view(torch.int64)[:] = tm

    def h2d_bytes(self) -> int:
        return self.layout.total * 4

    def upload(self) -> None:
        """One host-to-device copy of the whole packed buffer."""
        self.dev.copy_(self.host, non_blocking=True)
