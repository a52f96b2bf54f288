"""DSA (top-k sparse attention with a pooled indexer) operators. CUDA: ``csrc/dsa.cu`` and the gathered form
of ``csrc/latent.cu``; CPU: FP32 oracles restating the same arithmetic (reference: kernels/dsa.cu:99-425,
kernels/dsa_topk.cuh).

Storage is contiguous per sequence: token ``t`` of sequence ``s`` is global row ``seq_start[s] + t`` of
``latent`` [rows, D], ``idx_key`` [rows, 128] and ``pool_logit`` [rows, 128]; pool ``p`` of the sequence is
global pool row ``pool_start[s] + p`` and covers tokens ``4p .. 4p+3``.
"""
from __future__ import annotations

import math
from ctypes import c_float

import torch

from . import _count, _require, workspace
from .lib import check, kernels, ptr, status_tensor, stream_ptr

POOL, DIM, HEADS, TOPK = 4, 128, 32, 512
BF16 = torch.bfloat16


def _r(x: torch.Tensor) -> torch.Tensor:
    return x.to(BF16).float()


def pool_keys(idx_key: torch.Tensor, pool_logit: torch.Tensor, ape: torch.Tensor, seq_start: torch.Tensor,
              seq_len: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (pooled [sum(len // 4), 128] bf16, pool_start [sequences] int32)."""
    npool = (seq_len // POOL).to(torch.int32)
    pool_start = (torch.cumsum(npool, 0) - npool).to(torch.int32)
    total = int(npool.sum().item())
    pooled = torch.zeros(max(total, 1), DIM, dtype=BF16, device=idx_key.device)
    if total == 0:
        return pooled[:0], pool_start
    if not idx_key.is_cuda:
        for s in range(seq_len.numel()):
            for p in range(int(npool[s])):
                t0 = int(seq_start[s]) + p * POOL
                lg = pool_logit[t0: t0 + POOL].float() + ape.float()
                pr = _r(torch.softmax(lg, dim=0))
                pooled[int(pool_start[s]) + p] = _r(pr * idx_key[t0: t0 + POOL].float()).sum(0).to(BF16)
        return pooled, pool_start
    _require(idx_key.is_contiguous() and pool_logit.is_contiguous() and ape.is_contiguous(), "dsa pool: layout")
    rc = kernels().ff_dsa_pool(ptr(idx_key), ptr(pool_logit), ptr(ape), ptr(seq_start), ptr(seq_len), ptr(pool_start),
                               ptr(pooled), seq_len.numel(), int(npool.max().item()), stream_ptr())
    check(rc, "ff_dsa_pool")
    _count()
    return pooled, pool_start


def index_scores_ref(q: torch.Tensor, w: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
    """q [32, 128], w [32], pooled [P, 128] -> [P] FP32."""
    dots = q.float() @ pooled.float().t()                           # [32, P]
    return (torch.relu(dots * 0.0883883461356163) * (w.float() * 0.1767766922712326)[:, None]).sum(0)


def index_topk(q: torch.Tensor, w: torch.Tensor, pooled: torch.Tensor, pool_base: torch.Tensor, n_cand: torch.Tensor,
               k: int = TOPK) -> tuple[torch.Tensor, torch.Tensor]:
    """q [rows, 32, 128] bf16, w [rows, 32] bf16; row r scores pools pool_base[r] .. +n_cand[r].
    -> (selected [rows, k] int32 sequence-local pool ids, score descending, ties to the lower id, -1 padded;
    scores [rows, k] FP32)."""
    rows = q.shape[0]
    if not q.is_cuda:
        sel = torch.full((rows, k), -1, dtype=torch.int32)
        val = torch.full((rows, k), -math.inf)
        for r in range(rows):
            n = int(n_cand[r])
            if n == 0:
                continue
            sc = index_scores_ref(q[r], w[r], pooled[int(pool_base[r]): int(pool_base[r]) + n])
            order = sorted(range(n), key=lambda i: (-float(sc[i]), i))[:k]
            sel[r, : len(order)] = torch.tensor(order, dtype=torch.int32)
            val[r, : len(order)] = sc[order]
        return sel, val
    _require(q.is_contiguous() and w.is_contiguous() and pooled.is_contiguous() and k <= TOPK, "dsa index_topk: layout")
    max_cand = int(n_cand.max().item()) if rows else 0
    ld = max(max_cand, 1)
    scores = workspace(q.device).ensure("dsa_scores", rows * ld)[: rows * ld].view(rows, ld)
    sel = torch.empty(rows, k, dtype=torch.int32, device=q.device)
    val = torch.empty(rows, k, dtype=torch.float32, device=q.device)
    rc = kernels().ff_dsa_index_topk(ptr(q), ptr(w), ptr(pooled), ptr(pool_base), ptr(n_cand), ptr(scores), ld, rows,
                                     max_cand, k, ptr(sel), ptr(val), stream_ptr())
    check(rc, "ff_dsa_index_topk")
    _count(2)
    return sel, val


def expand(selected: torch.Tensor, seq_base: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """-> indices [rows, k*4 + 3] int32 global token rows (-1 = unused): tokens of the selected pools, then the
    tokens after the last complete pool up to ``pos`` (sequence-local, inclusive)."""
    rows, k = selected.shape
    width = k * POOL + POOL - 1
    if not selected.is_cuda:
        out = torch.full((rows, width), -1, dtype=torch.int32)
        for r in range(rows):
            npools = (int(pos[r]) + 1) // POOL
            nsel = min(k, npools)
            for j in range(nsel):
                p = int(selected[r, j])
                if p >= 0:
                    out[r, j * POOL: (j + 1) * POOL] = torch.arange(4, dtype=torch.int32) + int(seq_base[r]) + p * POOL
            ntail = int(pos[r]) + 1 - npools * POOL
            out[r, nsel * POOL: nsel * POOL + ntail] = torch.arange(ntail, dtype=torch.int32) + int(seq_base[r]) + npools * POOL
        return out
    out = torch.empty(rows, width, dtype=torch.int32, device=selected.device)
    rc = kernels().ff_dsa_expand(ptr(selected), ptr(seq_base), ptr(pos), rows, k, ptr(out), stream_ptr())
    check(rc, "ff_dsa_expand")
    _count()
    return out


def sparse_attention(q: torch.Tensor, latent: torch.Tensor, indices: torch.Tensor, sink: torch.Tensor,
                     scale: float | None = None) -> torch.Tensor:
    """q [rows, heads, D] bf16 (absorbed queries), latent [tokens, D] bf16 (key = value), indices [rows, W],
    sink [heads] f32 -> out [rows, heads, D]: soft-max over the selected rows with the sink logit in the
    denominator only (blocked in 64 keys, P rounded to BF16, see ``latent_ops``)."""
    rows, heads, d = q.shape
    scale = scale if scale is not None else d ** -0.5
    if not q.is_cuda:
        out = torch.zeros(rows, heads, d)
        for r in range(rows):
            idx = indices[r]
            kk = torch.zeros(idx.numel(), d)
            live = idx >= 0
            kk[live] = latent[idx[live].long()].float()
            s = (q[r].float() @ kk.t()) * scale
            s[:, ~live] = -math.inf
            acc = torch.zeros(heads, d); m_run = torch.full((heads,), -math.inf); ssum = torch.zeros(heads)
            for t in range(0, idx.numel(), 64):
                blk = s[:, t: t + 64]
                bmax = torch.maximum(m_run, blk.max(dim=1).values)
                seen = m_run > -math.inf
                rsc = torch.where(seen, torch.exp(m_run - bmax), torch.ones(heads))
                acc *= rsc[:, None]; ssum *= rsc
                p = torch.where(blk > -math.inf, torch.exp(blk - bmax[:, None]), torch.zeros_like(blk))
                p = torch.nan_to_num(p, nan=0.0)
                ssum += p.sum(1)
                acc += p.to(BF16).float() @ kk[t: t + 64]
                m_run = bmax
            tail = torch.where(m_run > -math.inf, torch.exp(sink.float() - m_run), torch.ones(heads))
            out[r] = (acc / (ssum + tail)[:, None]).to(BF16).float()
        return out.to(BF16)
    _require(q.is_contiguous() and latent.is_contiguous() and indices.is_contiguous() and d % 64 == 0 and d <= 512,
             "dsa sparse_attention: layout")
    out = torch.empty_like(q)
    rc = kernels().ff_latent_sparse_attention(ptr(q), ptr(latent), ptr(indices), ptr(sink), ptr(out), rows, heads, d,
                                              indices.shape[1], latent.shape[0], c_float(scale),
                                              ptr(status_tensor(q.device)), stream_ptr())
    check(rc, "ff_latent_sparse_attention")
    _count()
    return out


class StateSnapshot:
    """Rows of a set of per-token state tables, saved by :func:`checkpoint_save`."""
    def __init__(self, tables, rows, data, meta):
        self.tables, self.rows, self.data, self.meta = tables, rows, data, meta


def _table_meta(tables: list[torch.Tensor]):
    dev = tables[0].device
    vecs = [t.shape[1] * t.element_size() // 16 for t in tables]
    ptrs = torch.tensor([t.data_ptr() for t in tables], dtype=torch.int64, device=dev)
    return ptrs, torch.tensor(vecs, dtype=torch.int32, device=dev), torch.tensor([t.shape[0] for t in tables],
                                                                                   dtype=torch.int32, device=dev), max(vecs)


def checkpoint_save(tables: list[torch.Tensor], rows: torch.Tensor) -> StateSnapshot:
    """Save rows ``rows`` (int32 [n], global row ids) of every 2-D table (any dtype, row bytes a multiple of 16) so that
    a speculative round that overwrites them can be rolled back: one launch for all tables."""
    n = rows.numel()
    if not tables[0].is_cuda:
        return StateSnapshot(tables, rows.clone(), [t[rows.long()].clone() for t in tables], None)
    for t in tables:
        _require(t.dim() == 2 and t.is_contiguous() and (t.shape[1] * t.element_size()) % 16 == 0, "checkpoint: table layout")
    meta = _table_meta(tables)
    ptrs, vecs, trows, mx = meta
    data = torch.empty(len(tables) * n * mx * 16, dtype=torch.uint8, device=rows.device)
    rows = rows.to(torch.int32).contiguous()
    rc = kernels().ff_dsa_checkpoint(ptr(ptrs), ptr(vecs), ptr(trows), len(tables), ptr(rows), n, ptr(data), mx, 0,
                                     ptr(status_tensor(rows.device)), stream_ptr())
    check(rc, "ff_dsa_checkpoint(save)")
    _count()
    return StateSnapshot(tables, rows, data, meta)


def checkpoint_restore(snap: StateSnapshot) -> None:
    """Write the saved rows back into their tables."""
    if snap.meta is None:
        for t, d in zip(snap.tables, snap.data):
            t[snap.rows.long()] = d
        return
    ptrs, vecs, trows, mx = snap.meta
    rc = kernels().ff_dsa_checkpoint(ptr(ptrs), ptr(vecs), ptr(trows), len(snap.tables), ptr(snap.rows), snap.rows.numel(),
                                     ptr(snap.data), mx, 1, ptr(status_tensor(snap.rows.device)), stream_ptr())
    check(rc, "ff_dsa_checkpoint(restore)")
    _count()
