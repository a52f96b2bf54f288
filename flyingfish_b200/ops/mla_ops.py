"""Multi-head latent attention operators: latent cache write, absorbed attention over the paged
latent cache, per-head batched projections. CUDA: ``csrc/mla.cu`` (+ the grouped tcgen05 GEMM for the
per-head W_UK / W_UV products); CPU: FP32 oracles."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_longlong

import torch

from . import _count, _require, workspace
from .lib import check, kernels, ptr, status_tensor, stream_ptr

F32 = torch.float32


def cache_write(c: torch.Tensor, k_rope: torch.Tensor, slots: torch.Tensor, cache: torch.Tensor) -> None:
    """cache: [blocks, 1, block_size, kv_lora + rope]; row r goes to ``slots[r]`` (negative skips)."""
    nb, _, bs, d = cache.shape
    if not c.is_cuda:
        ok = slots >= 0
        blk = torch.div(slots[ok], bs, rounding_mode="floor").long()
        off = (slots[ok] % bs).long()
        cache[blk, 0, off, :] = torch.cat([c, k_rope], dim=1)[ok].to(cache.dtype)
        return
    _require(c.shape[1] == 512 and k_rope.shape[1] == 64 and bs == 64 and d == 576, "MLA kernel: kv_lora 512 + rope 64")
    _require(c.stride(1) == 1 and k_rope.stride(1) == 1 and cache.is_contiguous(), "mla cache_write: layout")
    check(kernels().ff_mla_cache_write(ptr(c), ptr(k_rope), ptr(slots), ptr(cache), c.shape[0], c.stride(0),
                                       k_rope.stride(0), nb, ptr(status_tensor(c.device)), stream_ptr()), "ff_mla_cache_write")
    _count()


def attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
              q_lens: torch.Tensor, ctx_lens: torch.Tensor, max_q: int, max_ctx: int, scale: float, kv_lora: int
              ) -> torch.Tensor:
    """q: [rows, heads, kv_lora + rope] (absorbed queries). Returns out_lat [rows, heads, kv_lora]."""
    rows, heads, d = q.shape
    batch = block_table.shape[0]
    if not q.is_cuda:
        out = torch.zeros(rows, heads, kv_lora, dtype=q.dtype)
        bs = cache.shape[2]
        for b in range(batch):
            ql, ctx, qs = int(q_lens[b]), int(ctx_lens[b]), int(q_start[b])
            if ql == 0:
                continue
            nblk = (ctx + bs - 1) // bs
            kv = cache[block_table[b, :nblk].long(), 0].reshape(nblk * bs, d)[:ctx].to(F32)
            qq = q[qs: qs + ql].to(F32)
            s = torch.einsum("qhd,kd->hqk", qq, kv) * scale
            pos_q = torch.arange(ql)[:, None] + (ctx - ql)
            vis = torch.arange(ctx)[None, :] <= pos_q
            s = s.masked_fill(~vis[None], float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[qs: qs + ql] = torch.einsum("hqk,kd->qhd", p, kv[:, :kv_lora]).to(q.dtype)
        return out
    _require(d == 576 and kv_lora == 512 and q.is_contiguous(), "MLA kernel: contiguous [rows, heads, 576]")
    lib = kernels()
    po, pml = c_longlong(0), c_longlong(0)
    nsplit = lib.ff_mla_plan(batch, heads, max_q, max_ctx, ctypes.byref(po), ctypes.byref(pml))
    ws = workspace(q.device)
    part_o = ws.ensure("attn_o", po.value // 4) if nsplit > 1 else None
    part_ml = ws.ensure("attn_ml", pml.value // 4) if nsplit > 1 else None
    out = torch.empty(rows, heads, kv_lora, dtype=torch.bfloat16, device=q.device)
    rc = lib.ff_mla_attn(ptr(q), ptr(cache), ptr(block_table), ptr(q_start), ptr(q_lens), ptr(ctx_lens), ptr(out),
                         ptr(part_o), ptr(part_ml), batch, heads, max_q, block_table.shape[1], cache.shape[0], nsplit,
                         c_float(scale), ptr(status_tensor(q.device)), stream_ptr())
    check(rc, "ff_mla_attn")
    _count(2 if nsplit > 1 else 1)
    return out


def per_head_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y[r, h] = x[r, h] @ w[h].T`` for x [rows, heads, k], w [heads, n, k] -> [rows, heads, n]."""
    rows, heads, k = x.shape
    n = w.shape[1]
    if not x.is_cuda:
        return torch.einsum("rhk,hnk->rhn", x.to(torch.float64), w.to(torch.float64)).to(x.dtype)
    from . import moe_cuda
    _require(n % 128 == 0 and k % 8 == 0, "per_head_linear: n % 128 == 0")
    pad = (rows + 15) // 16 * 16
    xs = torch.zeros(heads, pad, k, dtype=torch.bfloat16, device=x.device)
    xs[:, :rows] = x.permute(1, 0, 2)
    seg_off = (torch.arange(heads + 1, dtype=torch.int32, device=x.device) * pad)
    counts = torch.full((heads,), rows, dtype=torch.int32, device=x.device)
    y = moe_cuda.grouped_gemm(xs.view(heads * pad, k), w.contiguous(), seg_off, counts, heads * pad, epi=0)
    return y.view(heads, pad, n)[:, :rows].permute(1, 0, 2).contiguous()
