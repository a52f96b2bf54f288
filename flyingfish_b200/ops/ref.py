"""Plain PyTorch oracles for every operator (run on CPU, FP32 math, explicit rounding points).

These are the numerics contracts the CUDA kernels are tested against, and they are also the
implementation the framework uses when it runs on a CPU (the tiny-MoE host configuration). The
rounding points follow the reference's kernel contracts:

* residual add + RMSNorm rounds the sum to the storage dtype before normalising
  (kernels/norm.cu:8-21),
* RoPE rounds cos/sin to BF16 and rotates in BF16 arithmetic (kernels/rope_kv.cu:34-43),
* SwiGLU has numbered rounding modes (kernels/act.cu:220-262),
* argmax and top-k break ties towards the lower index (kernels/sample.cu:3-6,
  kernels/moe_route.cu:17-22),
* MoE combine sums contributions in ascending expert id in FP32 and rounds once
  (kernels/moe_combine.cu:1-10).
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32


def _r(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round an FP32 tensor to `dtype` and come back to FP32."""
    return x.to(dtype).to(F32)


# ------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------
def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``y = x @ w.T``, one rounding to the output dtype. The products are accumulated in FP64 so
    the oracle does not depend on how a BLAS blocks the sum for a given batch size (results are
    batch-invariant, as the device kernels' are)."""
    y = x.to(torch.float64) @ w.to(torch.float64).t()
    return y.to(out_dtype or x.dtype)


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, mode: int = 0) -> torch.Tensor:
    """Fused gate/up projection + SwiGLU for a weight whose rows are interleaved per 64:
    rows [128*t, 128*t+64) are gate rows for outputs [64*t, 64*t+64), the next 64 the
    matching up rows (one 128-row weight tile of the decode GEMM holds both)."""
    y = (x.to(torch.float64) @ w_interleaved.to(torch.float64).t()).to(F32)
    n = y.shape[-1]
    y = y.view(*y.shape[:-1], n // 128, 2, 64)
    gate, up = y[..., 0, :], y[..., 1, :]
    gu = torch.cat([gate.reshape(*y.shape[:-3], -1), up.reshape(*y.shape[:-3], -1)], dim=-1).to(x.dtype)
    return silu_mul(gu, mode=mode)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Build the per-64 interleaved [2f, h] weight used by the fused SwiGLU GEMM epilogues."""
    f, h = w_gate.shape
    assert f % 64 == 0
    g = w_gate.view(f // 64, 1, 64, h)
    u = w_up.view(f // 64, 1, 64, h)
    return torch.cat([g, u], dim=1).reshape(2 * f, h).contiguous()


# ------------------------------------------------------------------------------------------
# norms / embedding
# ------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, unit_offset: bool = False) -> torch.Tensor:
    xf = x.to(F32)
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.to(F32) + (1.0 if unit_offset else 0.0)
    return (xf * rstd * wf).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float,
                unit_offset: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (new residual, normalised). The sum is rounded to the storage dtype first and the
    rounded value is what gets normalised."""
    new_res = (res.to(F32) + x.to(F32)).to(res.dtype)
    return new_res, rmsnorm(new_res, w, eps, unit_offset)


def embed_rmsnorm(ids: torch.Tensor, table: torch.Tensor, w: torch.Tensor, eps: float,
                  unit_offset: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    x = table[ids.long()]
    return x, rmsnorm(x, w, eps, unit_offset)


# ------------------------------------------------------------------------------------------
# RoPE
# ------------------------------------------------------------------------------------------
def rope_inv_freq(rot_dim: int, theta: float) -> torch.Tensor:
    i = torch.arange(0, rot_dim // 2, dtype=F32)
    return 1.0 / torch.pow(torch.tensor(theta, dtype=F32), (2.0 * i) / rot_dim)


def rope_rotate_half(x: torch.Tensor, positions: torch.Tensor, theta: float, rot_dim: int | None = None,
                     inv_freq: torch.Tensor | None = None) -> torch.Tensor:
    """x: [rows, heads, dim]. Rotate-half RoPE. For BF16 inputs cos/sin are rounded to BF16 and
    every product and sum rounds to BF16; FP32 inputs use FP32 arithmetic."""
    dim = x.shape[-1]
    rot_dim = rot_dim or dim
    half, rhalf = dim // 2, rot_dim // 2
    inv = inv_freq if inv_freq is not None else rope_inv_freq(rot_dim, theta)
    ang = positions.to(F32)[:, None] * inv.to(F32)[None, :]          # [rows, rhalf]
    cos, sin = torch.cos(ang), torch.sin(ang)
    dt = x.dtype
    lo = x[..., :half].to(F32).clone()
    hi = x[..., half:].to(F32).clone()
    x1, x2 = lo[..., :rhalf], hi[..., :rhalf]
    if dt == torch.float32:
        c, s = cos[:, None, :], sin[:, None, :]
        o1 = x1 * c - x2 * s
        o2 = x2 * c + x1 * s
    else:
        c, s = _r(cos, dt)[:, None, :], _r(sin, dt)[:, None, :]
        o1 = _r(_r(x1 * c, dt) - _r(x2 * s, dt), dt)
        o2 = _r(_r(x2 * c, dt) + _r(x1 * s, dt), dt)
    lo[..., :rhalf] = o1
    hi[..., :rhalf] = o2
    return torch.cat([lo, hi], dim=-1).to(dt)


def rope_kv_paged(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor,
                  vcache: torch.Tensor, hq: int, hkv: int, dim: int, theta: float, rot_dim: int | None = None,
                  inv_freq: torch.Tensor | None = None) -> None:
    """In place: rotates Q and K inside the packed rows, writes K and V to the paged cache
    ``[blocks, hkv, block_size, dim]`` at ``slots`` (slot = block * block_size + offset, < 0 skips)."""
    rows = qkv.shape[0]
    bs = kcache.shape[2]
    q = qkv[:, : hq * dim].reshape(rows, hq, dim)
    k = qkv[:, hq * dim: (hq + hkv) * dim].reshape(rows, hkv, dim)
    v = qkv[:, (hq + hkv) * dim: (hq + 2 * hkv) * dim].reshape(rows, hkv, dim)
    q2 = rope_rotate_half(q, positions, theta, rot_dim, inv_freq)
    k2 = rope_rotate_half(k, positions, theta, rot_dim, inv_freq)
    qkv[:, : hq * dim] = q2.reshape(rows, -1)
    qkv[:, hq * dim: (hq + hkv) * dim] = k2.reshape(rows, -1)
    ok = slots >= 0
    blk = torch.div(slots[ok], bs, rounding_mode="floor").long()
    off = (slots[ok] % bs).long()
    kcache[blk, :, off, :] = k2[ok].to(kcache.dtype)
    vcache[blk, :, off, :] = v[ok].to(vcache.dtype)


# ------------------------------------------------------------------------------------------
# activations
# ------------------------------------------------------------------------------------------
def silu_mul(gu: torch.Tensor, mode: int = 0, limit: float = 0.0) -> torch.Tensor:
    """gu: [..., 2f] = gate | up. Modes: 0 = silu rounded then product rounded, 1 = single rounding,
    2 = tanh-GELU twice rounded, 4 = clamped SwiGLU in FP32 (gate <= limit, |up| <= limit)."""
    f = gu.shape[-1] // 2
    dt = gu.dtype
    g, u = gu[..., :f].to(F32), gu[..., f:].to(F32)
    if mode == 0:
        y = _r(g * torch.sigmoid(g), dt) * u
    elif mode == 1:
        y = g * torch.sigmoid(g) * u
    elif mode == 2:
        t = torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))
        y = _r(0.5 * g * (1 + t), dt) * u
    elif mode == 4:
        g = torch.clamp(g, max=limit)
        u = torch.clamp(u, min=-limit, max=limit)
        y = g * torch.sigmoid(g) * u
    else:
        raise ValueError(f"unknown SwiGLU mode {mode}")
    return y.to(dt)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return (cap * torch.tanh(x.to(F32) / cap)).to(x.dtype)


# ------------------------------------------------------------------------------------------
# attention over the paged cache
# ------------------------------------------------------------------------------------------
def gather_kv(cache: torch.Tensor, block_table_row: torch.Tensor, ctx: int) -> torch.Tensor:
    """cache [blocks, hkv, bs, dim] -> [ctx, hkv, dim] for one sequence."""
    bs = cache.shape[2]
    nblk = (ctx + bs - 1) // bs
    blocks = cache[block_table_row[:nblk].long()]             # [nblk, hkv, bs, dim]
    return blocks.permute(0, 2, 1, 3).reshape(nblk * bs, cache.shape[1], cache.shape[3])[:ctx]


def attention_paged(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    q_start: torch.Tensor, q_lens: torch.Tensor, ctx_lens: torch.Tensor, hq: int, hkv: int,
                    dim: int, scale: float, tree_mask: torch.Tensor | None = None, window: int = 0,
                    sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of packed query rows against the paged cache. ``sinks`` (float [hq]): learnable soft-max, one
    extra logit per head that takes probability mass but contributes no value.

    q: [rows, >= hq*dim] (head h at columns h*dim). Sequence b owns rows
    ``q_start[b] : q_start[b]+q_lens[b]`` and ``ctx_lens[b]`` cached keys; its query i sits at
    position ``ctx - q_len + i``. ``tree_mask`` (int64 [B, q_len]) replaces causality inside the
    last q_len positions by an ancestor bit set. Returns [rows, hq*dim]."""
    rows = q.shape[0]
    out = torch.zeros(rows, hq * dim, dtype=q.dtype, device=q.device)
    g = hq // hkv
    for b in range(block_table.shape[0]):
        ql, ctx, qs = int(q_lens[b]), int(ctx_lens[b]), int(q_start[b])
        if ql == 0:
            continue
        k = gather_kv(kcache, block_table[b], ctx).to(F32)    # [ctx, hkv, dim]
        v = gather_kv(vcache, block_table[b], ctx).to(F32)
        qb = q[qs: qs + ql, : hq * dim].reshape(ql, hq, dim).to(F32)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", qb, k) * scale
        pos_q = torch.arange(ql)[:, None] + (ctx - ql)
        pos_k = torch.arange(ctx)[None, :]
        vis = pos_k <= pos_q if window >= 0 else torch.ones(ql, ctx, dtype=torch.bool)   # window < 0: bidirectional
        if window > 0:
            vis &= pos_k > pos_q - window
        if tree_mask is not None:
            tail = ctx - ql
            bits = tree_mask[b, :ql].to(torch.int64)
            rel = torch.arange(ql)
            anc = ((bits[:, None] >> rel[None, :]) & 1).bool()  # [q, tail keys]
            vis[:, tail:] &= anc
        s = s.masked_fill(~vis[None].to(s.device), float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks.to(F32)[:, None, None].expand(hq, ql, 1)], dim=-1)
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        if sinks is not None:
            p = p[..., :-1]
        o = torch.einsum("hqk,khd->qhd", p, v)
        out[qs: qs + ql] = o.reshape(ql, hq * dim).to(q.dtype)
    return out


# ------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------
def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """Greedy ids; ties go to the lower index."""
    lf = logits.to(F32)
    mx = lf.max(dim=-1, keepdim=True).values
    idx = torch.arange(lf.shape[-1], device=lf.device).expand_as(lf)
    big = torch.full_like(idx, lf.shape[-1])
    return torch.where(lf == mx, idx, big).min(dim=-1).values.to(torch.int32)


def philox4x32_10(key: tuple[int, int], ctr: tuple[int, int, int, int]) -> tuple[int, int, int, int]:
    """Philox4x32-10 block function (host reference of the device generator)."""
    m0, m1, w0, w1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    k0, k1 = key
    c0, c1, c2, c3 = ctr
    mask = 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c3 ^ k1) & mask, p0 & mask
        k0, k1 = (k0 + w0) & mask, (k1 + w1) & mask
    return c0, c1, c2, c3


def philox_uniform(n: int, seed: int, offset: int = 0) -> torch.Tensor:
    out = []
    for i in range((n + 3) // 4):
        c = offset + i
        r = philox4x32_10((seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF), (c & 0xFFFFFFFF, (c >> 32) & 0xFFFFFFFF, 0, 0))
        out.extend(((v >> 8) + 0.5) / 16777216.0 for v in r)
    return torch.tensor(out[:n], dtype=F32)


def sampling_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, rep_penalty: float = 1.0,
                   history: torch.Tensor | None = None) -> torch.Tensor:
    """Probabilities after repetition penalty, temperature, top-k and top-p for one row
    (src/sampling.rs:4-105 of the reference): the kept set is the smallest prefix of the
    descending order whose mass reaches top_p, capped at top_k elements, renormalised."""
    lg = logits.to(F32).clone()
    if history is not None and rep_penalty != 1.0:
        ids = history[history >= 0].long().unique()
        v = logits.to(F32)[ids]
        lg[ids] = torch.where(v > 0, v / rep_penalty, v * rep_penalty)
    p = torch.softmax(lg / temperature, dim=-1)
    order = torch.argsort(p, descending=True, stable=True)
    sp = p[order]
    csum = torch.cumsum(sp, 0)
    keep_n = int((csum < top_p).sum().item()) + 1
    if top_k > 0:
        keep_n = min(keep_n, top_k)
    keep_n = min(keep_n, p.numel())
    thr = sp[keep_n - 1]
    kept = p >= thr
    out = torch.where(kept, p, torch.zeros_like(p))
    return out / out.sum()


def sample_row(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, step: int, row: int,
               rep_penalty: float = 1.0, history: torch.Tensor | None = None) -> int:
    p = sampling_probs(logits, temperature, top_k, top_p, rep_penalty, history)
    r = philox4x32_10((seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF),
                      (step & 0xFFFFFFFF, (step >> 32) & 0xFFFFFFFF, row, 0))
    u = ((r[0] >> 8) + 0.5) / 16777216.0
    c = torch.cumsum(p, 0)
    idx = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=F32)).item())
    nz = torch.nonzero(p > 0).flatten()
    idx = min(idx, int(nz[-1]))
    while p[idx] == 0:
        idx += 1
    return idx


# ------------------------------------------------------------------------------------------
# MoE
# ------------------------------------------------------------------------------------------
def topk_lower_tie(scores: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Deterministic top-k along the last dim: larger score first, ties -> lower index."""
    n = scores.shape[-1]
    idx = torch.arange(n, device=scores.device).expand_as(scores)
    # sort by (-score, index): stable sort on descending scores keeps lower index first
    order = torch.argsort(scores, dim=-1, descending=True, stable=True)
    top = order[..., :k]
    return torch.gather(scores, -1, top), top


def moe_route(x: torch.Tensor, w_router: torch.Tensor, top_k: int, score: str = "softmax",
              bias: torch.Tensor | None = None, n_groups: int = 1, topk_groups: int = 1,
              routed_scaling: float = 1.0, renormalize: bool = True,
              logits_dtype: torch.dtype | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Router (kernels/moe_route.cu:1-30, 155-390 of the reference).

    * logits = x @ w_router.T accumulated in FP32, rounded to the activation dtype;
    * ``softmax``: softmax over all experts, top-k, renormalise;
    * ``sigmoid``: sigmoid scores, top-k, renormalise;
    * ``noaux``: selection on ``sigmoid(logit) + bias`` restricted to the ``topk_groups`` best of
      ``n_groups`` groups (group score = sum of its two best biased scores), weights are the
      unbiased scores renormalised and multiplied by ``routed_scaling``;
    * ``sqrt_softplus``: as ``noaux`` with scores ``sqrt(softplus(logit))`` (the DeepSeek-V4.1 router).
    Returns (weights FP32 [rows, k], ids int32 [rows, k]) with ids in selection order."""
    dt = logits_dtype or x.dtype
    logits = _r((x.to(torch.float64) @ w_router.to(torch.float64).t()).to(F32), dt)
    if score == "softmax":
        s = torch.softmax(logits, dim=-1)
        w, ids = topk_lower_tie(s, top_k)
    elif score == "sigmoid":
        s = torch.sigmoid(logits)
        w, ids = topk_lower_tie(s, top_k)
    elif score in ("noaux", "sqrt_softplus"):
        s = torch.sigmoid(logits) if score == "noaux" else torch.sqrt(torch.nn.functional.softplus(logits))
        sb = s + (bias.to(F32) if bias is not None else 0.0)
        rows, e = sb.shape
        if n_groups > 1:
            gs = sb.view(rows, n_groups, e // n_groups)
            gscore = topk_lower_tie(gs, 2)[0].sum(-1)                       # [rows, groups]
            _, gidx = topk_lower_tie(gscore, topk_groups)
            gmask = torch.zeros(rows, n_groups, dtype=torch.bool, device=x.device)
            gmask.scatter_(1, gidx, True)
            sel = sb.masked_fill(~gmask[:, :, None].expand_as(gs).reshape(rows, e), float("-inf"))
        else:
            sel = sb
        _, ids = topk_lower_tie(sel, top_k)
        w = torch.gather(s, -1, ids)
    else:
        raise ValueError(score)
    if renormalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    w = w * routed_scaling
    return w.to(F32), ids.to(torch.int32)


def expert_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, mode: int = 0) -> torch.Tensor:
    """One SwiGLU expert: down(silu_mul(x @ [gate|up].T))."""
    gu = linear(x, w_gate_up)
    return linear(silu_mul(gu, mode), w_down)


def moe_forward(x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, shared_gate_up: torch.Tensor | None = None,
                shared_down: torch.Tensor | None = None, mode: int = 0) -> torch.Tensor:
    """Routed experts + optional shared expert. Contributions of a row are rounded to the storage
    dtype, multiplied by their routing weight and summed in ascending expert id in FP32, the sum
    is rounded once; the shared expert is then added in the storage dtype."""
    rows, h = x.shape
    dt = x.dtype
    n_exp = w_gate_up.shape[0]
    contrib = torch.zeros(rows, ids.shape[1], h, dtype=F32, device=x.device)
    for e in range(n_exp):
        r, c = torch.nonzero(ids == e, as_tuple=True)
        if r.numel() == 0:
            continue
        y = expert_ffn(x[r], w_gate_up[e], w_down[e], mode).to(F32)
        contrib[r, c] = y * weights[r, c, None]
    order = torch.argsort(ids.long(), dim=-1, stable=True)                   # ascending expert id
    ordered = torch.gather(contrib, 1, order[:, :, None].expand_as(contrib))
    acc = torch.zeros(rows, h, dtype=F32, device=x.device)
    for j in range(ids.shape[1]):
        acc = acc + ordered[:, j]
    out = acc.to(dt)
    if shared_gate_up is not None:
        sh = expert_ffn(x, shared_gate_up, shared_down, mode)
        out = (out.to(F32) + sh.to(F32)).to(dt)
    return out
