"""Latent window attention operators (DeepSeek-V4.1-style mixer): per-32 E4M3/E8M0 quantisation,
the FP8 latent ring, and attention over the ring with a per-head sink, blocked soft-max with BF16 P
rounding and the inverse rotary on the output tail. CUDA: ``csrc/latent.cu``; CPU: FP32 oracles that
restate the same arithmetic (reference: kernels/latent_window_attention.cu:51-275, 307-348,
kernels/q38_contract.cuh:153-170)."""
from __future__ import annotations

import math
from ctypes import c_float, c_longlong

import torch

from . import _count, _require
from .lib import check, kernels, ptr, status_tensor, stream_ptr

BLOCK = 32          # codes per E8M0 scale
KEYS = 64           # keys per soft-max block


def quant32_ref(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """codes uint8 [..., D] (E4M3), scales uint8 [..., D/32] (E8M0 = exponent + 127)."""
    xf = x.float()
    g = xf.reshape(*xf.shape[:-1], xf.shape[-1] // BLOCK, BLOCK)
    amax = g.abs().amax(-1).clamp_min(1e-4)
    ratio = amax / 448.0
    mant, ex = torch.frexp(ratio)
    exponent = torch.where(mant == 0.5, ex - 1, ex)
    scale = torch.ldexp(torch.ones_like(ratio), exponent)
    codes = (g / scale[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes.reshape(x.shape), (exponent + 127).to(torch.uint8)


def dequant32(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    v = codes.view(torch.float8_e4m3fn).float()
    s = torch.ldexp(torch.ones(scales.shape, dtype=torch.float32, device=scales.device), scales.to(torch.int32) - 127)
    return (v.reshape(*scales.shape, BLOCK) * s[..., None]).reshape(codes.shape)


def act_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Linear layout: codes [rows, D], scales [rows, D/32]."""
    rows, d = x.shape
    if not x.is_cuda:
        return quant32_ref(x)
    _require(d % BLOCK == 0 and x.stride(1) == 1 and x.dtype == torch.bfloat16, "act_quant: bf16 rows, D % 32 == 0")
    codes = torch.empty(rows, d, dtype=torch.uint8, device=x.device)
    scales = torch.empty(rows, d // BLOCK, dtype=torch.uint8, device=x.device)
    rc = kernels().ff_latent_quant(ptr(x), ptr(codes), ptr(scales), None, None, c_longlong(rows), d, x.stride(0), 0, 0,
                                   ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_latent_quant")
    _count()
    return codes, scales


def ring_write(k: torch.Tensor, ring_ids: torch.Tensor, positions: torch.Tensor, codes: torch.Tensor,
               scales: torch.Tensor) -> None:
    """k [rows, D] post-RoPE rows; row r -> slot ``positions[r] % window`` of ring ``ring_ids[r]``.
    codes [rings, window, D] uint8, scales [rings, window, D/32] uint8."""
    rings, window, d = codes.shape
    if not k.is_cuda:
        c, s = quant32_ref(k)
        slot = positions.long() % window
        codes[ring_ids.long(), slot] = c
        scales[ring_ids.long(), slot] = s
        return
    _require(k.dtype == torch.bfloat16 and k.stride(1) == 1 and codes.is_contiguous() and scales.is_contiguous(),
             "ring_write: layout")
    rc = kernels().ff_latent_quant(ptr(k), ptr(codes), ptr(scales), ptr(ring_ids), ptr(positions), c_longlong(k.shape[0]), d,
                                   k.stride(0), window, rings, ptr(status_tensor(k.device)), stream_ptr())
    check(rc, "ff_latent_quant(ring)")
    _count()


def rotary_table(positions: torch.Tensor, rope_tail: int, theta: float, inverse: bool = False) -> torch.Tensor:
    """[B, rope_tail] FP32: (cos, sin) of the (inverse) angle of every adjacent pair of the tail."""
    i = torch.arange(rope_tail // 2, dtype=torch.float32, device=positions.device)
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32, device=positions.device), 2 * i / max(rope_tail, 1))
    ang = positions.float()[:, None] * inv[None, :]
    if inverse:
        ang = -ang
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).reshape(positions.shape[0], rope_tail).contiguous()


def inverse_rotary(positions: torch.Tensor, rope_tail: int, theta: float) -> torch.Tensor:
    return rotary_table(positions, rope_tail, theta, inverse=True)


def rope_pair_tail(x: torch.Tensor, cs: torch.Tensor, heads: int, d: int, rope_tail: int) -> None:
    """In place: rotate the adjacent pairs of the last ``rope_tail`` dims of every head of x [rows, heads * d] by the
    angles of ``cs`` [rows, rope_tail] (:func:`rotary_table`); FP32 arithmetic, one rounding to BF16."""
    rows = x.shape[0]
    if not x.is_cuda:
        v = x.view(rows, heads, d)[:, :, d - rope_tail:].float().reshape(rows, heads, rope_tail // 2, 2)
        c = cs.reshape(rows, 1, rope_tail // 2, 2)
        a, b = v[..., 0], v[..., 1]
        rot = torch.stack([a * c[..., 0] - b * c[..., 1], a * c[..., 1] + b * c[..., 0]], -1).reshape(rows, heads, rope_tail)
        x.view(rows, heads, d)[:, :, d - rope_tail:] = rot.to(x.dtype)
        return
    _require(x.dtype == torch.bfloat16 and x.stride(1) == 1 and cs.is_contiguous() and cs.dtype == torch.float32
             and cs.shape == (rows, rope_tail), "rope_pair_tail: layout")
    rc = kernels().ff_rope_pair_tail(ptr(x), ptr(cs), c_longlong(rows), heads, d, x.stride(0), rope_tail, stream_ptr())
    check(rc, "ff_rope_pair_tail")
    _count()


def window_attention_ref(q, codes, scales, ring_ids, positions, sink, inv_rot, rope_tail, scale, visible=None):
    b_, heads, d = q.shape
    window = codes.shape[1]
    visible = visible or window
    out = torch.zeros(b_, heads, d, dtype=torch.float32)
    for b in range(b_):
        pos, ring = int(positions[b]), int(ring_ids[b])
        nvis = min(pos + 1, visible)
        first = (pos + 1 - nvis) % window
        slots = [(first + j) % window for j in range(nvis)]
        k = dequant32(codes[ring, slots], scales[ring, slots]).to(torch.bfloat16).float()      # [nvis, d]
        s = (q[b].float() @ k.t()) * scale                                                     # [heads, nvis]
        acc = torch.zeros(heads, d)
        m_run = torch.full((heads,), -math.inf)
        ssum = torch.zeros(heads)
        for t in range(0, nvis, KEYS):
            blk = s[:, t: t + KEYS]
            bmax = torch.maximum(m_run, blk.max(dim=1).values)
            if t > 0:
                r = torch.exp(m_run - bmax)
                acc *= r[:, None]
                ssum *= r
            p = torch.exp(blk - bmax[:, None])
            ssum += p.sum(1)
            acc += p.to(torch.bfloat16).float() @ k[t: t + KEYS]
            m_run = bmax
        denom = ssum + torch.exp(sink.float() - m_run)
        o = (acc / denom[:, None]).to(torch.bfloat16).float()
        if rope_tail:
            tail = o[:, d - rope_tail:].reshape(heads, rope_tail // 2, 2)
            cs = inv_rot[b].reshape(rope_tail // 2, 2)
            a, c = tail[..., 0], tail[..., 1]
            o[:, d - rope_tail:] = torch.stack([a * cs[:, 0] - c * cs[:, 1], a * cs[:, 1] + c * cs[:, 0]], -1).reshape(heads, rope_tail)
        out[b] = o
    return out.to(torch.bfloat16)


def window_attention(q: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, ring_ids: torch.Tensor,
                     positions: torch.Tensor, sink: torch.Tensor, rope_tail: int, theta: float,
                     scale: float | None = None, visible: int | None = None, inv_rot: torch.Tensor | None = None
                     ) -> torch.Tensor:
    """q [B, heads, D] bf16 post-RoPE -> out [B, heads, D] bf16 (value = K content, inverse rotary on the
    last ``rope_tail`` dims). The query's own K row must already be in its ring. ``visible`` (default: the ring
    length) is the attention window; a ring longer than the window lets one launch serve the rows of a prefill chunk
    (row of position p in slot p % ring length, every query reading the ``visible`` positions up to its own).
    ``inv_rot``: the table of :func:`inverse_rotary` when the caller already has it."""
    b_, heads, d = q.shape
    rings, window, _ = codes.shape
    scale = scale if scale is not None else d ** -0.5
    visible = visible or window
    _require(0 < visible <= window, "window_attention: visible")
    if inv_rot is None:
        inv_rot = inverse_rotary(positions, rope_tail, theta) if rope_tail else torch.zeros(b_, 0, device=q.device)
    if not q.is_cuda:
        return window_attention_ref(q, codes, scales, ring_ids, positions, sink, inv_rot, rope_tail, scale, visible)
    _require(q.is_contiguous() and q.dtype == torch.bfloat16 and d % 64 == 0 and d <= 512, "window_attention: q layout")
    _require(codes.is_contiguous() and scales.is_contiguous() and sink.dtype == torch.float32, "window_attention: ring layout")
    out = torch.empty_like(q)
    rc = kernels().ff_latent_window_attention(ptr(q), ptr(codes), ptr(scales), ptr(ring_ids), ptr(positions), ptr(sink),
                                              ptr(inv_rot), ptr(out), b_, heads, d, window, visible, rings, rope_tail,
                                              c_float(scale), ptr(status_tensor(q.device)), stream_ptr())
    check(rc, "ff_latent_window_attention")
    _count()
    return out
