"""Gated DeltaNet operators: depthwise causal conv + SiLU with carried history, q/k preparation, and the
recurrent state update. CUDA: ``csrc/gdn.cu``; CPU: FP32 oracles (reference: kernels/gdn/gdn_conv.cu:1-8,
gdn_prep.cu:1-4, gdn_recurrent.cuh:1-16)."""
from __future__ import annotations

from ctypes import c_float

import torch

from . import _count
from .lib import check, kernels, ptr, stream_ptr

BF16 = torch.bfloat16
D = 128


def conv(x: torch.Tensor, weight: torch.Tensor, history: torch.Tensor, commit: bool = True) -> torch.Tensor:
    """x [rows, channels] bf16 (rows of one sequence in order), weight [channels, 4] bf16, history
    [channels, 3] f32 (updated in place when ``commit``)."""
    rows, ch = x.shape
    if not x.is_cuda:
        full = torch.cat([history.t(), x.float()], dim=0)                          # [3 + rows, ch]
        w = weight.float()
        acc = sum(full[t: t + rows] * w[:, t] for t in range(4))
        y = acc.to(BF16).float()
        out = (y * torch.sigmoid(y)).to(BF16)
        if commit:
            history.copy_(full[rows: rows + 3].t())
        return out
    out = torch.empty_like(x)
    check(kernels().ff_gdn_conv(ptr(x), ptr(weight), ptr(history), ptr(out), rows, ch, int(commit), stream_ptr()), "ff_gdn_conv")
    _count()
    return out


def prep(conv_out: torch.Tensor, heads: int, kheads: int, eps: float = 1e-6):
    """conv_out [rows, (2*kheads + heads) * 128] bf16 -> q, k, v [rows, heads, 128] f32."""
    rows = conv_out.shape[0]
    if not conv_out.is_cuda:
        x = conv_out.float()
        qk = x[:, : 2 * kheads * D].reshape(rows, 2, kheads, D)
        rep = heads // kheads
        q = qk[:, 0].repeat_interleave(rep, dim=1); k = qk[:, 1].repeat_interleave(rep, dim=1)
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + eps) * (D ** -0.5)
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + eps)
        return q.contiguous(), k.contiguous(), x[:, 2 * kheads * D:].reshape(rows, heads, D).contiguous()
    q = torch.empty(rows, heads, D, dtype=torch.float32, device=conv_out.device); k = torch.empty_like(q); v = torch.empty_like(q)
    check(kernels().ff_gdn_prep(ptr(conv_out), ptr(q), ptr(k), ptr(v), rows, heads, kheads, c_float(eps), stream_ptr()), "ff_gdn_prep")
    _count()
    return q, k, v


def recurrent(q, k, v, beta, g, state: torch.Tensor, row_start: torch.Tensor) -> torch.Tensor:
    """q, k, v [rows, heads, 128] f32, beta / g [rows, heads] f32, state [sequences, heads, 128, 128] f32 (updated
    in place), row_start [sequences + 1] int32 -> out [rows, heads, 128] bf16."""
    rows, heads, _ = q.shape
    if not q.is_cuda:
        out = torch.zeros(rows, heads, D)
        for s in range(row_start.numel() - 1):
            for r in range(int(row_start[s]), int(row_start[s + 1])):
                S = state[s] * torch.exp(g[r])[:, None, None]
                kv = torch.einsum("hk,hkv->hv", k[r], S)
                delta = (v[r] - kv) * beta[r][:, None]
                S = S + k[r][:, :, None] * delta[:, None, :]
                out[r] = torch.einsum("hk,hkv->hv", q[r], S)
                state[s] = S
        return out.to(BF16)
    out = torch.empty(rows, heads, D, dtype=BF16, device=q.device)
    check(kernels().ff_gdn_recurrent(ptr(q), ptr(k), ptr(v), ptr(beta), ptr(g), ptr(state), ptr(out), ptr(row_start),
                                     row_start.numel() - 1, heads, stream_ptr()), "ff_gdn_recurrent")
    _count()
    return out


# ------------------------------------------------------------------------------------------------
# batched forms used by a model's forward: packed rows of several sequences, state addressed by slot
# ------------------------------------------------------------------------------------------------
def conv_batched(x: torch.Tensor, weight: torch.Tensor, history: torch.Tensor, row_start: torch.Tensor,
                 slots: torch.Tensor, commit: bool = True) -> torch.Tensor:
    """x [rows, >= channels] bf16 (the first ``channels`` columns are convolved), history [slots, channels, 3] f32,
    row_start [sequences + 1] / slots [sequences] int32 -> [rows, channels] bf16."""
    ch = weight.shape[0]
    if not x.is_cuda:
        out = torch.empty(x.shape[0], ch, dtype=BF16)
        for s in range(slots.numel()):
            r0, r1 = int(row_start[s]), int(row_start[s + 1])
            if r1 > r0:
                out[r0:r1] = conv(x[r0:r1, :ch].contiguous(), weight, history[int(slots[s])], commit)
        return out
    out = torch.empty(x.shape[0], ch, dtype=BF16, device=x.device)
    check(kernels().ff_gdn_conv_batched(ptr(x), ptr(weight), ptr(history), ptr(out), ptr(row_start), ptr(slots),
                                        slots.numel(), ch, x.stride(0), int(commit), stream_ptr()), "ff_gdn_conv_batched")
    _count()
    return out


def recurrent_slots(q, k, v, beta, g, state: torch.Tensor, row_start: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """Like :func:`recurrent` with sequence s using ``state[slots[s]]``."""
    if not q.is_cuda:
        rows, heads, _ = q.shape
        out = torch.zeros(rows, heads, D, dtype=BF16)
        for s in range(slots.numel()):
            r0, r1 = int(row_start[s]), int(row_start[s + 1])
            if r1 > r0:
                sl = int(slots[s])
                out[r0:r1] = recurrent(q[r0:r1], k[r0:r1], v[r0:r1], beta[r0:r1], g[r0:r1], state[sl: sl + 1],
                                       torch.tensor([0, r1 - r0], dtype=torch.int32))
        return out
    rows, heads, _ = q.shape
    out = torch.empty(rows, heads, D, dtype=BF16, device=q.device)
    check(kernels().ff_gdn_recurrent_slots(ptr(q), ptr(k), ptr(v), ptr(beta), ptr(g), ptr(state), ptr(out), ptr(row_start),
                                           ptr(slots), slots.numel(), heads, stream_ptr()), "ff_gdn_recurrent_slots")
    _count()
    return out


CHUNK_MIN_ROWS = 32          # shortest sequence segment of a launch for which the chunked form is used


def chunked_slots(q, k, v, beta, g, state: torch.Tensor, row_start: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """Prefill form of :func:`recurrent_slots`: the same recurrence evaluated 64 tokens at a time through the WY
    representation on tensor cores (``csrc/gdn_chunk.cu``; reference: kernels/gdn/gdn_chunkwise_p1.cu, gdn_cw_p2.cu).
    Matrix products take BF16 operands, so results agree with the token-by-token form to BF16 accuracy, not bit for
    bit. CPU tensors run the recurrent oracle."""
    if not q.is_cuda:
        return recurrent_slots(q, k, v, beta, g, state, row_start, slots)
    rows, heads, d = q.shape
    assert d == D and state.shape[-2:] == (D, D)
    out = torch.empty(rows, heads, D, dtype=BF16, device=q.device)
    check(kernels().ff_gdn_chunked_slots(ptr(q.contiguous()), ptr(k.contiguous()), ptr(v.contiguous()), ptr(beta), ptr(g),
                                         ptr(state), ptr(out), ptr(row_start), ptr(slots), slots.numel(), heads, stream_ptr()),
          "ff_gdn_chunked_slots")
    _count()
    return out
