"""Quantised linears and quantisation operators.

CUDA: ``csrc/quantize.cu`` (activation / weight codecs) and ``csrc/gemm_fp8.cu`` (block-scaled FP8
GEMM on tcgen05 with per-K-block promotion). CPU: the oracles of :mod:`flyingfish_b200.loaders.quant`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_longlong

import torch

from ..loaders import quant as qref
from . import _count, _require, linear, workspace
from .lib import check, kernels, ptr, status_tensor, stream_ptr


def quant_fp8_act(x: torch.Tensor, ue8m0: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [M, K] -> (E4M3 codes uint8 [M, K], FP32 scales [M, K/128])."""
    if not x.is_cuda:
        if ue8m0:
            q, e = qref.quantize_act_ue8m0(x, 128)
            return q, qref.e8m0_decode(e)
        return qref.quantize_fp8_act(x)
    m, k = x.shape
    _require(x.dtype == torch.bfloat16 and x.stride(1) == 1 and k % 128 == 0, "quant_fp8_act: bf16 rows, K % 128 == 0")
    q = torch.empty(m, k, dtype=torch.uint8, device=x.device)
    s = torch.empty(m, k // 128, dtype=torch.float32, device=x.device)
    check(kernels().ff_quant_fp8_1x128(ptr(x), ptr(q), ptr(s), m, k, x.stride(0), int(ue8m0), stream_ptr()),
          "ff_quant_fp8_1x128")
    _count()
    return q, s


def linear_fp8(x: torch.Tensor, w_codes: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """W8A8 block-scaled linear: ``x`` BF16 [M, K]; weight E4M3 codes [N, K] + FP32 128x128 scales."""
    if not x.is_cuda:
        return qref.fp8_block_linear(x, w_codes, w_scale)
    m, k = x.shape
    n = w_codes.shape[0]
    xq, xs = quant_fp8_act(x)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    lib = kernels()
    sb, cb = c_longlong(0), c_longlong(0)
    splits = lib.ff_gemm_fp8_plan(m, n, k, ctypes.byref(sb), ctypes.byref(cb))
    ws = workspace(x.device)
    scratch = ws.ensure("gemm_scratch", sb.value // 4) if splits > 1 else None
    _require(cb.value // 4 <= ws.gemm_counters.numel(), "linear_fp8: too many tiles for the counters")
    rc = lib.ff_gemm_fp8(ptr(xq), ptr(xs), ptr(w_codes), ptr(w_scale), ptr(y), None, None, 1, m, n, k, n, 0, splits,
                         ptr(scratch), ptr(ws.gemm_counters), ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_gemm_fp8")
    _count()
    return y


def grouped_gemm_fp8(xs_codes, xs_scale, w_codes, w_scale, seg_off, counts, capacity: int, epi: int,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped W8A8 GEMM over 16-row padded expert segments (see moe_cuda.dispatch_local)."""
    el, nw, k = w_codes.shape
    n_out = nw // 2 if epi == 1 else nw
    y = out if out is not None else torch.empty(capacity, n_out, dtype=torch.bfloat16, device=xs_codes.device)
    rc = kernels().ff_gemm_fp8(ptr(xs_codes), ptr(xs_scale), ptr(w_codes), ptr(w_scale), ptr(y), ptr(seg_off), ptr(counts),
                               el, capacity, nw, k, n_out, epi, 1, None, None, ptr(status_tensor(y.device)), stream_ptr())
    check(rc, "ff_gemm_fp8(grouped)")
    _count()
    return y


# ------------------------------------------------------------------------------------------
# FP8-resident weights: what a model holds when ``linear_format`` / ``expert_format`` is fp8_block
# ------------------------------------------------------------------------------------------
class Fp8Weight:
    """[N, K] linear weight kept as E4M3 codes + one FP32 scale per 128x128 block (the published DeepSeek-V3 layout,
    the reference's ``LinearWeightRef::Fp8Block``, src/backend/cuda/linear.rs). ``ops.linear`` accepts it in place
    of a BF16 matrix and runs the W8A8 block-scaled GEMM."""

    def __init__(self, codes: torch.Tensor, scale: torch.Tensor):
        assert codes.dtype == torch.uint8 and codes.dim() == 2 and scale.dtype == torch.float32
        self.codes, self.scale = codes.contiguous(), scale.contiguous()

    @classmethod
    def from_dense(cls, w: torch.Tensor) -> "Fp8Weight":
        q, s = qref.quantize_fp8_block_weight(w)
        return cls(q, s)

    @property
    def shape(self) -> tuple[int, int]:
        return tuple(self.codes.shape)

    @property
    def device(self) -> torch.device:
        return self.codes.device

    def nbytes(self) -> int:
        return self.codes.numel() + self.scale.numel() * 4

    def dense(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return dequant_fp8_block(self.codes, self.scale).to(dtype)

    def stride(self, dim: int) -> int:
        return self.codes.stride(dim)


class Fp8Experts:
    """Stacked expert matrices [E, N, K] as E4M3 codes with [E, N/128, K/128] FP32 block scales. ``interleaved``:
    gate/up rows alternate in groups of 64 (what the grouped kernel's SwiGLU epilogue expects)."""

    def __init__(self, codes: torch.Tensor, scale: torch.Tensor, interleaved: bool = False):
        self.codes, self.scale, self.interleaved = codes.contiguous(), scale.contiguous(), interleaved

    @classmethod
    def from_dense(cls, w: torch.Tensor, interleave: bool = False) -> "Fp8Experts":
        if interleave:
            e, n2, k = w.shape
            f = n2 // 2
            w = torch.stack([w[:, :f].reshape(e, f // 64, 64, k), w[:, f:].reshape(e, f // 64, 64, k)], dim=2).reshape(e, n2, k)
        qs = [qref.quantize_fp8_block_weight(w[i]) for i in range(w.shape[0])]
        return cls(torch.stack([q for q, _ in qs]), torch.stack([s for _, s in qs]), interleave)

    @property
    def shape(self) -> tuple[int, int, int]:
        return tuple(self.codes.shape)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scale.numel() * 4

    def expert(self, i: int) -> Fp8Weight:
        return Fp8Weight(self.codes[i], self.scale[i])


def _deinterleave_cols(gu: torch.Tensor) -> torch.Tensor:
    """[rows, 2f] with gate/up alternating per 64 columns -> [gate | up]."""
    m, n = gu.shape
    g = gu.view(m, n // 128, 2, 64)
    return torch.cat([g[:, :, 0].reshape(m, n // 2), g[:, :, 1].reshape(m, n // 2)], dim=1)


def experts_forward_fp8(x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, gate_up: Fp8Experts, down: Fp8Experts,
                        e_lo: int = 0, n_experts_total: int | None = None) -> torch.Tensor:
    """Routed experts with FP8-resident weights. CUDA: dispatch -> 1x128 activation quantisation -> grouped W8A8
    GEMM with SwiGLU -> quantisation -> grouped W8A8 down GEMM -> combine in ascending expert id. CPU: the same
    program with the oracle linears, expert by expert."""
    rows, hidden = x.shape
    el = gate_up.shape[0]
    total = n_experts_total if n_experts_total is not None else el
    if not x.is_cuda:
        from . import ref
        acc = torch.zeros(rows, ids.shape[1], hidden, dtype=torch.float32)
        for le in range(el):
            r, c = torch.nonzero(ids == e_lo + le, as_tuple=True)
            if r.numel() == 0:
                continue
            gu = qref.fp8_block_linear(x[r], gate_up.codes[le], gate_up.scale[le])
            if gate_up.interleaved:
                gu = _deinterleave_cols(gu)
            h = ref.silu_mul(gu, 0)
            y = qref.fp8_block_linear(h, down.codes[le], down.scale[le])
            acc[r, c] = y.to(torch.float32) * weights[r, c, None]
        order = torch.argsort(ids.long(), dim=-1, stable=True)
        ordered = torch.gather(acc, 1, order[:, :, None].expand_as(acc))
        out = torch.zeros(rows, hidden, dtype=torch.float32)
        for j in range(ids.shape[1]):
            out = out + ordered[:, j]
        return out.to(x.dtype)
    from . import moe_cuda
    _require(gate_up.interleaved, "experts_forward_fp8: the gate/up experts must be interleaved per 64 rows")
    xs, pos, seg_off, counts, cap = moe_cuda.dispatch_local(x.contiguous(), ids.contiguous(), total, e_lo, e_lo + el)
    xq, xsc = quant_fp8_act(xs)
    h = grouped_gemm_fp8(xq, xsc, gate_up.codes, gate_up.scale, seg_off, counts, cap, epi=1)
    hq, hsc = quant_fp8_act(h)
    y = grouped_gemm_fp8(hq, hsc, down.codes, down.scale, seg_off, counts, cap, epi=0)
    return moe_cuda.combine(y, pos, ids, weights.contiguous(), rows, hidden)


def dequant_fp8_block(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    if not codes.is_cuda:
        return qref.dequantize_fp8_block(codes, scale)
    n, k = codes.shape
    out = torch.empty(n, k, dtype=torch.bfloat16, device=codes.device)
    check(kernels().ff_dequant_fp8_block(ptr(codes), ptr(scale), ptr(out), n, k, stream_ptr()), "ff_dequant_fp8_block")
    _count()
    return out


def dequant_nvfp4(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    if not packed.is_cuda:
        return qref.dequantize_nvfp4(packed, scales, global_scale)
    n = packed.shape[0]
    k = packed.shape[1] * 2
    out = torch.empty(n, k, dtype=torch.bfloat16, device=packed.device)
    gs = global_scale.reshape(1).to(torch.float32)
    check(kernels().ff_dequant_nvfp4(ptr(packed), ptr(scales), ptr(gs), ptr(out), c_longlong(n * k), stream_ptr()),
          "ff_dequant_nvfp4")
    _count()
    return out


def linear_nvfp4(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """W4A16: effective BF16 weights (E2M1 * E4M3 scale * global, rounded to BF16) times BF16
    activations, FP32 accumulation."""
    if not x.is_cuda:
        return qref.nvfp4_linear(x, packed, scales, global_scale)
    return linear(x, dequant_nvfp4(packed, scales, global_scale))


def quant_fp4(x: torch.Tensor, mode: str = "nvfp4", global_scale: torch.Tensor | None = None
              ) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 -> (packed E2M1, scale codes): ``nvfp4`` = E4M3 scale per 16 relative to ``global_scale``,
    ``mxfp4`` = E8M0 scale per 32."""
    gs = 16 if mode == "nvfp4" else 32
    _require(x.is_cuda and x.is_contiguous() and x.numel() % gs == 0, "quant_fp4: contiguous CUDA tensor")
    packed = torch.empty(x.numel() // 2, dtype=torch.uint8, device=x.device)
    scales = torch.empty(x.numel() // gs, dtype=torch.uint8, device=x.device)
    g = None if global_scale is None else global_scale.reshape(1).to(torch.float32)
    check(kernels().ff_quant_fp4(ptr(x), ptr(packed), ptr(scales), ptr(g), c_longlong(x.numel()),
                                 0 if mode == "nvfp4" else 1, stream_ptr()), "ff_quant_fp4")
    _count()
    return packed.view(*x.shape[:-1], x.shape[-1] // 2), scales.view(*x.shape[:-1], x.shape[-1] // gs)
