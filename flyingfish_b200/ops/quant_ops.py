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


def grouped_gemm_fp8(xs_codes, xs_scale, w_codes, w_scale, seg_off, counts, capacity: int, epi: int) -> torch.Tensor:
    """Grouped W8A8 GEMM over 16-row padded expert segments (see moe_cuda.dispatch_local)."""
    el, nw, k = w_codes.shape
    n_out = nw // 2 if epi == 1 else nw
    y = torch.empty(capacity, n_out, dtype=torch.bfloat16, device=xs_codes.device)
    rc = kernels().ff_gemm_fp8(ptr(xs_codes), ptr(xs_scale), ptr(w_codes), ptr(w_scale), ptr(y), ptr(seg_off), ptr(counts),
                               el, capacity, nw, k, n_out, epi, 1, None, None, ptr(status_tensor(y.device)), stream_ptr())
    check(rc, "ff_gemm_fp8(grouped)")
    _count()
    return y


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
