"""Quantised number formats of the published checkpoints, host side: E4M3 / E2M1 / E8M0 codecs,
block-scale shapes, reference quantisers and reference linears. These are the oracles for the
device kernels (``csrc/quantize.cu``, ``csrc/gemm_fp8.cu``, ``csrc/moe_fp4.cu``) and the code the
loaders use to validate scale tensor shapes (the reference's src/fp8.rs:69-147, 245-345).

Formats
  * FP8 E4M3 ("fn": no infinities, max 448), weights with one FP32 scale per 128x128 block,
    activations quantised on the fly with one FP32 scale per 1x128 (scale = amax / 448).
  * UE8M0: power-of-two scales (exponent byte, value 2**(e-127)); DeepSeek-style activation
    quantisation floors amax at 1e-4 and uses 2**ceil(log2(amax/448)) per 32 elements.
  * NVFP4: E2M1 values {0, .5, 1, 1.5, 2, 3, 4, 6} two per byte (low nibble first), one E4M3
    scale per 16 elements, one FP32 global scale per tensor; effective weight
    ``e2m1 * e4m3_scale * global`` rounded to BF16 before the dot product (W4A16).
  * MXFP4: E2M1 with one E8M0 scale per 32 elements.
"""
from __future__ import annotations

import torch

F32 = torch.float32
E4M3_MAX = 448.0
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=F32)


# ------------------------------------------------------------------------------------------
# E4M3
# ------------------------------------------------------------------------------------------
def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """Saturating round-to-nearest-even encode to FP8 E4M3 (returns uint8 codes)."""
    return x.to(F32).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(codes: torch.Tensor) -> torch.Tensor:
    return codes.view(torch.float8_e4m3fn).to(F32)


# ------------------------------------------------------------------------------------------
# E8M0
# ------------------------------------------------------------------------------------------
def e8m0_decode(codes: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, codes.to(F32) - 127.0)


def e8m0_encode_ceil(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x, as an exponent byte."""
    e = torch.ceil(torch.log2(x.to(F32).clamp_min(2.0 ** -127)))
    return (e + 127).clamp(0, 254).to(torch.uint8)


# ------------------------------------------------------------------------------------------
# E2M1
# ------------------------------------------------------------------------------------------
def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 code (4 bits: sign | 3-bit magnitude index), ties to the even index."""
    a = x.to(F32).abs().clamp(max=6.0)
    vals = E2M1_VALUES.to(x.device)
    d = (a[..., None] - vals).abs()
    idx = d.argmin(-1)
    # ties: argmin returns the first (lower) index; round-half-to-even wants the even index
    lo = idx
    hi = (idx + 1).clamp(max=7)
    tie = (d.gather(-1, lo[..., None])[..., 0] == d.gather(-1, hi[..., None])[..., 0]) & (hi != lo)
    idx = torch.where(tie & (lo % 2 == 1), hi, lo)
    sign = (x < 0).to(torch.uint8) << 3
    return (idx.to(torch.uint8) | sign)


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    vals = E2M1_VALUES.to(codes.device)
    mag = vals[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def e2m1_pack(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] 4-bit codes -> [..., K/2] bytes, element 2i in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def e2m1_unpack(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


# ------------------------------------------------------------------------------------------
# block-scale shapes
# ------------------------------------------------------------------------------------------
def fp8_block_scale_shape(n: int, k: int, block: int = 128) -> tuple[int, int]:
    return ((n + block - 1) // block, (k + block - 1) // block)


def nvfp4_scale_shape(n: int, k: int) -> tuple[int, int]:
    assert k % 16 == 0
    return (n, k // 16)


# ------------------------------------------------------------------------------------------
# quantisers
# ------------------------------------------------------------------------------------------
def quantize_fp8_block_weight(w: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (uint8 codes [N, K], FP32 scales [ceil(N/128), ceil(K/128)])."""
    n, k = w.shape
    sn, sk = fp8_block_scale_shape(n, k, block)
    wp = torch.zeros(sn * block, sk * block, dtype=F32, device=w.device)
    wp[:n, :k] = w.to(F32)
    blocks = wp.view(sn, block, sk, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / E4M3_MAX
    q = e4m3_encode(blocks / scale[:, None, :, None]).view(sn * block, sk * block)[:n, :k]
    return q.contiguous(), scale


def quantize_fp8_act(x: torch.Tensor, group: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (codes [M, K], FP32 scales [M, K/128]); scale = amax / 448
    (kernels/fp8_linear.cu:12-48 of the reference)."""
    m, k = x.shape
    assert k % group == 0
    g = x.to(F32).view(m, k // group, group)
    amax = g.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = e4m3_encode(g / scale[..., None]).view(m, k)
    return q, scale


def quantize_act_ue8m0(x: torch.Tensor, group: int = 32) -> tuple[torch.Tensor, torch.Tensor]:
    """DeepSeek-style activation quantisation: amax floored at 1e-4, power-of-two scale per 32."""
    m, k = x.shape
    g = x.to(F32).view(m, k // group, group)
    amax = g.abs().amax(-1).clamp_min(1e-4)
    e = e8m0_encode_ceil(amax / E4M3_MAX)
    scale = e8m0_decode(e)
    return e4m3_encode(g / scale[..., None]).view(m, k), e


def quantize_nvfp4(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[N, K] -> (packed E2M1 [N, K/2], E4M3 scale codes [N, K/16], FP32 global scale)."""
    n, k = w.shape
    wf = w.to(F32)
    gmax = wf.abs().max().clamp_min(1e-12)
    global_scale = gmax / (6.0 * E4M3_MAX)
    g = wf.view(n, k // 16, 16)
    amax = g.abs().amax(-1)
    s = e4m3_encode(amax / 6.0 / global_scale)
    sdec = e4m3_decode(s) * global_scale
    sdec = torch.where(sdec > 0, sdec, torch.ones_like(sdec))
    codes = e2m1_encode(g / sdec[..., None]).view(n, k)
    return e2m1_pack(codes), s, global_scale.reshape(())


def dequantize_nvfp4(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                     dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Effective weight ``e2m1 * e4m3 * global`` rounded to ``dtype``."""
    n = packed.shape[0]
    vals = e2m1_decode(e2m1_unpack(packed)).view(n, -1, 16)
    s = e4m3_decode(scales) * global_scale.to(F32)
    return (vals * s[..., None]).view(n, -1).to(dtype)


def dequantize_fp8_block(codes: torch.Tensor, scale: torch.Tensor, block: int = 128,
                         dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    n, k = codes.shape
    s = scale.repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return (e4m3_decode(codes) * s).to(dtype)


# ------------------------------------------------------------------------------------------
# reference linears
# ------------------------------------------------------------------------------------------
def fp8_block_linear(x: torch.Tensor, w_codes: torch.Tensor, w_scale: torch.Tensor,
                     out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """W8A8 block linear: activations quantised per 1x128, per-K-block partial dot products of the
    codes multiplied by (w_scale * x_scale) and accumulated in FP32
    (kernels/fp8_linear.cu:122-131 of the reference)."""
    m, k = x.shape
    n = w_codes.shape[0]
    xq, xs = quantize_fp8_act(x)
    xd = e4m3_decode(xq).view(m, k // 128, 128).to(torch.float64)
    wd = e4m3_decode(w_codes).view(n, k // 128, 128).to(torch.float64)
    part = torch.einsum("mbk,nbk->mnb", xd, wd).to(F32)                       # exact products, per block
    ws = w_scale.repeat_interleave(128, 0)[:n]                                # [n, kb]
    y = (part * xs[:, None, :] * ws[None, :, :]).sum(-1)
    return y.to(out_dtype)


def nvfp4_linear(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                 out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """W4A16: BF16 effective weights, FP32 accumulation."""
    w = dequantize_nvfp4(packed, scales, global_scale, torch.bfloat16)
    return (x.to(torch.float64) @ w.to(torch.float64).t()).to(out_dtype)
