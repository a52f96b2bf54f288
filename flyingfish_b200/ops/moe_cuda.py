"""CUDA side of the MoE operators (see :mod:`flyingfish_b200.ops.moe_ops`): router top-k kernel,
device-side dispatch (count / scan / permute), grouped tcgen05 GEMMs with SwiGLU in the gate/up
epilogue, deterministic combine -- ``csrc/moe.cu``."""
from __future__ import annotations

import os
import weakref

from ctypes import c_float

import torch

from . import _count, _require, linear, workspace
from .lib import check, kernels, ptr, status_tensor, stream_ptr

SCORE_MODES = {"softmax": 0, "sigmoid": 1, "noaux": 2, "sqrt_softplus": 3}


def route(x, w_router, top_k, score, bias, n_groups, topk_groups, routed_scaling, renormalize):
    rows = x.shape[0]
    e = w_router.shape[0]
    logits = linear(x, w_router)                       # FP32 accumulate, rounded to BF16
    out_w = torch.empty(rows, top_k, dtype=torch.float32, device=x.device)
    out_ids = torch.empty(rows, top_k, dtype=torch.int32, device=x.device)
    rc = kernels().ff_moe_topk(ptr(logits), ptr(bias), ptr(out_w), ptr(out_ids), rows, e, top_k, SCORE_MODES[score],
                               n_groups, topk_groups, c_float(routed_scaling), int(renormalize), logits.stride(0),
                               ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_moe_topk")
    _count()
    return out_w, out_ids


def interleave64(w_gate_up: torch.Tensor) -> torch.Tensor:
    """[E, 2f, h] with rows [gate | up] -> rows interleaved per 64 (64 gate rows, the matching 64
    up rows, ...) so a 128-row weight tile carries both halves of 64 outputs."""
    e, two_f, h = w_gate_up.shape
    f = two_f // 2
    _require(f % 64 == 0, "expert FFN width must be a multiple of 64")
    g = w_gate_up[:, :f].reshape(e, f // 64, 1, 64, h)
    u = w_gate_up[:, f:].reshape(e, f // 64, 1, 64, h)
    return torch.cat([g, u], dim=2).reshape(e, two_f, h).contiguous()


_i64_cache: dict[int, tuple[weakref.ref, torch.Tensor]] = {}


def _gu_interleaved(w_gate_up: torch.Tensor) -> torch.Tensor:
    """Per-64 interleaved copy of an expert gate/up stack, cached per source tensor OBJECT: an address alone can be
    reused by a later tensor of the same shape once the first one is freed."""
    key = w_gate_up.data_ptr()
    hit = _i64_cache.get(key)
    if hit is not None and hit[0]() is w_gate_up:
        return hit[1]
    for k in [k for k, (r, _) in _i64_cache.items() if r() is None]:
        del _i64_cache[k]
    t = interleave64(w_gate_up)
    _i64_cache[key] = (weakref.ref(w_gate_up), t)
    return t


class _MoeWorkspace:
    def __init__(self):
        self.sorted: torch.Tensor | None = None


_moe_ws: dict[int, _MoeWorkspace] = {}


def _sorted_buffer(device, capacity: int, hidden: int) -> torch.Tensor:
    ws = _moe_ws.setdefault(device.index or 0, _MoeWorkspace())
    need = capacity * hidden
    if ws.sorted is None or ws.sorted.numel() < need:
        _require(not torch.cuda.is_current_stream_capturing(), "MoE workspace too small during graph capture")
        ws.sorted = torch.zeros(int(need * 1.2) + 16 * hidden, dtype=torch.bfloat16, device=device)
    return ws.sorted[:need].view(capacity, hidden)


def dispatch_local(x, ids, n_experts_total: int, e_lo: int, e_hi: int):
    """Device-side count / scan / permute for the experts [e_lo, e_hi) owned locally.
    Returns (sorted rows, pos, seg_off, counts, capacity)."""
    rows, hidden = x.shape
    top_k = ids.shape[1]
    el = e_hi - e_lo
    capacity = ((rows * top_k + 16 * el + 15) // 16) * 16
    dev = x.device
    meta = torch.empty(3 * el + 1, dtype=torch.int32, device=dev)
    counts, seg_off, cursors = meta[:el], meta[el: 2 * el + 1], meta[2 * el + 1:]
    pos = torch.empty(rows * top_k, dtype=torch.int32, device=dev)
    sorted_x = _sorted_buffer(dev, capacity, hidden)
    rc = kernels().ff_moe_dispatch_local(ptr(x), ptr(ids), rows, top_k, hidden, x.stride(0), n_experts_total, e_lo, e_hi,
                                         ptr(counts), ptr(seg_off), ptr(cursors), ptr(sorted_x), ptr(pos), capacity,
                                         ptr(status_tensor(dev)), stream_ptr())
    check(rc, "ff_moe_dispatch_local")
    _count(3)
    return sorted_x, pos, seg_off, counts, capacity


TILED_MIN_ROWS = int(os.environ.get("FF_MOE_TILED_MIN", "96"))


def grouped_gemm(xs, w, seg_off, counts, capacity: int, epi: int, rows_per_expert: float = 0.0,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """``rows_per_expert`` is the caller's estimate of the mean segment length (assignments / local experts; the
    true counts stay on the device): from ``TILED_MIN_ROWS`` on, the 128-row-tile kernel (tokens on the UMMA M
    side, double-buffered accumulators) runs instead of the swap-AB kernel that streams each weight slice once."""
    el, nw, k = w.shape
    n_out = nw // 2 if epi == 1 else nw
    y = out if out is not None else torch.empty(capacity, n_out, dtype=torch.bfloat16, device=xs.device)
    tiled = rows_per_expert >= TILED_MIN_ROWS and (epi == 0 or nw % 256 == 0)
    fn = kernels().ff_moe_grouped_gemm_tiled if tiled else kernels().ff_moe_grouped_gemm
    rc = fn(ptr(xs), ptr(w), ptr(y), ptr(seg_off), ptr(counts), el, nw, k, capacity, n_out, epi,
            ptr(status_tensor(xs.device)), stream_ptr())
    check(rc, "ff_moe_grouped_gemm")
    _count()
    return y


def combine(y, pos, ids, weights, rows: int, hidden: int, out: torch.Tensor | None = None,
            accumulate: bool = False) -> torch.Tensor:
    top_k = ids.shape[1]
    if out is None:
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=y.device)
    rc = kernels().ff_moe_combine(ptr(y), ptr(pos), ptr(ids), ptr(weights), ptr(out), rows, hidden, top_k, y.stride(0),
                                  int(accumulate), stream_ptr())
    check(rc, "ff_moe_combine")
    _count()
    return out


def experts_forward(x, weights, ids, w_gate_up, w_down, mode, e_lo: int = 0, n_experts_total: int | None = None):
    """Routed experts on one device: dispatch -> gate/up grouped GEMM (+SwiGLU) -> down grouped
    GEMM -> combine. ``w_gate_up`` is [E_local, 2f, h] in [gate | up] row order."""
    _require(mode == 0, "grouped GEMM epilogue implements SwiGLU rounding mode 0")
    rows, hidden = x.shape
    el = w_gate_up.shape[0]
    total = n_experts_total if n_experts_total is not None else el
    wgu = _gu_interleaved(w_gate_up)
    xs, pos, seg_off, counts, cap = dispatch_local(x.contiguous(), ids.contiguous(), total, e_lo, e_lo + el)
    rpe = rows * ids.shape[1] / max(total, 1)
    h = grouped_gemm(xs, wgu, seg_off, counts, cap, epi=1, rows_per_expert=rpe)
    y = grouped_gemm(h, w_down, seg_off, counts, cap, epi=0, rows_per_expert=rpe)
    return combine(y, pos, ids, weights.contiguous(), rows, hidden)


# ------------------------------------------------------------------------------------------------
# NVFP4 experts (W4A16): weights stay packed in HBM, csrc/moe_fp4.cu expands them inside the GEMM
# ------------------------------------------------------------------------------------------------
class Nvfp4Experts:
    """Packed expert stack: ``codes`` [E, N, K/2] uint8 (two E2M1 per byte, low nibble first), ``scales`` [E, N, K/16]
    uint8 (E4M3 per 16 weights), ``global_scale`` [E] f32. Gate/up stacks are kept interleaved per 64 rows (the
    order the SwiGLU epilogue expects); the interleave is a row permutation, so it applies to codes and scales alike."""

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor, gate_up: bool = False):
        _require(codes.dtype == torch.uint8 and scales.dtype == torch.uint8 and codes.dim() == 3, "nvfp4 experts: uint8 stacks")
        if gate_up:
            codes, scales = interleave64(codes), interleave64(scales)
        self.codes, self.scales = codes.contiguous(), scales.contiguous()
        self.global_scale = global_scale.to(torch.float32).reshape(-1).contiguous()
        self.experts, self.n, self.k = codes.shape[0], codes.shape[1], codes.shape[2] * 2
        _require(self.global_scale.numel() == self.experts and scales.shape == (self.experts, self.n, self.k // 16),
                 "nvfp4 experts: scale shapes")

    @classmethod
    def quantize(cls, w: torch.Tensor, gate_up: bool = False) -> "Nvfp4Experts":
        """[E, N, K] weights -> packed stack on the same device: per-expert global scale ``amax / (6 * 448)``, E4M3
        scale per 16 relative to it (device quantiser ``ff_quant_fp4`` on CUDA, ``loaders.quant`` on the host)."""
        if not w.is_cuda:
            from ..loaders import quant
            parts = [quant.quantize_nvfp4(w[e].float()) for e in range(w.shape[0])]
            return cls(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]),
                       torch.stack([p[2] for p in parts]), gate_up)
        from .quant_ops import quant_fp4
        gs = (w.float().abs().amax(dim=(1, 2)).clamp_min(1e-12) / (6.0 * 448.0)).contiguous()
        codes, scales = [], []
        for e in range(w.shape[0]):
            c, sc = quant_fp4(w[e].to(torch.bfloat16).contiguous(), "nvfp4", gs[e])
            codes.append(c)
            scales.append(sc)
        return cls(torch.stack(codes), torch.stack(scales), gs, gate_up)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel() + 4 * self.experts

    def supported(self) -> bool:
        return self.n % 128 == 0 and self.k % 128 == 0


def grouped_gemm_nvfp4(xs, w: Nvfp4Experts, seg_off, counts, capacity: int, epi: int,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    n_out = w.n // 2 if epi == 1 else w.n
    y = out if out is not None else torch.empty(capacity, n_out, dtype=torch.bfloat16, device=xs.device)
    rc = kernels().ff_moe_grouped_gemm_nvfp4(ptr(xs), ptr(w.codes), ptr(w.scales), ptr(w.global_scale), ptr(y), ptr(seg_off),
                                             ptr(counts), w.experts, w.n, w.k, capacity, n_out, epi,
                                             ptr(status_tensor(xs.device)), stream_ptr())
    check(rc, "ff_moe_grouped_gemm_nvfp4")
    _count()
    return y


def experts_forward_nvfp4(x, weights, ids, gate_up: Nvfp4Experts, down: Nvfp4Experts, e_lo: int = 0,
                          n_experts_total: int | None = None) -> torch.Tensor:
    """Routed experts with packed NVFP4 weights: dispatch -> gate/up (+SwiGLU) -> down -> combine, the weights
    expanded inside the two grouped GEMMs."""
    rows, hidden = x.shape
    total = n_experts_total if n_experts_total is not None else gate_up.experts
    xs, pos, seg_off, counts, cap = dispatch_local(x.contiguous(), ids.contiguous(), total, e_lo, e_lo + gate_up.experts)
    h = grouped_gemm_nvfp4(xs, gate_up, seg_off, counts, cap, epi=1)
    y = grouped_gemm_nvfp4(h, down, seg_off, counts, cap, epi=0)
    return combine(y, pos, ids, weights.contiguous(), rows, hidden)


FP4_DECODE_MAX_ROWS = int(os.environ.get("FF_FP4_MAX_ROWS_PER_EXPERT", "32"))


def pack_experts_nvfp4(weights) -> int:
    """Adds a packed NVFP4 copy of every MoE layer's routed experts (``lw.extra["experts_fp4"]``); decode-sized calls
    then read a quarter of the expert bytes. The BF16 stacks stay for prefill-sized calls. Returns the packed bytes."""
    total = 0
    for lw in weights.layers:
        if lw.router is None or lw.experts_gu is None or not lw.experts_gu.is_cuda:
            continue
        gu, dn = Nvfp4Experts.quantize(lw.experts_gu, gate_up=True), Nvfp4Experts.quantize(lw.experts_down)
        if gu.supported() and dn.supported():
            lw.extra["experts_fp4"] = (gu, dn)
            total += gu.nbytes() + dn.nbytes()
    return total
