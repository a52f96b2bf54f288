"""Operator API of the framework.

Every function takes PyTorch tensors. On a CUDA device the hand-written sm_100a kernel runs
(through ``_ff_kernels.so``; a missing library is an error, never a silent fallback); on a CPU
tensor the plain PyTorch oracle from :mod:`flyingfish_b200.ops.ref` runs, which is how the tiny
host-only configuration and the CPU test-suite execute the same model code.

Host-side contract checks (shapes, strides, dtypes, alignment) happen here before a launch, in
the spirit of the reference's typed tensor views (src/backend/cuda/contracts.rs:81-139); the
kernels report what only the device can see (bad token ids, bad block ids, timed-out waits)
through the status word (:func:`flyingfish_b200.ops.lib.check_status`).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import ref
from .lib import DeviceStatusError, KernelError, check, check_status, kernels, ptr, read_status, status_tensor, stream_ptr

__all__ = [
    "linear", "linear_swiglu", "rmsnorm", "add_rmsnorm", "embed_rmsnorm", "embed", "rope_kv_paged", "silu_mul",
    "attn_decode", "attn_prefill", "argmax_rows", "sample_rows", "residual_add", "softcap", "check_status",
    "read_status", "KernelError", "DeviceStatusError", "launch_count", "reset_launch_count",
]

BF16 = torch.bfloat16
_launches = 0


def launch_count() -> int:
    """Number of kernel launches issued through this module since the last reset."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _rows2d(t: torch.Tensor) -> tuple[int, int]:
    _require(t.dim() == 2 and t.stride(1) == 1, "expected a 2-D tensor with unit inner stride")
    return t.shape[0], t.stride(0)


# ------------------------------------------------------------------------------------------
# workspace (split-K partials, attention split partials): one per device, grown outside of
# graph capture only
# ------------------------------------------------------------------------------------------
class _Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self.gemm_scratch = torch.empty(8 << 20, dtype=torch.float32, device=device)      # 32 MiB
        self.gemm_counters = torch.zeros(4096, dtype=torch.int32, device=device)
        self.attn_o = torch.empty(4 << 20, dtype=torch.float32, device=device)             # 16 MiB
        self.attn_ml = torch.empty(1 << 18, dtype=torch.float32, device=device)
        self.attn_counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)     # one per (sequence, kv head, row tile)

    def ensure(self, name: str, numel: int) -> torch.Tensor:
        t = getattr(self, name, None)
        if t is None:                      # scratch of an optional operator family: FP32, created on first use
            t = torch.empty(0, dtype=torch.float32, device=self.device)
        if t.numel() < numel:
            _require(not torch.cuda.is_current_stream_capturing(), f"workspace {name} too small during graph capture")
            t = torch.empty(int(numel * 1.25), dtype=t.dtype, device=self.device)
            setattr(self, name, t)
        return t


_workspaces: dict[int, _Workspace] = {}


def workspace(device: torch.device) -> _Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = _Workspace(torch.device("cuda", idx))
        _workspaces[idx] = ws
    return ws


# ------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------
SKINNY_MAX_M = 128
FP8_DENSE_ROWS = 256         # more rows than this: FP8-resident weights are expanded to BF16 for the call
FP8_MAX_K = 32768            # deepest reduction the W8A8 kernel stages activation scales for
# decode-shape epilogue fusions (FLYINGFISH_FUSE_SWIGLU=0 / FLYINGFISH_FUSE_ROPE=0 fall back to separate kernels)
FUSE_SWIGLU = os.environ.get("FLYINGFISH_FUSE_SWIGLU", "1") != "0"
FUSE_ROPE = os.environ.get("FLYINGFISH_FUSE_ROPE", "1") != "0"
FUSE_ATTN_MERGE = os.environ.get("FLYINGFISH_FUSE_ATTN_MERGE", "0") == "1"
# prefill attention: the tcgen05 kernel (csrc/attention_tc.cu); FF_ATTN_PREFILL=mma selects the mma.sync kernel
ATTN_PREFILL_TC = os.environ.get("FF_ATTN_PREFILL", "tc") != "mma"


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``y[M,N] = x[M,K] @ w[N,K].T`` (BF16 operands, FP32 accumulation).

    CUDA path: tcgen05 kernels -- the weight-streaming decode kernel of ``csrc/gemm_skinny.cu`` (tokens on
    the UMMA M side, cluster split-K or stream-K) for M <= 128, the persistent 128x256x64 kernel of
    ``csrc/gemm_bf16.cu`` otherwise. ``w`` may be an FP8-resident weight (``quant_ops.Fp8Weight``): the block-scaled
    W8A8 GEMM of ``csrc/gemm_fp8.cu`` (CPU: its oracle) runs instead."""
    if not isinstance(w, torch.Tensor):
        from . import quant_ops
        tok = min(128, (x.shape[0] + 15) // 16 * 16)
        if x.shape[0] > FP8_DENSE_ROWS or w.shape[1] > FP8_MAX_K or (w.shape[1] // 128) * tok * 4 > 64 * 1024:
            # prefill-sized calls: the weight is expanded to BF16 for this call and the large-tile BF16 GEMM runs
            # (W8A16), as the reference does for many rows (kernels/fp8_linear.cu materialises + cuBLAS); the W8A8
            # kernel keeps tokens on the narrow UMMA side and is meant for decode batches
            return linear(x, w.dense(), out=out, out_dtype=out_dtype)
        y = quant_ops.linear_fp8(x, w.codes, w.scale)
        if out_dtype is not None and y.dtype != out_dtype:
            y = y.to(out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if not _is_cuda(x):
        y = ref.linear(x, w, out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _require(x.dtype == BF16 and w.dtype == BF16, "linear: BF16 operands required on CUDA")
    m, ldx = _rows2d(x)
    n, ldw = _rows2d(w)
    k = x.shape[1]
    _require(w.shape[1] == k, "linear: inner dimensions differ")
    odt = out_dtype or BF16
    if out is None:
        out = torch.empty(m, n, dtype=odt, device=x.device)
    _require(out.shape == (m, n) and out.stride(1) == 1 and out.dtype == odt, "linear: bad output tensor")
    lib = kernels()
    st = status_tensor(x.device)
    if m <= SKINNY_MAX_M and odt == BF16:
        scratch_b, counter_b = c_longlong(0), c_longlong(0)
        splits = lib.ff_gemm_skinny_plan(m, n, k, ctypes.byref(scratch_b), ctypes.byref(counter_b))
        ws = workspace(x.device)
        scratch = ws.ensure("gemm_scratch", scratch_b.value // 4) if scratch_b.value > 0 else None
        _require(counter_b.value // 4 <= ws.gemm_counters.numel(), "linear: too many column tiles for counters")
        rc = lib.ff_gemm_skinny(ptr(x), ptr(w), ptr(out), m, n, k, ldx, ldw, out.stride(0), splits, ptr(scratch),
                                ptr(ws.gemm_counters), ptr(st), stream_ptr())
        check(rc, "ff_gemm_skinny")
    else:
        epi = 0 if odt == BF16 else 2
        _require(odt in (BF16, torch.float32), "linear: output dtype must be bf16 or fp32")
        rc = lib.ff_gemm_bf16(ptr(x), ptr(w), ptr(out), m, n, k, ldx, ldw, out.stride(0), epi, ptr(st), stream_ptr())
        check(rc, "ff_gemm_bf16")
    _count()
    return out


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor | None = None,
                  mode: int = 0) -> torch.Tensor:
    """Gate/up projection with the SwiGLU activation fused into the GEMM epilogue. The weight is
    the per-64 interleaved ``[2f, h]`` matrix built by :func:`ref.interleave_gate_up`."""
    if not _is_cuda(x):
        return ref.linear_swiglu(x, w_interleaved, mode)
    m, ldx = _rows2d(x)
    n, ldw = _rows2d(w_interleaved)
    k = x.shape[1]
    _require(n % 256 == 0, "linear_swiglu: N must be a multiple of 256")
    if out is None:
        out = torch.empty(m, n // 2, dtype=BF16, device=x.device)
    if mode != 0:
        # the GEMM epilogues implement rounding mode 0; other gates (tanh-GELU, clamped) run as the activation kernel
        return silu_mul_interleaved(linear(x, w_interleaved), out, mode)
    if m <= SKINNY_MAX_M and not FUSE_SWIGLU:
        return silu_mul_interleaved(linear(x, w_interleaved), out)
    if m <= SKINNY_MAX_M:
        # decode shapes: the weight-streaming kernel applies SwiGLU row-wise in its epilogue
        lib = kernels()
        scratch_b, counter_b = c_longlong(0), c_longlong(0)
        grid = lib.ff_gemm_skinny_plan_epi(m, n, k, 1, ctypes.byref(scratch_b), ctypes.byref(counter_b))
        check(min(grid, 0), "ff_gemm_skinny_plan_epi")
        ws = workspace(x.device)
        scratch = ws.ensure("gemm_scratch", scratch_b.value // 4) if scratch_b.value > 0 else None
        _require(counter_b.value // 4 <= ws.gemm_counters.numel(), "linear_swiglu: too many column tiles for counters")
        rc = lib.ff_gemm_skinny_swiglu(ptr(x), ptr(w_interleaved), ptr(out), m, n, k, ldx, ldw, out.stride(0), grid,
                                       ptr(scratch), ptr(ws.gemm_counters), ptr(status_tensor(x.device)), stream_ptr())
        check(rc, "ff_gemm_skinny_swiglu")
        _count()
        return out
    rc = kernels().ff_gemm_bf16(ptr(x), ptr(w_interleaved), ptr(out), m, n, k, ldx, ldw, out.stride(0), 1,
                                ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_gemm_bf16(swiglu)")
    _count()
    return out


def silu_mul_interleaved(gu: torch.Tensor, out: torch.Tensor | None = None, mode: int = 0) -> torch.Tensor:
    """SwiGLU on the per-64 interleaved gate/up layout produced by the fused weight."""
    return silu_mul(gu, mode=mode, out=out, interleaved=True)


# ------------------------------------------------------------------------------------------
# norms / embedding
# ------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, unit_offset: bool = False,
            out: torch.Tensor | None = None) -> torch.Tensor:
    if not _is_cuda(x):
        return ref.rmsnorm(x, w, eps, unit_offset)
    rows, ldx = _rows2d(x)
    hidden = x.shape[1]
    _require(x.dtype == BF16 and w.dtype == BF16 and w.numel() == hidden, "rmsnorm: bad operands")
    if out is None:
        out = torch.empty(rows, hidden, dtype=BF16, device=x.device)
    rc = kernels().ff_rmsnorm(ptr(x), ptr(w), ptr(out), rows, hidden, ldx, c_float(eps), int(unit_offset),
                              ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_rmsnorm")
    _count()
    return out


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float, unit_offset: bool = False,
                out: torch.Tensor | None = None, capture: torch.Tensor | None = None) -> torch.Tensor:
    """``res += x`` (rounded to the storage dtype, in place) and returns ``rmsnorm(res) * w``.
    ``capture`` ([rows, hidden] view of a ``[rows, taps, hidden]`` slab) also receives the new
    residual for a draft model's hidden-state taps."""
    if not _is_cuda(x):
        new_res, n = ref.add_rmsnorm(x, res, w, eps, unit_offset)
        res.copy_(new_res)
        if capture is not None:
            capture.copy_(new_res)
        return n
    rows, ldx = _rows2d(x)
    hidden = x.shape[1]
    _require(res.is_contiguous() and res.shape == (rows, hidden), "add_rmsnorm: residual must be contiguous")
    if out is None:
        out = torch.empty(rows, hidden, dtype=BF16, device=x.device)
    cstride = capture.stride(0) if capture is not None else 0
    rc = kernels().ff_add_rmsnorm(ptr(x), ptr(res), ptr(w), ptr(out), ptr(capture), cstride, rows, hidden, ldx,
                                  c_float(eps), int(unit_offset), ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_add_rmsnorm")
    _count()
    return out


def embed_rmsnorm(ids: torch.Tensor, table: torch.Tensor, w: torch.Tensor, eps: float, unit_offset: bool = False
                  ) -> tuple[torch.Tensor, torch.Tensor]:
    """Embedding gather fused with the first layer's RMSNorm: returns (residual, normalised)."""
    if not _is_cuda(table):
        return ref.embed_rmsnorm(ids, table, w, eps, unit_offset)
    rows = ids.numel()
    vocab, hidden = table.shape
    _require(ids.dtype == torch.int32 and ids.is_contiguous(), "embed_rmsnorm: ids must be contiguous int32")
    res = torch.empty(rows, hidden, dtype=BF16, device=table.device)
    out = torch.empty(rows, hidden, dtype=BF16, device=table.device)
    rc = kernels().ff_embed_rmsnorm(ptr(ids), ptr(table), ptr(w), ptr(res), ptr(out), rows, hidden, vocab,
                                    c_float(eps), int(unit_offset), ptr(status_tensor(table.device)), stream_ptr())
    check(rc, "ff_embed_rmsnorm")
    _count()
    return res, out


def embed(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if not _is_cuda(table):
        x = table[ids.long()]
        return x if scale == 1.0 else (x.to(torch.float32) * scale).to(table.dtype)
    rows = ids.numel()
    vocab, hidden = table.shape
    out = torch.empty(rows, hidden, dtype=BF16, device=table.device)
    rc = kernels().ff_embed(ptr(ids), ptr(table), ptr(out), rows, hidden, vocab, c_float(scale),
                            ptr(status_tensor(table.device)), stream_ptr())
    check(rc, "ff_embed")
    _count()
    return out


def residual_add(res: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    if not _is_cuda(res):
        res.copy_((res.to(torch.float32) + x.to(torch.float32)).to(res.dtype))
        return res
    _require(res.is_contiguous() and x.is_contiguous() and res.numel() == x.numel(), "residual_add: contiguous only")
    check(kernels().ff_residual_add(ptr(res), ptr(x), c_longlong(res.numel()), stream_ptr()), "ff_residual_add")
    _count()
    return res


# ------------------------------------------------------------------------------------------
# rope + kv write, activation
# ------------------------------------------------------------------------------------------
def rope_kv_paged(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor,
                  vcache: torch.Tensor, hq: int, hkv: int, dim: int, theta: float, rot_dim: int | None = None,
                  inv_freq: torch.Tensor | None = None) -> None:
    """In place on ``qkv`` ([rows, (hq+2*hkv)*dim], Q and K rotated) and the paged cache."""
    if not _is_cuda(qkv):
        ref.rope_kv_paged(qkv, positions, slots, kcache, vcache, hq, hkv, dim, theta, rot_dim, inv_freq)
        return
    rows, ld = _rows2d(qkv)
    _require(qkv.shape[1] >= (hq + 2 * hkv) * dim, "rope_kv_paged: packed row too short")
    _require(positions.dtype == torch.int32 and slots.dtype == torch.int32, "rope_kv_paged: int32 metadata")
    _require(kcache.is_contiguous() and vcache.is_contiguous() and kcache.dim() == 4, "rope_kv_paged: cache layout")
    nb, ch, bs, cd = kcache.shape
    _require(ch == hkv and cd == dim, "rope_kv_paged: cache geometry differs from the heads")
    rc = kernels().ff_rope_kv_paged(ptr(qkv), ptr(positions), ptr(slots), ptr(kcache), ptr(vcache), ptr(inv_freq),
                                    rows, hq, hkv, dim, rot_dim or dim, bs, nb, c_float(theta), ld,
                                    ptr(status_tensor(qkv.device)), stream_ptr())
    check(rc, "ff_rope_kv_paged")
    _count()


def rope_table(positions: torch.Tensor, rot_dim: int, theta: float, inv_freq: torch.Tensor | None = None) -> torch.Tensor:
    """``[rows, rot_dim/2, 2]`` FP32 (cos, sin) of ``position * inv_freq``, rounded to BF16 as the rotation
    kernels round them. Computed once per step and shared by every layer's fused QKV epilogue."""
    rows = positions.shape[0]
    out = torch.empty(rows, rot_dim // 2, 2, dtype=torch.float32, device=positions.device)
    if not _is_cuda(positions):
        i = torch.arange(rot_dim // 2, dtype=torch.float32)
        inv = inv_freq.float() if inv_freq is not None else 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2 * i / rot_dim)
        ang = positions.float()[:, None] * inv[None, :]
        out[..., 0] = torch.cos(ang).to(BF16).float()
        out[..., 1] = torch.sin(ang).to(BF16).float()
        return out
    rc = kernels().ff_rope_table(ptr(positions), ptr(inv_freq), ptr(out), rows, rot_dim, c_float(theta), stream_ptr())
    check(rc, "ff_rope_table")
    _count()
    return out


def linear_rope_kv(x: torch.Tensor, wqkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                   kcache: torch.Tensor, vcache: torch.Tensor, hq: int, hkv: int, dim: int, theta: float,
                   rot_dim: int | None = None, inv_freq: torch.Tensor | None = None,
                   cos_sin: torch.Tensor | None = None) -> torch.Tensor:
    """Fused QKV projection + rotary embedding + paged KV write: ``qkv = x @ wqkv.T`` with Q and K
    rotated and K/V stored at ``slots``. Decode shapes with 128-dim heads run as one kernel (the
    rotation and the cache write are the GEMM's epilogue; ``cos_sin`` from :func:`rope_table` is
    reused across layers); everything else as GEMM + rope kernel."""
    m = x.shape[0]
    n = wqkv.shape[0]
    fused = (FUSE_ROPE and _is_cuda(x) and m <= SKINNY_MAX_M and dim == 128 and n == (hq + 2 * hkv) * 128 and x.dtype == BF16
             and kcache.dim() == 4 and kcache.is_contiguous() and vcache.is_contiguous())
    if not fused:
        qkv = linear(x, wqkv)
        rope_kv_paged(qkv, positions, slots, kcache, vcache, hq, hkv, dim, theta, rot_dim, inv_freq)
        return qkv
    _require(positions.dtype == torch.int32 and slots.dtype == torch.int32, "linear_rope_kv: int32 metadata")
    nb, ch, bs, cd = kcache.shape
    _require(ch == hkv and cd == dim, "linear_rope_kv: cache geometry differs from the heads")
    _, ldx = _rows2d(x)
    _, ldw = _rows2d(wqkv)
    k = x.shape[1]
    out = torch.empty(m, n, dtype=BF16, device=x.device)
    lib = kernels()
    scratch_b, counter_b = c_longlong(0), c_longlong(0)
    grid = lib.ff_gemm_skinny_plan_epi(m, n, k, 2, ctypes.byref(scratch_b), ctypes.byref(counter_b))
    check(min(grid, 0), "ff_gemm_skinny_plan_epi")
    ws = workspace(x.device)
    scratch = ws.ensure("gemm_scratch", scratch_b.value // 4) if scratch_b.value > 0 else None
    _require(counter_b.value // 4 <= ws.gemm_counters.numel(), "linear_rope_kv: too many column tiles for counters")
    if cos_sin is None:
        cos_sin = rope_table(positions, rot_dim or dim, theta, inv_freq)
    _require(cos_sin.shape == (m, (rot_dim or dim) // 2, 2) and cos_sin.is_contiguous(), "linear_rope_kv: cos/sin table shape")
    rc = lib.ff_gemm_skinny_rope_kv(ptr(x), ptr(wqkv), ptr(out), m, n, k, ldx, ldw, n, grid, ptr(scratch),
                                    ptr(ws.gemm_counters), ptr(cos_sin), ptr(slots), ptr(kcache), ptr(vcache),
                                    hq, hkv, rot_dim or dim, bs, nb, ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_gemm_skinny_rope_kv")
    _count()
    return out


def silu_mul(gu: torch.Tensor, mode: int = 0, limit: float = 0.0, out: torch.Tensor | None = None,
             interleaved: bool = False) -> torch.Tensor:
    if not _is_cuda(gu):
        if interleaved:
            m, n = gu.shape
            g = gu.view(m, n // 128, 2, 64)
            gu = torch.cat([g[:, :, 0].reshape(m, n // 2), g[:, :, 1].reshape(m, n // 2)], dim=1)
        return ref.silu_mul(gu, mode, limit)
    rows, ld = _rows2d(gu)
    f = gu.shape[1] // 2
    if out is None:
        out = torch.empty(rows, f, dtype=BF16, device=gu.device)
    rc = kernels().ff_silu_mul(ptr(gu), ptr(out), rows, f, ld, out.stride(0), mode, c_float(limit), int(interleaved), stream_ptr())
    check(rc, "ff_silu_mul")
    _count()
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    if not _is_cuda(x):
        return ref.softcap(x, cap)
    _require(x.is_contiguous() and x.dtype == BF16, "softcap: contiguous bf16")
    check(kernels().ff_softcap(ptr(x), c_longlong(x.numel()), c_float(cap), stream_ptr()), "ff_softcap")
    _count()
    return x


# ------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------
def attn_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                ctx_lens: torch.Tensor, hq: int, hkv: int, dim: int, scale: float, nq: int = 1,
                tree_mask: torch.Tensor | None = None, max_ctx: int | None = None,
                out: torch.Tensor | None = None, window: int = 0, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Decode / multi-row verify attention. ``q`` holds ``batch * nq`` rows (heads at columns
    ``h*dim``; it may be the packed QKV buffer). ``ctx_lens[b]`` counts the keys visible to the last
    of the ``nq`` rows. ``window > 0``: every row sees only its last ``window`` keys (local-attention
    layers; not together with a tree mask). ``sinks`` (float32 [hq]): learnable soft-max, one sink logit per head in the
    denominator. Returns ``[batch*nq, hq*dim]``."""
    batch = block_table.shape[0]
    _require(not (window > 0 and tree_mask is not None), "attn_decode: window and tree mask are exclusive")
    _require(not (sinks is not None and tree_mask is not None), "attn_decode: sinks and tree mask are exclusive")
    if not _is_cuda(q):
        q_start = torch.arange(batch, dtype=torch.int32) * nq
        q_lens = torch.full((batch,), nq, dtype=torch.int32)
        tm = None if tree_mask is None else tree_mask.view(batch, nq)
        return ref.attention_paged(q, kcache, vcache, block_table, q_start, q_lens, ctx_lens, hq, hkv, dim, scale, tm,
                                   window, sinks)
    rows, ldq = _rows2d(q)
    _require(rows == batch * nq, "attn_decode: q rows must equal batch * nq")
    _require(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attn_decode: block table int32")
    _require(ctx_lens.dtype == torch.int32, "attn_decode: ctx_lens int32")
    nb = kcache.shape[0]
    _require(kcache.shape[2] == 64 and kcache.shape[3] == dim == 128, "attn_decode: block 64 / head_dim 128 only")
    if max_ctx is None:
        max_ctx = block_table.shape[1] * 64
    lib = kernels()
    po, pml = c_longlong(0), c_longlong(0)
    nsplit = lib.ff_attn_decode_plan(batch, hq, hkv, nq, max_ctx, ctypes.byref(po), ctypes.byref(pml))
    ws = workspace(q.device)
    part_o = ws.ensure("attn_o", po.value // 4) if nsplit > 1 else None
    part_ml = ws.ensure("attn_ml", pml.value // 4) if nsplit > 1 else None
    if out is None:
        out = torch.empty(rows, hq * dim, dtype=BF16, device=q.device)
    if tree_mask is not None:
        _require(tree_mask.dtype == torch.int64 and tree_mask.numel() == batch * nq, "attn_decode: tree mask int64")
    # optionally the last split of a (sequence, kv head, row tile) merges in place of a second kernel; measured
    # slower on B200 (81.8 vs 75.6 us at batch 64 / context 1100: every CTA pays a fence and an atomic), so off
    items = batch * hkv * ((nq * (hq // hkv) + 15) // 16)
    counters = ws.attn_counters if (FUSE_ATTN_MERGE and nsplit > 1 and items <= ws.attn_counters.numel()) else None
    if sinks is not None:
        _require(sinks.dtype == torch.float32 and sinks.numel() == hq and sinks.is_contiguous(), "attn_decode: sinks float32 [hq]")
        counters = None
        rc = lib.ff_attn_decode_sink(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), ptr(ctx_lens), ptr(out),
                                     ptr(part_o), ptr(part_ml), batch, hq, hkv, dim, nq, ldq, block_table.shape[1], nb,
                                     nsplit, c_float(scale), max(window, 0), ptr(sinks), ptr(status_tensor(q.device)),
                                     stream_ptr())
    elif window > 0:
        rc = lib.ff_attn_decode_window(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), ptr(ctx_lens), ptr(out),
                                       ptr(part_o), ptr(part_ml), batch, hq, hkv, dim, nq, ldq, block_table.shape[1], nb,
                                       nsplit, c_float(scale), window, ptr(counters), ptr(status_tensor(q.device)),
                                       stream_ptr())
    else:
        rc = lib.ff_attn_decode(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), ptr(ctx_lens), ptr(tree_mask),
                                ptr(out), ptr(part_o), ptr(part_ml), batch, hq, hkv, dim, nq, ldq, block_table.shape[1],
                                nb, nsplit, c_float(scale), ptr(counters), ptr(status_tensor(q.device)), stream_ptr())
    check(rc, "ff_attn_decode")
    _count(1 if (nsplit == 1 or counters is not None) else 2)
    return out


def attn_decode_mixed(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, compact, layer: int,
                      block_table: torch.Tensor, ctx_lens: torch.Tensor, kv_start: torch.Tensor, group_table: torch.Tensor,
                      hq: int, hkv: int, dim: int, scale: float, max_ctx: int | None = None) -> torch.Tensor:
    """Decode attention (one query row per sequence) over a cache whose older keys are sealed in the 8-bit store
    ``compact`` (``engine.kv_compact.CompactKV``): keys ``[0, 64)`` and ``[kv_start[b], ctx)`` come from BF16 pages,
    keys ``[64, kv_start[b])`` from the sealed groups named by ``group_table[b]`` (dequantised as
    ``bf16(code * scale + lo)``). CUDA: the paged BF16 kernel writes its split partials, ``csrc/kv_affine8.cu`` adds
    one partial per chunk of sealed groups, one merge. Returns ``[batch, hq * dim]``."""
    batch = block_table.shape[0]
    max_groups = group_table.shape[1]
    if not _is_cuda(q):
        out = torch.zeros(batch, hq * dim, dtype=q.dtype)
        g = hq // hkv
        for b in range(batch):
            ctx, ks = int(ctx_lens[b]), int(kv_start[b])
            if ctx == 0:
                continue
            kk, vv = [], []
            for p0 in range(0, ctx, 64):
                n = min(64, ctx - p0)
                if p0 >= 64 and p0 < ks:
                    slot = int(group_table[b, p0 // 128])
                    kd, vd = compact.dequant(layer, slot)
                    o = p0 % 128
                    kk.append(kd[:, o: o + n]); vv.append(vd[:, o: o + n])
                else:
                    blk = int(block_table[b, p0 // 64])
                    kk.append(kcache[blk][:, :n].to(torch.bfloat16)); vv.append(vcache[blk][:, :n].to(torch.bfloat16))
            k = torch.cat(kk, 1).float(); v = torch.cat(vv, 1).float()            # [hkv, ctx, D]
            qb = q[b, : hq * dim].float().view(hkv, g, dim)
            sc = torch.einsum("hgd,htd->hgt", qb, k) * scale
            p = torch.softmax(sc, dim=-1)
            out[b] = torch.einsum("hgt,htd->hgd", p, v).reshape(hq * dim).to(q.dtype)
        return out
    rows, ldq = _rows2d(q)
    _require(rows == batch and dim == 128 and kcache.shape[2] == 64, "attn_decode_mixed: one row per sequence, block 64, d128")
    _require(block_table.dtype == torch.int32 and kv_start.dtype == torch.int32 and group_table.dtype == torch.int32
             and group_table.is_contiguous(), "attn_decode_mixed: int32 metadata")
    from ..engine.kv_compact import GROUPS_PER_CHUNK
    if max_ctx is None:
        max_ctx = block_table.shape[1] * 64
    lib = kernels()
    nsplit = lib.ff_attn_decode_plan(batch, hq, hkv, 1, max_ctx, None, None)
    chunks = (max_groups + GROUPS_PER_CHUNK - 1) // GROUPS_PER_CHUNK
    pstride = nsplit + chunks
    ws = workspace(q.device)
    part_o = ws.ensure("attn_o", batch * pstride * hq * dim)
    part_ml = ws.ensure("attn_ml", batch * pstride * hq * 2)
    out = torch.empty(rows, hq * dim, dtype=BF16, device=q.device)
    st = status_tensor(q.device)
    nb = kcache.shape[0]
    rc = lib.ff_attn_decode_partial(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), ptr(ctx_lens), ptr(kv_start),
                                    ptr(part_o), ptr(part_ml), batch, hq, hkv, dim, ldq, block_table.shape[1], nb, nsplit,
                                    pstride, c_float(scale), ptr(st), stream_ptr())
    check(rc, "ff_attn_decode_partial")
    rc = lib.ff_attn_sealed(ptr(q), ptr(compact.k_codes[layer]), ptr(compact.v_codes[layer]), ptr(compact.k_stats[layer]),
                            ptr(compact.v_stats[layer]), ptr(kcache), ptr(vcache), ptr(block_table), ptr(group_table),
                            ptr(kv_start), ptr(part_o), ptr(part_ml), batch, hq, hkv, dim, ldq, block_table.shape[1], nb,
                            max_groups, compact.slots, GROUPS_PER_CHUNK, nsplit, pstride, c_float(scale), ptr(st),
                            stream_ptr())
    check(rc, "ff_attn_sealed")
    rc = lib.ff_attn_merge(ptr(part_o), ptr(part_ml), ptr(out), batch, hq, pstride, stream_ptr())
    check(rc, "ff_attn_merge")
    _count(3)
    return out


def attn_prefill(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                 q_start: torch.Tensor, q_lens: torch.Tensor, ctx_lens: torch.Tensor, max_q_len: int, hq: int,
                 hkv: int, dim: int, scale: float, window: int = 0, out: torch.Tensor | None = None,
                 sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Causal chunked-prefill attention of packed query rows against the paged cache. ``window < 0`` makes it
    bidirectional: every query row sees all ``ctx_lens`` keys of its sequence (encoders, vision towers). ``sinks``
    (float32 [hq]): learnable soft-max, one sink logit per head in the denominator (tcgen05 kernel only)."""
    if not _is_cuda(q):
        return ref.attention_paged(q, kcache, vcache, block_table, q_start, q_lens, ctx_lens, hq, hkv, dim, scale,
                                   None, window, sinks)
    rows, ldq = _rows2d(q)
    batch = block_table.shape[0]
    if out is None:
        out = torch.empty(rows, hq * dim, dtype=BF16, device=q.device)
    nb = kcache.shape[0]
    _require(kcache.shape[2] == 64 and dim == 128, "attn_prefill: block 64 / head_dim 128 only")
    if sinks is not None:
        _require(sinks.dtype == torch.float32 and sinks.numel() == hq and sinks.is_contiguous(), "attn_prefill: sinks float32 [hq]")
        _require(out.stride(0) % 8 == 0 and ldq % 8 == 0, "attn_prefill: sinks need the tcgen05 kernel (16-byte aligned rows)")
    if (ATTN_PREFILL_TC or sinks is not None) and out.stride(0) % 8 == 0 and ldq % 8 == 0:
        # tcgen05 kernel: Q Kᵀ and P V on the tensor cores with S and O in tensor memory
        rc = kernels().ff_attn_prefill_tc(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), ptr(q_start), ptr(q_lens),
                                          ptr(ctx_lens), ptr(out), batch, rows, max_q_len, hq, hkv, dim, ldq, out.stride(0),
                                          block_table.shape[1], nb, c_float(scale), window, ptr(sinks),
                                          ptr(status_tensor(q.device)), stream_ptr())
        check(rc, "ff_attn_prefill_tc")
        _count()
        return out
    rc = kernels().ff_attn_prefill(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), ptr(q_start), ptr(q_lens),
                                   ptr(ctx_lens), ptr(out), batch, max_q_len, hq, hkv, dim, ldq, out.stride(0),
                                   block_table.shape[1], nb, c_float(scale), window, ptr(status_tensor(q.device)),
                                   stream_ptr())
    check(rc, "ff_attn_prefill")
    _count()
    return out


# ------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------
def argmax_rows(logits: torch.Tensor, out: torch.Tensor | None = None, id_offset: int = 0,
                out_vals: torch.Tensor | None = None) -> torch.Tensor:
    """Greedy token per row, ties -> lower id. ``out_vals`` additionally receives the row maxima
    (for merging vocab-parallel shards)."""
    if not _is_cuda(logits):
        ids = ref.argmax_rows(logits) + id_offset
        if out_vals is not None:
            out_vals.copy_(logits.to(torch.float32).max(-1).values)
        return ids
    rows, ld = _rows2d(logits)
    vocab = logits.shape[1]
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    dt = 0 if logits.dtype == BF16 else 1
    _require(logits.dtype in (BF16, torch.float32), "argmax_rows: bf16 or fp32 logits")
    rc = kernels().ff_argmax_rows(ptr(logits), ptr(out), ptr(out_vals), rows, vocab, ld, dt, id_offset, None,
                                  ptr(status_tensor(logits.device)), stream_ptr())
    check(rc, "ff_argmax_rows")
    _count()
    return out


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, step: int,
                rep_penalty: float = 1.0, history: torch.Tensor | None = None) -> torch.Tensor:
    """Stochastic sampler (temperature, top-k, top-p, repetition penalty, Philox4x32-10)."""
    if not _is_cuda(logits):
        return torch.tensor([ref.sample_row(logits[r], temperature, top_k, top_p, seed, step, r, rep_penalty,
                                            None if history is None else history[r])
                             for r in range(logits.shape[0])], dtype=torch.int32)
    lg = logits.to(torch.float32).contiguous()
    rows, vocab = lg.shape
    work = torch.empty_like(lg)
    out = torch.empty(rows, dtype=torch.int32, device=lg.device)
    hl = 0 if history is None else history.shape[1]
    rc = kernels().ff_sample_rows(ptr(lg), ptr(out), ptr(work), rows, vocab, c_float(temperature), top_k,
                                  c_float(top_p), c_float(rep_penalty), ptr(history), hl, c_ulonglong(seed),
                                  c_ulonglong(step), stream_ptr())
    check(rc, "ff_sample_rows")
    _count()
    return out


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, heads: int, dim: int, theta: float,
                 inv_freq: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate-half RoPE on a standalone [rows, heads*dim] tensor (no cache write); same numerics
    contract as :func:`rope_kv_paged`."""
    if not _is_cuda(x):
        rows = x.shape[0]
        y = ref.rope_rotate_half(x[:, : heads * dim].reshape(rows, heads, dim), positions, theta, None, inv_freq)
        x[:, : heads * dim] = y.reshape(rows, -1)
        return x
    rows, ld = _rows2d(x)
    _require(dim % 16 == 0 and positions.dtype == torch.int32, "rope_inplace: dim % 16 == 0, int32 positions")
    rc = kernels().ff_rope_kv_paged(ptr(x), ptr(positions), None, None, None, ptr(inv_freq), rows, heads, 0, dim, dim, 64, 0,
                                    c_float(theta), ld, ptr(status_tensor(x.device)), stream_ptr())
    check(rc, "ff_rope_kv_paged(rope only)")
    _count()
    return x
