"""Decode-step projection chain (``csrc/gemm_chain.cu``): the projections of a dense decoder layer
and the residual-add + RMSNorm steps between them as one persistent kernel launch.

``layer_chain`` takes the attention output of layer ``i`` and returns the final-normed activations
(after the last layer) or the rotated, cache-written QKV rows of layer ``i + 1``. The phases are
ordered inside the kernel by device counters; the buffers those counters and the stream-K partial
sums live in are allocated once per device here and must be zero before the first launch
(:func:`reset_workspace` restores that state after a failed step).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .lib import check, kernels, ptr, status_tensor, stream_ptr

# Off unless FLYINGFISH_CHAIN=1: on one B200 the chain measured 7.2 ms per Llama-3-8B-shape decode step (batch 64)
# against 6.2 ms for the operator-by-operator path (4.4 against 4.0 ms at batch 1): every phase boundary costs
# dependent L2 round trips (publish partials -> reduce -> publish rows -> activation load) of about 2 us each, which
# the weight look-ahead does not hide, while separately launched kernels overlap theirs through programmatic
# dependent launch.
ENABLED = os.environ.get("FLYINGFISH_CHAIN", "0") == "1"
MAX_ROWS = 128
MAX_HIDDEN = 8192


class _Phase(ctypes.Structure):
    _fields_ = [("kind", c_int), ("epi", c_int), ("N", c_int), ("K", c_int),
                ("X", c_void_p), ("ldx", c_int), ("W", c_void_p), ("ldw", c_int), ("Y", c_void_p), ("ldy", c_int),
                ("nx", c_void_p), ("res", c_void_p), ("nw", c_void_p), ("eps", c_float), ("unit_offset", c_int)]


class _Rope(ctypes.Structure):
    _fields_ = [("cos_sin", c_void_p), ("slots", c_void_p), ("kcache", c_void_p), ("vcache", c_void_p),
                ("hq", c_int), ("hkv", c_int), ("rot_dim", c_int), ("block_size", c_int), ("num_blocks", c_int)]


class _Workspace:
    def __init__(self, device: torch.device):
        sb, cb, yb = c_longlong(0), c_longlong(0), c_longlong(0)
        check(kernels().ff_decode_chain_workspace(MAX_ROWS, ctypes.byref(sb), ctypes.byref(cb), ctypes.byref(yb)),
              "ff_decode_chain_workspace")
        self.scratch = torch.empty(sb.value // 4, dtype=torch.float32, device=device)
        self.counters = torch.zeros(cb.value // 4, dtype=torch.int32, device=device)
        self.sync = torch.zeros(yb.value // 4, dtype=torch.int32, device=device)


_workspaces: dict[int, _Workspace] = {}


def _ws(device: torch.device) -> _Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _workspaces.get(idx)
    if w is None:
        w = _Workspace(torch.device("cuda", idx))
        _workspaces[idx] = w
    return w


def reset_workspace(device: torch.device | None = None) -> None:
    """Zero the phase counters (after a step that ended with a device-side time-out)."""
    for idx, w in _workspaces.items():
        if device is None or device.index in (None, idx):
            w.counters.zero_()
            w.sync.zero_()


def gemm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, epi: int = 0) -> _Phase:
    p = _Phase()
    p.kind, p.epi, p.N, p.K = 0, epi, w.shape[0], w.shape[1]
    p.X, p.ldx, p.W, p.ldw, p.Y, p.ldy = x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), y.data_ptr(), y.stride(0)
    return p


def add_norm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float,
             unit_offset: bool = False) -> _Phase:
    p = _Phase()
    p.kind, p.N = 1, res.shape[1]
    p.nx, p.res, p.nw, p.Y, p.eps, p.unit_offset = x.data_ptr(), res.data_ptr(), w.data_ptr(), out.data_ptr(), eps, int(unit_offset)
    return p


def run(phases: list[_Phase], rows: int, device: torch.device, rope: _Rope | None = None) -> None:
    ws = _ws(device)
    arr = (_Phase * len(phases))(*phases)
    rc = kernels().ff_decode_chain(arr, len(phases), rows, ctypes.byref(rope) if rope is not None else None,
                                   ptr(ws.scratch), ptr(ws.counters), ptr(ws.sync), ptr(status_tensor(device)),
                                   stream_ptr())
    check(rc, "ff_decode_chain")


def layer_chain(attn_out: torch.Tensor, res: torch.Tensor, wo: torch.Tensor, post_ln: torch.Tensor, wgu: torch.Tensor,
                wdown: torch.Tensor, next_ln: torch.Tensor, eps: float, next_wqkv: torch.Tensor | None = None,
                rope: dict | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """O projection -> add + norm -> gate/up with SwiGLU -> down -> add + norm [-> next layer's QKV projection with
    rotary embedding and KV-cache write]. ``res`` (the residual stream) is updated in place. Returns (normed
    activations, next layer's QKV rows or None)."""
    m, dev = attn_out.shape[0], attn_out.device
    hidden = res.shape[1]
    bf = torch.bfloat16
    tmp = torch.empty(m, hidden, dtype=bf, device=dev)
    n1 = torch.empty(m, hidden, dtype=bf, device=dev)
    hmid = torch.empty(m, wgu.shape[0] // 2, dtype=bf, device=dev)
    n2 = torch.empty(m, hidden, dtype=bf, device=dev)
    phases = [gemm(attn_out, wo, tmp), add_norm(tmp, res, post_ln, n1, eps), gemm(n1, wgu, hmid, epi=1),
              gemm(hmid, wdown, tmp), add_norm(tmp, res, next_ln, n2, eps)]
    qkv, rp = None, None
    if next_wqkv is not None:
        qkv = torch.empty(m, next_wqkv.shape[0], dtype=bf, device=dev)
        phases.append(gemm(n2, next_wqkv, qkv, epi=2))
        kc, vc = rope["kcache"], rope["vcache"]
        rp = _Rope()
        rp.cos_sin, rp.slots, rp.kcache, rp.vcache = rope["cos_sin"].data_ptr(), rope["slots"].data_ptr(), kc.data_ptr(), vc.data_ptr()
        rp.hq, rp.hkv, rp.rot_dim, rp.block_size, rp.num_blocks = rope["hq"], rope["hkv"], rope["rot_dim"], kc.shape[2], kc.shape[0]
    run(phases, m, dev, rp)
    return n2, qkv
