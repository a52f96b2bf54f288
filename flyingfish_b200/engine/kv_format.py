"""KV cache formats: ``bf16`` (paged, the default) and ``affine8`` (8-bit codes for everything older than
64 sink + 2048 recent tokens, which stay BF16 in a ring). Geometry, byte accounting and the pack/unpack
operators; mirrors src/kv.rs:5-133 and kernels/kv_cache.cuh of the reference (format identities, sealed
boundary, ring slots, compact block sizes).

The attention kernels of this engine read BF16 pages; ``Affine8Store`` is the compact store behind them:
``seal`` packs every group that has left the recent window, ``materialise`` rebuilds BF16 rows for a token
range (used when a sequence is paged back in or handed to another rank)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

SINK_TOKENS, RECENT_TOKENS, GROUP_TOKENS, TENTATIVE_TOKENS = 64, 2048, 128, 5   # tentative = most rows one verify step appends
RING_TOKENS = SINK_TOKENS + RECENT_TOKENS + GROUP_TOKENS - 1 + TENTATIVE_TOKENS
TAGS = {"bf16": "BF16", "affine8": "UINT8_KC128_VT_F32_S64_R2048_MUL_ADD_BF16_RNE_V1"}


def from_tag(tag: str) -> str:
    for name, t in TAGS.items():
        if t == tag:
            return name
    raise ValueError("unknown KV format identity")


def sealed_until(committed: int) -> int:
    """Tokens below this position are (or may be) stored as codes: whole 128-token groups older than the
    recent window."""
    return max(0, committed - RECENT_TOKENS) // GROUP_TOKENS * GROUP_TOKENS


def ring_slot(position: int, ring: int) -> int:
    if not (ring > 0 and (position < ring or ring > SINK_TOKENS)):
        raise ValueError("KV ring cannot address position")
    if position < SINK_TOKENS:
        return position
    return SINK_TOKENS + (position - SINK_TOKENS) % (ring - SINK_TOKENS)


@dataclass(frozen=True)
class KvLayout:
    capacity: int
    ring: int
    ring_elements: int      # per K and per V, BF16 elements
    codes: int              # per K and per V, bytes
    k_stats: int            # FP32 values
    v_stats: int
    bytes: int


def layout(fmt: str, capacity: int, heads: int, dim: int) -> KvLayout:
    if capacity <= 0 or heads <= 0 or dim <= 0:
        raise ValueError("empty KV layout")
    if capacity > (1 << 48):
        raise ValueError("KV size overflow")
    if fmt == "bf16":
        ring, codes, k_stats, v_stats = capacity, 0, 0, 0
    elif fmt == "affine8":
        ring = min(capacity, RING_TOKENS)
        codes = heads * capacity * dim
        k_stats = heads * -(-capacity // GROUP_TOKENS) * dim * 2
        v_stats = heads * capacity * 2
    else:
        raise ValueError(f"unknown KV format {fmt}")
    ring_elements = heads * ring * dim
    nbytes = ring_elements * 4 + codes * 2 + (k_stats + v_stats) * 4 + (0 if fmt == "bf16" else 16)
    return KvLayout(capacity, ring, ring_elements, codes, k_stats, v_stats, nbytes)


def block_bytes(fmt: str, start: int, tokens: int, prefix: int, heads: int, dim: int) -> int:
    """Bytes a prefix block [start, start + tokens) of a committed prefix occupies when exported."""
    end = start + tokens
    if not (tokens > 0 and end <= prefix):
        raise ValueError("KV block outside prefix")
    if fmt == "bf16":
        return heads * tokens * dim * 4
    if start % GROUP_TOKENS:
        raise ValueError("compact KV block must start on a 128-token group")
    sealed = sealed_until(prefix)
    live = sum(1 for p in range(start, end) if p < SINK_TOKENS or p >= sealed)
    encoded = max(0, min(end, sealed) - start)
    stats = encoded // GROUP_TOKENS * dim * 2 + encoded * 2
    return heads * (encoded * dim * 2 + stats * 4 + live * dim * 4)


# ---- pack / unpack --------------------------------------------------------------------------------
def _pack_ref(x: torch.Tensor, dims: tuple[int, ...]):
    xf = x.float()
    lo = xf.amin(dims, keepdim=True); hi = xf.amax(dims, keepdim=True)
    span = hi - lo
    scale = torch.where(span == 0, torch.ones_like(span), span / 255.0)
    codes = torch.clamp((xf - lo) / scale, 0, 255).round().to(torch.uint8)     # round(): half to even, as cvt.rni
    return codes, lo, scale


def pack_k(src: torch.Tensor, codes: torch.Tensor, stats: torch.Tensor, group0: int, groups: int) -> None:
    """src [heads, capacity, D] bf16 -> codes [heads, capacity, D] uint8, stats [heads, G, D, 2] f32 for groups
    [group0, group0 + groups)."""
    heads, cap, d = src.shape
    if not src.is_cuda:
        for g in range(group0, group0 + groups):
            sl = slice(g * GROUP_TOKENS, (g + 1) * GROUP_TOKENS)
            c, lo, sc = _pack_ref(src[:, sl], (1,))
            codes[:, sl] = c
            stats[:, g, :, 0] = lo[:, 0]; stats[:, g, :, 1] = sc[:, 0]
        return
    from ..ops import _count
    from ..ops.lib import check, kernels, ptr, status_tensor, stream_ptr
    rc = kernels().ff_kv_pack_k(ptr(src), ptr(codes), ptr(stats), heads, cap, d, group0, groups,
                                ptr(status_tensor(src.device)), stream_ptr())
    check(rc, "ff_kv_pack_k")
    _count()


def pack_v(src: torch.Tensor, codes: torch.Tensor, stats: torch.Tensor, pos0: int, tokens: int) -> None:
    """Per-token statistics: stats [heads, capacity, 2]."""
    heads, cap, d = src.shape
    if not src.is_cuda:
        sl = slice(pos0, pos0 + tokens)
        c, lo, sc = _pack_ref(src[:, sl], (2,))
        codes[:, sl] = c
        stats[:, sl, 0] = lo[..., 0]; stats[:, sl, 1] = sc[..., 0]
        return
    from ..ops import _count
    from ..ops.lib import check, kernels, ptr, status_tensor, stream_ptr
    rc = kernels().ff_kv_pack_v(ptr(src), ptr(codes), ptr(stats), heads, cap, d, pos0, tokens,
                                ptr(status_tensor(src.device)), stream_ptr())
    check(rc, "ff_kv_pack_v")
    _count()


def unpack(codes: torch.Tensor, stats: torch.Tensor, dst: torch.Tensor, pos0: int, tokens: int, is_k: bool) -> None:
    heads, cap, d = codes.shape
    if not codes.is_cuda:
        sl = slice(pos0, pos0 + tokens)
        c = codes[:, sl].float()
        if is_k:
            g = torch.arange(pos0, pos0 + tokens) // GROUP_TOKENS
            lo, sc = stats[:, g, :, 0], stats[:, g, :, 1]
        else:
            lo, sc = stats[:, sl, 0:1], stats[:, sl, 1:2]
        dst[:, sl] = (c * sc + lo).to(torch.bfloat16)
        return
    from ..ops import _count
    from ..ops.lib import check, kernels, ptr, stream_ptr
    rc = kernels().ff_kv_unpack(ptr(codes), ptr(stats), ptr(dst), heads, cap, d, pos0, tokens, int(is_k), stream_ptr())
    check(rc, "ff_kv_unpack")
    _count()


class Affine8Store:
    """Compact K/V of one layer and sequence: codes + statistics for sealed groups."""

    def __init__(self, heads: int, capacity: int, dim: int, device):
        groups = -(-capacity // GROUP_TOKENS)
        self.heads, self.capacity, self.dim = heads, capacity, dim
        self.k_codes = torch.zeros(heads, capacity, dim, dtype=torch.uint8, device=device)
        self.v_codes = torch.zeros_like(self.k_codes)
        self.k_stats = torch.zeros(heads, groups, dim, 2, dtype=torch.float32, device=device)
        self.v_stats = torch.zeros(heads, capacity, 2, dtype=torch.float32, device=device)
        self.sealed = 0

    def seal(self, k_full: torch.Tensor, v_full: torch.Tensor, committed: int) -> int:
        """Pack every group that left the recent window; k_full / v_full [heads, capacity, D] bf16. Returns the
        new sealed boundary."""
        target = sealed_until(committed)
        if target > self.sealed:
            g0, g1 = self.sealed // GROUP_TOKENS, target // GROUP_TOKENS
            pack_k(k_full, self.k_codes, self.k_stats, g0, g1 - g0)
            pack_v(v_full, self.v_codes, self.v_stats, self.sealed, target - self.sealed)
            self.sealed = target
        return self.sealed

    def materialise(self, k_out: torch.Tensor, v_out: torch.Tensor, pos0: int, tokens: int) -> None:
        """BF16 rows of sealed tokens [pos0, pos0 + tokens) (positions below 64 are never read from codes by
        the attention path: the sink stays BF16)."""
        assert pos0 + tokens <= self.sealed
        unpack(self.k_codes, self.k_stats, k_out, pos0, tokens, True)
        unpack(self.v_codes, self.v_stats, v_out, pos0, tokens, False)
