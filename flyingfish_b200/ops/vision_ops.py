"""Vision-tower and 3-D compute operators. CUDA: ``csrc/vision.cu`` (plus the table-driven rotary entry of
``csrc/rope_act_sample.cu`` and the bidirectional mode of the paged prefill attention); CPU: FP32 oracles that
restate the same arithmetic. Reference counterparts: kernels/vision_ops.cu (bias + GELU variants, sparse gathers,
rotary_spatial_f32), src/sparse.rs (site tables), src/convrot.rs:1-60 (Hadamard rotate-quantise INT8 linear).
No graphics API is involved anywhere: everything here is plain compute."""
from __future__ import annotations

import math
from ctypes import c_float, c_longlong

import torch

from . import _count, _require, linear
from .lib import check, kernels, ptr, status_tensor, stream_ptr

BF16 = torch.bfloat16
ACTS = {"none": 0, "gelu_tanh": 1, "quick_gelu": 2, "gelu": 3, "silu": 4, "relu": 5}


def _r(x: torch.Tensor) -> torch.Tensor:
    return x.to(BF16).float()


# ------------------------------------------------------------------------------------------------
# dense tower pieces
# ------------------------------------------------------------------------------------------------
def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, eps: float) -> torch.Tensor:
    """[rows, hidden] bf16 -> bf16; statistics in FP32, one rounding."""
    if not x.is_cuda:
        xf = x.float()
        mean = xf.mean(-1, keepdim=True)
        var = ((xf - mean) ** 2).mean(-1, keepdim=True)
        y = (xf - mean) * torch.rsqrt(var + eps) * w.float()
        return (y + b.float() if b is not None else y).to(x.dtype)
    rows, hidden = x.shape
    _require(x.dtype == BF16 and x.stride(1) == 1 and w.is_contiguous() and (b is None or b.is_contiguous()),
             "layernorm: bf16 rows")
    y = torch.empty(rows, hidden, dtype=BF16, device=x.device)
    rc = kernels().ff_layernorm(ptr(x), ptr(w), ptr(b), ptr(y), rows, hidden, x.stride(0), hidden, c_float(eps), stream_ptr())
    check(rc, "ff_layernorm")
    _count()
    return y


def act_ref(x: torch.Tensor, act: str) -> torch.Tensor:
    if act == "gelu_tanh":
        return 0.5 * x * (1 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    if act == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if act == "gelu":
        return 0.5 * x * (1 + torch.erf(x * 0.7071067811865476))
    if act == "silu":
        return x * torch.sigmoid(x)
    if act == "relu":
        return torch.relu(x)
    return x


def bias_act_(x: torch.Tensor, bias: torch.Tensor | None, act: str = "none") -> torch.Tensor:
    """In place: ``x = act(bf16(x + bias))``."""
    if not x.is_cuda:
        s = _r(x.float() + (bias.float() if bias is not None else 0.0))
        x.copy_(act_ref(s, act).to(x.dtype))
        return x
    rows, n = x.shape
    _require(x.dtype == BF16 and x.stride(1) == 1 and (bias is None or bias.is_contiguous()), "bias_act: bf16 rows")
    rc = kernels().ff_bias_act(ptr(x), ptr(bias), c_longlong(rows), n, x.stride(0), ACTS[act], stream_ptr())
    check(rc, "ff_bias_act")
    _count()
    return x


def sigmoid_gate(a: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``bf16(a * sigmoid(gate))`` row-wise; ``gate`` may be a column slice of a wider projection."""
    if not a.is_cuda:
        return (a.float() * torch.sigmoid(gate.float())).to(a.dtype)
    rows, n = a.shape
    _require(a.dtype == BF16 and gate.dtype == BF16 and a.stride(1) == 1 and gate.stride(1) == 1 and gate.shape == a.shape,
             "sigmoid_gate: bf16 rows")
    y = torch.empty(rows, n, dtype=BF16, device=a.device)
    rc = kernels().ff_sigmoid_gate(ptr(a), ptr(gate), ptr(y), c_longlong(rows), n, a.stride(0), gate.stride(0), n, stream_ptr())
    check(rc, "ff_sigmoid_gate")
    _count()
    return y


def group_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, groups: int, eps: float = 1e-5, act: str = "none") -> torch.Tensor:
    """Group normalisation of channels-last activations ``x`` [n, positions, C] (BF16): statistics over the positions and
    the ``C / groups`` channels of a group, per sample; then ``act(y * w + b)``. ``w`` / ``b``: [C] FP32."""
    n, positions, c = x.shape
    if not x.is_cuda:
        xf = x.float().reshape(n, positions, groups, c // groups)
        mean = xf.mean(dim=(1, 3), keepdim=True)
        var = ((xf - mean) ** 2).mean(dim=(1, 3), keepdim=True)
        y = ((xf - mean) * torch.rsqrt(var + eps)).reshape(n, positions, c) * w.float() + (b.float() if b is not None else 0.0)
        return act_ref(y, act).to(x.dtype)
    _require(x.dtype == BF16 and x.is_contiguous() and w.dtype == torch.float32 and c % groups == 0 and c % 8 == 0, "group_norm: layout")
    y = torch.empty_like(x)
    part = torch.empty(n * groups * 64 * 2, dtype=torch.float32, device=x.device)
    rc = kernels().ff_group_norm(ptr(x), ptr(w), ptr(b), ptr(y), ptr(part), n, positions, c, groups, c_float(eps), ACTS[act], stream_ptr())
    check(rc, "ff_group_norm")
    _count(2)
    return y


def conv3d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, act: str = "none") -> torch.Tensor:
    """Dense 3-D convolution, stride 1, "same" padding, channels-last: ``x`` [n, D, H, W, C] BF16, ``weight``
    [C_out, C, k, k, k] -> [n, D, H, W, C_out]. CUDA: the taps are gathered into rows (im2col) and one tensor-core GEMM
    against the weight in (tap, channel) order does the rest; the bias and activation follow in one pass."""
    n, d, h, w_, c = x.shape
    co, ci, k = weight.shape[0], weight.shape[1], weight.shape[2]
    _require(ci == c and weight.shape[3] == k and weight.shape[4] == k and k % 2 == 1, "conv3d: weight [C_out, C, k, k, k], odd k")
    pad = k // 2
    if not x.is_cuda:
        y = torch.nn.functional.conv3d(x.float().permute(0, 4, 1, 2, 3), weight.float(), None, padding=pad).permute(0, 2, 3, 4, 1)
        y = _r(y)
        if bias is not None or act != "none":
            y = act_ref(_r(y + (bias.float() if bias is not None else 0.0)), act)
        return y.to(x.dtype)
    _require(x.dtype == BF16 and x.is_contiguous() and c % 8 == 0, "conv3d: bf16 channels-last input, C % 8 == 0")
    rows = n * d * h * w_
    cols = torch.empty(rows, k * k * k * c, dtype=BF16, device=x.device)
    rc = kernels().ff_im2col3d(ptr(x), ptr(cols), n, d, h, w_, c, k, pad, stream_ptr())
    check(rc, "ff_im2col3d")
    _count()
    wmat = weight.permute(0, 2, 3, 4, 1).reshape(co, k * k * k * c).to(BF16).contiguous()
    y = linear_bias_act(cols, wmat, bias.to(BF16).contiguous() if bias is not None else None, act)
    return y.reshape(n, d, h, w_, co)


def neighborhood_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel: int) -> torch.Tensor:
    """2-D neighbourhood attention: ``q``, ``k``, ``v`` [n, H, W, heads, d] BF16; the query at (i, j) attends to the
    ``kernel x kernel`` keys of the window centred on it, shifted inwards at the borders (always ``kernel ** 2`` keys)."""
    n, h, w, heads, d = q.shape
    _require(kernel % 2 == 1 and kernel <= h and kernel <= w, "neighborhood_attention: odd window inside the grid")
    if not q.is_cuda:
        qf, kf, vf = q.float(), k.float(), v.float()
        out = torch.empty_like(qf)
        i0 = (torch.arange(h) - kernel // 2).clamp(0, h - kernel)
        j0 = (torch.arange(w) - kernel // 2).clamp(0, w - kernel)
        for i in range(h):
            for j in range(w):
                kk = kf[:, i0[i]: i0[i] + kernel, j0[j]: j0[j] + kernel].reshape(n, kernel * kernel, heads, d)
                vv = vf[:, i0[i]: i0[i] + kernel, j0[j]: j0[j] + kernel].reshape(n, kernel * kernel, heads, d)
                sc = torch.einsum("nhd,nkhd->nhk", qf[:, i, j], kk) / math.sqrt(d)
                out[:, i, j] = torch.einsum("nhk,nkhd->nhd", torch.softmax(sc, -1), vv)
        return out.to(q.dtype)
    _require(q.dtype == BF16 and q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and d % 32 == 0 and d <= 256,
             "neighborhood_attention: contiguous bf16, head width a multiple of 32 up to 256")
    out = torch.empty_like(q)
    rc = kernels().ff_neighborhood_attn(ptr(q), ptr(k), ptr(v), ptr(out), n, h, w, heads, d, kernel, c_float(1.0 / math.sqrt(d)), stream_ptr())
    check(rc, "ff_neighborhood_attn")
    _count()
    return out


def linear_bias_act(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, act: str = "none") -> torch.Tensor:
    y = linear(x, w)
    if bias is None and act == "none":
        return y
    return bias_act_(y, bias, act)


def rotary_2d_table(rows_hw: torch.Tensor, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """(row, column) positions [tokens, 2] -> cos/sin table [tokens, dim/2, 2] FP32 (BF16-rounded values) of the
    2-D rotary scheme of Qwen-style vision towers: the first dim/4 frequencies turn with the row index, the next
    dim/4 with the column index; pairs are (i, i + dim/2) ("rotate half")."""
    quarter = dim // 4
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), torch.arange(quarter, dtype=torch.float32) * 2 / (dim // 2))
    pos = rows_hw.float().cpu()
    ang = torch.cat([pos[:, :1] * inv[None, :], pos[:, 1:2] * inv[None, :]], dim=1)        # [tokens, dim/2]
    tab = torch.stack([_r(torch.cos(ang)), _r(torch.sin(ang))], dim=-1).contiguous()
    return tab.to(rows_hw.device)


def rope_table_apply_(qkv: torch.Tensor, table: torch.Tensor, heads: int, dim: int, rot_dim: int | None = None,
                      slots: torch.Tensor | None = None, kcache: torch.Tensor | None = None,
                      vcache: torch.Tensor | None = None, kv_heads: int = 0) -> None:
    """In place: rotates the first ``heads + kv_heads`` heads of every packed row by the per-row cos/sin ``table``
    ([rows, rot_dim/2, 2]); with ``slots`` the K and V heads are also written into the paged layout
    ``[blocks, kv_heads, 64, dim]``. BF16 arithmetic like the decoder's rotary kernel."""
    rot = rot_dim or dim
    rows = qkv.shape[0]
    if not qkv.is_cuda:
        half = rot // 2
        nrot = heads + kv_heads
        x = qkv[:, : nrot * dim].reshape(rows, nrot, dim).to(torch.float32, copy=True)
        cs, sn = table[..., 0][:, None, :], table[..., 1][:, None, :]
        x1, x2 = x[..., :half].clone(), x[..., dim // 2: dim // 2 + half].clone()
        x[..., :half] = _r(_r(x1 * cs) - _r(x2 * sn))
        x[..., dim // 2: dim // 2 + half] = _r(_r(x2 * cs) + _r(x1 * sn))
        qkv[:, : nrot * dim] = x.reshape(rows, -1).to(qkv.dtype)
        if slots is not None:
            bs = kcache.shape[2]
            ok = slots >= 0
            blk, off = (slots[ok] // bs).long(), (slots[ok] % bs).long()
            k = qkv[:, heads * dim: (heads + kv_heads) * dim].reshape(rows, kv_heads, dim)
            v = qkv[:, (heads + kv_heads) * dim: (heads + 2 * kv_heads) * dim].reshape(rows, kv_heads, dim)
            kcache[blk, :, off, :] = k[ok]
            vcache[blk, :, off, :] = v[ok]
        return
    _require(qkv.dtype == BF16 and qkv.stride(1) == 1 and table.is_contiguous() and table.dtype == torch.float32
             and table.shape == (rows, rot // 2, 2), "rope_table_apply: layout")
    nb, bs = (kcache.shape[0], kcache.shape[2]) if kcache is not None else (0, 64)
    rc = kernels().ff_rope_kv_paged_table(ptr(qkv), ptr(table), ptr(slots), ptr(kcache), ptr(vcache), rows, heads,
                                          kv_heads if slots is not None else 0, dim, rot, bs, nb, qkv.stride(0),
                                          ptr(status_tensor(qkv.device)), stream_ptr())
    check(rc, "ff_rope_kv_paged_table")
    _count()


# ------------------------------------------------------------------------------------------------
# sparse voxel operators
# ------------------------------------------------------------------------------------------------
def voxelize(points: torch.Tensor, batch: torch.Tensor | None, origin: tuple[float, float, float], voxel: float,
             dims: tuple[int, int, int]) -> torch.Tensor:
    """points [n, 3] f32 -> coords [n, 4] int32 (batch, x, y, z), all -1 for points outside the grid."""
    n = points.shape[0]
    if not points.is_cuda:
        inv = torch.tensor(1.0 / voxel, dtype=torch.float32)
        c = torch.floor((points.float() - torch.tensor(origin, dtype=torch.float32)) * inv).to(torch.int32)
        inside = ((c >= 0) & (c < torch.tensor(dims, dtype=torch.int32))).all(-1)
        b = batch.to(torch.int32) if batch is not None else torch.zeros(n, dtype=torch.int32)
        out = torch.cat([b[:, None], c], dim=1)
        out[~inside] = -1
        return out
    _require(points.dtype == torch.float32 and points.is_contiguous(), "voxelize: f32 points")
    out = torch.empty(n, 4, dtype=torch.int32, device=points.device)
    rc = kernels().ff_voxelize(ptr(points), ptr(batch), n, c_float(origin[0]), c_float(origin[1]), c_float(origin[2]),
                               c_float(voxel), dims[0], dims[1], dims[2], ptr(out), stream_ptr())
    check(rc, "ff_voxelize")
    _count()
    return out


class VoxelHash:
    """Coordinate -> lowest row index table over ``coords`` [n, 4] int32 (rows with negative entries are skipped)."""

    def __init__(self, coords: torch.Tensor):
        self.coords = coords.contiguous()
        self.n = coords.shape[0]
        self.cuda = coords.is_cuda
        if not self.cuda:
            self.table: dict[tuple, int] = {}
            for i, c in enumerate(self.coords.tolist()):
                if min(c) >= 0:
                    self.table.setdefault(tuple(c), i)
            return
        self.capacity = 1 << max(4, math.ceil(math.log2(max(2 * self.n, 2))))
        self.keys = torch.empty(self.capacity, dtype=torch.int64, device=coords.device)
        self.vals = torch.empty(self.capacity, dtype=torch.int32, device=coords.device)
        rc = kernels().ff_voxel_hash_build(ptr(self.coords), self.n, ptr(self.keys), ptr(self.vals), self.capacity,
                                           ptr(status_tensor(coords.device)), stream_ptr())
        check(rc, "ff_voxel_hash_build")
        _count()

    def first_mask(self) -> torch.Tensor:
        """bool [n]: row is the first (lowest index) holder of its coordinate -> unique sites in input order."""
        if not self.cuda:
            m = torch.zeros(self.n, dtype=torch.bool)
            for i in self.table.values():
                m[i] = True
            return m
        first = torch.empty(self.n, dtype=torch.int32, device=self.coords.device)
        rc = kernels().ff_voxel_first(ptr(self.coords), self.n, ptr(self.keys), ptr(self.vals), self.capacity, ptr(first),
                                      stream_ptr())
        check(rc, "ff_voxel_first")
        _count()
        return first.bool()

    def neighbor_map(self, offsets: torch.Tensor, query: torch.Tensor | None = None) -> torch.Tensor:
        """offsets [n_off, 3] -> int32 [n_off, m]: row of the site at query[i] + offset (same batch) or -1."""
        q = (self.coords if query is None else query).contiguous()
        m, n_off = q.shape[0], offsets.shape[0]
        if not self.cuda:
            out = torch.full((n_off, m), -1, dtype=torch.int32)
            ql = q.tolist()
            for o, d in enumerate(offsets.tolist()):
                for i, c in enumerate(ql):
                    if min(c) < 0:
                        continue
                    out[o, i] = self.table.get((c[0], c[1] + d[0], c[2] + d[1], c[3] + d[2]), -1)
            return out
        off4 = torch.zeros(n_off, 4, dtype=torch.int32, device=q.device)
        off4[:, 1:] = offsets.to(torch.int32).to(q.device)
        out = torch.empty(n_off, m, dtype=torch.int32, device=q.device)
        rc = kernels().ff_voxel_neighbor_map(ptr(q), m, ptr(off4), n_off, ptr(self.keys), ptr(self.vals), self.capacity,
                                             ptr(out), stream_ptr())
        check(rc, "ff_voxel_neighbor_map")
        _count()
        return out


def cube_offsets(k: int = 3) -> torch.Tensor:
    r = range(-(k // 2), k // 2 + 1)
    return torch.tensor([(x, y, z) for x in r for y in r for z in r], dtype=torch.int32)


def sparse_gather(feat: torch.Tensor, nbr: torch.Tensor) -> torch.Tensor:
    """feat [n_src, C] bf16, nbr [n_off, n] -> [n, n_off * C]: block o of row i is feat[nbr[o, i]] (zeros for -1)."""
    n_off, n = nbr.shape
    c = feat.shape[1]
    if not feat.is_cuda:
        out = torch.zeros(n, n_off, c, dtype=feat.dtype)
        for o in range(n_off):
            ok = nbr[o] >= 0
            out[ok, o] = feat[nbr[o][ok].long()]
        return out.reshape(n, n_off * c)
    _require(feat.dtype == BF16 and feat.is_contiguous() and nbr.is_contiguous() and c % 8 == 0, "sparse_gather: layout")
    out = torch.empty(n, n_off * c, dtype=BF16, device=feat.device)
    rc = kernels().ff_sparse_gather(ptr(feat), ptr(nbr), n, n_off, c, feat.shape[0], ptr(out),
                                    ptr(status_tensor(feat.device)), stream_ptr())
    check(rc, "ff_sparse_gather")
    _count()
    return out


def sparse_conv3d(feat: torch.Tensor, coords: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                  act: str = "none", k: int = 3) -> torch.Tensor:
    """Submanifold sparse convolution: output sites = input sites. feat [n, Cin] bf16, coords [n, 4] int32 (unique),
    weight [Cout, k^3 * Cin] (offset-major, the order of :func:`cube_offsets`). The gather builds the im2col
    operand; the contraction over offsets and channels is one tensor-core GEMM with FP32 accumulation."""
    table = VoxelHash(coords)
    nbr = table.neighbor_map(cube_offsets(k).to(coords.device))
    cols = sparse_gather(feat, nbr)
    return linear_bias_act(cols, weight, bias, act)


# ------------------------------------------------------------------------------------------------
# Hadamard-rotated INT8 linear
# ------------------------------------------------------------------------------------------------
_H4 = torch.tensor([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=torch.float32)


def hadamard(group: int) -> torch.Tensor:
    """Regular Hadamard of a power-of-four ``group``: kron of H4 / 2."""
    _require(group >= 4 and math.log(group, 4) == int(math.log(group, 4)), "hadamard: group must be a power of 4")
    h = torch.ones(1, 1)
    while h.shape[0] < group:
        h = torch.kron(_H4 * 0.5, h)
    return h


def rotate_quant(x: torch.Tensor, group: int) -> tuple[torch.Tensor, torch.Tensor]:
    """x [rows, k] bf16 -> (codes int8 [rows, k], scales f32 [rows]): every ``group`` activations are rotated by
    the regular Hadamard (FP32), rounded to BF16, then quantised with the row's ``max(|xR|, 1e-12) / 127``."""
    rows, k = x.shape
    if not x.is_cuda:
        h = hadamard(group)
        xr = _r((x.float().reshape(rows, k // group, group) @ h).reshape(rows, k))
        s = xr.abs().amax(-1).clamp_min(1e-12) / 127.0
        q = torch.round(xr / s[:, None]).clamp(-127, 127).to(torch.int8)
        return q, s
    _require(x.dtype == BF16 and x.stride(1) == 1 and k % group == 0, "rotate_quant: layout")
    codes = torch.empty(rows, k, dtype=torch.int8, device=x.device)
    scales = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = kernels().ff_rotate_quant(ptr(x), rows, k, group, x.stride(0), ptr(codes), ptr(scales), stream_ptr())
    check(rc, "ff_rotate_quant")
    _count()
    return codes, scales


def int8_linear(x: torch.Tensor, qweight: torch.Tensor, wscale: torch.Tensor, group: int) -> torch.Tensor:
    """``y = bf16((q(x R) @ qweight^T) * s_x * wscale)`` with INT32 products (qweight [n, k] int8 holds the rotated,
    quantised weight; wscale [n] f32)."""
    q, s = rotate_quant(x, group)
    rows, k = q.shape
    n = qweight.shape[0]
    if not x.is_cuda:
        acc = q.to(torch.int32) @ qweight.to(torch.int32).t()
        return (acc.float() * s[:, None] * wscale[None, :].float()).to(BF16)
    _require(qweight.dtype == torch.int8 and qweight.is_contiguous() and wscale.dtype == torch.float32 and k % 16 == 0,
             "int8_linear: layout")
    y = torch.empty(rows, n, dtype=BF16, device=x.device)
    rc = kernels().ff_int8_linear(ptr(q), ptr(s), ptr(qweight), ptr(wscale), ptr(y), rows, n, k, n, stream_ptr())
    check(rc, "ff_int8_linear")
    _count()
    return y


def quantize_weight_rotated(w: torch.Tensor, group: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Offline side of :func:`int8_linear`: w [n, k] -> (int8 codes of w R, per-row scales). Because R is
    orthogonal, ``(x R)(w R)^T = x w^T``."""
    n, k = w.shape
    wr = (w.float().cpu().reshape(n, k // group, group) @ hadamard(group)).reshape(n, k)
    s = wr.abs().amax(-1).clamp_min(1e-12) / 127.0
    return torch.round(wr / s[:, None]).clamp(-127, 127).to(torch.int8), s
