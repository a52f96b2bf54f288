"""Vision side of the MiniCPM-V 4.x family: a SigLIP-style tower with a window-attention merger in its middle and a
2x2 merger at its end, 16 patches per output token in total.

Layout (tensor names of the published checkpoints; src/backend/cuda/engine_vision.rs:998-1110 and :2509-2643 of the
reference, position ids and gather orders src/vision_input.rs:46-159):

* ``model.vision_tower.embeddings``: patch projection (a ``patch x patch`` convolution, i.e. one GEMM over packed patch
  rows in raster order) plus a learned ``side x side`` position table addressed by the nearest bucket of each patch's
  relative position in its own grid, so any grid size reuses the one table.
* ``model.vision_tower.encoder.layers.N``: pre-norm blocks (LayerNorm, separate q / k / v / out projections with bias,
  bidirectional attention inside one view, tanh-GELU MLP).
* ``model.vision_tower.vit_merger``, after block ``insert_layer``: the rows are regrouped into 2x2 windows; attention
  inside each window (4 tokens) with a residual, then the window's 4 rows are concatenated, normalised and projected
  back to one row (``linear_1`` -> GELU -> ``linear_2``) on top of the window mean. The remaining blocks run on a
  quarter of the rows.
* ``model.vision_tower.post_layernorm``, then ``model.merger.mlp.0``: the rows are regrouped 2x2 once more, the
  concatenated group is normalised and goes through ``linear_1`` -> GELU -> ``linear_2`` into the language model's width.

B200 mapping as in ``models/vision.py``: every projection is the tcgen05 GEMM with a fused bias + activation pass,
attention inside a view is the tcgen05 prefill kernel in bidirectional mode over a scratch page cache (heads widened to
128 lanes; K / V are filed by the rotary kernel with an identity table). The 4-token window attention is 16 scores per
head and window: it runs as two batched products on the device."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import vision_ops as vo

BF16 = torch.bfloat16
PAGE = 64
LANES = 128


@dataclass
class MiniCpmVisionSpec:
    hidden: int = 1152
    heads: int = 16
    depth: int = 27
    intermediate: int = 4304
    patch: int = 14
    channels: int = 3
    image_size: int = 980                 # the position table is (image_size / patch)^2
    insert_layer: int = 6
    out_hidden: int = 4096
    eps: float = 1e-6
    window: int = 2                       # window merger: window x window patches -> one row
    merge: int = 2                        # final merger: merge x merge rows -> one token

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def position_side(self) -> int:
        return self.image_size // self.patch

    @property
    def patch_dim(self) -> int:
        return self.channels * self.patch * self.patch

    @property
    def patches_per_token(self) -> int:
        return (self.window * self.merge) ** 2

    def check(self) -> None:
        if self.hidden % self.heads or self.head_dim % 2 or self.head_dim > LANES:
            raise ValueError("unsupported vision head geometry")
        if self.image_size % self.patch or not (0 <= self.insert_layer < self.depth):
            raise ValueError("image size is not a patch multiple, or the insert layer lies outside the tower")
        if self.hidden % 8 or self.intermediate % 8:
            raise ValueError("row widths must be multiples of 8")

    @classmethod
    def from_config(cls, root: dict) -> "MiniCpmVisionSpec":
        """``config.json`` of a MiniCPM-V checkpoint (``vision_config`` + the merger settings beside it)."""
        v = root.get("vision_config")
        if not isinstance(v, dict) or v.get("hidden_act") != "gelu_pytorch_tanh":
            raise ValueError("vision_config missing or with an unsupported activation")
        for key in ("window_kernel_size",):
            if key in v and list(v[key]) != [2, 2]:
                raise ValueError(f"unsupported {key}: {v[key]}")
        if "merge_kernel_size" in root and list(root["merge_kernel_size"]) != [2, 2]:
            raise ValueError(f"unsupported merge_kernel_size: {root['merge_kernel_size']}")
        if int(root.get("merger_times", 1)) != 1 or root.get("downsample_mode") != "16x":
            raise ValueError("unsupported merger_times / downsample_mode")
        spec = cls(hidden=int(v["hidden_size"]), heads=int(v["num_attention_heads"]), depth=int(v["num_hidden_layers"]),
                   intermediate=int(v["intermediate_size"]), patch=int(v["patch_size"]), channels=int(v.get("num_channels", 3)),
                   image_size=int(v["image_size"]), insert_layer=int(root["insert_layer_id"]),
                   out_hidden=int(root["text_config"]["hidden_size"]), eps=float(v.get("layer_norm_eps", 1e-6)))
        spec.check()
        return spec

    def expected_tensors(self) -> dict[str, tuple[int, ...]]:
        h, i, w4, m4 = self.hidden, self.intermediate, self.window ** 2, self.merge ** 2
        out: dict[str, tuple[int, ...]] = {
            "model.vision_tower.embeddings.patch_embedding.weight": (h, self.channels, self.patch, self.patch),
            "model.vision_tower.embeddings.patch_embedding.bias": (h,),
            "model.vision_tower.embeddings.position_embedding.weight": (self.position_side ** 2, h),
            "model.vision_tower.post_layernorm.weight": (h,), "model.vision_tower.post_layernorm.bias": (h,)}

        def attention(prefix: str) -> None:
            for n in ("q", "k", "v", "out"):
                out[f"{prefix}.self_attn.{n}_proj.weight"] = (h, h)
                out[f"{prefix}.self_attn.{n}_proj.bias"] = (h,)
        for layer in range(self.depth):
            p = f"model.vision_tower.encoder.layers.{layer}"
            for n in ("layer_norm1", "layer_norm2"):
                out[f"{p}.{n}.weight"], out[f"{p}.{n}.bias"] = (h,), (h,)
            attention(p)
            out[f"{p}.mlp.fc1.weight"], out[f"{p}.mlp.fc1.bias"] = (i, h), (i,)
            out[f"{p}.mlp.fc2.weight"], out[f"{p}.mlp.fc2.bias"] = (h, i), (h,)
        p = "model.vision_tower.vit_merger"
        attention(p)
        out[f"{p}.layer_norm1.weight"], out[f"{p}.layer_norm1.bias"] = (h,), (h,)
        out[f"{p}.pre_norm.weight"], out[f"{p}.pre_norm.bias"] = (w4 * h,), (w4 * h,)
        out[f"{p}.linear_1.weight"], out[f"{p}.linear_1.bias"] = (w4 * i, w4 * h), (w4 * i,)
        out[f"{p}.linear_2.weight"], out[f"{p}.linear_2.bias"] = (h, w4 * i), (h,)
        p = "model.merger.mlp.0"
        out[f"{p}.pre_norm.weight"], out[f"{p}.pre_norm.bias"] = (m4 * h,), (m4 * h,)
        out[f"{p}.linear_1.weight"], out[f"{p}.linear_1.bias"] = (m4 * h, m4 * h), (m4 * h,)
        out[f"{p}.linear_2.weight"], out[f"{p}.linear_2.bias"] = (self.out_hidden, m4 * h), (self.out_hidden,)
        return out


def minicpm_vision_tiny() -> MiniCpmVisionSpec:
    spec = MiniCpmVisionSpec(hidden=64, heads=2, depth=3, intermediate=96, patch=4, channels=3, image_size=32, insert_layer=0,
                             out_hidden=48)
    spec.check()
    return spec


# ------------------------------------------------------------------------------------------------
# geometry: position buckets and gather orders (host)
# ------------------------------------------------------------------------------------------------
def nearest_position_ids(grids: list[tuple[int, int]], side: int) -> torch.Tensor:
    """Id into the ``side x side`` position table for every patch (raster order, view after view): the bucket of the
    patch's relative row ``r / h`` and column ``c / w`` among the boundaries ``(j + 1) / side`` (a value on a boundary
    belongs to the bucket above), computed in FP32 like the published processor's ``bucketize(right=True)``."""
    if side <= 0:
        raise ValueError("zero position table side")
    bounds = (torch.arange(1, side + 1, dtype=torch.float64) / side).float()
    ids = []
    for h, w in grids:
        if h <= 0 or w <= 0:
            raise ValueError("empty patch grid")
        br = torch.bucketize(torch.arange(h, dtype=torch.float32) / h, bounds, right=True).clamp_(max=side - 1)
        bc = torch.bucketize(torch.arange(w, dtype=torch.float32) / w, bounds, right=True).clamp_(max=side - 1)
        ids.append((br[:, None] * side + bc[None, :]).reshape(-1))
    return torch.cat(ids).to(torch.int64)


def block_order(grids: list[tuple[int, int]], block: int) -> torch.Tensor:
    """Row order that makes every ``block x block`` square of a raster grid contiguous (squares in raster order, rows
    inside a square in raster order), view after view."""
    out, base = [], 0
    for h, w in grids:
        if h % block or w % block:
            raise ValueError(f"patch grid {h}x{w} is not aligned to {block}")
        idx = torch.arange(h * w).reshape(h // block, block, w // block, block).permute(0, 2, 1, 3).reshape(-1)
        out.append(idx + base)
        base += h * w
    return torch.cat(out)


# ------------------------------------------------------------------------------------------------
# the tower
# ------------------------------------------------------------------------------------------------
def _widen_rows(w: torch.Tensor, heads: int, d: int) -> torch.Tensor:
    """[heads * d, k] -> [heads * 128, k]: each half of a head (d / 2 rows) opens a 64-row half."""
    if d == LANES:
        return w
    k = w.shape[1]
    out = torch.zeros(heads, 2, LANES // 2, k, dtype=w.dtype)
    out[:, :, : d // 2] = w.reshape(heads, 2, d // 2, k)
    return out.reshape(heads * LANES, k)


class MiniCpmVisionTower:
    def __init__(self, spec: MiniCpmVisionSpec, state: dict[str, torch.Tensor], device: torch.device | str = "cpu"):
        spec.check()
        for name, shape in spec.expected_tensors().items():
            if name not in state:
                raise ValueError(f"vision tensor missing: {name}")
            if tuple(state[name].shape) != shape:
                raise ValueError(f"vision tensor {name} has shape {tuple(state[name].shape)}, expected {shape}")
        self.spec, self.device = spec, torch.device(device)
        s, h, d = spec, spec.heads, spec.head_dim
        t = {k: v.float() for k, v in state.items() if k in spec.expected_tensors()}

        def dev(x: torch.Tensor) -> torch.Tensor:
            return x.to(BF16).contiguous().to(self.device)

        def qkv(prefix: str):
            w = torch.cat([_widen_rows(t[f"{prefix}.self_attn.{n}_proj.weight"], h, d) for n in ("q", "k", "v")], 0)
            b = torch.cat([_widen_rows(t[f"{prefix}.self_attn.{n}_proj.bias"][:, None], h, d)[:, 0] for n in ("q", "k", "v")], 0)
            wo = _widen_rows(t[f"{prefix}.self_attn.out_proj.weight"].t().contiguous(), h, d).t().contiguous()
            return dev(w), dev(b), dev(wo), dev(t[f"{prefix}.self_attn.out_proj.bias"])

        def pair(prefix: str):
            return dev(t[prefix + ".weight"]), dev(t[prefix + ".bias"])
        e = "model.vision_tower.embeddings."
        # packed patch rows are padded to a multiple of 8 values (16-byte rows for the GEMM's TMA loads; 588 -> 592)
        self.patch_pad = (-s.patch_dim) % 8
        self.patch = (dev(F.pad(t[e + "patch_embedding.weight"].reshape(s.hidden, -1), (0, self.patch_pad))), dev(t[e + "patch_embedding.bias"]))
        self.positions = dev(t[e + "position_embedding.weight"])
        self.blocks = []
        for i in range(s.depth):
            p = f"model.vision_tower.encoder.layers.{i}"
            self.blocks.append(dict(ln1=pair(p + ".layer_norm1"), attn=qkv(p), ln2=pair(p + ".layer_norm2"), fc1=pair(p + ".mlp.fc1"),
                                    fc2=pair(p + ".mlp.fc2")))
        p = "model.vision_tower.vit_merger"
        # the window attention works on the un-widened heads (batched 4 x 4 products)
        self.window = dict(ln1=pair(p + ".layer_norm1"),
                           wqkv=dev(torch.cat([t[f"{p}.self_attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0)),
                           bqkv=dev(torch.cat([t[f"{p}.self_attn.{n}_proj.bias"] for n in ("q", "k", "v")], 0)),
                           out=pair(p + ".self_attn.out_proj"), pre=pair(p + ".pre_norm"), fc1=pair(p + ".linear_1"), fc2=pair(p + ".linear_2"))
        self.post = pair("model.vision_tower.post_layernorm")
        m = "model.merger.mlp.0"
        self.merger = dict(pre=pair(m + ".pre_norm"), fc1=pair(m + ".linear_1"), fc2=pair(m + ".linear_2"))
        self.scale = d ** -0.5

    @staticmethod
    def random_state(spec: MiniCpmVisionSpec, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        out = {}
        for name, shape in spec.expected_tensors().items():
            x = torch.randn(*shape, generator=g) * std
            if name.endswith("norm.weight") or "layer_norm1.weight" in name or "layer_norm2.weight" in name or name.endswith("post_layernorm.weight"):
                x = x + 1.0
            out[name] = x
        return out

    @classmethod
    def random(cls, spec: MiniCpmVisionSpec, device="cpu", seed: int = 0) -> "MiniCpmVisionTower":
        return cls(spec, cls.random_state(spec, seed), device)

    # -- pieces --------------------------------------------------------------------------------------
    def _attention_setup(self, lens: list[int]):
        """Scratch page cache and sequence metadata for views of ``lens`` rows, each starting on a page boundary."""
        dev, h = self.device, self.spec.heads
        starts, blocks_per, total = [], [], 0
        for n in lens:
            starts.append(total * PAGE)
            blocks_per.append((n + PAGE - 1) // PAGE)
            total += blocks_per[-1]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        slots = i32([st + j for st, n in zip(starts, lens) for j in range(n)])
        bt = torch.zeros(len(lens), max(blocks_per), dtype=torch.int32)
        b0 = 0
        for i, nb in enumerate(blocks_per):
            bt[i, :nb] = torch.arange(b0, b0 + nb, dtype=torch.int32)
            b0 += nb
        q_start, acc = [], 0
        for n in lens:
            q_start.append(acc)
            acc += n
        kc = torch.zeros(total, h, PAGE, LANES, dtype=BF16, device=dev)
        rows = sum(lens)
        ident = torch.zeros(rows, self.spec.head_dim // 2, 2, dtype=torch.float32, device=dev)
        ident[..., 0] = 1.0                                               # cos 1, sin 0: K / V are filed unrotated
        return dict(slots=slots, bt=bt.to(dev), q_start=i32(q_start), q_lens=i32(lens), kc=kc, vc=torch.zeros_like(kc), ident=ident,
                    max_len=max(lens))

    def _block(self, x: torch.Tensor, blk: dict, at: dict) -> torch.Tensor:
        s, h = self.spec, self.spec.heads
        wqkv, bqkv, wo, bo = blk["attn"]
        n1 = vo.layernorm(x, *blk["ln1"], s.eps)
        qkv = vo.linear_bias_act(n1, wqkv, bqkv)
        vo.rope_table_apply_(qkv, at["ident"], h, LANES, rot_dim=s.head_dim, slots=at["slots"], kcache=at["kc"], vcache=at["vc"], kv_heads=h)
        a = ops.attn_prefill(qkv, at["kc"], at["vc"], at["bt"], at["q_start"], at["q_lens"], at["q_lens"], at["max_len"], h, h, LANES,
                             self.scale, window=-1)
        x = x + vo.linear_bias_act(a, wo, bo)
        n2 = vo.layernorm(x, *blk["ln2"], s.eps)
        f = vo.linear_bias_act(n2, *blk["fc1"], "gelu_tanh")
        return x + vo.linear_bias_act(f, *blk["fc2"])

    def _window_merger(self, x: torch.Tensor, grids: list[tuple[int, int]]) -> torch.Tensor:
        """Rows [n, hidden] in raster order -> [n / 4, hidden] in raster order of the halved grids."""
        s, w = self.spec, self.window
        k = s.window * s.window
        order = block_order(grids, s.window).to(x.device)
        g = x.index_select(0, order)                                       # windows contiguous
        n1 = vo.layernorm(g, *w["ln1"], s.eps)
        qkv = vo.linear_bias_act(n1, w["wqkv"], w["bqkv"]).reshape(-1, k, 3, s.heads, s.head_dim)
        q, kk, v = (qkv[:, :, j].permute(0, 2, 1, 3).float() for j in range(3))            # [windows, heads, 4, d]
        att = torch.softmax(torch.matmul(q, kk.transpose(-1, -2)) * self.scale, dim=-1)
        core = torch.matmul(att, v).permute(0, 2, 1, 3).reshape(-1, s.hidden).to(BF16)
        g = g + vo.linear_bias_act(core.contiguous(), *w["out"])
        mean = g.reshape(-1, k, s.hidden).float().mean(dim=1).to(BF16)
        cat = vo.layernorm(g.reshape(-1, k * s.hidden), *w["pre"], s.eps)
        f = vo.linear_bias_act(cat, *w["fc1"], "gelu_tanh")
        return vo.linear_bias_act(f, *w["fc2"]) + mean

    def forward(self, patches: list[torch.Tensor], grids: list[tuple[int, int]]) -> list[torch.Tensor]:
        """``patches[i]`` [gh * gw, patch_dim] in raster order with ``grids[i] = (gh, gw)`` (multiples of 4). Returns one
        [gh * gw / 16, out_hidden] BF16 tensor per view."""
        s, dev = self.spec, self.device
        step = s.window * s.merge
        for p, (gh, gw) in zip(patches, grids):
            if p.shape != (gh * gw, s.patch_dim) or gh % step or gw % step:
                raise ValueError(f"view of {tuple(p.shape)} patches does not match its {gh}x{gw} grid (multiples of {step})")
        packed = torch.cat([p.to(BF16) for p in patches], 0)
        if self.patch_pad:
            packed = F.pad(packed, (0, self.patch_pad))
        x = vo.linear_bias_act(packed.contiguous().to(dev), *self.patch)
        x = x + self.positions.index_select(0, nearest_position_ids(grids, s.position_side).to(dev))
        at = self._attention_setup([gh * gw for gh, gw in grids])
        small = [(gh // s.window, gw // s.window) for gh, gw in grids]
        for i, blk in enumerate(self.blocks):
            x = self._block(x, blk, at)
            if i == s.insert_layer:
                x = self._window_merger(x, grids)
                at = self._attention_setup([gh * gw for gh, gw in small])
        x = vo.layernorm(x, *self.post, s.eps)
        m = self.merger
        grouped = x.index_select(0, block_order(small, s.merge).to(dev)).reshape(-1, s.merge * s.merge * s.hidden)
        y = vo.linear_bias_act(vo.layernorm(grouped, *m["pre"], s.eps), *m["fc1"], "gelu_tanh")
        y = vo.linear_bias_act(y, *m["fc2"])
        out, o = [], 0
        for gh, gw in grids:
            n = gh * gw // s.patches_per_token
            out.append(y[o:o + n])
            o += n
        return out

    def reference_forward(self, patches: list[torch.Tensor], grids: list[tuple[int, int]], state: dict[str, torch.Tensor]) -> list[torch.Tensor]:
        """Plain FP32 PyTorch restatement on the checkpoint tensors, one view at a time (the numerics oracle)."""
        s = self.spec
        t = {k: v.float() for k, v in state.items()}
        h, d = s.heads, s.head_dim
        ln = lambda x, p: F.layer_norm(x, (x.shape[-1],), t[p + ".weight"], t[p + ".bias"], s.eps)
        lin = lambda x, p: F.linear(x, t[p + ".weight"], t[p + ".bias"])
        gelu = lambda x: F.gelu(x, approximate="tanh")

        def attend(x, p, group):
            """Attention among consecutive groups of ``group`` rows."""
            n = x.shape[0]
            q, k, v = (lin(x, f"{p}.self_attn.{nm}_proj").reshape(n // group, group, h, d).transpose(1, 2) for nm in ("q", "k", "v"))
            a = torch.softmax(q @ k.transpose(-1, -2) * d ** -0.5, -1) @ v
            return lin(a.transpose(1, 2).reshape(n, s.hidden), f"{p}.self_attn.out_proj")
        outs = []
        for pt, (gh, gw) in zip(patches, grids):
            e = "model.vision_tower.embeddings."
            x = pt.float() @ t[e + "patch_embedding.weight"].reshape(s.hidden, -1).t() + t[e + "patch_embedding.bias"]
            x = x + t[e + "position_embedding.weight"][nearest_position_ids([(gh, gw)], s.position_side)]
            for i in range(s.depth):
                p = f"model.vision_tower.encoder.layers.{i}"
                x = x + attend(ln(x, p + ".layer_norm1"), p, x.shape[0])
                x = x + lin(gelu(lin(ln(x, p + ".layer_norm2"), p + ".mlp.fc1")), p + ".mlp.fc2")
                if i == s.insert_layer:
                    p = "model.vision_tower.vit_merger"
                    k = s.window ** 2
                    g = x[block_order([(gh, gw)], s.window)]
                    g = g + attend(ln(g, p + ".layer_norm1"), p, k)
                    mean = g.reshape(-1, k, s.hidden).mean(1)
                    x = lin(gelu(lin(ln(g.reshape(-1, k * s.hidden), p + ".pre_norm"), p + ".linear_1")), p + ".linear_2") + mean
            x = ln(x, "model.vision_tower.post_layernorm")
            m = "model.merger.mlp.0"
            g = x[block_order([(gh // s.window, gw // s.window)], s.merge)].reshape(-1, s.merge ** 2 * s.hidden)
            outs.append(lin(gelu(lin(ln(g, m + ".pre_norm"), m + ".linear_1")), m + ".linear_2"))
        return outs


def expand_view_tokens(ids: list[int], image_token: int, plans: list[tuple[int, int, int, int]], start: int, end: int,
                       slice_start: int, slice_end: int, newline: int) -> list[int]:
    """Every ``image_token`` of ``ids`` becomes the token span of one sliced image: ``start, thumb tokens, end`` and then,
    tile row after tile row (a newline token between rows), ``slice_start, tile tokens, slice_end`` per tile
    (src/serve/image.rs:1140-1200 of the reference). ``plans[i] = (thumb tokens, tile rows, tile columns, tokens per tile)``."""
    out, k = [], 0
    for tok in ids:
        if tok != image_token:
            out.append(tok)
            continue
        if k >= len(plans):
            raise ValueError("more image placeholders than images")
        thumb, rows, cols, per = plans[k]
        k += 1
        out += [start] + [image_token] * thumb + [end]
        for r in range(rows):
            if r:
                out.append(newline)
            for _ in range(cols):
                out += [slice_start] + [image_token] * per + [slice_end]
    if k != len(plans):
        raise ValueError("fewer image placeholders than images")
    return out
