"""Vision tower of a vision-language decoder (Qwen-VL family layout): patch embedding over packed
``temporal x patch x patch`` pixel blocks, learned position table interpolated to the image grid, pre-norm
transformer blocks with bidirectional attention inside each image and 2-D rotary embedding, then a 2x2 patch
merger that projects into the language model's hidden size.

B200 mapping: every projection is the tcgen05 GEMM (``ops.linear``) followed by a fused bias + activation pass;
attention is the paged prefill kernel in bidirectional mode over a scratch cache (each image starts on a 64-token
page boundary, so an image is one "sequence" whose block table is a plain range); 2-D rotary goes through the
table-driven rotary + KV-write kernel. Heads narrower than 128 are widened to 128 lanes at load time (each rotary
half padded to 64 with zero weights), which leaves the attention result unchanged.

The reference drives the same model family through src/vision_input.rs and kernels/vision_ops.cu /
kernels/vision_attn.cu; its image preprocessing is src/serve/image.rs:386-815 (here ``serve/image.py``).
"""
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
class VisionSpec:
    hidden: int = 1024
    heads: int = 8
    depth: int = 4
    intermediate: int = 4096
    patch: int = 16
    temporal: int = 2
    merge: int = 2
    out_hidden: int = 2048
    pos_side: int = 48                 # the learned position table is pos_side x pos_side
    act: str = "gelu_tanh"
    eps: float = 1e-6
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def patch_dim(self) -> int:
        return 3 * self.temporal * self.patch * self.patch


def _widen_rows(w: torch.Tensor, heads: int, d: int) -> torch.Tensor:
    """[heads * d, k] -> [heads * 128, k]: each half of a head (d/2 rows) lands at the start of a 64-row half."""
    if d == LANES:
        return w
    k = w.shape[1]
    out = torch.zeros(heads, 2, LANES // 2, k, dtype=w.dtype)
    out[:, :, : d // 2] = w.reshape(heads, 2, d // 2, k)
    return out.reshape(heads * LANES, k)


@dataclass
class VisionBlock:
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    wqkv: torch.Tensor                 # [3 * heads * 128, hidden] (Q heads, K heads, V heads)
    bqkv: torch.Tensor
    wo: torch.Tensor                   # [hidden, heads * 128]
    bo: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor


class VisionTower:
    def __init__(self, spec: VisionSpec, state: dict[str, torch.Tensor], device: torch.device | str = "cpu"):
        """``state`` uses the checkpoint names of the Qwen-VL vision tower (prefix ``visual.`` stripped):
        ``patch_embed.proj.{weight,bias}``, ``pos_embed.weight``, ``blocks.N.{norm1,norm2}.{weight,bias}``,
        ``blocks.N.attn.{qkv,proj}.{weight,bias}``, ``blocks.N.mlp.{linear_fc1,linear_fc2}.{weight,bias}``,
        ``merger.{norm,linear_fc1,linear_fc2}.{weight,bias}``."""
        self.spec, self.device = spec, torch.device(device)
        s, d, h = spec, spec.head_dim, spec.heads
        assert d % 2 == 0 and d <= LANES and s.hidden % 8 == 0

        def dev(t: torch.Tensor) -> torch.Tensor:
            return t.to(BF16).contiguous().to(self.device)

        self.patch_w = dev(state["patch_embed.proj.weight"].reshape(s.hidden, -1))
        self.patch_b = dev(state["patch_embed.proj.bias"])
        self.pos_table = state["pos_embed.weight"].float()                   # host: interpolated per image grid
        self.blocks: list[VisionBlock] = []
        for i in range(s.depth):
            p = f"blocks.{i}."
            wqkv, bqkv = state[p + "attn.qkv.weight"].float(), state[p + "attn.qkv.bias"].float()
            wq = torch.cat([_widen_rows(wqkv[j * s.hidden: (j + 1) * s.hidden], h, d) for j in range(3)], 0)
            bq = torch.cat([_widen_rows(bqkv[j * s.hidden: (j + 1) * s.hidden, None], h, d)[:, 0] for j in range(3)], 0)
            wo = _widen_rows(state[p + "attn.proj.weight"].float().t().contiguous(), h, d).t().contiguous()
            self.blocks.append(VisionBlock(
                dev(state[p + "norm1.weight"]), dev(state[p + "norm1.bias"]), dev(wq), dev(bq), dev(wo),
                dev(state[p + "attn.proj.bias"]), dev(state[p + "norm2.weight"]), dev(state[p + "norm2.bias"]),
                dev(state[p + "mlp.linear_fc1.weight"]), dev(state[p + "mlp.linear_fc1.bias"]),
                dev(state[p + "mlp.linear_fc2.weight"]), dev(state[p + "mlp.linear_fc2.bias"])))
        self.m_ln_w, self.m_ln_b = dev(state["merger.norm.weight"]), dev(state["merger.norm.bias"])
        self.m_w1, self.m_b1 = dev(state["merger.linear_fc1.weight"]), dev(state["merger.linear_fc1.bias"])
        self.m_w2, self.m_b2 = dev(state["merger.linear_fc2.weight"]), dev(state["merger.linear_fc2.bias"])
        self.scale = d ** -0.5

    # -- construction ------------------------------------------------------------------------------
    @staticmethod
    def random_state(spec: VisionSpec, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        rn = lambda *shape: torch.randn(*shape, generator=g) * std
        s = spec
        st = {"patch_embed.proj.weight": rn(s.hidden, s.patch_dim), "patch_embed.proj.bias": rn(s.hidden),
              "pos_embed.weight": rn(s.pos_side * s.pos_side, s.hidden)}
        for i in range(s.depth):
            p = f"blocks.{i}."
            st.update({p + "norm1.weight": torch.ones(s.hidden) + rn(s.hidden), p + "norm1.bias": rn(s.hidden),
                       p + "norm2.weight": torch.ones(s.hidden) + rn(s.hidden), p + "norm2.bias": rn(s.hidden),
                       p + "attn.qkv.weight": rn(3 * s.hidden, s.hidden), p + "attn.qkv.bias": rn(3 * s.hidden),
                       p + "attn.proj.weight": rn(s.hidden, s.hidden), p + "attn.proj.bias": rn(s.hidden),
                       p + "mlp.linear_fc1.weight": rn(s.intermediate, s.hidden), p + "mlp.linear_fc1.bias": rn(s.intermediate),
                       p + "mlp.linear_fc2.weight": rn(s.hidden, s.intermediate), p + "mlp.linear_fc2.bias": rn(s.hidden)})
        mh = s.hidden * s.merge * s.merge
        st.update({"merger.norm.weight": torch.ones(s.hidden) + rn(s.hidden), "merger.norm.bias": rn(s.hidden),
                   "merger.linear_fc1.weight": rn(mh, mh), "merger.linear_fc1.bias": rn(mh),
                   "merger.linear_fc2.weight": rn(s.out_hidden, mh), "merger.linear_fc2.bias": rn(s.out_hidden)})
        return st

    @classmethod
    def random(cls, spec: VisionSpec, device="cpu", seed: int = 0) -> "VisionTower":
        return cls(spec, cls.random_state(spec, seed), device)

    # -- geometry ------------------------------------------------------------------------------------
    def _grid_positions(self, gh: int, gw: int) -> torch.Tensor:
        """(row, col) of every patch in merge-block order (the order ``serve.image.pack_patches`` emits)."""
        m = self.spec.merge
        rows = torch.arange(gh).reshape(gh // m, m, 1, 1).expand(gh // m, m, gw // m, m)
        cols = torch.arange(gw).reshape(1, 1, gw // m, m).expand(gh // m, m, gw // m, m)
        order = (0, 2, 1, 3)                                   # block row, block col, inner row, inner col
        return torch.stack([rows.permute(order).reshape(-1), cols.permute(order).reshape(-1)], dim=1)

    def _pos_embed(self, gh: int, gw: int) -> torch.Tensor:
        s = self.spec
        tab = self.pos_table.reshape(1, s.pos_side, s.pos_side, s.hidden).permute(0, 3, 1, 2)
        grid = F.interpolate(tab, size=(gh, gw), mode="bilinear", align_corners=True)[0].permute(1, 2, 0)   # [gh, gw, hidden]
        rc = self._grid_positions(gh, gw)
        return grid[rc[:, 0], rc[:, 1]]

    # -- forward -------------------------------------------------------------------------------------
    def forward(self, patches: list[torch.Tensor], grids: list[tuple[int, int, int]]) -> list[torch.Tensor]:
        """patches[i] [gh*gw, patch_dim] (merge-block order), grids[i] = (t, gh, gw) with t == 1.
        Returns one [gh*gw / merge^2, out_hidden] bf16 tensor per image."""
        s, dev = self.spec, self.device
        h = s.heads
        lens = [p.shape[0] for p in patches]
        # every image starts on a page boundary of the scratch cache
        starts, blocks_per, total_blocks = [], [], 0
        for n in lens:
            starts.append(total_blocks * PAGE)
            blocks_per.append((n + PAGE - 1) // PAGE)
            total_blocks += blocks_per[-1]
        x_in = torch.cat([p.to(BF16) for p in patches], 0).to(dev)
        pos = torch.cat([self._pos_embed(g[1], g[2]) for g in grids], 0).to(BF16).to(dev)
        rc = torch.cat([self._grid_positions(g[1], g[2]) for g in grids], 0)
        table = vo.rotary_2d_table(rc, s.head_dim, s.rope_theta).to(dev)
        q_start, acc = [], 0
        for n in lens:
            q_start.append(acc)
            acc += n
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        slots = i32([st + j for st, n in zip(starts, lens) for j in range(n)])
        max_blocks = max(blocks_per)
        bt = torch.zeros(len(lens), max_blocks, dtype=torch.int32)
        b0 = 0
        for i, nb in enumerate(blocks_per):
            bt[i, :nb] = torch.arange(b0, b0 + nb, dtype=torch.int32)
            b0 += nb
        bt = bt.to(dev)
        q_start_t, q_lens_t = i32(q_start), i32(lens)
        kc = torch.zeros(total_blocks, h, PAGE, LANES, dtype=BF16, device=dev)
        vc = torch.zeros_like(kc)

        x = vo.linear_bias_act(x_in, self.patch_w, self.patch_b)
        x = x + pos
        for blk in self.blocks:
            n1 = vo.layernorm(x, blk.ln1_w, blk.ln1_b, s.eps)
            qkv = vo.linear_bias_act(n1, blk.wqkv, blk.bqkv)
            vo.rope_table_apply_(qkv, table, h, LANES, rot_dim=s.head_dim, slots=slots, kcache=kc, vcache=vc, kv_heads=h)
            a = ops.attn_prefill(qkv, kc, vc, bt, q_start_t, q_lens_t, q_lens_t, max(lens), h, h, LANES, self.scale,
                                 window=-1)
            x = x + vo.linear_bias_act(a, blk.wo, blk.bo)
            n2 = vo.layernorm(x, blk.ln2_w, blk.ln2_b, s.eps)
            f = vo.linear_bias_act(n2, blk.w1, blk.b1, s.act)
            x = x + vo.linear_bias_act(f, blk.w2, blk.b2)
        m2 = s.merge * s.merge
        y = vo.layernorm(x, self.m_ln_w, self.m_ln_b, s.eps).reshape(-1, s.hidden * m2)
        y = vo.linear_bias_act(y, self.m_w1, self.m_b1, "gelu")
        y = vo.linear_bias_act(y, self.m_w2, self.m_b2)
        out, o = [], 0
        for n in lens:
            out.append(y[o: o + n // m2])
            o += n // m2
        return out

    def reference_forward(self, patches: list[torch.Tensor], grids: list[tuple[int, int, int]],
                          state: dict[str, torch.Tensor]) -> list[torch.Tensor]:
        """Plain FP32 PyTorch restatement on the un-widened checkpoint tensors (the numerics oracle)."""
        s = self.spec
        d, h = s.head_dim, s.heads
        outs = []
        for p, g in zip(patches, grids):
            x = p.float() @ state["patch_embed.proj.weight"].reshape(s.hidden, -1).float().t() + state["patch_embed.proj.bias"].float()
            x = x + self._pos_embed(g[1], g[2])
            rc = self._grid_positions(g[1], g[2])
            tab = vo.rotary_2d_table(rc, d, s.rope_theta)
            cs, sn = tab[..., 0][:, None, :], tab[..., 1][:, None, :]

            def rot(t):
                t1, t2 = t[..., : d // 2], t[..., d // 2:]
                return torch.cat([t1 * cs - t2 * sn, t2 * cs + t1 * sn], -1)
            for i in range(s.depth):
                q = f"blocks.{i}."
                n1 = F.layer_norm(x, (s.hidden,), state[q + "norm1.weight"].float(), state[q + "norm1.bias"].float(), s.eps)
                qkv = n1 @ state[q + "attn.qkv.weight"].float().t() + state[q + "attn.qkv.bias"].float()
                qq, kk, vv = (t.reshape(-1, h, d) for t in qkv.split(s.hidden, dim=-1))
                qq, kk = rot(qq), rot(kk)
                att = torch.softmax(torch.einsum("qhd,khd->hqk", qq, kk) * self.scale, -1)
                a = torch.einsum("hqk,khd->qhd", att, vv).reshape(-1, s.hidden)
                x = x + a @ state[q + "attn.proj.weight"].float().t() + state[q + "attn.proj.bias"].float()
                n2 = F.layer_norm(x, (s.hidden,), state[q + "norm2.weight"].float(), state[q + "norm2.bias"].float(), s.eps)
                f = vo.act_ref(n2 @ state[q + "mlp.linear_fc1.weight"].float().t() + state[q + "mlp.linear_fc1.bias"].float(), s.act)
                x = x + f @ state[q + "mlp.linear_fc2.weight"].float().t() + state[q + "mlp.linear_fc2.bias"].float()
            m2 = s.merge * s.merge
            y = F.layer_norm(x, (s.hidden,), state["merger.norm.weight"].float(), state["merger.norm.bias"].float(), s.eps)
            y = y.reshape(-1, s.hidden * m2)
            y = vo.act_ref(y @ state["merger.linear_fc1.weight"].float().t() + state["merger.linear_fc1.bias"].float(), "gelu")
            outs.append(y @ state["merger.linear_fc2.weight"].float().t() + state["merger.linear_fc2.bias"].float())
        return outs
