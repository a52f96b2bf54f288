"""Paged 8-bit store behind the BF16 block cache (``--kv-format affine8``).

Whole 128-token groups of a sequence that have left the recent window are *sealed*: the two BF16 blocks of the group
are packed into one slot of a per-layer pool (K codes with per-channel statistics over the group, V codes with
per-token statistics, the reference's ``UINT8_KC128_VT_F32`` layout, src/kv.rs:5-133, kernels/kv_cache.cuh:6-33) and
the blocks go back to the allocator, except block 0: the first 64 tokens (the sink) stay BF16. A sealed token costs
``2 * (D + 8/128 * D + 8)`` bytes per KV head instead of ``4 * D``. Decode attention reads the sealed groups in place
(``ops.attn_decode_mixed``: the BF16 kernel covers the sink and the recent pages, ``csrc/kv_affine8.cu`` the sealed
groups, one merge). Prefill chunks and speculative verification read BF16 only, so sealing starts when a prompt is
complete and the mode excludes speculation and prefix sharing.
"""
from __future__ import annotations

import torch

from .kv_format import GROUP_TOKENS, RECENT_TOKENS

GROUPS_PER_CHUNK = 4          # sealed groups one CTA of the sealed-part kernel walks


def sealed_until(committed: int, recent: int = RECENT_TOKENS) -> int:
    return max(0, committed - recent) // GROUP_TOKENS * GROUP_TOKENS


class CompactKV:
    def __init__(self, layers: int, kv_heads: int, head_dim: int, slots: int, device, recent: int = RECENT_TOKENS):
        assert head_dim % 32 == 0
        self.layers, self.kv_heads, self.head_dim, self.slots, self.recent = layers, kv_heads, head_dim, slots, recent
        self.device = torch.device(device)
        z = lambda *shape, dt=torch.uint8: torch.zeros(*shape, dtype=dt, device=self.device)
        self.k_codes = [z(slots, kv_heads, GROUP_TOKENS, head_dim) for _ in range(layers)]
        self.v_codes = [z(slots, kv_heads, GROUP_TOKENS, head_dim) for _ in range(layers)]
        self.k_stats = [z(slots, kv_heads, head_dim, 2, dt=torch.float32) for _ in range(layers)]
        self.v_stats = [z(slots, kv_heads, GROUP_TOKENS, 2, dt=torch.float32) for _ in range(layers)]
        self._free = list(range(slots - 1, -1, -1))
        self.groups: dict[int, list[int]] = {}            # sequence id -> pool slot of every sealed group, in order
        self.stats = {"sealed_groups": 0, "released_blocks": 0}

    # -- accounting ------------------------------------------------------------------------------------------
    @staticmethod
    def bytes_per_slot(layers: int, kv_heads: int, head_dim: int) -> int:
        return layers * kv_heads * (2 * GROUP_TOKENS * head_dim + head_dim * 8 + GROUP_TOKENS * 8)

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def sealed_tokens(self, seq_id: int) -> int:
        return len(self.groups.get(seq_id, ())) * GROUP_TOKENS

    def free_sequence(self, seq_id: int) -> None:
        self._free.extend(self.groups.pop(seq_id, ()))

    # -- sealing ---------------------------------------------------------------------------------------------
    def seal(self, kv, seq_id: int) -> int:
        """Seal every group of the sequence that has left the recent window; returns the number of groups sealed.
        ``kv`` is the block cache (its sequence record supplies the blocks and receives -1 for the released ones)."""
        s = kv.seqs[seq_id]
        mine = self.groups.setdefault(seq_id, [])
        target = sealed_until(s.length, self.recent) // GROUP_TOKENS
        todo = list(range(len(mine), target))
        if not todo:
            return 0
        if len(todo) > len(self._free):
            todo = todo[: len(self._free)]                # pool exhausted: the rest stays BF16 until slots come back
            if not todo:
                return 0
        per = GROUP_TOKENS // kv.block_size
        assert per == 2, "the compact store packs two 64-token blocks per group"
        blk_a = [s.blocks[g * per] for g in todo]
        blk_b = [s.blocks[g * per + 1] for g in todo]
        slots = [self._free.pop() for _ in todo]
        assert all(b >= 0 for b in blk_a + blk_b), "sealing a released block"
        self._pack(kv, blk_a, blk_b, slots)
        mine.extend(slots)
        for g in todo:
            for j in (g * per, g * per + 1):
                if j == 0:
                    continue                               # the sink block stays BF16
                kv.alloc.release(s.blocks[j])
                s.blocks[j] = -1
                self.stats["released_blocks"] += 1
        self.stats["sealed_groups"] += len(todo)
        return len(todo)

    def _pack(self, kv, blk_a: list[int], blk_b: list[int], slots: list[int]) -> None:
        dev = self.device
        a, b, sl = (torch.tensor(x, dtype=torch.int32, device=dev) for x in (blk_a, blk_b, slots))
        if dev.type == "cuda":
            from ..ops import _count
            from ..ops.lib import check, kernels, ptr, status_tensor, stream_ptr
            for i in range(self.layers):
                rc = kernels().ff_kv_seal_groups(ptr(kv.k[i]), ptr(kv.v[i]), ptr(a), ptr(b), ptr(sl), len(slots),
                                                 ptr(self.k_codes[i]), ptr(self.v_codes[i]), ptr(self.k_stats[i]),
                                                 ptr(self.v_stats[i]), self.kv_heads, self.head_dim, kv.k[i].shape[0],
                                                 self.slots, ptr(status_tensor(dev)), stream_ptr())
                check(rc, "ff_kv_seal_groups")
                _count()
            return
        from .kv_format import _pack_ref
        for i in range(self.layers):
            for x, y, s_ in zip(blk_a, blk_b, slots):
                k = torch.cat([kv.k[i][x], kv.k[i][y]], dim=1)          # [hkv, 128, D]
                v = torch.cat([kv.v[i][x], kv.v[i][y]], dim=1)
                c, lo, sc = _pack_ref(k, (1,))
                self.k_codes[i][s_] = c
                self.k_stats[i][s_, :, :, 0] = lo[:, 0]; self.k_stats[i][s_, :, :, 1] = sc[:, 0]
                c, lo, sc = _pack_ref(v, (2,))
                self.v_codes[i][s_] = c
                self.v_stats[i][s_, :, :, 0] = lo[..., 0]; self.v_stats[i][s_, :, :, 1] = sc[..., 0]

    def dequant(self, layer: int, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """BF16 rows of one sealed group: (K [hkv, 128, D], V [hkv, 128, D]) = bf16(code * scale + lo)."""
        ks, vs = self.k_stats[layer][slot], self.v_stats[layer][slot]
        k = (self.k_codes[layer][slot].float() * ks[:, None, :, 1] + ks[:, None, :, 0]).to(torch.bfloat16)
        v = (self.v_codes[layer][slot].float() * vs[:, :, None, 1] + vs[:, :, None, 0]).to(torch.bfloat16)
        return k, v
