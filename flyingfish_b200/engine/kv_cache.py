"""Paged KV cache: block allocator, per-sequence block lists and the device tensors.

The reference keeps one contiguous head-major cache per layer for its single sequence
(kernels/rope_kv.cu:44-53, src/backend/cuda/engine.rs:1701-1702). Serving many sequences on a
180 GB part needs a block cache instead: every layer owns ``[num_blocks, kv_heads, 64, head_dim]``
K and V tensors, a sequence owns a list of block ids, and the kernels translate positions through
a block table. Blocks are reference-counted so committed prefixes can be shared (prefix cache)
and speculative rows can be rolled back by truncating a sequence's length.

The device tensors are zero-initialised: attention tiles always read whole 64-token blocks and
multiply masked probabilities (exact zeros) with whatever the tail of the last block holds, so
that tail must be finite.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


class OutOfBlocks(RuntimeError):
    pass


class BlockAllocator:
    """Free-list allocator with reference counts (host side, O(1) per operation)."""

    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))
        self._ref = [0] * num_blocks

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfBlocks("KV cache is out of blocks")
        b = self._free.pop()
        self._ref[b] = 1
        return b

    def share(self, block: int) -> None:
        assert self._ref[block] > 0, "sharing a free block"
        self._ref[block] += 1

    def release(self, block: int) -> None:
        assert self._ref[block] > 0, "double free of a KV block"
        self._ref[block] -= 1
        if self._ref[block] == 0:
            self._free.append(block)

    def refcount(self, block: int) -> int:
        return self._ref[block]


@dataclass
class SequenceKV:
    """Block list and committed length of one sequence."""
    seq_id: int
    blocks: list[int] = field(default_factory=list)
    length: int = 0                      # tokens whose K/V are committed in the cache


class PagedKVCache:
    """Device K/V tensors for every layer plus the allocator and per-sequence state."""

    def __init__(self, layers: int, kv_heads: int, head_dim: int, num_blocks: int, block_size: int = 64,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cpu",
                 v_head_dim: int | None = None):
        self.layers, self.kv_heads, self.head_dim = layers, kv_heads, head_dim
        self.block_size, self.num_blocks = block_size, num_blocks
        self.device = torch.device(device)
        vd = v_head_dim if v_head_dim is not None else head_dim
        self.k = [torch.zeros(num_blocks, kv_heads, block_size, head_dim, dtype=dtype, device=self.device)
                  for _ in range(layers)]
        self.v = [torch.zeros(num_blocks, kv_heads, block_size, vd, dtype=dtype, device=self.device)
                  for _ in range(layers)] if vd > 0 else [None] * layers
        self.alloc = BlockAllocator(num_blocks)
        self.seqs: dict[int, SequenceKV] = {}
        self.compact = None                 # engine.kv_compact.CompactKV when the cache format is affine8

    # -- sizing ----------------------------------------------------------------------------
    @staticmethod
    def bytes_per_block(layers: int, kv_heads: int, head_dim: int, block_size: int = 64, elem_bytes: int = 2,
                        v_head_dim: int | None = None) -> int:
        vd = head_dim if v_head_dim is None else v_head_dim
        return layers * kv_heads * block_size * (head_dim + vd) * elem_bytes

    # -- sequence life cycle ---------------------------------------------------------------
    def add_sequence(self, seq_id: int) -> SequenceKV:
        assert seq_id not in self.seqs
        s = SequenceKV(seq_id)
        self.seqs[seq_id] = s
        return s

    def free_sequence(self, seq_id: int) -> None:
        s = self.seqs.pop(seq_id)
        for b in s.blocks:
            if b >= 0:                      # -1: sealed into the compact store and released then
                self.alloc.release(b)
        if self.compact is not None:
            self.compact.free_sequence(seq_id)

    def blocks_needed(self, seq_id: int, new_tokens: int) -> int:
        s = self.seqs[seq_id]
        total = s.length + new_tokens
        need = (total + self.block_size - 1) // self.block_size
        return max(0, need - len(s.blocks))

    def reserve(self, seq_id: int, new_tokens: int) -> list[int]:
        """Make room for ``new_tokens`` more tokens and return their slots
        (slot = block * block_size + offset). Does not commit the length."""
        s = self.seqs[seq_id]
        need = self.blocks_needed(seq_id, new_tokens)
        if need > self.alloc.free_blocks:
            raise OutOfBlocks(f"sequence {seq_id} needs {need} blocks, {self.alloc.free_blocks} free")
        for _ in range(need):
            s.blocks.append(self.alloc.alloc())
        bs = self.block_size
        return [s.blocks[p // bs] * bs + p % bs for p in range(s.length, s.length + new_tokens)]

    def commit(self, seq_id: int, new_tokens: int) -> None:
        self.seqs[seq_id].length += new_tokens

    def truncate(self, seq_id: int, length: int) -> None:
        """Roll a sequence back to ``length`` committed tokens (speculative rejection); blocks past
        the new end are released."""
        s = self.seqs[seq_id]
        assert 0 <= length <= s.length
        s.length = length
        keep = (length + self.block_size - 1) // self.block_size
        while len(s.blocks) > max(keep, 0):
            self.alloc.release(s.blocks.pop())

    def fork_prefix(self, src_id: int, dst_id: int, tokens: int) -> SequenceKV:
        """New sequence sharing the first ``tokens`` (a multiple of the block size) of ``src``."""
        assert tokens % self.block_size == 0
        src = self.seqs[src_id]
        assert tokens <= src.length
        dst = self.add_sequence(dst_id)
        for b in src.blocks[: tokens // self.block_size]:
            self.alloc.share(b)
            dst.blocks.append(b)
        dst.length = tokens
        return dst

    def block_row(self, seq_id: int, width: int) -> list[int]:
        blocks = self.seqs[seq_id].blocks
        assert len(blocks) <= width, "block table too narrow for the sequence"
        return blocks + [0] * (width - len(blocks))

    def move_rows(self, seq_id: int, src_positions: list[int], dst_positions: list[int]) -> None:
        """Copy the K/V rows at ``src_positions`` of a sequence to ``dst_positions`` in every layer
        (gather first, then scatter, so overlapping sets are safe). Used to compact the accepted
        path of a verification tree onto consecutive positions (the reference's
        ``tree_kv_gather`` / ``tree_kv_scatter``, kernels/tree/meta.cu)."""
        if not src_positions:
            return
        s = self.seqs[seq_id]
        bs = self.block_size
        dev = self.device
        if dev.type == "cuda" and self.k[0].dtype == torch.bfloat16 and self.head_dim % 8 == 0 and \
                (self.v[0] is None or self.v[0].shape == self.k[0].shape):
            # two launches for all layers and both tensors (csrc/kv_util.cu)
            from ..ops.lib import check, kernels, ptr, status_tensor, stream_ptr
            if getattr(self, "_cache_ptrs", None) is None:
                ptrs = [t.data_ptr() for layer in range(self.layers) for t in (self.k[layer], self.v[layer]) if t is not None]
                self._cache_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=dev)
            n, tensors = len(src_positions), self._cache_ptrs.numel()
            slot = lambda ps: torch.tensor([s.blocks[p // bs] * bs + p % bs for p in ps], dtype=torch.int32, device=dev)
            staging = torch.empty(n * tensors * self.kv_heads * self.head_dim, dtype=torch.bfloat16, device=dev)
            src_slots, dst_slots = slot(src_positions), slot(dst_positions)       # both alive until the launches are queued
            rc = kernels().ff_kv_move_rows(ptr(self._cache_ptrs), tensors, ptr(src_slots), ptr(dst_slots), n,
                                           ptr(staging), self.kv_heads, bs, self.head_dim, self.k[0].shape[0],
                                           ptr(status_tensor(dev)), stream_ptr())
            check(rc, "ff_kv_move_rows")
            return
        sb = torch.tensor([s.blocks[p // bs] for p in src_positions], device=dev)
        so = torch.tensor([p % bs for p in src_positions], device=dev)
        db = torch.tensor([s.blocks[p // bs] for p in dst_positions], device=dev)
        do = torch.tensor([p % bs for p in dst_positions], device=dev)
        for layer in range(self.layers):
            for cache in (self.k[layer], self.v[layer]):
                if cache is None:
                    continue
                rows = cache[sb, :, so, :].clone()
                cache[db, :, do, :] = rows
