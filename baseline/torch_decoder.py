"""Library-call baseline: the same dense GQA decoder built from vendor libraries only.

This is the comparison arm of ``bench.py --impl baseline``. It has none of the framework's
kernels, engine or scheduler on its path: projections are ``torch.matmul`` (cuBLAS / cuBLASLt),
normalisation is ``torch.nn.functional.rms_norm``, attention is
``flash_attn.flash_attn_with_kvcache`` when that library runs on the device and
``scaled_dot_product_attention`` otherwise, tensor parallelism is NCCL ``all_reduce`` on the
row-parallel projections and ``all_gather`` for the vocabulary-parallel greedy pick, and the decode
step is replayed from one CUDA graph. It mirrors how the reference engine is put together (cuBLAS
linears chosen by calibration, src/backend/cuda/blas.rs:852-1080; one captured decode graph,
src/backend/cuda/engine.rs:4401) on the hardware and batch sizes of this build.

Weights are random N(0, 0.02) of the named shape; only throughput is measured with it.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _flash_kvcache():
    try:
        from flash_attn import flash_attn_with_kvcache
        return flash_attn_with_kvcache
    except Exception:
        return None


class TorchDecoder:
    """Dense Llama-style decoder, optionally tensor parallel (heads / FFN columns / vocabulary sharded)."""

    def __init__(self, spec, device: torch.device, batch: int, capacity: int, rank: int = 0, world: int = 1,
                 seed: int = 0, attention: str = "auto"):
        self.spec, self.device, self.batch, self.capacity = spec, device, batch, capacity
        self.rank, self.world = rank, world
        h, d = spec.hidden, spec.head_dim
        self.hq = spec.heads // world
        self.hkv = max(1, spec.kv_heads // world)
        self.d = d
        f = spec.ffn // world
        self.f = f
        g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
        bf = torch.bfloat16

        def rnd(*shape):
            return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(bf)

        self.layers = []
        for _ in range(spec.layers):
            self.layers.append({
                "ln1": torch.ones(h, dtype=bf, device=device), "ln2": torch.ones(h, dtype=bf, device=device),
                "wqkv": rnd((self.hq + 2 * self.hkv) * d, h), "wo": rnd(h, self.hq * d),
                "wgu": rnd(2 * f, h), "wdown": rnd(h, f),
            })
        self.embed = rnd(spec.vocab, h)
        self.final_ln = torch.ones(h, dtype=bf, device=device)
        vshard = (spec.vocab + world - 1) // world
        self.v0 = rank * vshard
        self.lm_head = rnd(min(vshard, spec.vocab - self.v0), h)
        # contiguous caches [batch, capacity, kv heads, dim] (flash_attn layout)
        self.k = [torch.zeros(batch, capacity, self.hkv, d, dtype=bf, device=device) for _ in range(spec.layers)]
        self.v = [torch.zeros(batch, capacity, self.hkv, d, dtype=bf, device=device) for _ in range(spec.layers)]
        inv = 1.0 / (spec.rope_theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
        pos = torch.arange(capacity, device=device, dtype=torch.float32)
        ang = pos[:, None] * inv[None, :]
        self.cos, self.sin = torch.cos(ang).to(bf), torch.sin(ang).to(bf)
        self.scale = 1.0 / math.sqrt(d)
        self.flash = _flash_kvcache() if (attention in ("auto", "flash") and device.type == "cuda") else None
        self.attention_impl = "flash_attn_with_kvcache" if self.flash is not None else "sdpa"
        # static decode inputs (graph-stable addresses)
        self.ids = torch.zeros(batch, dtype=torch.long, device=device)
        self.lens = torch.zeros(batch, dtype=torch.int32, device=device)      # tokens already cached per sequence
        self.graph = None
        self.out = None

    # -- pieces ------------------------------------------------------------------------------
    def _rope(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        x1, x2 = x[..., : self.d // 2], x[..., self.d // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    def _allreduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(x)
        return x

    def _mlp(self, lw, n: torch.Tensor) -> torch.Tensor:
        gu = n @ lw["wgu"].t()
        return self._allreduce((F.silu(gu[..., : self.f]) * gu[..., self.f:]) @ lw["wdown"].t())

    def _greedy(self, n: torch.Tensor) -> torch.Tensor:
        logits = n @ self.lm_head.t()
        val, idx = logits.float().max(dim=-1)
        idx = idx + self.v0
        if self.world == 1:
            return idx
        vals = [torch.empty_like(val) for _ in range(self.world)]
        idxs = [torch.empty_like(idx) for _ in range(self.world)]
        dist.all_gather(vals, val)
        dist.all_gather(idxs, idx)
        best = torch.stack(vals).argmax(dim=0, keepdim=True)
        return torch.stack(idxs).gather(0, best)[0]

    # -- prefill -----------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        """prompts: [batch, T] token ids; fills the caches and returns the first generated id per sequence."""
        b, t = prompts.shape
        s = self.spec
        x = self.embed[prompts]
        cos, sin = self.cos[:t][None, :, None, :], self.sin[:t][None, :, None, :]
        for i, lw in enumerate(self.layers):
            n = F.rms_norm(x, (s.hidden,), lw["ln1"], s.rms_eps)
            qkv = (n @ lw["wqkv"].t()).view(b, t, self.hq + 2 * self.hkv, self.d)
            q = self._rope(qkv[:, :, : self.hq], cos, sin)
            k = self._rope(qkv[:, :, self.hq: self.hq + self.hkv], cos, sin)
            v = qkv[:, :, self.hq + self.hkv:]
            self.k[i][:, :t] = k
            self.v[i][:, :t] = v
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=True).transpose(1, 2).reshape(b, t, -1)
            x = x + self._allreduce(a @ lw["wo"].t())
            n = F.rms_norm(x, (s.hidden,), lw["ln2"], s.rms_eps)
            x = x + self._mlp(lw, n)
        n = F.rms_norm(x[:, -1], (s.hidden,), self.final_ln, s.rms_eps)
        self.lens.fill_(t)
        return self._greedy(n)

    # -- decode ------------------------------------------------------------------------------
    @torch.no_grad()
    def _decode_body(self) -> torch.Tensor:
        s, b = self.spec, self.batch
        x = self.embed[self.ids]
        pos = self.lens.long()
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        rows = torch.arange(b, device=self.device)
        for i, lw in enumerate(self.layers):
            n = F.rms_norm(x, (s.hidden,), lw["ln1"], s.rms_eps)
            qkv = (n @ lw["wqkv"].t()).view(b, self.hq + 2 * self.hkv, self.d)
            q = self._rope(qkv[:, : self.hq], cos, sin)
            k = self._rope(qkv[:, self.hq: self.hq + self.hkv], cos, sin)
            v = qkv[:, self.hq + self.hkv:]
            if self.flash is not None:
                a = self.flash(q[:, None], self.k[i], self.v[i], k=k[:, None], v=v[:, None], cache_seqlens=self.lens,
                               softmax_scale=self.scale, causal=True).reshape(b, -1)
            else:
                self.k[i][rows, pos] = k
                self.v[i][rows, pos] = v
                mask = (torch.arange(self.capacity, device=self.device)[None, :] <= pos[:, None])[:, None, None, :]
                a = F.scaled_dot_product_attention(q[:, :, None], self.k[i].transpose(1, 2), self.v[i].transpose(1, 2),
                                                   attn_mask=mask, enable_gqa=True).reshape(b, -1)
            x = x + self._allreduce(a @ lw["wo"].t())
            n = F.rms_norm(x, (s.hidden,), lw["ln2"], s.rms_eps)
            x = x + self._mlp(lw, n)
        n = F.rms_norm(x, (s.hidden,), self.final_ln, s.rms_eps)
        return self._greedy(n)

    def capture(self) -> None:
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        saved = self.lens.clone()
        with torch.cuda.stream(side):
            for _ in range(2):
                self._decode_body()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = self._decode_body()
        self.lens.copy_(saved)

    def step(self) -> torch.Tensor:
        """One decode step of the whole batch from ``self.ids`` / ``self.lens``; advances ``lens`` on the device."""
        if self.graph is not None:
            self.graph.replay()
            out = self.out
        else:
            out = self._decode_body()
        self.lens.add_(1)
        return out
