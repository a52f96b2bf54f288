"""Device engine: owns the weights, the paged KV cache, the packed step metadata and the
CUDA graphs, and exposes prefill / decode / verify steps over sets of sequences.

This is the counterpart of the reference's ``Engine`` (src/backend/cuda/engine.rs:699-777:
``prefill`` :4009, ``decode`` :4262, ``capture`` :4401) re-designed for many concurrent
sequences: chunked prefill over a block cache, decode batches replayed from one CUDA graph per
batch bucket (the reference captures one graph for its single sequence), one pinned
host-to-device copy of the step metadata and one device-to-host read of the sampled ids per step.

Failure policy follows the reference's poisoning rule (engine.rs:1941-1944): an exception inside
a step marks the engine poisoned and every later entry point refuses until ``reset``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from .. import ops
from ..config import ModelSpec, Settings
from ..utils.log import log_json
from .batch import BatchLayout, ForwardBatch
from .kv_cache import OutOfBlocks, PagedKVCache


class EnginePoisoned(RuntimeError):
    pass


DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def bucket_for(n: int) -> int:
    for b in DECODE_BUCKETS:
        if n <= b:
            return b
    raise ValueError(f"decode batch {n} exceeds the largest bucket {DECODE_BUCKETS[-1]}")


@dataclass
class Sequence:
    seq_id: int
    prompt: list[int]
    output: list[int] = field(default_factory=list)
    prefilled: int = 0                 # prompt tokens whose KV is committed
    pending: int | None = None         # token sampled but not yet fed through the model
    finished: bool = False
    state_slot: int = -1               # slot of the per-sequence recurrent state (hybrid linear-attention models)
    mm_positions: list[int] | None = None      # prompt indices whose embedding row comes from ``mm_embeds``
    mm_embeds: torch.Tensor | None = None      # [len(mm_positions), hidden] (vision-tower output)

    @property
    def all_tokens(self) -> list[int]:
        return self.prompt + self.output


class _Graph:
    def __init__(self):
        self.graph: torch.cuda.CUDAGraph | None = None
        self.batch: ForwardBatch | None = None
        self.out: torch.Tensor | None = None


class Engine:
    def __init__(self, model, spec: ModelSpec, settings: Settings, num_blocks: int, device: torch.device | str,
                 max_prefill_rows: int = 8192):
        self.model, self.spec, self.settings = model, spec, settings
        self.device = torch.device(device)
        tp = model.w.tp.size
        hkv = max(1, spec.kv_heads // tp)
        dtype = model.w.embed.dtype
        if spec.mla is not None:       # one latent row per token: [kv_lora | rope key], no separate V
            self.kv = PagedKVCache(spec.layers, 1, spec.mla.kv_lora_rank + spec.mla.qk_rope_dim, num_blocks,
                                   settings.kv_block, dtype, self.device, v_head_dim=0)
        elif getattr(model, "owns_token_state", False):
            # the model keeps its per-token state itself (latent rings, sparse tables): the block cache only accounts
            # for positions and capacity
            self.kv = PagedKVCache(spec.layers, 1, 8, num_blocks, settings.kv_block, dtype, self.device, v_head_dim=0)
        else:
            self.kv = PagedKVCache(spec.layers, hkv, spec.head_dim, num_blocks, settings.kv_block, dtype, self.device)
        # 8-bit store behind the block cache: groups that leave the recent window are sealed after every step
        self.max_groups = 0
        if settings.kv_format == "affine8":
            from .kv_compact import CompactKV
            if spec.mla is not None or getattr(model, "state_slot_count", 0) or getattr(model, "owns_token_state", False) \
                    or spec.head_dim != 128 or settings.kv_block != 64 or spec.extra.get("gemma"):
                raise ValueError("--kv-format affine8 needs a GQA decoder with 128-wide heads and 64-token blocks")
            self.kv.compact = CompactKV(spec.layers, hkv, spec.head_dim, max(num_blocks // 2, 1), self.device,
                                        recent=settings.kv_recent)
            self.max_groups = max(settings.capacity // 128, 1)
        self.max_blocks = (settings.capacity + settings.kv_block - 1) // settings.kv_block
        self.max_batch = max(settings.max_batch, 1)
        self.max_prefill_rows = max_prefill_rows
        self.take_limit = getattr(model, "prefill_take_limit", None) or max_prefill_rows   # rows of ONE sequence per chunk
        # models that encode a prompt bidirectionally need all of it in one chunk: a prompt is never split, it waits
        # for a chunk with room (and is refused when it is longer than a chunk)
        self.whole_prompt = bool(getattr(model, "whole_prompt_prefill", False))
        self.prefill_batch = ForwardBatch(BatchLayout(self.max_batch, max(max_prefill_rows, self.max_batch),
                                                      self.max_blocks), self.device)
        self.graphs: dict[tuple[int, int], _Graph] = {}
        self.eager_decode_batch: dict[int, ForwardBatch] = {}
        self.seqs: dict[int, Sequence] = {}
        self._next_id = 0
        self.poisoned = False
        self.use_graph = settings.graph and self.device.type == "cuda"
        # models with per-sequence recurrent state (gated-delta-net mixers) address it by slot; the last slot
        # is scratch for the padding rows of a decode bucket. Their step is not graph-captured.
        self.state_slots: list[int] | None = None
        if getattr(model, "state_slot_count", 0):
            self.state_slots = list(range(model.state_slot_count - 1))
            self.scratch_slot = model.state_slot_count - 1
            # a model whose state kernels take their slots from the packed step metadata can be captured
            if not getattr(model, "graph_safe_state", False):
                self.use_graph = False
        self.stats = {"prefill_tokens": 0, "decode_steps": 0, "decode_tokens": 0, "graph_replays": 0,
                      "captures": 0, "h2d_bytes": 0, "d2h_bytes": 0}
        self.fail_next_step = False      # host-side fault injection hook for tests

    # -- sequence management ---------------------------------------------------------------
    def add_sequence(self, prompt: list[int], mm_positions: list[int] | None = None,
                     mm_embeds: torch.Tensor | None = None) -> Sequence:
        """``mm_positions`` / ``mm_embeds``: prompt indices whose embedding rows are supplied by the caller (the
        vision tower's output for image placeholder tokens) instead of the embedding table."""
        self._check()
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) + 1 > self.settings.capacity:
            raise ValueError(f"prompt of {len(prompt)} tokens exceeds the KV capacity {self.settings.capacity}")
        sid = self._next_id
        self._next_id += 1
        s = Sequence(sid, list(prompt))
        if mm_positions:
            if mm_embeds is None or mm_embeds.shape[0] != len(mm_positions) or mm_embeds.shape[1] != self.spec.hidden:
                raise ValueError("mm_embeds must hold one hidden-sized row per mm position")
            s.mm_positions, s.mm_embeds = list(mm_positions), mm_embeds
        if self.state_slots is not None:
            if not self.state_slots:
                raise ValueError("no free recurrent-state slot: too many live sequences")
            s.state_slot = self.state_slots.pop()
            self.model.reset_state(s.state_slot)
        self.seqs[sid] = s
        self.kv.add_sequence(sid)
        return s

    def free_sequence(self, seq_id: int) -> None:
        s = self.seqs.pop(seq_id, None)
        if s is not None and self.state_slots is not None and s.state_slot >= 0:
            self.state_slots.append(s.state_slot)
            s.state_slot = -1
        if seq_id in self.kv.seqs:
            self.kv.free_sequence(seq_id)

    def reset(self) -> None:
        for sid in list(self.kv.seqs):
            self.kv.free_sequence(sid)
        self.seqs.clear()
        if self.state_slots is not None:
            self.state_slots = list(range(self.model.state_slot_count - 1))
        self.poisoned = False
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            ops.read_status(self.device)
            from ..ops import chain
            chain.reset_workspace(self.device)      # phase counters of the decode chain, in case a step timed out

    def _check(self) -> None:
        if self.poisoned:
            raise EnginePoisoned("engine is poisoned by an earlier failure; call reset()")

    # -- prefill -----------------------------------------------------------------------------
    def prefill(self, seqs: list[Sequence], chunk: int | None = None) -> list[int]:
        """Prefill the given sequences to the end of their prompts (chunked) and return the first
        generated token of each. Sequences are packed row-wise into chunks of at most ``chunk``
        rows; only the chunk that contains a sequence's last prompt token computes its logits."""
        self._check()
        chunk = min(chunk or self.settings.chunk or self.max_prefill_rows, self.max_prefill_rows)
        first: dict[int, int] = {}
        try:
            pending = [s for s in seqs if s.prefilled < len(s.prompt)]
            while pending:
                rows_left = chunk
                part: list[tuple[Sequence, int]] = []
                for s in pending:
                    if rows_left <= 0 or len(part) >= self.max_batch:
                        break
                    take = min(len(s.prompt) - s.prefilled, rows_left, self.take_limit)
                    if self.whole_prompt and take < len(s.prompt) - s.prefilled:
                        if not part and len(s.prompt) > min(chunk, self.take_limit):
                            raise ValueError(f"prompt of {len(s.prompt)} tokens does not fit one prefill chunk of {chunk} rows")
                        break
                    part.append((s, take))
                    rows_left -= take
                toks = self._prefill_chunk(part)
                for (s, take), t in zip(part, toks):
                    if s.prefilled == len(s.prompt):
                        first[s.seq_id] = t
                        s.pending = t
                        s.output.append(t)
                pending = [s for s in pending if s.prefilled < len(s.prompt)]
        except Exception:
            self.poisoned = True
            raise
        return [first[s.seq_id] for s in seqs if s.seq_id in first]

    def prefill_some(self, seqs: list[Sequence], max_rows: int) -> list[Sequence]:
        """ONE packed prefill chunk of at most ``max_rows`` prompt rows over ``seqs`` (in order, each contributing as
        many of its remaining prompt tokens as fit). Returns the sequences whose prompt was completed by this chunk;
        their first generated token is in ``pending`` / ``output``. This is the unit the scheduler interleaves with
        decode steps, so that a long prompt does not stall the sequences that are already generating."""
        self._check()
        rows_left = min(max_rows, self.max_prefill_rows)
        part: list[tuple[Sequence, int]] = []
        for s in seqs:
            if rows_left <= 0 or len(part) >= self.max_batch:
                break
            rem = len(s.prompt) - s.prefilled
            if rem <= 0:
                continue
            take = min(rem, rows_left, self.take_limit)
            if self.whole_prompt and take < rem:
                if not part and rem > min(self.max_prefill_rows, self.take_limit):
                    raise ValueError(f"prompt of {rem} tokens does not fit one prefill chunk of {self.max_prefill_rows} rows")
                break
            part.append((s, take))
            rows_left -= take
        if not part:
            return []
        try:
            toks = self._prefill_chunk(part)
        except OutOfBlocks:
            raise
        except Exception:
            self.poisoned = True
            raise
        done = []
        for (s, _), t in zip(part, toks):
            if s.prefilled == len(s.prompt):
                s.pending = t
                s.output.append(t)
                done.append(s)
        return done

    def _need_blocks(self, items: list[tuple[int, int]]) -> None:
        """Refuse a step before it reserves anything when the (sequence, new tokens) pairs do not all fit: a step
        either reserves for every sequence or for none."""
        need = sum(self.kv.blocks_needed(sid, n) for sid, n in items)
        if need > self.kv.alloc.free_blocks:
            raise OutOfBlocks(f"step needs {need} KV blocks, {self.kv.alloc.free_blocks} free")

    def _prefill_chunk(self, part: list[tuple[Sequence, int]]) -> list[int]:
        self._need_blocks([(s.seq_id, take) for s, take in part])
        fb = self.prefill_batch
        ids, positions, slots, q_lens, ctx_lens, block_rows, logit_rows = [], [], [], [], [], [], []
        row = 0
        for s, take in part:
            kvs = self.kv.seqs[s.seq_id]
            sl = self.kv.reserve(s.seq_id, take)
            ids += s.prompt[s.prefilled: s.prefilled + take]
            positions += list(range(kvs.length, kvs.length + take))
            slots += sl
            q_lens.append(take)
            ctx_lens.append(kvs.length + take)
            block_rows.append(list(kvs.blocks))
            logit_rows.append(row + take - 1)
            row += take
        mult = getattr(self.model.comm, "size", 1) * 128 if getattr(self.model.comm, "fused", False) else 1
        if mult > 1 and row >= mult and (row + mult - 1) // mult * mult <= fb.layout.max_rows:
            # sequence-parallel prefill shards rows over the ranks in 128-row blocks: pad with rows
            # that belong to no sequence (no KV write, no logits)
            pad = (row + mult - 1) // mult * mult - row
            ids += [0] * pad; positions += [0] * pad; slots += [-1] * pad
        fb.fill(ids=ids, positions=positions, slots=slots, q_lens=q_lens, ctx_lens=ctx_lens, block_rows=block_rows,
                logit_rows=logit_rows, is_decode=False,
                state_slots=[s.state_slot for s, _ in part] if self.state_slots is not None else None)
        fb.upload()
        fb.state_slots = [s.state_slot for s, _ in part]
        out = self.model.forward(fb, self.kv, inputs_embeds=self._mm_embeds(part, fb, len(ids)))
        toks = [int(t) for t in out.cpu().tolist()]
        self._after_sync()
        for s, take in part:
            self.kv.commit(s.seq_id, take)
            s.prefilled += take
        self.stats["prefill_tokens"] += row
        return toks

    def _mm_embeds(self, part: list[tuple[Sequence, int]], fb: ForwardBatch, rows: int) -> torch.Tensor | None:
        """Embedding rows of a prefill chunk with the multimodal rows replaced, or None for text-only chunks."""
        dst, src_rows, row = [], [], 0
        for s, take in part:
            if s.mm_positions:
                lo, hi = s.prefilled, s.prefilled + take
                for j, p in enumerate(s.mm_positions):
                    if lo <= p < hi:
                        dst.append(row + p - lo)
                        src_rows.append(s.mm_embeds[j])
            row += take
        if not dst:
            return None
        from .. import ops
        w = self.model.w
        emb = ops.embed(fb.ids, w.embed)
        emb[torch.tensor(dst, dtype=torch.long, device=emb.device)] = torch.stack(src_rows).to(emb.dtype).to(emb.device)
        return emb

    # -- decode ------------------------------------------------------------------------------
    def _fill_decode(self, fb: ForwardBatch, seqs: list[Sequence], bucket: int) -> None:
        self._need_blocks([(s.seq_id, 1) for s in seqs])
        ids, positions, slots, q_lens, ctx_lens, block_rows = [], [], [], [], [], []
        for s in seqs:
            kvs = self.kv.seqs[s.seq_id]
            sl = self.kv.reserve(s.seq_id, 1)
            ids.append(s.pending)
            positions.append(kvs.length)
            slots += sl
            q_lens.append(1)
            ctx_lens.append(kvs.length + 1)
            block_rows.append(list(kvs.blocks))
        pad = bucket - len(seqs)
        ids += [0] * pad; positions += [0] * pad; slots += [-1] * pad
        q_lens += [1] * pad; ctx_lens += [0] * pad; block_rows += [[]] * pad
        kv_start = group_rows = None
        if self.kv.compact is not None:
            c = self.kv.compact
            kv_start = [c.sealed_tokens(s.seq_id) for s in seqs]
            group_rows = [c.groups.get(s.seq_id, []) for s in seqs]
        st = None
        if self.state_slots is not None:
            st = [s.state_slot for s in seqs] + [self.scratch_slot] * pad
        fb.fill(ids=ids, positions=positions, slots=slots, q_lens=q_lens, ctx_lens=ctx_lens, block_rows=block_rows,
                logit_rows=list(range(bucket)), is_decode=True, nq=1, kv_start=kv_start, group_rows=group_rows,
                state_slots=st)
        fb.max_ctx = self.settings.capacity      # fixed launch geometry (graph-stable)

    def _decode_batch(self, bucket: int) -> ForwardBatch:
        fb = self.eager_decode_batch.get(bucket)
        if fb is None:
            fb = ForwardBatch(BatchLayout(bucket, bucket, self.max_blocks, self.max_groups), self.device)
            self.eager_decode_batch[bucket] = fb
        return fb

    def capture(self, bucket: int) -> _Graph:
        """Capture the decode step for a batch bucket: one eager warm-up on padding rows (which
        write no KV), then stream capture of the same step."""
        key = (bucket, 1)
        g = self.graphs.get(key)
        if g is not None:
            return g
        t0 = time.perf_counter()
        g = _Graph()
        fb = self._decode_batch(bucket)
        fb.fill(ids=[0] * bucket, positions=[0] * bucket, slots=[-1] * bucket, q_lens=[1] * bucket,
                ctx_lens=[0] * bucket, block_rows=[[]] * bucket, logit_rows=list(range(bucket)), is_decode=True,
                state_slots=[self.scratch_slot] * bucket if self.state_slots is not None else None)
        fb.max_ctx = self.settings.capacity
        fb.upload()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(fb, self.kv)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.model.forward(fb, self.kv)
        g.graph, g.batch, g.out = graph, fb, out
        self.graphs[key] = g
        self.stats["captures"] += 1
        log_json("graph_capture", bucket=bucket, ms=(time.perf_counter() - t0) * 1e3, verbose_only=True)
        return g

    def decode(self, seqs: list[Sequence]) -> list[int]:
        """One decode step for the given sequences (each must have a pending token)."""
        self._check()
        if self.fail_next_step:
            self.fail_next_step = False
            self.poisoned = True
            raise RuntimeError("injected step failure")
        try:
            n = len(seqs)
            bucket = bucket_for(n)
            provider = getattr(self.model, "expert_provider", None)
            if provider is not None:
                provider.begin_token()
            for s in seqs:
                if self.kv.seqs[s.seq_id].length + 1 > self.settings.capacity:
                    raise OutOfBlocks(f"sequence {s.seq_id} reached the KV capacity {self.settings.capacity}")
            if self.use_graph and provider is None:
                g = self.capture(bucket)
                fb = g.batch
                self._fill_decode(fb, seqs, bucket)
                fb.upload()
                g.graph.replay()
                out = g.out
                self.stats["graph_replays"] += 1
            else:
                fb = self._decode_batch(bucket)
                self._fill_decode(fb, seqs, bucket)
                fb.upload()
                out = self.model.forward(fb, self.kv)
            toks = [int(t) for t in out[:n].cpu().tolist()]
            if provider is not None:
                provider.finish_token()
            self.stats["h2d_bytes"] += fb.h2d_bytes()
            self.stats["d2h_bytes"] += 4 * bucket
            self._after_sync()
            for s, t in zip(seqs, toks):
                self.kv.commit(s.seq_id, 1)
                s.pending = t
                s.output.append(t)
            self._seal(seqs)
            self.stats["decode_steps"] += 1
            self.stats["decode_tokens"] += n
            return toks
        except OutOfBlocks:
            raise                      # nothing was reserved or launched: the caller may preempt and retry
        except Exception:
            self.poisoned = True
            raise

    def _seal(self, seqs: list[Sequence]) -> None:
        """Affine8 cache: pack the groups that left the recent window and give their BF16 blocks back. Runs between
        steps on the launching stream; prompts are sealed once they are complete (prefill chunks read BF16 only)."""
        c = self.kv.compact
        if c is None:
            return
        for s in seqs:
            if s.prefilled >= len(s.prompt):
                c.seal(self.kv, s.seq_id)

    def _no_compact(self, what: str) -> None:
        if self.kv.compact is not None:
            raise ValueError(f"{what} reads BF16 pages only and is not available with --kv-format affine8")

    def capture_verify(self, bucket: int, nq: int) -> _Graph:
        """Capture the verification step of ``nq`` rows per sequence for a batch bucket (decode-style attention over
        ``nq`` query rows; the reference captures its draft and verify steps per row count,
        src/backend/cuda/engine.rs:5347-5440). The graph's outputs are the greedy token of every row and the
        residual rows (for multi-token-prediction heads)."""
        key = (bucket, nq)
        g = self.graphs.get(key)
        if g is not None:
            return g
        t0 = time.perf_counter()
        g = _Graph()
        rows = bucket * nq
        fb = ForwardBatch(BatchLayout(bucket, rows, self.max_blocks), self.device)
        fb.fill(ids=[0] * rows, positions=[0] * rows, slots=[-1] * rows, q_lens=[nq] * bucket, ctx_lens=[0] * bucket,
                block_rows=[[]] * bucket, logit_rows=list(range(rows)), is_decode=True, nq=nq)
        fb.max_ctx = self.settings.capacity
        fb.upload()

        def step():
            n = self.model.hidden_states(fb, self.kv)
            return self.model.greedy(self.model.logits(n, fb)), self.model.last_residual, n
        # a caller may be collecting the final-normed rows of every forward (multi-token prediction): the warm-up and
        # capture passes are not its forwards; replays hand it the captured rows instead
        sink, self.model.normed_sink = getattr(self.model, "normed_sink", None), None
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out, hid, normed = step()
        self.model.normed_sink = sink
        g.graph, g.batch, g.out, g.hidden, g.normed = graph, fb, out, hid, normed
        self.graphs[key] = g
        self.stats["captures"] += 1
        self.stats["capture_ms"] = self.stats.get("capture_ms", 0.0) + (time.perf_counter() - t0) * 1e3
        return g

    # -- speculative verification --------------------------------------------------------------
    def verify(self, seqs: list[Sequence], drafts: list[list[int]], return_hidden: bool = False,
               device_out: bool = False):
        """Feed every sequence's pending token plus its draft tokens (same count k for all) through
        the target in ONE forward of k+1 rows per sequence and return the target's greedy token
        after each row: ``[[t_0 .. t_k]]`` per sequence. Nothing is committed; call
        :meth:`commit_verified` with the number of accepted drafts. Rows of rejected drafts leave
        stale K/V behind the committed length, which later steps simply overwrite (the paged
        cache needs no copy-back, unlike the reference's gather/scatter of tree rows,
        kernels/tree/meta.cu)."""
        self._check()
        self._no_compact("speculative verification")
        if self.fail_next_step:
            self.fail_next_step = False
            self.poisoned = True
            raise RuntimeError("injected step failure")
        try:
            k = len(drafts[0])
            assert all(len(d) == k for d in drafts), "all sequences must carry the same number of drafts"
            nq = k + 1
            # graph path: decode-style batch of nq rows per sequence in a bucket, replayed from a capture per (bucket, nq)
            graphed = (self.use_graph and getattr(self.model, "expert_provider", None) is None and nq <= 8
                       and self.state_slots is None and self.settings.spec_graph)
            bucket = bucket_for(len(seqs)) if graphed else len(seqs)
            g = self.capture_verify(bucket, nq) if graphed else None
            fb = g.batch if graphed else self.prefill_batch
            ids, positions, slots, q_lens, ctx_lens, block_rows = [], [], [], [], [], []
            for s, d in zip(seqs, drafts):
                kvs = self.kv.seqs[s.seq_id]
                if kvs.length + nq > self.settings.capacity:
                    raise OutOfBlocks(f"sequence {s.seq_id}: no KV headroom for {nq} verification rows")
                sl = self.kv.reserve(s.seq_id, nq)
                ids += [s.pending] + list(d)
                positions += list(range(kvs.length, kvs.length + nq))
                slots += sl
                q_lens.append(nq)
                ctx_lens.append(kvs.length + nq)
                block_rows.append(list(kvs.blocks))
            rows = len(ids)
            if graphed:
                pad = bucket - len(seqs)
                ids += [0] * (pad * nq); positions += [0] * (pad * nq); slots += [-1] * (pad * nq)
                q_lens += [nq] * pad; ctx_lens += [0] * pad; block_rows += [[]] * pad
                fb.fill(ids=ids, positions=positions, slots=slots, q_lens=q_lens, ctx_lens=ctx_lens, block_rows=block_rows,
                        logit_rows=list(range(bucket * nq)), is_decode=True, nq=nq)
                fb.max_ctx = self.settings.capacity
                fb.upload()
                g.graph.replay()
                out, hid_all = g.out[:rows], g.hidden
                if getattr(self.model, "normed_sink", None) is not None:
                    self.model.normed_sink.append(g.normed[:rows])
                self.stats["graph_replays"] += 1
                self.stats["verify_graph_replays"] = self.stats.get("verify_graph_replays", 0) + 1
            else:
                fb.fill(ids=ids, positions=positions, slots=slots, q_lens=q_lens, ctx_lens=ctx_lens, block_rows=block_rows,
                        logit_rows=list(range(rows)), is_decode=False)
                fb.upload()
                n = self.model.hidden_states(fb, self.kv)
                out = self.model.greedy(self.model.logits(n, fb))
                hid_all = self.model.last_residual
            if device_out:
                # the caller decides acceptance on the device and reads one verdict back (then calls _after_sync)
                self.stats["verify_rows"] = self.stats.get("verify_rows", 0) + rows
                return out
            toks = [int(t) for t in out.cpu().tolist()]
            self._after_sync()
            self.stats["verify_rows"] = self.stats.get("verify_rows", 0) + rows
            res = [toks[i * nq: (i + 1) * nq] for i in range(len(seqs))]
            if return_hidden:
                hid = hid_all
                return res, [hid[i * nq: (i + 1) * nq] for i in range(len(seqs))]
            return res
        except Exception:
            self.poisoned = True
            raise

    def forward_rows(self, seq: Sequence, tokens: list[int], return_logits: bool = True) -> torch.Tensor:
        """Uncommitted forward of ``tokens`` placed after the sequence's committed prefix (causal);
        returns the logits (or greedy ids) of every row. The K/V rows written stay behind the
        committed length and are overwritten by whatever runs next."""
        self._check()
        self._no_compact("an uncommitted multi-row forward")
        kvs = self.kv.seqs[seq.seq_id]
        n = len(tokens)
        sl = self.kv.reserve(seq.seq_id, n)
        fb = self.prefill_batch
        fb.fill(ids=tokens, positions=list(range(kvs.length, kvs.length + n)), slots=sl, q_lens=[n],
                ctx_lens=[kvs.length + n], block_rows=[list(kvs.blocks)], logit_rows=list(range(n)), is_decode=False)
        fb.upload()
        return self.model.forward(fb, self.kv, return_logits=return_logits)

    def verify_tree(self, seq: Sequence, tokens: list[int], depths: list[int], masks: list[int]) -> list[int]:
        """Verify a draft tree in one forward: row i holds ``tokens[i]`` at sequence position
        ``committed + depths[i]`` and cache slot ``committed + i``; ``masks[i]`` (bit j = row j is an
        ancestor-or-self) restricts what it sees among the tree rows. Returns the target's greedy
        token after every row."""
        self._check()
        self._no_compact("tree verification")
        try:
            kvs = self.kv.seqs[seq.seq_id]
            n = len(tokens)
            assert n <= 64 and tokens[0] == seq.pending
            if kvs.length + n > self.settings.capacity:
                raise OutOfBlocks("no KV headroom for the verification tree")
            sl = self.kv.reserve(seq.seq_id, n)
            fb = self._decode_batch(1) if n == 1 else self.prefill_batch
            fb = self.prefill_batch
            fb.fill(ids=tokens, positions=[kvs.length + d for d in depths], slots=sl, q_lens=[n],
                    ctx_lens=[kvs.length + n], block_rows=[list(kvs.blocks)], logit_rows=list(range(n)),
                    is_decode=True, nq=n, tree_mask=masks)
            fb.max_ctx = self.settings.capacity
            fb.upload()
            out = self.model.forward(fb, self.kv)
            toks = [int(t) for t in out.cpu().tolist()]
            self._after_sync()
            return toks
        except Exception:
            self.poisoned = True
            raise

    def commit_tree_path(self, seq: Sequence, path_rows: list[int], emitted: list[int]) -> None:
        """Compact the K/V of the accepted tree path onto consecutive positions and commit it."""
        kvs = self.kv.seqs[seq.seq_id]
        base = kvs.length
        src = [base + r for r in path_rows]
        dst = [base + j for j in range(len(path_rows))]
        moves = [(s_, d_) for s_, d_ in zip(src, dst) if s_ != d_]
        if moves:
            self.kv.move_rows(seq.seq_id, [m[0] for m in moves], [m[1] for m in moves])
        self.kv.commit(seq.seq_id, len(path_rows))
        seq.output.extend(emitted)
        seq.pending = emitted[-1]

    def commit_verified(self, seq: Sequence, emitted: list[int], n_draft_accepted: int) -> None:
        """Commit the pending token and the accepted drafts (their K/V rows are already in place),
        publish ``emitted`` and make its last token the new pending one."""
        self.kv.commit(seq.seq_id, n_draft_accepted + 1)
        seq.output.extend(emitted)
        seq.pending = emitted[-1]

    def _after_sync(self) -> None:
        """Runs right after a device-to-host read (an existing sync point): surface device status."""
        if self.device.type == "cuda":
            code = ops.read_status(self.device)
            if code[0] != 0:
                raise ops.DeviceStatusError(*code)

    # -- convenience ---------------------------------------------------------------------------
    def generate(self, prompts: list[list[int]], max_new_tokens: int, eos: int | None = None,
                 ignore_eos: bool = True, on_token=None) -> list[list[int]]:
        """Greedy generation for a batch of prompts; returns the generated ids per prompt
        (``generated[0]`` is the token emitted by prefill, as in the reference's ``generate``)."""
        seqs = [self.add_sequence(p) for p in prompts]
        try:
            self.prefill(seqs)
            if on_token:
                for s in seqs:
                    on_token(s.seq_id, s.output[-1])
            live = list(seqs)
            while live:
                live = [s for s in live if len(s.output) < max_new_tokens and
                        not (not ignore_eos and eos is not None and s.output[-1] == eos)]
                if not live:
                    break
                toks = self.decode(live)
                if on_token:
                    for s, t in zip(live, toks):
                        on_token(s.seq_id, t)
            return [list(s.output) for s in seqs]
        finally:
            for s in seqs:
                self.free_sequence(s.seq_id)
