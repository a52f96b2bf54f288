"""Library surface: ``Model`` and ``generate_plain``.

Mirrors the reference's model façade (src/model.rs:185-405 ``Model::{load, prefill, decode,
capture, reset, embed, ...}``, ``generate_plain`` :89-127, ``GenerationOutput``) on top of the
batched engine: the single-sequence calls operate on an implicit "current" sequence, the batched
calls (``generate_batch``) expose continuous batching.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .config import ModelSpec, Settings, named_shape, read_model_spec
from .engine.engine import Engine, Sequence
from .models.decoder import DecoderModel
from .models.weights import TPInfo, random_decoder_weights
from .planner.plan import plan_engine
from .utils.log import log_json


@dataclass
class GenerationOutput:
    ids: list[int]
    prefill_ms: float = 0.0
    capture_ms: float = 0.0
    decode_ms: float = 0.0
    decode_steps: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def decode_tok_s(self) -> float:
        return 1000.0 * self.decode_steps / self.decode_ms if self.decode_ms > 0 else 0.0


class Model:
    """A loaded model bound to one device (or one tensor/expert-parallel rank)."""

    def __init__(self, engine: Engine, spec: ModelSpec, settings: Settings, tokenizer=None, name: str | None = None):
        self.engine, self.spec, self.settings = engine, spec, settings
        self.tokenizer = tokenizer
        self.name = name or spec.name
        self._seq: Sequence | None = None
        self.load_ms = 0.0
        self.vision = None                 # models.vision.VisionTower of vision-language checkpoints

    # -- construction ------------------------------------------------------------------------
    @classmethod
    def load(cls, model: "str | ModelSpec", settings: Settings | None = None, device: str | torch.device | None = None,
             random_init: bool | None = None, seed: int = 0, comm=None, ep=None) -> "Model":
        """Load a checkpoint directory, or a named shape with seeded random weights
        (``random_init``; implied when ``model`` names a shape rather than a directory)."""
        t0 = time.perf_counter()
        settings = settings or Settings()
        if device is None:
            device = f"cuda:{settings.device}" if torch.cuda.is_available() else "cpu"
        device = torch.device(device)
        tokenizer = None
        preset: ModelSpec | None = None
        if isinstance(model, ModelSpec):          # an explicit (possibly modified) shape: random-init weights
            preset, model = model, model.name
        path = Path(model)
        tp = TPInfo(comm.rank, comm.size) if comm is not None else TPInfo()
        epi = TPInfo(ep.rank, ep.size) if ep is not None else TPInfo()
        if preset is None and path.is_dir() and not random_init:
            from .loaders.checkpoint import load_decoder_weights
            from .loaders.tokenizer import load_tokenizer
            spec = read_model_spec(path)
            if spec.extra.get("hrm"):
                # looped two-stack decoder: its own weight assembly over the published tensor names (text side only)
                from .loaders.checkpoint import checkpoint_source
                from .models.hrm import build_hrm_weights
                source, close = checkpoint_source(path, spec, device)
                try:
                    weights = build_hrm_weights(spec, source, device)
                finally:
                    close()
            else:
                weights = load_decoder_weights(path, spec, device, tp, epi)
            tokenizer = load_tokenizer(path)
            name = path.name
        else:
            spec = preset if preset is not None else (read_model_spec(path) if path.is_dir() else named_shape(model))
            if spec.extra.get("v41"):
                from .models.deepseek_v41 import build_v41_weights
                from .models.weights import DTYPES, synthetic_source
                weights = build_v41_weights(spec, seed, device, synthetic_source(spec, seed, device, DTYPES[spec.dtype]),
                                            tp, epi)
            elif spec.extra.get("hrm"):
                from .models.hrm import random_hrm_weights
                weights = random_hrm_weights(spec, seed, device)
            elif spec.mla is not None:
                from .models.deepseek import build_deepseek_weights
                from .models.weights import DTYPES, synthetic_source
                weights = build_deepseek_weights(spec, synthetic_source(spec, seed, device, DTYPES[spec.dtype]),
                                                 device, tp, epi)
            else:
                weights = random_decoder_weights(spec, seed, device, tp, epi)
            name = spec.name
        if (spec.moe is not None and spec.moe.expert_format == "nvfp4" and device.type == "cuda" and spec.mla is None
                and ep is None and os.environ.get("FLYINGFISH_FP4_EXPERTS", "1") != "0"):
            from .ops.moe_cuda import pack_experts_nvfp4
            log_json("nvfp4_experts_packed", verbose_only=True, bytes=pack_experts_nvfp4(weights))
        if spec.mla is not None:
            from .models.deepseek import DeepseekModel
            net = DeepseekModel(weights, comm=comm)
        elif spec.extra.get("v41"):
            from .models.deepseek_v41 import DeepseekV41Model
            net = DeepseekV41Model(weights, comm=comm, max_sequences=settings.max_batch, max_len=settings.capacity,
                                   max_chunk=min(settings.chunk or 256, 256), seed=seed)
        elif spec.extra.get("hrm"):
            from .models.hrm import HrmModel
            net = HrmModel(weights, comm=comm)
        elif spec.extra.get("flint"):
            from .models.flint import FlintModel
            net = FlintModel(weights, comm=comm, seed=seed, state=weights.extra.get("state"))
        elif spec.extra.get("gemma"):
            from .models.gemma import GemmaModel
            net = GemmaModel(weights, comm=comm, seed=seed)
        elif spec.extra.get("gdn"):
            from .models.hybrid import HybridModel
            net = HybridModel(weights, comm=comm, max_sequences=settings.max_batch, seed=seed)
        else:
            net = DecoderModel(weights, comm=comm)
        if ep is not None:
            net.ep = ep
        if device.type == "cuda":
            # measured kernel choices of an earlier ``ff calibrate`` for this model, device and kernel build
            try:
                from .planner.calibrate import apply_kernel_choices, load_calibration
                applied = apply_kernel_choices(load_calibration(str(model), settings, device))
                if applied:
                    log_json("kernel_choices_applied", verbose_only=True, count=applied)
            except (OSError, ValueError, RuntimeError):
                pass
        plan = plan_engine(spec, settings, device, weights_bytes=weights.nbytes(), tp=tp.size)
        log_json("prefill_memory_plan", verbose_only=True, **plan.to_json())
        chunk = plan.prefill_chunk
        if ep is not None and getattr(ep, "arena", None) is not None and getattr(ep, "max_rows", 0) > 0:
            chunk = min(chunk, ep.max_rows)          # the expert-parallel receive buffers are sized for this many rows per call
        engine = Engine(net, spec, settings, plan.kv_blocks, device, max_prefill_rows=chunk)
        m = cls(engine, spec, settings, tokenizer, name)
        if spec.extra.get("vision") and spec.extra["vision"].get("kind") == "minicpm":
            from .models.minicpm_vision import MiniCpmVisionSpec, MiniCpmVisionTower
            vspec = MiniCpmVisionSpec(**{k: v for k, v in spec.extra["vision"].items() if k != "kind"})
            if path.is_dir() and not random_init:
                from .loaders.safetensors_io import MappedCheckpoint
                ckpt = MappedCheckpoint(path)
                m.vision = MiniCpmVisionTower(vspec, {n: ckpt.tensor(n) for n in vspec.expected_tensors() if ckpt.has(n)}, device)
            else:
                m.vision = MiniCpmVisionTower.random(vspec, device, seed + 1)
            engine.mm_encoder = m.encode_images
        elif spec.extra.get("vision"):
            from .models.vision import VisionSpec, VisionTower
            vspec = VisionSpec(**spec.extra["vision"])
            if path.is_dir() and not random_init:
                from .loaders.checkpoint import load_prefixed_tensors
                m.vision = VisionTower(vspec, load_prefixed_tensors(path, ("visual.", "model.visual.")), device)
            else:
                m.vision = VisionTower.random(vspec, device, seed + 1)
            engine.mm_encoder = m.encode_images
        m.load_ms = (time.perf_counter() - t0) * 1e3
        log_json("backend_device", verbose_only=True, device=str(device), model=name, load_ms=m.load_ms)
        return m

    # -- single-sequence surface -------------------------------------------------------------
    def reset(self) -> None:
        self.engine.reset()
        self._seq = None

    def prefill(self, ids: list[int]) -> int:
        """Start a sequence with ``ids``; returns the first generated token."""
        if self._seq is not None:
            self.engine.free_sequence(self._seq.seq_id)
            self._seq = None
        store = self.prefix_store()
        if store is not None:
            self._seq = store.restore(self, ids)
        if self._seq is None:
            self._seq = self.engine.add_sequence(ids)
        first = self.engine.prefill([self._seq])[0]
        if store is not None:
            store.store(self, self._seq)
        return first

    def prefix_store(self):
        """The on-disk prefix cache of ``--prefix-cache true`` (under the runtime directory), or None."""
        if not self.settings.prefix_cache:
            return None
        if getattr(self, "_prefix_store", None) is None:
            from .utils.prefix_cache import PrefixStore
            self._prefix_store = PrefixStore(self.settings.resolved_runtime_dir() / "prefix")
        return self._prefix_store

    def encode_images(self, ids: list[int], images: list) -> tuple[list[int], list[int], torch.Tensor]:
        """Runs the vision tower over ``images`` (``serve.image.Image``) and expands every image placeholder of
        ``ids`` to the span the tower fills. Returns (expanded ids, placeholder positions, embedding rows)."""
        from .serve.image import expand_image_tokens, image_token_count, pack_patches
        if self.vision is None:
            raise ValueError("this model has no vision tower")
        vs = self.vision.spec
        if self.spec.extra["vision"].get("kind") == "minicpm":
            return self._encode_sliced_images(ids, images)
        packed = [pack_patches(im, patch=vs.patch, merge=vs.merge, temporal=vs.temporal) for im in images]
        patches = [torch.from_numpy(p) for p, _ in packed]
        grids = [g for _, g in packed]
        embeds = torch.cat(self.vision.forward(patches, grids), 0)
        token = int(self.spec.extra["image_token_id"])
        out = expand_image_tokens(ids, token, [image_token_count(g, vs.merge) for g in grids])
        positions = [i for i, t in enumerate(out) if t == token]
        return out, positions, embeds

    def _encode_sliced_images(self, ids: list[int], images: list) -> tuple[list[int], list[int], torch.Tensor]:
        """MiniCPM-V style: every image is shown whole (about ``slice_scale`` pixels a side) and, when it is large, as a
        grid of tiles; all views of all images go through the tower together, and an image's placeholder becomes
        ``start thumb end`` followed by ``slice_start tile slice_end`` per tile with a newline token between tile rows."""
        from .models.minicpm_vision import expand_view_tokens
        from .serve.image import pack_slices
        vs, ex = self.vision.spec, self.spec.extra
        patches, grids, plans = [], [], []
        for im in images:
            views, plan = pack_slices(im, patch=vs.patch, max_slices=int(ex.get("max_slices", 9)), scale=int(ex.get("slice_scale", 448)))
            vg = [(g[1], g[2]) for g in plan.grids(vs.patch)]
            patches += [torch.from_numpy(v) for v in views]
            grids += vg
            per = vs.patches_per_token
            plans.append((vg[0][0] * vg[0][1] // per, plan.rows, plan.cols, vg[1][0] * vg[1][1] // per if plan.rows else 0))
        embeds = torch.cat(self.vision.forward(patches, grids), 0)
        token = int(ex["image_token_id"])
        out = expand_view_tokens(ids, token, plans, int(ex["image_start_id"]), int(ex["image_end_id"]), int(ex["slice_start_id"]),
                                 int(ex["slice_end_id"]), int(ex["newline_id"]))
        positions = [i for i, t in enumerate(out) if t == token]
        if len(positions) != embeds.shape[0]:
            raise RuntimeError(f"{len(positions)} image rows in the prompt for {embeds.shape[0]} rows from the tower")
        return out, positions, embeds

    def prefill_multimodal(self, ids: list[int], images: list) -> int:
        """Like :meth:`prefill` for a prompt with one image placeholder token per image."""
        ids, positions, embeds = self.encode_images(ids, images)
        if self._seq is not None:
            self.engine.free_sequence(self._seq.seq_id)
        self._seq = self.engine.add_sequence(ids, positions, embeds)
        return self.engine.prefill([self._seq])[0]

    def decode(self) -> int:
        """One greedy decode step for the current sequence."""
        assert self._seq is not None, "prefill first"
        return self.engine.decode([self._seq])[0]

    def capture(self) -> float:
        """Capture the batch-1 decode graph ahead of time; returns milliseconds spent."""
        t0 = time.perf_counter()
        if self.engine.use_graph:
            self.engine.capture(1)
        return (time.perf_counter() - t0) * 1e3

    def graph_decode(self) -> bool:
        return self.engine.use_graph

    # -- generation --------------------------------------------------------------------------
    def generate_batch(self, prompts: list[list[int]], max_new_tokens: int, ignore_eos: bool = True,
                       on_token=None) -> list[list[int]]:
        return self.engine.generate(prompts, max_new_tokens, self.spec.eos_token_id, ignore_eos, on_token)


def generate_plain(model: Model, ids: list[int], count: int, ignore_eos: bool = False, graph: bool = True,
                   on_token=None) -> GenerationOutput:
    """Greedy loop: prefill -> optional graph capture -> decode until EOS or ``count`` tokens.
    ``ids[0]`` of the result is the token emitted by prefill."""
    eng = model.engine
    eng.use_graph = graph and eng.device.type == "cuda"
    sync = (lambda: torch.cuda.synchronize(eng.device)) if eng.device.type == "cuda" else (lambda: None)
    t0 = time.perf_counter()
    first = model.prefill(ids)
    sync()
    t1 = time.perf_counter()
    out = [first]
    if on_token:
        on_token(first)
    cap_ms = model.capture() if eng.use_graph else 0.0
    t2 = time.perf_counter()
    eos = model.spec.eos_token_id
    steps = 0
    while len(out) < count and not (not ignore_eos and eos is not None and out[-1] == eos):
        tok = model.decode()
        steps += 1
        out.append(tok)
        if on_token:
            on_token(tok)
    sync()
    t3 = time.perf_counter()
    return GenerationOutput(ids=out, prefill_ms=(t1 - t0) * 1e3, capture_ms=cap_ms, decode_ms=(t3 - t2) * 1e3,
                            decode_steps=steps)
