"""Trace comparison: error metrics between two operator traces (max-abs, RMSE, BF16 half-ULP
ratio, bit mismatches after BF16 rounding, top-two logit margin), optional per-tensor limit files,
and JSON-lines log comparison (the reference's ``verify`` / ``compare-prefill`` / ``compare-log``,
src/verify.rs:89-120, 458-712, 876-960)."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..loaders.safetensors_io import SafetensorsFile


def tensor_metrics(a: torch.Tensor, b: torch.Tensor) -> dict:
    a, b = a.to(torch.float32).flatten(), b.to(torch.float32).flatten()
    if a.shape != b.shape:
        return {"shape_mismatch": [list(a.shape), list(b.shape)]}
    diff = (a - b).abs()
    # half a BF16 ULP at the reference magnitude: 2**(floor(log2|b|) - 8)
    mag = b.abs().clamp_min(1e-30)
    half_ulp = torch.pow(2.0, torch.floor(torch.log2(mag)) - 8.0)
    bits = (a.to(torch.bfloat16).view(torch.int16) != b.to(torch.bfloat16).view(torch.int16)).sum().item()
    out = {"max_abs": diff.max().item() if diff.numel() else 0.0,
           "rmse": diff.pow(2).mean().sqrt().item() if diff.numel() else 0.0,
           "half_ulp_ratio": (diff / half_ulp).max().item() if diff.numel() else 0.0,
           "bf16_bit_mismatches": int(bits), "numel": a.numel()}
    return out


def top_two_margin(logits: torch.Tensor) -> float:
    v = torch.topk(logits.to(torch.float32).flatten(), 2).values
    return float(v[0] - v[1])


def compare_traces(trace: str | Path, reference: str | Path, limits: str | Path | None = None) -> dict:
    ta, tb = SafetensorsFile(trace), SafetensorsFile(reference)
    lim = json.loads(Path(limits).read_text()) if limits else {}
    report, failures = {}, []
    try:
        for name in sorted(set(ta.tensors) | set(tb.tensors)):
            if name not in ta.tensors or name not in tb.tensors:
                report[name] = {"missing_in": "trace" if name not in ta.tensors else "reference"}
                failures.append(name)
                continue
            m = tensor_metrics(ta.tensor(name), tb.tensor(name))
            if name.endswith("logits"):
                m["top_two_margin"] = top_two_margin(tb.tensor(name))
            report[name] = m
            bound = lim.get(name, lim.get("*"))
            if "shape_mismatch" in m or (bound is not None and m["max_abs"] > bound):
                failures.append(name)
        return {"tensors": report, "failures": failures, "ok": not failures,
                "devices": [ta.metadata.get("device"), tb.metadata.get("device")]}
    finally:
        ta.close(); tb.close()


def compare_logs(a: str | Path, b: str | Path) -> dict:
    """Compare two JSON-lines result logs field by field (generated ids must be identical)."""
    def load(p):
        return [json.loads(l) for l in Path(p).read_text().splitlines() if l.strip().startswith("{")]
    la, lb = load(a), load(b)
    diffs = []
    for i, (x, y) in enumerate(zip(la, lb)):
        for k in ("generated_ids", "input_ids", "text"):
            if k in x or k in y:
                if x.get(k) != y.get(k):
                    diffs.append({"record": i, "field": k})
    if len(la) != len(lb):
        diffs.append({"record_count": [len(la), len(lb)]})
    return {"records": min(len(la), len(lb)), "differences": diffs, "ok": not diffs}
