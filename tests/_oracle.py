"""Shared check: a model loaded on the GPU against the same model on the CPU (FP32-math oracle operators).

Test-sized random weights are drawn on the host for every device, so the two models hold identical tensors; what
differs is BF16 kernel arithmetic against FP32 oracle arithmetic, hence a tolerance relative to the activations' scale."""
import torch

from flyingfish_b200.models.encoder import run_whole


def assert_hidden_close(cpu_model, gpu_model, prompts, rel: float = 0.06) -> None:
    a = run_whole(cpu_model, prompts, "hidden")
    b = run_whole(gpu_model, prompts, "hidden")
    for x, y in zip(a, b):
        x, y = x.float().cpu(), y.float().cpu()
        assert torch.isfinite(y).all()
        scale = max(x.abs().max().item(), 1e-3)
        err = (x - y).abs().max().item()
        assert err <= rel * scale, f"hidden states differ: max err {err} at scale {scale}"
        cos = torch.nn.functional.cosine_similarity(x.flatten(), y.flatten(), dim=0).item()
        assert cos > 0.995, f"cosine {cos}"


def assert_tokens_equal_up_to_ties(model, prompt, want, got, tol: float = 0.08) -> None:
    """``got`` must equal ``want`` token by token; where they part, the two candidates must be a near-tie in
    ``model``'s own logits for that position (different summation orders may resolve a tie differently), and the
    comparison stops there because the continuations are then different texts."""
    for p, (w, g) in enumerate(zip(want, got)):
        if w == g:
            continue
        lg = run_whole(model, [list(prompt) + list(want[:p])], "logits")[0][-1].float().cpu()
        margin = abs(lg[w].item() - lg[g].item())
        scale = max(lg.abs().max().item(), 1e-3)
        assert margin <= tol * scale, f"token {p}: {w} vs {g} differ by {margin} (scale {scale}): not a tie"
        return
    assert len(want) == len(got)


def assert_rows_mostly_close(cpu_model, gpu_model, prompts, rel: float = 0.06, frac: float = 0.9) -> None:
    """For mixture-of-experts models: a router score that is a near-tie may pick a different expert on the two
    devices, which changes that row discretely. So the bound is on rows: at least ``frac`` of the final hidden rows
    must agree within ``rel`` of the activations' scale, and all must be finite."""
    from flyingfish_b200.models.encoder import run_whole as _rw
    import torch as _t
    good = total = 0
    for p in prompts:
        for n in (len(p),):
            x = _rw(cpu_model, [p[:n]], "hidden")[0].float().cpu()
            y = _rw(gpu_model, [p[:n]], "hidden")[0].float().cpu()
            assert _t.isfinite(y).all()
            scale = max(x.abs().max().item(), 1e-3)
            good += int(((x - y).abs().max(dim=-1).values <= rel * scale).sum())
            total += x.shape[0]
    assert good >= frac * total, f"only {good} of {total} rows agree"
