"""Canary-style attention encoder-decoder: task prompt, position rows, the cached decoder against a plain teacher-forced
PyTorch decoder, configuration and checkpoint contract, and the CUDA path against the CPU path."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from flyingfish_b200.loaders.safetensors_io import save_safetensors
from flyingfish_b200.models.conformer import random_tensors
from flyingfish_b200.speech import CanaryModel, CanarySpec, canary_prompt, canary_tiny
from flyingfish_b200.speech.canary import sinusoidal_rows


def test_prompt_maps_languages_and_punctuation():
    table = {"<|startofcontext|>": 7, "<|startoftranscript|>": 4, "<|emo:undefined|>": 16, "<|en|>": 64, "<|de|>": 78, "<|pnc|>": 5,
             "<|nopnc|>": 6, "<|noitn|>": 9, "<|notimestamp|>": 11, "<|nodiarize|>": 13}
    enc = lambda text: [table.get(text, 0)]
    assert canary_prompt(enc, "en", "en", True) == [7, 4, 16, 64, 64, 5, 9, 11, 13]
    assert canary_prompt(enc, "en", "de", False) == [7, 4, 16, 64, 78, 6, 9, 11, 13]
    with pytest.raises(ValueError, match="unsupported Canary language zz"):
        canary_prompt(enc, "en", "zz", True)
    with pytest.raises(ValueError, match="not atomic"):
        canary_prompt(lambda text: [1, 2], "en", "en", True)


def test_position_rows():
    rows = sinusoidal_rows(16, 1024)
    assert rows.shape == (16, 1024)
    assert rows[0, :512].abs().max() == 0 and torch.allclose(rows[0, 512:], torch.full((512,), 1 / 32.0))
    assert abs(float(rows[3, 0]) - math.sin(3.0) / 32.0) < 1e-6
    slowest = 10000.0 ** ((1024 - 2.0) / 1024)
    assert abs(float(rows[5, 511]) - math.sin(5.0 / slowest) / 32.0) < 1e-6


def _plain_logits(spec, tensors, enc_rows, ids):
    """Teacher-forced FP32 decoder over ``ids`` with cross-attention over ``enc_rows`` [T, hidden]: logits [len, vocab]."""
    W = {k: v.float() for k, v in tensors.items()}
    h, nh = spec.hidden, spec.heads
    n = len(ids)
    ln = lambda x, name: F.layer_norm(x, (h,), W[f"{name}.weight"], W[f"{name}.bias"], 1e-5)
    lin = lambda x, name: x @ W[f"{name}.weight"].t() + W[f"{name}.bias"]
    x = W["model.decoder.embed_tokens.weight"][torch.tensor(ids)] + sinusoidal_rows(n, h)
    x = ln(x, "model.decoder.embedding_layernorm")
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))

    def attend(q, k, v, mask):
        q, k, v = (t.reshape(t.shape[0], nh, 128).transpose(0, 1) for t in (q, k, v))
        sc = q @ k.transpose(1, 2) / math.sqrt(128.0)
        if mask is not None:
            sc = sc.masked_fill(~mask[None], float("-inf"))
        return (torch.softmax(sc, -1) @ v).transpose(0, 1).reshape(-1, h)

    for i in range(spec.decoder_layers):
        p = f"model.decoder.layers.{i}"
        y = ln(x, f"{p}.input_layernorm")
        a = attend(lin(y, f"{p}.self_attn.q_proj"), lin(y, f"{p}.self_attn.k_proj"), lin(y, f"{p}.self_attn.v_proj"), causal)
        x = x + lin(a, f"{p}.self_attn.o_proj")
        y = ln(x, f"{p}.post_attention_layernorm")
        a = attend(lin(y, f"{p}.encoder_attn.q_proj"), lin(enc_rows, f"{p}.encoder_attn.k_proj"), lin(enc_rows, f"{p}.encoder_attn.v_proj"), None)
        x = x + lin(a, f"{p}.encoder_attn.o_proj")
        y = ln(x, f"{p}.final_layernorm")
        x = x + lin(torch.relu(lin(y, f"{p}.mlp.fc1")), f"{p}.mlp.fc2")
    return lin(ln(x, "model.decoder.norm"), "proj_out")


def _tensors(spec, seed):
    t = random_tensors(spec.expected_tensors(), seed, std=0.08)
    t["proj_out.weight"] = t["model.decoder.embed_tokens.weight"].clone()
    # weights as the BF16 GEMMs see them
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 else v) for k, v in t.items()}


def _waves():
    g = torch.Generator().manual_seed(31)
    return [0.1 * torch.randn(16000, generator=g), 0.1 * torch.randn(7000, generator=g)]


def _check_generation(spec, tensors, model, outs, prompt, tol):
    """Every generated token is the arg-max of the plain decoder's logits given the encoder rows the model produced, or
    a near-tie with it (the comparison stops at the first tie)."""
    feat, valid = model.mel.extract(_waves())
    encoded, rows = model.encoder.encode(feat, valid.tolist())
    for b, ids in enumerate(outs):
        enc_rows = encoded[b, : rows[b]].float().cpu()
        lg = _plain_logits(spec, tensors, enc_rows, ids[:-1])
        for t in range(len(prompt) - 1, len(ids) - 1):
            best, got = int(lg[t].argmax()), ids[t + 1]
            if best != got:
                assert float(lg[t, best] - lg[t, got]) <= tol * float(lg[t].abs().max()), (b, t, best, got)
                break


def test_cached_decoder_matches_teacher_forcing_cpu():
    spec = canary_tiny()
    tensors = _tensors(spec, 3)
    model = CanaryModel(spec, tensors)
    prompt = [7, 4, 16, 64, 64, 5, 9, 11, 13]
    outs = model.generate(_waves(), prompt, max_new=12)
    assert all(o[: len(prompt)] == prompt and len(o) <= len(prompt) + 12 for o in outs)
    assert all(spec.eos not in o[len(prompt):-1] for o in outs)
    _check_generation(spec, tensors, model, outs, prompt, tol=0.03)
    # one utterance alone decodes to the same ids as inside the batch
    alone = model.generate(_waves()[1:], prompt, max_new=12)[0]
    assert alone == outs[1]
    with pytest.raises(ValueError):
        model.generate(_waves(), [spec.vocab], max_new=2)


def test_config_contract_and_checkpoint(tmp_path):
    spec = CanarySpec()
    exp = spec.expected_tensors()
    assert exp["model.decoder.layers.7.encoder_attn.k_proj.weight"] == ("F32", (1024, 1024)) and exp["proj_out.bias"] == ("F32", (16384,))
    assert exp["model.encoder.layers.0.self_attn.q_proj.bias"] == ("F32", (1024,)) and exp["model.decoder.layers.0.mlp.fc1.weight"] == ("F32", (4096, 1024))
    assert CanarySpec.from_json(*spec.to_json()) == spec
    tiny = canary_tiny()
    d = tmp_path / "canary"
    d.mkdir()
    for name, obj in zip(("config.json", "processor_config.json", "generation_config.json"), tiny.to_json()):
        (d / name).write_text(json.dumps(obj))
    tensors = random_tensors(tiny.expected_tensors(), 5)
    save_safetensors(d / "model.safetensors", tensors)
    with pytest.raises(ValueError, match="differ"):
        CanaryModel.load(d)                                     # the output projection must be the embedding table
    (d / "model.safetensors").unlink()
    tensors["proj_out.weight"] = tensors["model.decoder.embed_tokens.weight"].clone()
    save_safetensors(d / "model.safetensors", tensors)
    loaded = CanaryModel.load(d)
    assert loaded.spec == tiny
    prompt = [7, 4, 16, 64, 64, 5, 9, 11, 13]
    assert loaded.generate(_waves(), prompt, max_new=6) == CanaryModel(tiny, tensors).generate(_waves(), prompt, max_new=6)
    bad = json.loads((d / "config.json").read_text())
    bad["tie_word_embeddings"] = False
    with pytest.raises(ValueError):
        CanarySpec.from_json(bad, *tiny.to_json()[1:])


@pytest.mark.gpu
def test_generation_on_device(cuda):
    from flyingfish_b200 import ops
    spec = canary_tiny()
    tensors = _tensors(spec, 3)
    model = CanaryModel(spec, tensors, cuda)
    prompt = [7, 4, 16, 64, 64, 5, 9, 11, 13]
    before = ops.launch_count()
    outs = model.generate(_waves(), prompt, max_new=12)
    assert ops.launch_count() > before
    ops.check_status()
    _check_generation(spec, tensors, model, outs, prompt, tol=0.06)


def test_transcribe_command_with_languages(tmp_path, capsys):
    from tokenizers import AddedToken, Tokenizer, decoders, models
    from flyingfish_b200 import cli
    from flyingfish_b200.speech import write_wav
    spec = canary_tiny()
    d = tmp_path / "canary"
    d.mkdir()
    for name, obj in zip(("config.json", "processor_config.json", "generation_config.json"), spec.to_json()):
        (d / name).write_text(json.dumps(obj))
    tensors = random_tensors(spec.expected_tensors(), 5)
    tensors["proj_out.weight"] = tensors["model.decoder.embed_tokens.weight"].clone()
    save_safetensors(d / "model.safetensors", tensors)
    specials = ["<unk>", "<s>", "<pad>", "</s>", "<|startoftranscript|>", "<|pnc|>", "<|nopnc|>", "<|startofcontext|>", "<|noitn|>",
                "<|notimestamp|>", "<|nodiarize|>", "<|emo:undefined|>", "<|en|>", "<|de|>"]
    vocab = {t: i for i, t in enumerate(specials)}
    for i in range(len(specials), spec.vocab):
        vocab[("▁" if i % 2 else "") + f"w{i}"] = i
    tk = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tk.add_special_tokens([AddedToken(t, special=True) for t in specials])
    tk.decoder = decoders.Metaspace()
    tk.save(str(d / "tokenizer.json"))
    g = torch.Generator().manual_seed(2)
    write_wav(tmp_path / "a.wav", 0.2 * torch.randn(12000, generator=g), 16000)
    base = ["--cpu", "--model", str(d), "transcribe", str(tmp_path / "a.wav"), "--format", "json"]
    assert cli.main(base + ["--source-lang", "en", "--target-lang", "de"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert isinstance(out["text"], str) and all("<|" not in s["text"] for s in out["segments"])
    if out["segments"]:
        assert out["segments"][0]["start"] == 0.0 and abs(out["segments"][0]["end"] - 0.75) < 1e-9
    model = CanaryModel.load(d)
    assert model.prompt("en", "de", False) == [7, 4, 11, 12, 13, 6, 8, 9, 10]
    with pytest.raises(ValueError, match="unsupported Canary language"):
        cli.main(base + ["--target-lang", "xx"])
