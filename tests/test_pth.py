"""``.pth`` / ``.nemo`` readers: zero-copy tensors, refusal of code-carrying pickles."""
import io
import pickle
import tarfile
import warnings

import pytest
import torch

from flyingfish_b200.loaders import pth


def _state():
    g = torch.Generator().manual_seed(0)
    big = torch.randn(6, 8, generator=g)
    return {"a.weight": big.to(torch.bfloat16), "b": {"bias": torch.arange(5, dtype=torch.int64), "view": big[1:4, ::2]},
            "flag": torch.tensor([True, False])}


def test_pth_roundtrip_without_unpickling(tmp_path):
    p = tmp_path / "m.pth"
    torch.save(_state(), p)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        f = pth.read_pth(p)
        t = f.tensors()
    s = _state()
    assert set(t) == {"a.weight", "b.bias", "b.view", "flag"}
    assert torch.equal(t["a.weight"], s["a.weight"]) and torch.equal(t["b.bias"], s["b"]["bias"])
    assert torch.equal(t["b.view"], s["b"]["view"]) and torch.equal(t["flag"], s["flag"])
    f.close()


def test_pth_refuses_code(tmp_path):
    import zipfile

    class Evil:
        def __reduce__(self):
            return (print, ("pwned",))
    p = tmp_path / "evil.pth"
    with zipfile.ZipFile(p, "w", zipfile.ZIP_STORED) as z:
        z.writestr("archive/data.pkl", pickle.dumps({"x": Evil()}, protocol=2))
    with pytest.raises(pth.UnsafePickle):
        pth.read_pth(p)


def test_nemo_archive(tmp_path):
    ck = tmp_path / "model_weights.ckpt"
    torch.save({"enc.w": torch.ones(3, 4)}, ck)
    cfg = tmp_path / "model_config.yaml"
    cfg.write_text("target: test\nhidden: 4\n")
    arc = tmp_path / "m.nemo"
    with tarfile.open(arc, "w:") as tar:
        tar.add(cfg, arcname="./model_config.yaml"); tar.add(ck, arcname="./model_weights.ckpt")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        text, f = pth.read_nemo(arc)
        assert "hidden: 4" in text and torch.equal(f.tensor("enc.w"), torch.ones(3, 4))
    f.close()
    bad = tmp_path / "bad.nemo"
    with tarfile.open(bad, "w:") as tar:
        tar.add(cfg, arcname="model_config.yaml")
    with pytest.raises(ValueError):
        pth.read_nemo(bad)
