"""Dense-layer streaming: placement arithmetic on CPU, streamed == resident on the device."""
import pytest
import torch

from flyingfish_b200.planner import streaming as st


def test_placement_arithmetic():
    layers = [100] * 10
    p = st.plan_layer_streaming(layers, device_budget=2000, host_budget=0, h2d_gbs=50, disk_gbs=5, compute_ms_per_layer=0.1)
    assert p.streamed == () and p.slots == 0 and p.bound == "compute"
    p = st.plan_layer_streaming(layers, device_budget=650, host_budget=250, h2d_gbs=1e-6, disk_gbs=1e-7, compute_ms_per_layer=0.1)
    assert p.resident == (0, 1, 2, 3) and p.streamed == tuple(range(4, 10)) and p.slots == 2
    assert p.host_layers == (4, 5) and p.disk_layers == (6, 7, 8, 9) and p.device_bytes == 600
    assert p.bound == "disk" and abs(p.decode_ms - 400 / (1e-7 * 1e6)) < 1e-6
    with pytest.raises(ValueError):
        st.plan_layer_streaming(layers, device_budget=150, host_budget=0, h2d_gbs=1, disk_gbs=1, compute_ms_per_layer=1)


@pytest.mark.gpu
def test_streamed_layers_match_resident_model():
    import dataclasses

    from flyingfish_b200.config import Settings, named_shape
    from flyingfish_b200.engine.engine import Engine
    from flyingfish_b200.models.decoder import DecoderModel
    from flyingfish_b200.models.weights import random_decoder_weights
    dev = torch.device("cuda")
    spec = dataclasses.replace(named_shape("tiny-llama"), layers=6)
    settings = Settings(capacity=256, max_batch=2, graph=False)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (40, 17)]

    def run(stream: bool):
        w = random_decoder_weights(spec, 0, dev)
        sl = None
        if stream:
            sizes = [sum(t.numel() * t.element_size() for t in vars(l).values() if isinstance(t, torch.Tensor)) for l in w.layers]
            place = st.plan_layer_streaming(sizes, device_budget=3 * max(sizes) + 1, host_budget=1 << 40, h2d_gbs=50, disk_gbs=5,
                                            compute_ms_per_layer=0.05)
            assert place.resident == (0,) and place.slots == 2 and len(place.streamed) == 5
            sl = st.StreamedLayers(w.layers, place, dev)
            w.layers = sl
        eng = Engine(DecoderModel(w), spec, settings, 64, dev, max_prefill_rows=256)
        out = eng.generate(prompts, 6, None, True, None)
        torch.cuda.synchronize()
        return out, sl

    want, _ = run(False)
    got, sl = run(True)
    assert got == want
    assert sl.stats["copies"] > 5 * 3           # five streamed layers are re-copied on every step through two slots
