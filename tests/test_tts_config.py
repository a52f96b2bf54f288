"""Text-to-speech request contract: prompt prefix and sampling settings."""
import pytest

from flyingfish_b200.speech import tts_config as tc

PUBLISHED = {"bos_token_id": 2, "depth_decoder_do_sample": True, "depth_decoder_temperature": 0.9, "do_sample": True, "eos_token_id": [1],
             "max_new_tokens": 750, "pad_token_id": 0, "temperature": 0.9, "transformers_version": "4.57.3"}


def test_prompt_and_published_settings():
    assert tc.plain_prompt("Hello") == "[S0]Hello" and tc.plain_prompt("[笑] 欢迎") == "[S0][笑] 欢迎"
    cfg = tc.speak_config(PUBLISHED)
    assert (cfg.temperature, cfg.top_k, cfg.top_p, cfg.repetition_penalty, cfg.max_new_tokens) == (0.9, 50, 1.0, 1.1, 750)
    assert cfg.max_seconds == pytest.approx(60.0)
    assert tc.speak_config(dict(PUBLISHED, top_k=20, top_p=0.8, repetition_penalty=1.0)).top_k == 20
    for bad in (dict(PUBLISHED, depth_decoder_temperature=0.8), dict(PUBLISHED, max_new_tokens=751), dict(PUBLISHED, do_sample=False),
                dict(PUBLISHED, eos_token_id=1), dict(PUBLISHED, extra=1), dict(PUBLISHED, top_p=0.0),
                {k: v for k, v in PUBLISHED.items() if k != "temperature"}):
        with pytest.raises(ValueError):
            tc.speak_config(bad)
