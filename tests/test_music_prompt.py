"""Prompt assembly of the text-to-music family against published examples."""
import pytest

from flyingfish_b200.utils import music_prompt as mp

CASES = [
    ("A warm acoustic pop song with intimate female vocals.", "[verse]\nMorning light",
     "<|im_start|><|caption_start|>A warm acoustic pop song with intimate female vocals.<|caption_end|><|lyrics_start|>[start]\n[verse]\n"
     "Morning light<|lyrics_end|><|im_end|><|audio_start|>"),
    ("## Global Metadata\n<|bpm 92|>\n- **Genre**: Electric Blues\n• Hammond organ\n    indented line",
     "[Verse] these words are dropped\n[Chorus] Softly the world begins\n[Bridge]\nReturn ^ again",
     "<|im_start|><|caption_start|>Global Metadata\nbpm is 92\nGenre: Electric Blues\nHammond organ\nindented line<|caption_end|>"
     "<|lyrics_start|>[start]\n[verse]\n[chorus]\n[bridge]\nReturn\nagain<|lyrics_end|><|im_end|><|audio_start|>"),
    ("**Ambient** soundscape\n\n\nSecond paragraph", "[Chorus]\nSoftly the world begins to breathe\n[Instrumental]\n(open strings)",
     "<|im_start|><|caption_start|>Ambient soundscape\nSecond paragraph<|caption_end|><|lyrics_start|>[start]\n[chorus]\n"
     "Softly the world begins to breathe\n[instrumental]\n(open strings)<|lyrics_end|><|im_end|><|audio_start|>"),
]


def test_published_examples():
    for prompt, lyrics, want in CASES:
        assert mp.assemble_prompt(prompt, lyrics) == want


def test_caption_and_lyric_rules():
    assert mp.clean_caption("*soft* and **loud**, 2 * 3 stays") == "soft and loud, 2 * 3 stays"
    assert mp.clean_caption("title\n-----\n* item\n+ other") == "title\nitem\nother"
    assert mp.clean_caption("<|key D minor|> and <|solo|>") == "key is D minor and solo"
    assert mp.clean_caption("#hashtag stays\n####### seven stays") == "#hashtag stays\n####### seven stays"
    assert mp.normalize_lyrics("Line one [Outro] fade") == "[start]\nLine one\n[outro]\nfade"
    assert mp.normalize_lyrics("[A][B]  words") == "[start]\n[a][b]"
    assert mp.normalize_lyrics("open [bracket") == "[start]\nopen\n[bracket"
    with pytest.raises(ValueError):
        mp.assemble_prompt(" ", "[verse]\nx")
    with pytest.raises(ValueError):
        mp.assemble_prompt("x", "\n")


def test_paired_ids_and_stereo():
    encode = lambda text: [7] + [ord(c) % 50 + 10 for c in text[:20]] + [98, 99]
    ids = mp.paired_prompt_ids(*CASES[0][:2], encode)
    half = len(ids) // 2
    assert len(ids) == 2 * half and ids[0] == ids[half] == 7 and ids[half - 2: half] == ids[-2:] == [98, 99]
    assert all(t == mp.UNCONDITIONAL_FILL for t in ids[half + 1: -2]) and ids[1:half - 2] != ids[half + 1:-2]
    with pytest.raises(ValueError):
        mp.paired_prompt_ids(*CASES[0][:2], lambda t: [1, 2])
    with pytest.raises(ValueError):
        mp.paired_prompt_ids(*CASES[0][:2], lambda t: [1] * 5001)
    assert mp.interleave_stereo([1.0, 2.0, 3.0, 4.0, 5.0, 6.0]) == [1.0, 4.0, 2.0, 5.0, 3.0, 6.0]
    with pytest.raises(ValueError):
        mp.interleave_stereo([1.0])
