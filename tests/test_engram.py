"""Engram n-gram hashing and the LFU row service."""
import numpy as np
import pytest

from flyingfish_b200 import engram as eg


def _setup():
    return eg.EngramHashSetup.build([3, 7], tokenizer_vocab=1000, compressed_vocab=300, ngram=3, heads=4, table_rows=1000, seed=1)


def test_hashes_are_deterministic_incremental_and_respect_padding():
    s = _setup()
    assert s.hash_width == 8 and len({p for l in s.primes for z in l for p in z}) == 16
    ids = [5, 17, 999, 17, 42, 8]
    h1 = eg.NgramHistory(s, 64).prepare(ids, 0)
    hist = eg.NgramHistory(s, 64)
    parts = [hist.prepare(ids[:2], 0), hist.prepare(ids[2:], 2)]
    assert [a + b for a, b in zip(*parts)] == h1                     # incremental == whole
    assert len(h1[0]) == len(ids) * s.hash_width and all(0 <= r < s.table_rows(0) for r in h1[0])
    # position 0 has no history: its n-grams are padded; the same first token gives the same rows
    assert eg.NgramHistory(s, 8).prepare([5, 1], 0)[0][:8] == h1[0][:8]
    # a non-text token blocks every n-gram that covers it
    masked = eg.NgramHistory(s, 64).prepare(ids, 0, [True, True, False, True, True, True])
    assert masked[0][:16] == h1[0][:16] and masked[0][16:24] != h1[0][16:24]
    assert masked[0][40:48] == h1[0][40:48]                          # position 5: tokens 5,4,3 do not touch position 2
    with pytest.raises(ValueError):
        eg.NgramHistory(s, 4).prepare(ids, 0)
    with pytest.raises(ValueError):
        eg.NgramHistory(s, 64).prepare([5], 3)                       # gap in the history


def test_row_service_lfu_and_decoding(tmp_path):
    rng = np.random.default_rng(0)
    rows = rng.integers(0, 256, (50, eg.ROW_BYTES), dtype=np.uint8)
    rows[:, eg.HEAD_DIM:] = 125
    path = tmp_path / "table.bin"
    rows.tofile(path)
    svc = eg.RowService(str(path), 50, cache_rows=3)
    got = svc.gather([1, 2, 1, 3, 1, 4, 2])
    assert np.array_equal(got, rows[[1, 2, 1, 3, 1, 4, 2]])
    # 1 (freq 3) and the most recent survive; 2 was evicted for 4 only after 3 (lower recency at equal frequency)
    assert svc.stats["evictions"] == 2 and 1 in svc.cache and svc.stats["hits"] == 2
    dec = eg.decode_rows(rows[:2])
    assert dec.shape == (2, 256) and np.allclose(dec[0, 0], np.int8(rows[0, 0]) * 0.25)
    with pytest.raises(IndexError):
        svc.gather([50])
    svc.close()
