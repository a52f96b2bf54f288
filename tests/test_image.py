"""Image input processing: the reference's golden grid sizes, PNG data URLs, resampling and packing."""
import base64
import struct
import zlib

import numpy as np
import pytest

from flyingfish_b200.serve import image as im


def _png(w, h, rgba_rows, color=6):
    def chunk(t, b):
        return struct.pack(">I", len(b)) + t + b + struct.pack(">I", zlib.crc32(t + b))
    raw = b"".join(b"\x00" + bytes(r) for r in rgba_rows)
    return b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, color, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b"")


def test_smart_resize_golden_grid():
    assert im.smart_resize(1024, 1024, 65536, 16777216) == (1024, 1024)
    assert im.smart_resize(1500, 900, 65536, 16777216) == (1504, 896)
    assert im.smart_resize(64, 64, 65536, 16777216) == (256, 256)
    assert im.smart_resize(80, 80, 1024, 16777216) == (64, 64)
    for bad in ((0, 32), (1, 201)):
        with pytest.raises(ValueError):
            im.smart_resize(*bad, 65536, 16777216)


def test_png_data_url_rgb_without_alpha_compositing_and_refusals():
    data = base64.b64encode(_png(2, 1, [[255, 0, 0, 0, 0, 128, 255, 255]])).decode()
    img = im.load_image(f"data:image/png;base64,{data}")
    assert (img.width, img.height) == (2, 1) and img.pixels.reshape(-1).tolist() == [255, 0, 0, 0, 128, 255]
    for bad in (f"data:image/jpeg;base64,{data}", "https://example.com/image.png", "file:///etc/passwd",
                "data:image/gif;base64,R0lGODlh"):
        with pytest.raises(ValueError):
            im.load_image(bad)


def test_resize_pack_and_token_expansion():
    rng = np.random.default_rng(0)
    img = im.Image(90, 70, rng.integers(0, 256, (70, 90, 3), dtype=np.uint8))
    flat = im.resize_bicubic(np.full((10, 10, 3), 77, dtype=np.uint8), 32, 64)
    assert np.allclose(flat, 77.0)                                   # normalised weights keep constants
    patches, grid = im.pack_patches(img, min_pixels=65536)
    assert grid[1] * grid[2] == patches.shape[0] and patches.shape[1] == 3 * 2 * 16 * 16
    n = im.image_token_count(grid)
    assert n == (grid[1] // 2) * (grid[2] // 2)
    assert im.expand_image_tokens([1, 9, 2, 9], 9, [n, 3]) == [1] + [9] * n + [2] + [9] * 3
    with pytest.raises(ValueError):
        im.expand_image_tokens([1, 9], 9, [])
