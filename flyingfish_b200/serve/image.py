"""Image input processing for vision-language requests: data-URL loading (PNG through the standard library,
no network, no file URLs), Qwen-style ``smart_resize`` to multiples of 32 inside a pixel budget, separable
bicubic resampling, normalisation, patch packing (temporal x 2, merge 2 x 2) and the expansion of an image
placeholder into its token span. Mirrors src/serve/image.rs:386-815, :1404-1436 of the reference (same rounding
rule, aspect and budget guards; its tests give the golden grid sizes used in tests/test_image.py)."""
from __future__ import annotations

import base64
import math
import struct
import zlib
from dataclasses import dataclass

import numpy as np

MAX_PIXELS_HARD = 16_777_216
FACTOR = 32                      # patch 16 x spatial merge 2


@dataclass
class Image:
    width: int
    height: int
    pixels: np.ndarray           # uint8 [H, W, 3]


def _round_ties_even(x: float) -> int:
    return int(np.rint(x))


def smart_resize(height: int, width: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    if height <= 0 or width <= 0 or height * width > (1 << 40):
        raise ValueError("invalid image dimensions")
    if max(height, width) / min(height, width) > 200.0:
        raise ValueError("image aspect ratio exceeds 200")
    if not (0 < min_pixels <= max_pixels <= MAX_PIXELS_HARD):
        raise ValueError("invalid image pixel budget")
    h, w = float(height), float(width)
    out_h = _round_ties_even(h / FACTOR) * FACTOR
    out_w = _round_ties_even(w / FACTOR) * FACTOR
    if out_h * out_w > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        out_h = max(int(math.floor(h / beta / FACTOR)) * FACTOR, FACTOR)
        out_w = max(int(math.floor(w / beta / FACTOR)) * FACTOR, FACTOR)
    elif out_h * out_w < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        out_h = int(math.ceil(h * beta / FACTOR)) * FACTOR
        out_w = int(math.ceil(w * beta / FACTOR)) * FACTOR
    if not (out_h > 0 and out_w > 0 and out_h * out_w <= max_pixels):
        raise ValueError("resized image exceeds pixel budget")
    return out_h, out_w


# ---- PNG (8-bit gray / RGB / RGBA / palette, non-interlaced) ----------------------------------------------
def _paeth(a: int, b: int, c: int) -> int:
    p = a + b - c
    pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
    return a if pa <= pb and pa <= pc else (b if pb <= pc else c)


def decode_png(data: bytes) -> Image:
    if data[:8] != b"\x89PNG\r\n\x1a\n":
        raise ValueError("not a PNG")
    pos, idat, palette, hdr = 8, bytearray(), None, None
    while pos + 8 <= len(data):
        (length,), ctype = struct.unpack(">I", data[pos: pos + 4]), data[pos + 4: pos + 8]
        body = data[pos + 8: pos + 8 + length]
        if len(body) != length:
            raise ValueError("truncated PNG chunk")
        if zlib.crc32(ctype + body) != struct.unpack(">I", data[pos + 8 + length: pos + 12 + length])[0]:
            raise ValueError("PNG chunk checksum")
        if ctype == b"IHDR":
            hdr = struct.unpack(">IIBBBBB", body)
        elif ctype == b"PLTE":
            palette = np.frombuffer(body, dtype=np.uint8).reshape(-1, 3)
        elif ctype == b"IDAT":
            idat += body
        elif ctype == b"IEND":
            break
        pos += 12 + length
    if hdr is None:
        raise ValueError("PNG without header")
    w, h, depth, ctype_, _, _, interlace = hdr
    if depth != 8 or interlace != 0 or w == 0 or h == 0 or w * h > MAX_PIXELS_HARD:
        raise ValueError("unsupported PNG (8-bit, non-interlaced only)")
    ch = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}.get(ctype_)
    if ch is None:
        raise ValueError("unsupported PNG colour type")
    raw = zlib.decompress(bytes(idat))
    stride = w * ch
    if len(raw) != h * (stride + 1):
        raise ValueError("PNG payload size")
    out = np.zeros((h, stride), dtype=np.uint8)
    prev = np.zeros(stride, dtype=np.int32)
    for y in range(h):
        f = raw[y * (stride + 1)]
        line = np.frombuffer(raw, dtype=np.uint8, count=stride, offset=y * (stride + 1) + 1).astype(np.int32)
        cur = np.zeros(stride, dtype=np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 255
        else:
            for x in range(stride):
                a = cur[x - ch] if x >= ch else 0
                b = prev[x]
                c = prev[x - ch] if x >= ch else 0
                pred = a if f == 1 else ((a + b) >> 1 if f == 3 else (_paeth(int(a), int(b), int(c)) if f == 4 else None))
                if pred is None:
                    raise ValueError("PNG filter")
                cur[x] = (line[x] + pred) & 255
        out[y] = cur
        prev = cur
    px = out.reshape(h, w, ch)
    if ctype_ == 0:
        rgb = np.repeat(px, 3, axis=2)
    elif ctype_ == 3:
        if palette is None:
            raise ValueError("palette PNG without PLTE")
        rgb = palette[px[:, :, 0]]
    elif ctype_ == 4:
        rgb = np.repeat(px[:, :, :1], 3, axis=2)
    else:
        rgb = px[:, :, :3]                               # alpha is dropped, not composited
    return Image(w, h, np.ascontiguousarray(rgb, dtype=np.uint8))


def load_image(url: str) -> Image:
    """Only ``data:image/png;base64,...`` is accepted: no network, no file access."""
    if not url.startswith("data:"):
        raise ValueError("only data URLs are accepted")
    head, _, payload = url.partition(",")
    if head != "data:image/png;base64":
        raise ValueError("unsupported image media type")
    return decode_png(base64.b64decode(payload, validate=True))


# ---- resampling and packing --------------------------------------------------------------------------------
def _cubic(x: np.ndarray) -> np.ndarray:
    x = np.abs(x)
    return np.where(x < 1, ((1.5 * x - 2.5) * x) * x + 1, np.where(x < 2, ((-0.5 * x + 2.5) * x - 4) * x + 2, 0.0))


def _resize_axis(a: np.ndarray, out: int, axis: int) -> np.ndarray:
    n = a.shape[axis]
    scale = n / out
    support = 2.0 * max(scale, 1.0)                      # antialias when shrinking
    centers = (np.arange(out) + 0.5) * scale
    lo = np.floor(centers - support).astype(int)
    taps = int(math.ceil(2 * support)) + 2
    idx = lo[:, None] + np.arange(taps)[None, :]
    wts = _cubic((idx + 0.5 - centers[:, None]) / max(scale, 1.0))
    wts = np.where((idx >= 0) & (idx < n), wts, 0.0)
    wts /= wts.sum(1, keepdims=True)
    a = np.moveaxis(a, axis, 0)
    res = np.einsum("ot,ot...->o...", wts, a[np.clip(idx, 0, n - 1)])
    return np.moveaxis(res, 0, axis)


def resize_bicubic(pixels: np.ndarray, out_h: int, out_w: int) -> np.ndarray:
    x = pixels.astype(np.float64)
    return _resize_axis(_resize_axis(x, out_h, 0), out_w, 1)


MEAN = np.array([0.48145466, 0.4578275, 0.40821073])
STD = np.array([0.26862954, 0.26130258, 0.27577711])


def pack_patches(img: Image, min_pixels: int = 65536, max_pixels: int = MAX_PIXELS_HARD, patch: int = 16, merge: int = 2,
                 temporal: int = 2) -> tuple[np.ndarray, tuple[int, int, int]]:
    """-> (patches [grid_h * grid_w, 3 * temporal * patch * patch] float32 in merge-block order, (t, grid_h, grid_w))."""
    oh, ow = smart_resize(img.height, img.width, min_pixels, max_pixels)
    x = np.clip(resize_bicubic(img.pixels, oh, ow), 0, 255) / 255.0
    x = ((x - MEAN) / STD).astype(np.float32).transpose(2, 0, 1)                   # [3, H, W]
    gh, gw = oh // patch, ow // patch
    x = np.repeat(x[None], temporal, axis=0)                                        # a still image fills the temporal pair
    x = x.reshape(temporal, 3, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.transpose(2, 5, 3, 6, 1, 0, 4, 7)                                         # blocks, inner 2x2, channel, t, py, px
    return np.ascontiguousarray(x.reshape(gh * gw, 3 * temporal * patch * patch)), (1, gh, gw)


def image_token_count(grid: tuple[int, int, int], merge: int = 2) -> int:
    t, gh, gw = grid
    return t * (gh // merge) * (gw // merge)


def expand_image_tokens(ids: list[int], image_token: int, counts: list[int]) -> list[int]:
    """Every occurrence of ``image_token`` becomes ``counts[i]`` copies (the span the vision tower fills)."""
    out, i = [], 0
    for t in ids:
        if t == image_token:
            if i >= len(counts):
                raise ValueError("more image placeholders than images")
            out.extend([image_token] * counts[i])
            i += 1
        else:
            out.append(t)
    if i != len(counts):
        raise ValueError("more images than placeholders")
    return out
