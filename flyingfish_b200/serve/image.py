"""Image input processing for vision-language requests: data-URL loading (PNG through the standard library, JPEG
through the decoder of the native host library; no network, no file URLs), MiniCPM-style slicing of large images into a
source view plus a grid of refined tiles, video frame sampling from container metadata, Qwen-style ``smart_resize`` to multiples of 32 inside a pixel budget, separable
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


_JPEG_ERRORS = {-1: "truncated file", -2: "not a JPEG file", -3: "unsupported JPEG variant (progressive, arithmetic, "
                "12-bit or multi-scan)", -4: "bad table", -5: "corrupt entropy-coded data", -6: "image exceeds the pixel limit",
                -7: "output buffer too small"}


def decode_jpeg(data: bytes, max_pixels: int = 4 * MAX_PIXELS_HARD) -> Image:
    """Baseline / extended-sequential JPEG (grayscale, YCbCr with any sampling, Adobe CMYK / YCCK) -> RGB, decoded by
    ``native/jpeg.cpp``. The pixel limit is checked from the frame header before anything is allocated."""
    import ctypes
    from ..ops.lib import host
    lib = host()
    buf = (ctypes.c_uint8 * len(data)).from_buffer_copy(data)
    w, h, c = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    rc = lib.ff_jpeg_info(buf, ctypes.c_size_t(len(data)), ctypes.byref(w), ctypes.byref(h), ctypes.byref(c))
    if rc == 0 and w.value * h.value > max_pixels:
        rc = -6
    if rc != 0:
        raise ValueError(f"JPEG: {_JPEG_ERRORS.get(rc, rc)}")
    out = np.empty((h.value, w.value, 3), dtype=np.uint8)
    rc = lib.ff_jpeg_decode(buf, ctypes.c_size_t(len(data)), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)),
                            ctypes.c_size_t(out.nbytes), ctypes.c_longlong(max_pixels))
    if rc != 0:
        raise ValueError(f"JPEG: {_JPEG_ERRORS.get(rc, rc)}")
    return Image(w.value, h.value, out)


def decode_image(data: bytes, mime: str | None = None) -> Image:
    """PNG or JPEG by signature; a declared media type must agree with the bytes."""
    kind = "png" if data[:8] == b"\x89PNG\r\n\x1a\n" else "jpeg" if data[:2] == b"\xff\xd8" else None
    if kind is None:
        raise ValueError("unsupported image format (PNG and JPEG are accepted)")
    if mime is not None and mime not in (f"image/{kind}", "image/jpg" if kind == "jpeg" else ""):
        raise ValueError(f"media type {mime} does not match the {kind.upper()} data")
    return decode_png(data) if kind == "png" else decode_jpeg(data)


def load_image(url: str) -> Image:
    """Only ``data:image/png;base64,...`` and ``data:image/jpeg;base64,...`` are accepted: no network, no file access."""
    if not url.startswith("data:"):
        raise ValueError("only data URLs are accepted")
    head, _, payload = url.partition(",")
    if head not in ("data:image/png;base64", "data:image/jpeg;base64", "data:image/jpg;base64"):
        raise ValueError("unsupported image media type")
    return decode_image(base64.b64decode(payload, validate=True), head[5:].split(";")[0])


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


# ---- MiniCPM-style slicing ---------------------------------------------------------------------------------------
# A large image is shown to the tower twice: once whole, resized to about scale x scale pixels (the source view), and
# once as rows x cols tiles cut from a refined resize whose tiles each are about scale x scale. The grid is the
# factorisation of the slice count (area / scale^2, capped) whose aspect ratio is closest to the image's in log space.
# All sizes are multiples of 4 patches. Mirrors the slicing rules of src/serve/image.rs:859-1104 of the reference
# (which follow the published MiniCPM-V image processor); its tests give the grids checked in tests/test_image.py.
SCALE_RESOLUTION = 448


def _ensure_divide(length: float, divisor: int) -> int:
    return max(int(np.rint(length / divisor)) * divisor, divisor)


def _best_resize(height: float, width: float, scale: int, patch: int, allow_upscale: bool) -> tuple[int, int]:
    if height * width > scale * scale or allow_upscale:
        aspect = width / height
        height = float(int(scale / math.sqrt(aspect)))
        width = float(int(height * aspect))
    return _ensure_divide(height, patch * 4), _ensure_divide(width, patch * 4)


def slice_grid(height: int, width: int, max_slices: int, scale: int = SCALE_RESOLUTION) -> tuple[int, int] | None:
    """(rows, cols) of the tile grid, or None when the image is shown whole only."""
    log_ratio = math.log(width / height)
    multiple = min(math.ceil(width * height / (scale * scale)), max_slices)
    if multiple <= 1:
        return None
    best, err_best = (1, 1), math.inf
    for n in (multiple - 1, multiple, multiple + 1):
        if n <= 1 or n > max_slices:
            continue
        for rows in range(1, n + 1):
            if n % rows:
                continue
            cols = n // rows
            err = abs(log_ratio - math.log(cols / rows))
            if err < err_best or (err == err_best and rows > best[0]):
                best, err_best = (rows, cols), err
    return best


@dataclass
class SlicePlan:
    source: tuple[int, int]                 # (height, width) of the whole-image view
    rows: int                               # tile grid (0 x 0: no tiles)
    cols: int
    refine: tuple[int, int]                 # (height, width) of the resize the tiles are cut from
    tile: tuple[int, int]                   # (height, width) of one tile

    def grids(self, patch: int) -> list[tuple[int, int, int]]:
        g = [(1, self.source[0] // patch, self.source[1] // patch)]
        return g + [(1, self.tile[0] // patch, self.tile[1] // patch)] * (self.rows * self.cols)


def slice_plan(height: int, width: int, patch: int = 14, max_slices: int = 9, scale: int = SCALE_RESOLUTION) -> SlicePlan:
    if height <= 0 or width <= 0:
        raise ValueError("empty image")
    grid = slice_grid(height, width, max_slices, scale)
    source = _best_resize(float(height), float(width), scale, patch, grid is None)
    if grid is None:
        return SlicePlan(source, 0, 0, (0, 0), (0, 0))
    rows, cols = grid
    rh, rw = _ensure_divide(float(height), rows), _ensure_divide(float(width), cols)
    bh, bw = _best_resize(rh / rows, rw / cols, scale, patch, True)
    refine = (bh * rows, bw * cols)
    if bh % patch or bw % patch:
        raise ValueError("slice resize is not patch aligned")
    return SlicePlan(source, rows, cols, refine, (bh, bw))


def slice_image(img: Image, patch: int = 14, max_slices: int = 9, scale: int = SCALE_RESOLUTION
                ) -> tuple[SlicePlan, list[np.ndarray]]:
    """-> (plan, views): views[0] is the whole image at ``plan.source``; then the tiles in row-major order (float64
    [h, w, 3] in 0..255, bicubic)."""
    plan = slice_plan(img.height, img.width, patch, max_slices, scale)
    views = [np.clip(resize_bicubic(img.pixels, *plan.source), 0, 255)]
    if plan.rows:
        fine = np.clip(resize_bicubic(img.pixels, *plan.refine), 0, 255)
        th, tw = plan.tile
        for r in range(plan.rows):
            for c in range(plan.cols):
                views.append(fine[r * th: (r + 1) * th, c * tw: (c + 1) * tw])
    return plan, views


def pack_slices(img: Image, patch: int = 14, max_slices: int = 9, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5),
                scale: int = SCALE_RESOLUTION) -> tuple[list[np.ndarray], SlicePlan]:
    """Every view as patches [grid_h * grid_w, 3 * patch * patch] float32, row-major patch order, normalised."""
    plan, views = slice_image(img, patch, max_slices, scale)
    out = []
    for v in views:
        x = ((v / 255.0 - np.asarray(mean)) / np.asarray(std)).astype(np.float32).transpose(2, 0, 1)
        gh, gw = x.shape[1] // patch, x.shape[2] // patch
        x = x.reshape(3, gh, patch, gw, patch).transpose(1, 3, 0, 2, 4)
        out.append(np.ascontiguousarray(x.reshape(gh * gw, 3 * patch * patch)))
    return out, plan


def slice_token_count(plan: SlicePlan, query_tokens: int = 64) -> int:
    """Tokens the sliced image expands to: every view is resampled to ``query_tokens`` by the tower's resampler and
    wrapped in a start and an end marker; the tile rows are separated by a newline token."""
    views = 1 + plan.rows * plan.cols
    return views * (query_tokens + 2) + max(plan.rows - 1, 0)


# ---- video frames -----------------------------------------------------------------------------------------------
@dataclass
class VideoMeta:
    total_frames: int
    fps: float
    duration: float                         # seconds


def sample_frame_indices(meta: VideoMeta, max_frames: int) -> list[int]:
    """Frame indices shown to the model: one per second while the clip is at most ``max_frames`` seconds long, else
    ``max_frames`` frames spread evenly over a 0.1-second grid (first and last grid points included). The container is
    decoded outside this process (frames arrive as images); this is the selection rule
    (src/serve/image.rs:65-125 of the reference)."""
    if max_frames <= 0 or meta.total_frames <= 0 or not (meta.fps > 0) or not (meta.duration > 0):
        raise ValueError("invalid video metadata")
    if meta.duration > max_frames:
        count = int(meta.duration / 0.1)
        out = min(count, max_frames)
        delta = (count - 1) / (out - 1) if out > 1 else 0.0
        idx = []
        for k in range(out):
            pos = 0 if out == 1 else k if out == count else count - 1 if k + 1 == out else int(delta * k)
            idx.append(min(int(pos / 10.0 * meta.fps), meta.total_frames - 1))
        return idx
    idx = []
    for i in range(math.ceil(meta.duration)):
        j = int(i * meta.fps)
        if j >= meta.total_frames:
            raise ValueError(f"video metadata: sampled frame {j} outside {meta.total_frames} frames")
        idx.append(j)
    if not idx:
        raise ValueError("video sampling produced no frames")
    return idx


def pack_video_frames(frames: list[Image], min_pixels: int = 65536, max_pixels: int = MAX_PIXELS_HARD // 8, patch: int = 16,
                      merge: int = 2, temporal: int = 2) -> tuple[np.ndarray, tuple[int, int, int]]:
    """Qwen-style video packing: frames (all the same size) are grouped in temporal pairs (the last one repeated when
    the count is odd), every pair packed like an image -> (patches, (t, grid_h, grid_w))."""
    if not frames:
        raise ValueError("video has no frames")
    if any((f.height, f.width) != (frames[0].height, frames[0].width) for f in frames):
        raise ValueError("video frames differ in size")
    if len(frames) % temporal:
        frames = frames + [frames[-1]] * (temporal - len(frames) % temporal)
    oh, ow = smart_resize(frames[0].height, frames[0].width, min_pixels, max_pixels)
    gh, gw = oh // patch, ow // patch
    xs = [((np.clip(resize_bicubic(f.pixels, oh, ow), 0, 255) / 255.0 - MEAN) / STD).astype(np.float32).transpose(2, 0, 1)
          for f in frames]
    out = []
    for t0 in range(0, len(xs), temporal):
        x = np.stack(xs[t0: t0 + temporal])                                      # [temporal, 3, H, W]
        x = x.reshape(temporal, 3, gh // merge, merge, patch, gw // merge, merge, patch).transpose(2, 5, 3, 6, 1, 0, 4, 7)
        out.append(x.reshape(gh * gw, 3 * temporal * patch * patch))
    return np.ascontiguousarray(np.concatenate(out, 0)), (len(xs) // temporal, gh, gw)
