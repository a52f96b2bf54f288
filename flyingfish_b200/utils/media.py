"""Output containers of the media and 3-D model families: PNG images, YUV4MPEG2 video (and MP4 through an external
muxer), triangle meshes as binary PLY or OBJ, and a reader for both mesh forms.

The reference writes these on the host one pixel or vertex at a time (src/media.rs:292-324 PNG, :376-466 Y4M, :476-592
MP4 through ``ffmpeg``, :784-1040 meshes). Here pixel and vertex arrays are tensors: colour conversion and chroma
pooling are whole-frame integer tensor operations (they run where the tensor lives, so a frame batch produced on the GPU
is converted there and crosses to the host as 1.5 bytes per pixel), and vertex records are assembled as one structured
byte block."""
from __future__ import annotations

import io
import os
import shutil
import struct
import subprocess
import tempfile
import zlib
from dataclasses import dataclass
from pathlib import Path
from typing import BinaryIO

import numpy as np
import torch

MUX_TIMEOUT_S = 600


def _open(target) -> tuple[BinaryIO, bool]:
    if hasattr(target, "write"):
        return target, False
    return open(target, "wb"), True


# ------------------------------------------------------------------------------------------------
# PNG
# ------------------------------------------------------------------------------------------------
def write_png(target, width: int, height: int, pixels, channels: int = 3, level: int = 6) -> None:
    """8-bit RGB (``channels`` 3) or RGBA (4) PNG; ``pixels`` is ``height x width x channels`` bytes (a uint8 tensor or a
    bytes-like object). RGBA keeps the alpha channel (image-to-3D inputs carry the removed background there)."""
    if channels not in (3, 4):
        raise ValueError("PNG colour type: 3 (RGB) or 4 (RGBA) channels")
    if not (0 < width < 2 ** 31 and 0 < height < 2 ** 31):
        raise ValueError("PNG dimensions")
    t = pixels if isinstance(pixels, torch.Tensor) else torch.frombuffer(bytearray(pixels), dtype=torch.uint8)
    if t.dtype != torch.uint8 or t.numel() != width * height * channels:
        raise ValueError("PNG pixel extent")
    rows = t.detach().cpu().reshape(height, width * channels)
    raw = torch.cat([torch.zeros(height, 1, dtype=torch.uint8), rows], dim=1).contiguous().numpy().tobytes()     # filter 0 per row

    def chunk(tag: bytes, body: bytes) -> bytes:
        return struct.pack(">I", len(body)) + tag + body + struct.pack(">I", zlib.crc32(tag + body) & 0xFFFFFFFF)
    out = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", width, height, 8, 2 if channels == 3 else 6, 0, 0, 0)) \
        + chunk(b"IDAT", zlib.compress(raw, level)) + chunk(b"IEND", b"")
    f, close = _open(target)
    try:
        f.write(out)
    finally:
        if close:
            f.close()


# ------------------------------------------------------------------------------------------------
# YUV4MPEG2 / MP4
# ------------------------------------------------------------------------------------------------
def _yuv_plane(rgb_sum: torch.Tensor, shift: int, row: tuple[int, int, int], offset: int) -> torch.Tensor:
    v = row[0] * rgb_sum[..., 0] + row[1] * rgb_sum[..., 1] + row[2] * rgb_sum[..., 2]
    return (((v + (1 << (shift - 1))) >> shift) + offset).clamp_(0, 255).to(torch.uint8)


def rgb_to_yuv420(video: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """RGB frames ``[frames, height, width, 3]`` uint8 -> full-range BT.601 planes (Y ``[f, h, w]``, U and V
    ``[f, h/2, w/2]``), in 16-bit fixed point: luma per pixel, chroma from the sum of each 2x2 block (two more bits of
    shift instead of a rounded average first). Runs on the tensor's device."""
    if video.dtype != torch.uint8 or video.dim() != 4 or video.shape[-1] != 3:
        raise ValueError("video must be [frames, height, width, 3] uint8")
    f, h, w, _ = video.shape
    if f == 0 or h == 0 or w == 0 or h % 2 or w % 2:
        raise ValueError("Y4M dimensions must be positive and even")
    x = video.to(torch.int64)
    y = _yuv_plane(x, 16, (19595, 38470, 7471), 0)
    blocks = x.reshape(f, h // 2, 2, w // 2, 2, 3).sum(dim=(2, 4))
    u = _yuv_plane(blocks, 18, (-11058, -21710, 32768), 128)
    v = _yuv_plane(blocks, 18, (32768, -27439, -5329), 128)
    return y, u, v


def write_y4m(target, video: torch.Tensor, fps: tuple[int, int]) -> None:
    """RGB frames -> a YUV4MPEG2 stream (4:2:0, JPEG chroma siting, full range)."""
    if not (fps[0] > 0 and fps[1] > 0):
        raise ValueError("invalid Y4M frame rate")
    y, u, v = rgb_to_yuv420(video)
    f, h, w = y.shape
    y, u, v = (p.cpu().contiguous().numpy() for p in (y, u, v))
    out, close = _open(target)
    try:
        out.write(f"YUV4MPEG2 W{w} H{h} F{fps[0]}:{fps[1]} Ip A1:1 C420jpeg XCOLORRANGE=FULL\n".encode())
        for i in range(f):
            out.write(b"FRAME\n")
            out.write(y[i].tobytes())
            out.write(u[i].tobytes())
            out.write(v[i].tobytes())
    finally:
        if close:
            out.close()


def write_wav_bytes(rate: int, channels: int, samples: torch.Tensor) -> bytes:
    """Interleaved float samples in [-1, 1] -> 16-bit PCM RIFF/WAVE bytes."""
    if rate <= 0 or channels <= 0 or samples.numel() % channels:
        raise ValueError("WAV extent")
    pcm = (samples.detach().float().cpu().clamp(-1.0, 1.0) * 32767.0).round().to(torch.int16).contiguous().numpy().tobytes()
    return b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVE" + b"fmt " + struct.pack(
        "<IHHIIHH", 16, 1, channels, rate, rate * channels * 2, channels * 2, 16) + b"data" + struct.pack("<I", len(pcm)) + pcm


def mux_mp4(output: str | Path, video: torch.Tensor, fps: tuple[int, int], audio: tuple[int, int, torch.Tensor] | None = None,
            tool: str = "ffmpeg") -> None:
    """Lossless H.264 MP4 of RGB frames (and optional ``(rate, channels, samples)`` audio as AAC) through an external
    muxer that reads the Y4M stream on its standard input. The output must not exist; a failed run leaves no file."""
    out = Path(output)
    if out.suffix != ".mp4":
        raise ValueError("MP4 output must end in .mp4")
    if out.exists():
        raise FileExistsError(f"output already exists: {out}")
    parent = out.parent if str(out.parent) else Path(".")
    if not parent.is_dir():
        raise FileNotFoundError("MP4 parent directory is missing")
    exe = tool if os.path.sep in tool else shutil.which(tool)
    if not exe:
        raise RuntimeError(f"{tool} is not installed: write the frames with write_y4m and mux them elsewhere")
    stream = io.BytesIO()
    write_y4m(stream, video, fps)
    scratch = None
    args = [exe, "-v", "warning", "-y", "-f", "yuv4mpegpipe", "-color_range", "jpeg", "-colorspace", "bt470bg", "-i", "pipe:0"]
    try:
        if audio is not None:
            fd, scratch = tempfile.mkstemp(suffix=".wav", dir=parent)
            with os.fdopen(fd, "wb") as f:
                f.write(write_wav_bytes(*audio))
            args += ["-i", scratch]
        args += ["-map", "0:v:0"]
        if audio is not None:
            args += ["-map", "1:a:0", "-c:a", "aac"]
        args += ["-c:v", "libx264", "-crf", "0", "-vf", "scale=in_range=full:out_range=full:in_color_matrix=bt601:out_color_matrix=bt601",
                 "-pix_fmt", "yuvj420p", "-color_range", "jpeg", "-colorspace", "bt470bg", "-color_primaries", "bt470bg",
                 "-color_trc", "bt709", str(out)]
        done = subprocess.run(args, input=stream.getvalue(), capture_output=True, timeout=MUX_TIMEOUT_S)
        if done.returncode != 0 or not out.is_file():
            raise RuntimeError(f"MP4 mux failed ({done.returncode}): {done.stderr.decode(errors='replace')[-400:]}")
    except BaseException:
        if out.exists():
            out.unlink()
        raise
    finally:
        if scratch is not None and os.path.exists(scratch):
            os.unlink(scratch)


# ------------------------------------------------------------------------------------------------
# triangle meshes
# ------------------------------------------------------------------------------------------------
@dataclass
class Mesh:
    positions: torch.Tensor                                  # [rows, 3] float32
    triangles: torch.Tensor                                  # [faces, 3] int32
    rgb: torch.Tensor | None = None                          # [rows, 3] uint8
    extras: tuple[tuple[str, torch.Tensor], ...] = ()        # named float channels [rows]

    def check(self) -> int:
        p = self.positions
        if p.dim() != 2 or p.shape[1] != 3 or p.shape[0] == 0:
            raise ValueError("mesh positions extent")
        if self.triangles.numel() and (self.triangles.dim() != 2 or self.triangles.shape[1] != 3):
            raise ValueError("mesh triangle extent")
        rows = p.shape[0]
        if self.rgb is not None and (tuple(self.rgb.shape) != (rows, 3) or self.rgb.dtype != torch.uint8):
            raise ValueError("mesh RGB extent")
        for name, values in self.extras:
            if values.numel() != rows:
                raise ValueError(f"mesh extra channel {name} extent")
            if not name or any(c.isspace() for c in name):
                raise ValueError("mesh extra channel names are single words")
        return rows


def write_ply(target, mesh: Mesh) -> None:
    """Binary little-endian PLY: float x y z, optional uchar red green blue, the named float extras, and triangles as
    uchar-count / int-index lists. Colours are stored as given (no transfer function is applied)."""
    rows = mesh.check()
    faces = mesh.triangles.shape[0] if mesh.triangles.numel() else 0
    header = f"ply\nformat binary_little_endian 1.0\nelement vertex {rows}\nproperty float x\nproperty float y\nproperty float z\n"
    fields = [("x", "<f4"), ("y", "<f4"), ("z", "<f4")]
    if mesh.rgb is not None:
        header += "property uchar red\nproperty uchar green\nproperty uchar blue\n"
        fields += [("red", "u1"), ("green", "u1"), ("blue", "u1")]
    for name, _ in mesh.extras:
        header += f"property float {name}\n"
        fields.append((f"e_{name}", "<f4"))
    header += f"element face {faces}\nproperty list uchar int vertex_index\nend_header\n"
    rec = np.zeros(rows, dtype=np.dtype(fields))
    pos = mesh.positions.detach().float().cpu().numpy()
    rec["x"], rec["y"], rec["z"] = pos[:, 0], pos[:, 1], pos[:, 2]
    if mesh.rgb is not None:
        c = mesh.rgb.cpu().numpy()
        rec["red"], rec["green"], rec["blue"] = c[:, 0], c[:, 1], c[:, 2]
    for name, values in mesh.extras:
        rec[f"e_{name}"] = values.detach().float().cpu().reshape(-1).numpy()
    face = np.zeros(faces, dtype=np.dtype([("n", "u1"), ("i", "<i4", (3,))]))
    if faces:
        face["n"] = 3
        face["i"] = mesh.triangles.detach().to(torch.int32).cpu().numpy()
    f, close = _open(target)
    try:
        f.write(header.encode())
        f.write(rec.tobytes())
        f.write(face.tobytes())
    finally:
        if close:
            f.close()


def write_obj(target, mesh: Mesh) -> None:
    """OBJ with ``v x y z [r g b]`` (vertex colours as [0, 1] floats, the common extension) and 1-based ``f`` triangles;
    extra channels have no OBJ slot and are not written."""
    rows = mesh.check()
    pos = mesh.positions.detach().float().cpu().numpy()
    col = mesh.rgb.cpu().numpy().astype(np.float32) / np.float32(255.0) if mesh.rgb is not None else None
    lines = []
    for r in range(rows):
        vals = [np.format_float_positional(v, unique=True, trim="-") for v in pos[r]]
        if col is not None:
            vals += [np.format_float_positional(v, unique=True, trim="-") for v in col[r]]
        lines.append("v " + " ".join(vals))
    if mesh.triangles.numel():
        for a, b, c in (mesh.triangles.detach().to(torch.int64).cpu() + 1).tolist():
            lines.append(f"f {a} {b} {c}")
    f, close = _open(target)
    try:
        f.write(("\n".join(lines) + "\n").encode())
    finally:
        if close:
            f.close()


_PLY_SIZES = {"float": 4, "float32": 4, "uchar": 1, "uint8": 1, "int": 4, "int32": 4}


def read_mesh(data: bytes, extension: str) -> Mesh:
    """Positions and triangles of a binary little-endian PLY in the layout ``write_ply`` emits (further vertex properties
    are skipped by their size) or of an OBJ (``v`` and triangular ``f`` lines; ``a/b/c`` references use the vertex
    index, negative indices count back from the vertices defined so far). Colours and extras are dropped."""
    if extension == "ply":
        marker = b"end_header\n"
        at = data.find(marker)
        if at < 0:
            raise ValueError("PLY end_header missing")
        header = data[: at + len(marker)].decode("ascii", errors="strict")
        if "format binary_little_endian 1.0" not in header:
            raise ValueError("only binary little-endian PLY is supported")
        rows = faces = stride = props = 0
        in_vertex = False
        for line in header.splitlines():
            w = line.split()
            if not w:
                continue
            if w[0] == "element":
                in_vertex = len(w) > 1 and w[1] == "vertex"
                if len(w) > 2 and w[1] in ("vertex", "face"):
                    if not w[2].isdigit():
                        raise ValueError(f"PLY {w[1]} count")
                    if w[1] == "vertex":
                        rows = int(w[2])
                    else:
                        faces = int(w[2])
            elif w[0] == "property" and in_vertex:
                if len(w) < 3 or w[1] not in _PLY_SIZES:
                    raise ValueError(f"unsupported PLY property type {w[1] if len(w) > 1 else None!r}")
                stride += _PLY_SIZES[w[1]]
                props += 1
        if props < 3 or stride < 12:
            raise ValueError("PLY vertex properties carry no x y z")
        body = memoryview(data)[at + len(marker):]
        if len(body) < rows * stride + faces * 13:
            raise ValueError("truncated PLY body")
        vert = np.frombuffer(body[: rows * stride], dtype=np.uint8).reshape(rows, stride)
        pos = vert[:, :12].copy().view("<f4").reshape(rows, 3)
        fdat = np.frombuffer(body[rows * stride: rows * stride + faces * 13], dtype=np.dtype([("n", "u1"), ("i", "<i4", (3,))]))
        if faces and (fdat["n"] != 3).any():
            raise ValueError("PLY face that is not a triangle")
        tri = fdat["i"].astype(np.int32).reshape(faces, 3)
        return Mesh(torch.from_numpy(pos.astype(np.float32)), torch.from_numpy(tri.copy()))
    if extension == "obj":
        pos: list[list[float]] = []
        tri: list[list[int]] = []
        for line in data.decode("utf-8").splitlines():
            w = line.split()
            if not w:
                continue
            if w[0] == "v":
                if len(w) < 4:
                    raise ValueError("OBJ vertex")
                pos.append([float(v) for v in w[1:4]])
            elif w[0] == "f":
                if len(w) != 4:
                    raise ValueError(f"OBJ face carries {len(w) - 1} vertex references; only triangles are supported")
                face = []
                for ref in w[1:]:
                    idx = int(ref.split("/")[0])
                    zero = idx - 1 if idx > 0 else len(pos) + idx
                    if not (0 <= zero < len(pos)):
                        raise ValueError(f"OBJ face index {idx} outside the {len(pos)} defined vertices")
                    face.append(zero)
                tri.append(face)
        return Mesh(torch.tensor(pos, dtype=torch.float32).reshape(-1, 3), torch.tensor(tri, dtype=torch.int32).reshape(-1, 3))
    raise ValueError(f"unsupported mesh extension {extension!r}")
