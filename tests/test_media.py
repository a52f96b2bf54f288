"""Output containers: PNG, YUV4MPEG2 / MP4 muxing, PLY / OBJ meshes."""
import io
import os
import stat

import pytest
import torch

from flyingfish_b200.serve.image import decode_png
from flyingfish_b200.utils import media


def test_png_round_trips_through_the_decoder():
    g = torch.Generator().manual_seed(0)
    rgb = torch.randint(0, 256, (5, 7, 3), generator=g, dtype=torch.uint8)
    buf = io.BytesIO()
    media.write_png(buf, 7, 5, rgb)
    img = decode_png(buf.getvalue())
    assert (img.width, img.height) == (7, 5)
    assert torch.equal(torch.from_numpy(img.pixels.copy()).reshape(5, 7, -1)[..., :3].to(torch.uint8), rgb)
    rgba = torch.randint(0, 256, (4, 6, 4), generator=g, dtype=torch.uint8)
    buf = io.BytesIO()
    media.write_png(buf, 6, 4, rgba.numpy().tobytes(), channels=4)
    data = buf.getvalue()
    assert data[:8] == b"\x89PNG\r\n\x1a\n" and data[25] == 6          # colour type 6 = RGBA
    with pytest.raises(ValueError):
        media.write_png(io.BytesIO(), 6, 4, rgba, channels=3)
    with pytest.raises(ValueError):
        media.write_png(io.BytesIO(), 0, 4, b"", channels=3)


def _yuv_scalar(rgb, shift):
    r, g, b = rgb
    q = lambda v, off: max(0, min(255, ((v + (1 << (shift - 1))) >> shift) + off))
    return q(19595 * r + 38470 * g + 7471 * b, 0), q(-11058 * r - 21710 * g + 32768 * b, 128), q(32768 * r - 27439 * g - 5329 * b, 128)


def test_y4m_matches_the_fixed_point_formula():
    g = torch.Generator().manual_seed(1)
    video = torch.randint(0, 256, (2, 4, 6, 3), generator=g, dtype=torch.uint8)
    video[0, 0, 0] = torch.tensor([255, 255, 255], dtype=torch.uint8)
    video[0, 0, 1] = torch.tensor([0, 0, 255], dtype=torch.uint8)
    buf = io.BytesIO()
    media.write_y4m(buf, video, (24, 1))
    data = buf.getvalue()
    head = b"YUV4MPEG2 W6 H4 F24:1 Ip A1:1 C420jpeg XCOLORRANGE=FULL\n"
    assert data.startswith(head)
    frame = 6 * 4 + 2 * (3 * 2)
    assert len(data) == len(head) + 2 * (6 + frame)
    off = len(head)
    for f in range(2):
        assert data[off:off + 6] == b"FRAME\n"
        body = data[off + 6: off + 6 + frame]
        px = video[f].tolist()
        want_y = bytes(_yuv_scalar(px[r][c], 16)[0] for r in range(4) for c in range(6))
        assert body[:24] == want_y
        sums = [[[sum(px[r + dy][c + dx][k] for dy in range(2) for dx in range(2)) for k in range(3)] for c in range(0, 6, 2)]
                for r in range(0, 4, 2)]
        assert body[24:30] == bytes(_yuv_scalar(sums[r][c], 18)[1] for r in range(2) for c in range(3))
        assert body[30:36] == bytes(_yuv_scalar(sums[r][c], 18)[2] for r in range(2) for c in range(3))
        off += 6 + frame
    assert _yuv_scalar((255, 255, 255), 16) == (255, 128, 128)
    with pytest.raises(ValueError):
        media.write_y4m(io.BytesIO(), video[:, :3], (24, 1))                 # odd height
    with pytest.raises(ValueError):
        media.write_y4m(io.BytesIO(), video, (0, 1))


def test_mp4_mux_runs_the_tool_and_cleans_up(tmp_path):
    video = torch.zeros(1, 2, 2, 3, dtype=torch.uint8)
    tool = tmp_path / "fakemux"
    # a stand-in muxer: checks that a Y4M stream arrives on standard input, writes its last argument
    tool.write_text("#!/bin/sh\nhead -c 9 > \"$0.head\"\ncat > /dev/null\nfor a; do out=\"$a\"; done\nprintf ok > \"$out\"\n")
    tool.chmod(tool.stat().st_mode | stat.S_IEXEC)
    out = tmp_path / "clip.mp4"
    media.mux_mp4(out, video, (24, 1), audio=(16000, 1, torch.zeros(160)), tool=str(tool))
    assert out.read_text() == "ok" and (tmp_path / "fakemux.head").read_bytes() == b"YUV4MPEG2"
    assert [p.name for p in tmp_path.iterdir() if p.suffix == ".wav"] == []      # the audio scratch file is gone
    with pytest.raises(FileExistsError):
        media.mux_mp4(out, video, (24, 1), tool=str(tool))
    with pytest.raises(ValueError):
        media.mux_mp4(tmp_path / "clip.mov", video, (24, 1), tool=str(tool))
    bad = tmp_path / "badmux"
    bad.write_text("#!/bin/sh\ncat > /dev/null\nfor a; do out=\"$a\"; done\nprintf partial > \"$out\"\nexit 3\n")
    bad.chmod(bad.stat().st_mode | stat.S_IEXEC)
    with pytest.raises(RuntimeError, match="mux failed"):
        media.mux_mp4(tmp_path / "other.mp4", video, (24, 1), tool=str(bad))
    assert not (tmp_path / "other.mp4").exists()                               # a failed run leaves no file
    with pytest.raises(RuntimeError, match="not installed"):
        media.mux_mp4(tmp_path / "third.mp4", video, (24, 1), tool="no-such-muxer-anywhere")


def _mesh():
    rows = 10
    pos = torch.stack([torch.arange(rows) * 0.5, -torch.arange(rows).float(), torch.arange(rows) + 0.25], dim=1).float()
    tri = torch.stack([torch.arange(rows - 2), torch.arange(1, rows - 1), torch.arange(2, rows)], dim=1).to(torch.int32)
    rgb = (torch.arange(rows * 3) * 7 % 256).to(torch.uint8).reshape(rows, 3)
    return media.Mesh(pos, tri, rgb, (("opacity", torch.linspace(0, 1, rows)), ("scale", torch.full((rows,), 2.5))))


def test_mesh_writers_and_reader_round_trip():
    mesh = _mesh()
    buf = io.BytesIO()
    media.write_ply(buf, mesh)
    data = buf.getvalue()
    header = data[: data.index(b"end_header\n") + 11].decode()
    assert header == ("ply\nformat binary_little_endian 1.0\nelement vertex 10\nproperty float x\nproperty float y\nproperty float z\n"
                      "property uchar red\nproperty uchar green\nproperty uchar blue\nproperty float opacity\nproperty float scale\n"
                      "element face 8\nproperty list uchar int vertex_index\nend_header\n")
    assert len(data) == len(header) + 10 * (12 + 3 + 8) + 8 * 13
    back = media.read_mesh(data, "ply")
    assert torch.equal(back.positions, mesh.positions) and torch.equal(back.triangles, mesh.triangles)
    # without colours and extras the vertex record is 12 bytes
    buf = io.BytesIO()
    media.write_ply(buf, media.Mesh(mesh.positions, mesh.triangles))
    assert torch.equal(media.read_mesh(buf.getvalue(), "ply").positions, mesh.positions)
    buf = io.BytesIO()
    media.write_obj(buf, mesh)
    text = buf.getvalue().decode()
    lines = text.splitlines()
    assert lines[0].split()[:4] == ["v", "0", "-0", "0.25"] and len(lines[0].split()) == 7
    assert lines[10] == "f 1 2 3" and lines[-1] == "f 8 9 10"
    back = media.read_mesh(buf.getvalue(), "obj")
    assert torch.equal(back.positions, mesh.positions) and torch.equal(back.triangles, mesh.triangles)
    # OBJ references: slashes, negative (relative) indices; polygons and bad indices are refused
    obj = b"v 0 0 0\nv 1 0 0\nv 0 1 0\nvn 0 0 1\nf 1/1/1 2/2/1 -1/3/1\n"
    assert media.read_mesh(obj, "obj").triangles.tolist() == [[0, 1, 2]]
    with pytest.raises(ValueError, match="triangles"):
        media.read_mesh(b"v 0 0 0\nv 1 0 0\nv 0 1 0\nv 1 1 0\nf 1 2 3 4\n", "obj")
    with pytest.raises(ValueError, match="outside"):
        media.read_mesh(b"v 0 0 0\nf 1 2 3\n", "obj")
    with pytest.raises(ValueError):
        media.read_mesh(data[:-5], "ply")
    with pytest.raises(ValueError):
        media.read_mesh(data.replace(b"binary_little_endian", b"ascii"), "ply")
    with pytest.raises(ValueError):
        media.read_mesh(b"", "stl")
    with pytest.raises(ValueError):
        media.write_ply(io.BytesIO(), media.Mesh(mesh.positions, mesh.triangles, mesh.rgb[:5]))
    with pytest.raises(ValueError):
        media.write_ply(io.BytesIO(), media.Mesh(mesh.positions, mesh.triangles, None, (("bad name", torch.zeros(10)),)))
