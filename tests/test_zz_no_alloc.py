"""The allocation-free GEMM entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at call time (a serving loop
whose allocator is frozen after start-up, a plugin with a fixed budget, a plain C host that owns
only its inputs and outputs). ``ff_gemm_skinny_noalloc`` keeps its split-K scratch in a fixed
array inside the library for them. The test compares it with the ordinary entry point (which
receives caller-allocated scratch) on two calls in a row -- both shapes run as stream-K, so the
second call reuses the partial-sum array the first one left dirty -- and checks that an oversized
problem is refused. The two entry points run the same decomposition, so their outputs must be
bit-identical."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from flyingfish_b200.ops import build
    lib = ctypes.CDLL(str(build.build_kernels()))
    lib.ff_gemm_skinny_noalloc.restype = ctypes.c_int
    lib.ff_gemm_skinny.restype = ctypes.c_int
    lib.ff_gemm_skinny_plan.restype = ctypes.c_int
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    for call, (m, n, k) in enumerate([(24, 28672, 4096), (48, 32768, 2048)]):
        g = torch.Generator().manual_seed(100 + call)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
        w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        y_new = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        y_old = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        sb, cb = ctypes.c_longlong(0), ctypes.c_longlong(0)
        splits = lib.ff_gemm_skinny_plan(m, n, k, ctypes.byref(sb), ctypes.byref(cb))
        assert splits > 1
        assert sb.value > 0, "both cases must exercise the scratch path (stream-K partials)"
        scratch = torch.empty(max(sb.value // 4, 1), dtype=torch.float32, device=dev)
        counters = torch.zeros(max(cb.value // 4, 1), dtype=torch.int32, device=dev)
        rc = lib.ff_gemm_skinny(_p(x), _p(w), _p(y_old), m, n, k, k, k, n, splits, _p(scratch), _p(counters), _p(status), stream)
        assert rc == 0
        rc = lib.ff_gemm_skinny_noalloc(_p(x), _p(w), _p(y_new), m, n, k, k, k, n, _p(status), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.cpu().tolist() == [0, 0, 0, 0], "a kernel reported a device-side error"
        ref = (x.float().cpu() @ w.float().cpu().t())
        err = (y_new.float().cpu() - ref).abs()
        assert (err <= 2e-2 + 2e-2 * ref.abs()).all(), f"call {call}: max err {err.max().item()}"
        assert torch.equal(y_new, y_old), f"call {call}: the two entry points must give identical bits"


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    dev = torch.device("cuda", 0)
    x = torch.zeros(256, 4096, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(4096, 4096, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(256, 4096, dtype=torch.bfloat16, device=dev)
    rc = lib.ff_gemm_skinny_noalloc(_p(x), _p(w), _p(y), 256, 4096, 4096, 4096, 4096, 4096, None,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -5
    # just past the scratch limit: 64 tokens of a wide layer need 2 * 148 * 64 * 128 * 4 bytes > 8 MiB
    w2 = torch.zeros(28672, 4096, dtype=torch.bfloat16, device=dev)
    y2 = torch.zeros(64, 28672, dtype=torch.bfloat16, device=dev)
    rc = lib.ff_gemm_skinny_noalloc(_p(x), _p(w2), _p(y2), 64, 28672, 4096, 4096, 4096, 28672, None,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -5
