"""Device-side waits that nobody answers must run out, report through the status word and leave the context
usable -- never hang, trap or fault.

The tests load the short-wait build of the kernel library (every bounded wait cut from 2 s to 5 ms, see
``ops/build.py``) next to the production one, make a wait run out by construction (a flag that no rank ever sets, a
counter target that cannot be reached), read the status word, and then run an ordinary kernel through the same
library to show that tensor memory was released and results are still right. One GPU, plain peer-style stores into
local buffers standing for the second rank's arena, no NVLS."""
import ctypes
from ctypes import c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TIMEOUT, KID_AR, KID_GEMM_AR, KID_CHAIN = 1, 10, 11, 30


@pytest.fixture(scope="module")
def sw():
    from flyingfish_b200.ops import build
    lib = ctypes.CDLL(str(build.build_kernels(short_wait=True)))
    lib.ff_arena_data_offset.restype = ctypes.c_longlong
    return lib


def _p(t):
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _fake_arena(lib, dev, slot_bytes):
    """Two local buffers laid out like the symmetric arenas of ranks 0 and 1; this process plays rank 0 and nothing
    ever writes rank 1's flags."""
    half = slot_bytes * 2
    size = lib.ff_arena_data_offset() + 2 * half
    bufs = [torch.zeros(size, dtype=torch.uint8, device=dev) for _ in range(2)]
    ptrs = (ctypes.c_ulonglong * 8)(*([b.data_ptr() for b in bufs] + [0] * 6))
    return bufs, ptrs, half


def _gemm_check(lib, dev, status):
    g = torch.Generator().manual_seed(7)
    m, n, k = 24, 2048, 1024
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    sb, cb = c_longlong(0), c_longlong(0)
    grid = lib.ff_gemm_skinny_plan(m, n, k, ctypes.byref(sb), ctypes.byref(cb))
    scratch = torch.empty(max(sb.value // 4, 1), dtype=torch.float32, device=dev)
    counters = torch.zeros(max(cb.value // 4, 1), dtype=torch.int32, device=dev)
    rc = lib.ff_gemm_skinny(_p(x), _p(w), _p(y), m, n, k, k, k, n, grid, _p(scratch), _p(counters), _p(status), _stream())
    assert rc == 0
    torch.cuda.synchronize()
    ref = x.float().cpu() @ w.float().cpu().t()
    err = (y.float().cpu() - ref).abs()
    assert (err <= 2e-2 + 2e-2 * ref.abs()).all()


def test_allreduce_wait_on_a_silent_peer_times_out(sw):
    dev = torch.device("cuda", 0)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    bufs, ptrs, half = _fake_arena(sw, dev, 1 << 16)
    x = torch.ones(4096, dtype=torch.bfloat16, device=dev)
    out = torch.zeros_like(x)
    rc = sw.ff_allreduce_oneshot(ptrs, 0, 2, c_longlong(half), c_longlong(1 << 16), _p(x), _p(out), c_longlong(x.numel()),
                                 _p(status), _stream())
    assert rc == 0
    torch.cuda.synchronize()                      # returns: the wait is bounded
    code, kid, who, _ = status.cpu().tolist()
    assert (code, kid, who) == (TIMEOUT, KID_AR, 1)
    status.zero_()
    _gemm_check(sw, dev, status)
    assert status.cpu().tolist() == [0, 0, 0, 0]


def test_fused_gemm_allreduce_times_out_and_frees_tensor_memory(sw):
    dev = torch.device("cuda", 0)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    m, n, k = 16, 1024, 512
    bufs, ptrs, half = _fake_arena(sw, dev, m * n * 2)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    y = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    sb, cb = c_longlong(0), c_longlong(0)
    grid = sw.ff_gemm_skinny_plan(m, n, k, ctypes.byref(sb), ctypes.byref(cb))
    scratch = torch.empty(max(sb.value // 4, 1), dtype=torch.float32, device=dev)
    counters = torch.zeros(max(cb.value // 4, 1), dtype=torch.int32, device=dev)
    rc = sw.ff_gemm_ar(ptrs, 0, 2, c_longlong(half), c_longlong(m * n * 2), _p(x), _p(w), _p(y), m, n, k, k, k, n, grid,
                       _p(scratch), _p(counters), ctypes.c_ulonglong(0), _p(status), _stream())
    assert rc == 0
    torch.cuda.synchronize()
    code, kid, who, _ = status.cpu().tolist()
    assert (code, kid, who) == (TIMEOUT, KID_GEMM_AR, 1)
    # the kernel's own contribution reached the "peer": its stores were issued before the wait
    slot_on_peer = bufs[1][sw.ff_arena_data_offset():]
    assert slot_on_peer.any().item()
    # tensor memory was released on the way out: the next tcgen05 kernel allocates and runs
    status.zero_()
    _gemm_check(sw, dev, status)
    assert status.cpu().tolist() == [0, 0, 0, 0]


def test_chain_phase_wait_runs_out_and_the_kernel_unwinds(sw):
    """The projection chain orders its phases by counters. With the recorded base of the first phase pushed out of
    reach, every CTA's wait for that phase runs out: producers, MMA issuers and epilogue warps leave through the
    abort flag, copies in flight get their grace period, tensor memory is freed. After zeroing the counters the
    same chain runs correctly."""
    from flyingfish_b200 import ops
    from flyingfish_b200.ops import chain
    dev = torch.device("cuda", 0)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    m, hidden, kq = 8, 1024, 512
    g = torch.Generator().manual_seed(5)
    a = torch.randn(m, kq, generator=g).to(torch.bfloat16).to(dev)
    wo = (torch.randn(hidden, kq, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    w2 = (torch.randn(hidden, hidden, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    ln = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
    res0 = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(dev)
    sb, cb, yb = c_longlong(0), c_longlong(0), c_longlong(0)
    assert sw.ff_decode_chain_workspace(128, ctypes.byref(sb), ctypes.byref(cb), ctypes.byref(yb)) == 0
    scratch = torch.empty(sb.value // 4, dtype=torch.float32, device=dev)
    counters = torch.zeros(cb.value // 4, dtype=torch.int32, device=dev)
    sync = torch.zeros(yb.value // 4, dtype=torch.int32, device=dev)

    def launch(res):
        tmp = torch.empty(m, hidden, dtype=torch.bfloat16, device=dev)
        n1 = torch.empty(m, hidden, dtype=torch.bfloat16, device=dev)
        out = torch.empty(m, hidden, dtype=torch.bfloat16, device=dev)
        phases = [chain.gemm(a, wo, tmp), chain.add_norm(tmp, res, ln, n1, 1e-5), chain.gemm(n1, w2, out)]
        arr = (chain._Phase * 3)(*phases)
        rc = sw.ff_decode_chain(arr, 3, m, None, _p(scratch), _p(counters), _p(sync), _p(status), _stream())
        assert rc == 0
        torch.cuda.synchronize()
        return out

    base_word = 8 * 32            # CH_SYNC_BASE: first word behind the eight counter lines
    sync[base_word] = 1 << 20     # phase 0 can never reach base + its units
    launch(res0.clone())
    code, kid, _, _ = status.cpu().tolist()
    assert (code, kid) == (TIMEOUT, KID_CHAIN)
    status.zero_(); sync.zero_(); counters.zero_()
    out = launch(res0.clone())
    assert status.cpu().tolist() == [0, 0, 0, 0]
    # reference of the same three phases through the ordinary operators
    o = ops.linear(a, wo)
    r = res0.clone()
    n1 = ops.add_rmsnorm(o, r, ln, 1e-5)
    want = ops.linear(n1, w2)
    torch.cuda.synchronize()
    err = (out.float() - want.float()).abs()
    assert (err <= 3e-2 + 3e-2 * want.float().abs()).all()
