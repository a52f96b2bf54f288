"""KV format geometry (golden numbers of the reference's src/kv.rs tests) and affine8 pack/unpack."""
import pytest
import torch

from flyingfish_b200.engine import kv_format as kf


def test_layout_and_block_bytes_golden_numbers():
    a = kf.layout("affine8", 262144, 4, 256)
    assert (a.codes * 2 + (a.k_stats + a.v_stats) * 4) * 16 == 8_992_587_776
    assert a.ring_elements * 4 * 16 == 147_062_784
    assert a.bytes * 16 == 9_139_650_816
    assert kf.layout("bf16", 262144, 4, 256).bytes * 16 == 17_179_869_184
    with pytest.raises(ValueError):
        kf.layout("affine8", 1 << 63, 4, 256)
    assert kf.block_bytes("affine8", 2048, 129, 2177, 4, 256) == 4 * 129 * 256 * 4
    assert kf.block_bytes("affine8", 128, 128, 2177, 4, 256) == 4 * 128 * 256 * 4
    assert kf.block_bytes("affine8", 0, 127, 127, 4, 256) == 4 * 127 * 256 * 4
    assert kf.from_tag(kf.TAGS["affine8"]) == "affine8"


def test_sealed_boundary_and_ring_slots():
    ring = kf.layout("affine8", 262144, 4, 256).ring
    for n in range(0, 16384, 37):
        start = kf.sealed_until(n)
        assert start % 128 == 0 and start <= max(0, n - 2048)
        end = n + kf.TENTATIVE_TOKENS
        slots = {kf.ring_slot(p, ring) for p in range(max(start, 64), end)}
        assert len(slots) == end - min(max(start, 64), end)
    assert [kf.sealed_until(n) for n in (2175, 2176, 2177)] == [0, 128, 128]
    assert kf.ring_slot(63, ring) == 63
    with pytest.raises(ValueError):
        kf.ring_slot(64, 64)


def test_affine8_store_roundtrip_cpu():
    g = torch.Generator().manual_seed(0)
    heads, cap, d = 2, 2048 + 384, 64
    k = torch.randn(heads, cap, d, generator=g).to(torch.bfloat16); v = torch.randn(heads, cap, d, generator=g).to(torch.bfloat16)
    k[0, 130:140, 3] = 7.0
    st = kf.Affine8Store(heads, cap, d, "cpu")
    assert st.seal(k, v, 2048 + 300) == 256
    ko = torch.zeros_like(k); vo = torch.zeros_like(v)
    st.materialise(ko, vo, 0, 256)
    span_k = (k[:, :256].float().amax(1) - k[:, :256].float().amin(1)).max().item()
    assert (ko[:, :256].float() - k[:, :256].float()).abs().max().item() <= span_k / 255 * 0.51 + 0.04
    assert (vo[:, :256].float() - v[:, :256].float()).abs().max().item() <= 0.06
    assert ko[:, 256:].abs().max() == 0


@pytest.mark.gpu
def test_affine8_cuda_bit_exact_with_cpu():
    from flyingfish_b200 import ops
    g = torch.Generator().manual_seed(1)
    heads, cap, d = 3, 640, 256
    k = (torch.randn(heads, cap, d, generator=g) * 3).to(torch.bfloat16); v = torch.randn(heads, cap, d, generator=g).to(torch.bfloat16)
    v[1, 5] = 0.25                                   # zero span -> scale 1
    cpu = kf.Affine8Store(heads, cap, d, "cpu"); gpu = kf.Affine8Store(heads, cap, d, "cuda")
    for st, kk, vv in ((cpu, k, v), (gpu, k.cuda(), v.cuda())):
        kf.pack_k(kk, st.k_codes, st.k_stats, 1, 3); kf.pack_v(vv, st.v_codes, st.v_stats, 100, 400)
    ops.check_status()
    assert torch.equal(gpu.k_stats.cpu(), cpu.k_stats) and torch.equal(gpu.v_stats.cpu(), cpu.v_stats)
    assert (gpu.k_codes.cpu().int() - cpu.k_codes.int()).abs().max() <= 1        # CPU division is not correctly-rounded fdiv
    assert (gpu.v_codes.cpu().int() - cpu.v_codes.int()).abs().max() <= 1
    ko = torch.zeros(heads, cap, d, dtype=torch.bfloat16, device="cuda")
    kf.unpack(gpu.k_codes, gpu.k_stats, ko, 128, 384, True)
    ref = torch.zeros(heads, cap, d, dtype=torch.bfloat16); kf.unpack(gpu.k_codes.cpu(), gpu.k_stats.cpu(), ref, 128, 384, True)
    assert (ko.cpu().float() - ref.float()).abs().max() <= 0.02
