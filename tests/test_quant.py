"""Quantised formats: host codecs (CPU) and the device kernels against them (GPU)."""
import pytest
import torch

from flyingfish_b200.loaders import quant as q


def test_e2m1_codec_roundtrip_and_ties():
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -6.0, 7.5, 0.25, 0.75, 2.5, 5.0])
    codes = q.e2m1_encode(vals)
    dec = q.e2m1_decode(codes)
    assert dec.tolist()[:10] == vals.tolist()[:10]
    assert dec[10] == 6.0                      # saturates
    assert dec[11] == 0.0 and dec[12] == 1.0   # ties go to the even code
    assert dec[13] == 2.0 and dec[14] == 4.0
    packed = q.e2m1_pack(codes[:14])
    assert torch.equal(q.e2m1_unpack(packed), codes[:14])


def test_e8m0_and_e4m3():
    assert q.e8m0_decode(torch.tensor([127, 128, 120], dtype=torch.uint8)).tolist() == [1.0, 2.0, 2.0 ** -7]
    assert q.e8m0_encode_ceil(torch.tensor([1.0, 1.1, 0.3])).tolist() == [127, 128, 126]
    x = torch.tensor([0.0, 1.0, -448.0, 1000.0, 0.0625])
    assert q.e4m3_decode(q.e4m3_encode(x)).tolist() == [0.0, 1.0, -448.0, 448.0, 0.0625]


def test_fp8_block_linear_close_to_fp32():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 256, generator=g).to(torch.bfloat16)
    w = torch.randn(130, 256, generator=g) * 0.1
    wq, ws = q.quantize_fp8_block_weight(w)
    assert ws.shape == q.fp8_block_scale_shape(130, 256)
    y = q.fp8_block_linear(x, wq, ws).float()
    ref = x.float() @ w.t()
    assert (y - ref).abs().max() < 0.06 * ref.abs().max()
    deq = q.dequantize_fp8_block(wq, ws, dtype=torch.float32)
    assert (deq - w).abs().max() < 0.07 * w.abs().max()


def test_nvfp4_roundtrip_and_linear():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(64, 128, generator=g) * 0.05
    packed, scales, gs = q.quantize_nvfp4(w)
    assert packed.shape == (64, 64) and scales.shape == q.nvfp4_scale_shape(64, 128)
    deq = q.dequantize_nvfp4(packed, scales, gs, torch.float32)
    assert (deq - w).abs().mean() < 0.12 * w.abs().mean() + 1e-3
    x = torch.randn(5, 128, generator=g).to(torch.bfloat16)
    y = q.nvfp4_linear(x, packed, scales, gs).float()
    assert (y - x.float() @ deq.to(torch.bfloat16).float().t()).abs().max() < 1e-2


@pytest.mark.gpu
def test_quant_kernels_match_codecs():
    from flyingfish_b200.ops import quant_ops
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(33, 512, generator=g) * 3).to(torch.bfloat16)
    x[5, 128:256] = 0
    cq, cs = q.quantize_fp8_act(x)
    gq, gsc = quant_ops.quant_fp8_act(x.cuda())
    assert torch.allclose(gsc.cpu(), cs, rtol=1e-6)
    mism = (gq.cpu() != cq).float().mean().item()
    assert mism < 1e-3, f"{mism} of the E4M3 codes differ"
    # power-of-two scales
    _, s2 = quant_ops.quant_fp8_act(x.cuda(), ue8m0=True)
    assert torch.equal(torch.log2(s2).round(), torch.log2(s2))
    # NVFP4 dequant is bit exact
    w = torch.randn(96, 256, generator=g) * 0.05
    packed, scales, gs = q.quantize_nvfp4(w)
    got = quant_ops.dequant_nvfp4(packed.cuda(), scales.cuda(), gs.cuda())
    assert torch.equal(got.cpu(), q.dequantize_nvfp4(packed, scales, gs))
    wq, ws = q.quantize_fp8_block_weight(w)
    assert torch.equal(quant_ops.dequant_fp8_block(wq.cuda(), ws.cuda()).cpu(), q.dequantize_fp8_block(wq, ws))
    # FP4 packers decode close to the input
    xb = (torch.randn(8, 128, generator=g)).to(torch.bfloat16)
    gsx = (xb.float().abs().max() / (6 * 448)).reshape(())
    p, sc = quant_ops.quant_fp4(xb.cuda(), "nvfp4", gsx.cuda())
    deq = q.dequantize_nvfp4(p.cpu(), sc.cpu(), gsx, torch.float32)
    assert (deq - xb.float()).abs().mean() < 0.15 * xb.float().abs().mean()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (16, 1536, 7168), (64, 512, 1024), (130, 384, 256), (200, 7168, 2048)])
def test_fp8_gemm_matches_reference(m, n, k):
    from flyingfish_b200 import ops
    from flyingfish_b200.ops import quant_ops
    g = torch.Generator().manual_seed(3)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g) * 0.05
    wq, ws = q.quantize_fp8_block_weight(w)
    got = quant_ops.linear_fp8(x.cuda(), wq.cuda(), ws.cuda())
    torch.cuda.synchronize()
    ops.check_status()
    # oracle on the codes the device quantiser produced, so the GEMM is checked on its own
    xq, xs = quant_ops.quant_fp8_act(x.cuda())
    xd = q.e4m3_decode(xq.cpu()).view(m, k // 128, 128).double()
    wd = q.e4m3_decode(wq).view(n, k // 128, 128).double()
    part = torch.einsum("mbk,nbk->mnb", xd, wd).float()
    ref = (part * xs.cpu()[:, None, :] * ws.repeat_interleave(128, 0)[:n][None]).sum(-1)
    err = (got.float().cpu() - ref).abs()
    assert (err <= 1e-2 + 1e-2 * ref.abs()).all(), f"max err {err.max().item()}"
    end2end = q.fp8_block_linear(x, wq, ws).float()
    assert (got.float().cpu() - end2end).abs().max() <= 0.03 * end2end.abs().max() + 0.05
    again = quant_ops.linear_fp8(x.cuda(), wq.cuda(), ws.cuda())
    assert torch.equal(got, again)


@pytest.mark.gpu
def test_nvfp4_linear_gpu():
    from flyingfish_b200.ops import quant_ops
    g = torch.Generator().manual_seed(4)
    w = torch.randn(512, 1024, generator=g) * 0.05
    x = torch.randn(7, 1024, generator=g).to(torch.bfloat16)
    packed, scales, gs = q.quantize_nvfp4(w)
    got = quant_ops.linear_nvfp4(x.cuda(), packed.cuda(), scales.cuda(), gs.cuda())
    ref = q.nvfp4_linear(x, packed, scales, gs).float()
    assert (got.float().cpu() - ref).abs().max() <= 2e-2 + 2e-2 * ref.abs().max()
