"""Block-scaled tensor-core path (tcgen05 kind::mxf8f6f4 + TMA + TMEM) against the CPU oracle, through the C-ABI.
The activation is FP8-quantised first (q8, sf); q8 * 2^(sf-127) must equal the oracle's fake_quant_fp8 bit for bit, so the
oracle GEMM on that bf16 tensor is the exact reference of the tensor-core result."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _deq(q8, sf):
    v = q8.view(torch.float8_e4m3fn).float().view(q8.shape[0], -1, 32) * torch.exp2(sf.float() - 127).unsqueeze(-1)
    return v.view(q8.shape[0], -1)


def test_quantize_rows_matches_fake_quant(mods, oracle, dev):
    torch.manual_seed(0)
    x = (torch.randn(9, 512) * 3).to(torch.bfloat16)
    x[0, :32] = 0
    x[1, :64] *= 1e-5
    q8, sf = mods.cukern.mx_quantize_rows(x.to(dev))
    ref = oracle.fake_quant_fp8(x, 32)
    assert torch.equal(_deq(q8.cpu(), sf.cpu()).to(torch.bfloat16).view(torch.int16), ref.view(torch.int16))
    idx = torch.tensor([3, 3, 0, 8], dtype=torch.int32)
    q8g, sfg = mods.cukern.mx_quantize_rows(x.to(dev), idx.to(dev))
    assert torch.equal(q8g.cpu(), q8.cpu()[idx.long()]) and torch.equal(sfg.cpu(), sf.cpu()[idx.long()])
    assert mods.cukern.device_error(dev) == 0


def _experts(E, N, K, seed, lo=112, hi=128):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 256, (E, N, K // 2), dtype=torch.uint8, generator=g), torch.randint(lo, hi, (E, N, K // 32), dtype=torch.uint8, generator=g), g)


@pytest.mark.parametrize("G,M,N,K,rows", [(1, 1, 128, 128, 32), (1, 5, 256, 512, 64), (3, 16, 512, 1024, 64), (4, 21, 384, 2304, 32), (2, 40, 256, 4096, 128)])
def test_mx_grouped_store(mods, oracle, dev, G, M, N, K, rows):
    E = 6
    w, s, g = _experts(E, N, K, 10 * G + M)
    x = (torch.randn(G * M, K, generator=g) * 2).to(torch.bfloat16)
    q8, sf = mods.cukern.mx_quantize_rows(x.to(dev))
    xq = oracle.fake_quant_fp8(x, 32)
    experts = torch.tensor([5, 2, 0, 3][:G], dtype=torch.int32)
    grp_start = torch.arange(0, G * M + 1, M, dtype=torch.int32)
    P = G * M
    wt = torch.rand(P, generator=g)
    out_rows = torch.randperm(P, generator=g).int()
    ref = oracle.fp4_pairs(xq, w, s, experts.repeat_interleave(M), torch.arange(P), out_rows, wt, P)
    y = mods.cukern.mx_grouped(w.to(dev), s.to(dev), q8, sf, experts.to(dev), grp_start.to(dev), None, out_rows.to(dev), wt.to(dev), P, rows_per_tile=rows)
    assert mods.cukern.device_error(dev) == 0
    assert rel_err(y, ref) < 2e-3


@pytest.mark.parametrize("M,N,K,rows,tpw", [(100, 512, 512, 256, 128), (70, 256, 1024, 128, 64), (33, 768, 256, 256, 32)])
def test_mx_grouped_wide_tiles(mods, oracle, dev, M, N, K, rows, tpw):
    E, G = 5, 2
    w, s, g = _experts(E, N, K, M + rows)
    x = (torch.randn(G * M, K, generator=g) * 2).to(torch.bfloat16)
    q8, sf = mods.cukern.mx_quantize_rows(x.to(dev))
    xq = oracle.fake_quant_fp8(x, 32)
    experts = torch.tensor([4, 1], dtype=torch.int32)
    grp_start = torch.arange(0, G * M + 1, M, dtype=torch.int32)
    P = G * M
    wt = torch.rand(P, generator=g)
    out_rows = torch.randperm(P, generator=g).int()
    ref = oracle.fp4_pairs(xq, w, s, experts.repeat_interleave(M), torch.arange(P), out_rows, wt, P)
    y = mods.cukern.mx_grouped(w.to(dev), s.to(dev), q8, sf, experts.to(dev), grp_start.to(dev), None, out_rows.to(dev), wt.to(dev), P, rows_per_tile=rows,
                               tokens_per_work=tpw)
    assert mods.cukern.device_error(dev) == 0
    assert rel_err(y, ref) < 2e-3


@pytest.mark.parametrize("rows,tpw,M", [(32, 16, 7), (64, 32, 7), (128, 128, 7), (128, 128, 70)])
def test_mx_grouped_swiglu_epilogue(mods, oracle, dev, rows, tpw, M):
    # 7 rows per expert take the staged small-tile epilogue, 70 the thread-per-row one (SwiGLU on the special-function unit)
    E, inter, K, G = 4, 256, 512, 3
    w, s, g = _experts(E, 2 * inter, K, 77, 112, 120)
    x = torch.randn(G * M, K, generator=g).to(torch.bfloat16)
    q8, sf = mods.cukern.mx_quantize_rows(x.to(dev))
    xq = oracle.fake_quant_fp8(x, 32)
    experts = torch.tensor([1, 3, 0], dtype=torch.int32)
    grp_start = torch.arange(0, G * M + 1, M, dtype=torch.int32)
    P = G * M
    wt = torch.rand(P, generator=g)
    gu = oracle.fp4_pairs(xq, w, s, experts.repeat_interleave(M), torch.arange(P), torch.arange(P), None, P)
    for limit in (10.0, 0.0):
        ref = oracle.swiglu_quant(gu, wt, inter, limit)
        h8, hsf = mods.cukern.mx_grouped(w.to(dev), s.to(dev), q8, sf, experts.to(dev), grp_start.to(dev), None, None, wt.to(dev), P, epilogue="swiglu_q8",
                                         limit=limit, rows_per_tile=rows, tokens_per_work=tpw)
        assert mods.cukern.device_error(dev) == 0
        h = _deq(h8.cpu(), hsf.cpu())
        # against the oracle's own GEMM: isolated elements sit on a rounding boundary (the fp32 summation order of the tensor cores
        # differs from the oracle's), so values are compared, not bits
        assert rel_err(h, ref) < 0.07
        assert ((h - ref.float()).abs() > 1e-6 * ref.float().abs().max()).float().mean() < 0.02
        # the epilogue's arithmetic alone: SwiGLU + FP8 quantisation of the SAME accumulator values (the kernel's fp32 store
        # epilogue, identical MMAs) by the oracle -> at least 99.9 % of the values bit-equal, like the stand-alone kernel
        gu_gpu = mods.cukern.mx_grouped(w.to(dev), s.to(dev), q8, sf, experts.to(dev), grp_start.to(dev), None, None, None, P, rows_per_tile=rows,
                                        tokens_per_work=tpw)
        ref2 = oracle.swiglu_quant(gu_gpu.float().cpu(), wt, inter, limit)
        assert (h == ref2.float()).float().mean() >= 0.999


def test_mx_dense_fp8(mods, oracle, dev):
    g = torch.Generator().manual_seed(5)
    N, K, M = 256, 1024, 19
    w = torch.randint(0, 256, (N, K), dtype=torch.uint8, generator=g)
    w[(w & 0x7F) == 0x7F] = 0
    s = torch.randint(110, 130, (N // 32, K // 32), dtype=torch.uint8, generator=g)
    x = (torch.randn(M, K, generator=g) * 2).to(torch.bfloat16)
    q8, sf = mods.cukern.mx_quantize_rows(x.to(dev))
    ref = oracle.fp8_gemm(oracle.fake_quant_fp8(x, 32), w, s)
    y = mods.cukern.mx_grouped(w.to(dev), s.to(dev), q8, sf, None, None, None, None, None, M, rows_per_tile=64)
    assert mods.cukern.device_error(dev) == 0
    assert rel_err(y, ref) < 2e-3
    yb = mods.cukern.mx_grouped(w.to(dev), s.to(dev), q8, sf, None, None, None, None, None, M, epilogue="bf16", rows_per_tile=64)
    assert yb.dtype == torch.bfloat16 and rel_err(yb, ref) < 1e-2
