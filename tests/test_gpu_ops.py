"""Parity of every CUDA operator with the CPU oracle, through the C-ABI (the Python modules only marshal pointers).
Sizes are chosen so the scalar oracle finishes in seconds.  Tolerances are the reference's own (dsv41/test_kernels.py:18-19,
dsv41/test_fused.py:81-88, dsv41/test_fused2_units.py:69-75)."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.contiguous().view(torch.int16)


def test_fake_quant_fp8_exact(mods, oracle, dev):
    torch.manual_seed(0)
    x = (torch.randn(3, 7, 4096) * 4).to(torch.bfloat16)
    x[0, 0, :32] = 0
    x[0, 1, :64] *= 1e-6
    x[0, 2, :64] *= 3000
    x[1, 0, 5] = 448 * 4
    y = mods.fused.fake_quant_fp8(x.to(dev), 32).cpu()
    ref = oracle.fake_quant_fp8(x, 32)
    assert torch.equal(_bits(y), _bits(ref))
    y2 = mods.quant.fake_quant_fp8(x.to(dev), 32).cpu()
    assert torch.equal(_bits(y2), _bits(ref))


@pytest.mark.parametrize("score_func", ["sqrtsoftplus", "sigmoid", "softmax"])
@pytest.mark.parametrize("B,E,topk", [(1, 384, 6), (5, 384, 6), (64, 384, 6), (3, 8, 2), (2, 1000, 8)])
def test_gate_topk(mods, oracle, dev, score_func, B, E, topk):
    g = torch.Generator().manual_seed(B * 1000 + E)
    sc = torch.randn(B, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.1
    e_ref, w_ref = oracle.gate_topk(sc, bias, 1.3, topk, 2.5, score_func, True)
    eid, wt = mods.fused2.gate_topk(sc.to(dev), bias.to(dev), 1.3, topk, 2.5, score_func, True)
    if B == 1:
        assert eid.shape == (topk,) and wt.shape == (topk,)
        eid, wt = eid.view(1, -1), wt.view(1, -1)
    assert torch.equal(eid.cpu(), e_ref)
    assert torch.allclose(wt.cpu(), w_ref, rtol=2e-5, atol=1e-9)
    # no renormalisation, no bias, preallocated outputs
    e_ref, w_ref = oracle.gate_topk(sc, None, 1.0, topk, 1.0, score_func, False)
    eo = torch.empty(B, topk, dtype=torch.int32, device=dev)
    wo = torch.empty(B, topk, dtype=torch.float32, device=dev)
    mods.fused2.gate_topk(sc.to(dev), None, 1.0, topk, 1.0, score_func, False, eid=eo, wt=wo)
    assert torch.equal(eo.cpu(), e_ref) and torch.allclose(wo.cpu(), w_ref, rtol=2e-5, atol=1e-9)


def test_gate_topk_tie_lowest_index(mods, dev):
    sc = torch.zeros(2, 384)
    sc[1, 100:110] = 1.0
    eid, _ = mods.fused2.gate_topk(sc.to(dev), torch.zeros(384, device=dev), 1.0, 6, 1.0, "softmax", True)
    assert eid.cpu().tolist() == [[0, 1, 2, 3, 4, 5], [100, 101, 102, 103, 104, 105]]


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("limit", [10.0, 0.0])
def test_swiglu_quant(mods, oracle, dev, in_dtype, limit):
    torch.manual_seed(1)
    inter = 2304
    gu = (torch.randn(9, 2 * inter) * 5).to(in_dtype)
    wt = torch.rand(9)
    for w in (wt, None):
        ref = oracle.swiglu_quant(gu.float(), w, inter, limit)
        y = mods.fused.swiglu_quant(gu.to(dev), w.to(dev) if w is not None else None, inter, limit).cpu()
        same = (_bits(y) == _bits(ref)).float().mean().item()
        assert same >= 0.999, same  # expf rounding may flip a bf16 boundary on isolated elements
        assert (y.float() - ref.float()).abs().max().item() <= 0.07 * ref.float().abs().max().item()
    yp = mods.fused.swiglu_quant(gu.to(dev), wt.to(dev), inter, limit, permute=True)
    y0 = mods.fused.swiglu_quant(gu.to(dev), wt.to(dev), inter, limit)
    assert torch.equal(yp, mods.cukern.permute_x(y0))


def test_permute_x(mods, dev):
    x = torch.arange(64, dtype=torch.float32).view(2, 32).to(torch.bfloat16)
    y = mods.cukern.permute_x(x.to(dev)).cpu()
    ref = x.view(2, 4, 8)[:, :, [0, 4, 2, 6, 1, 5, 3, 7]].reshape(2, 32)
    assert torch.equal(y, ref)


@pytest.mark.parametrize("M,N,K", [(1, 2304, 5120), (7, 5120, 2304), (64, 2304, 5120), (20, 4096, 2048), (3, 64, 128), (9, 48, 512)])
def test_fp4_gemm(mods, oracle, dev, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    s = torch.randint(110, 135, (N, K // 32), dtype=torch.uint8, generator=g)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = oracle.fp4_gemm(a, w, s)
    out = mods.kernels.fp4_gemm(a.to(dev), w.to(dev), s.to(dev))
    assert out.dtype == torch.float32 and out.shape == (M, N)
    assert rel_err(out, ref) < 2e-3


def test_fp4_scale_byte_zero_and_bf16_scales(mods, oracle, dev):
    g = torch.Generator().manual_seed(5)
    N, K, M = 64, 512, 3
    w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    s = torch.randint(120, 130, (N, K // 32), dtype=torch.uint8, generator=g)
    s[::3, ::2] = 0  # byte 0 decodes to 0 (dsv41/cpu/moe_cpu.cpp:190)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = oracle.fp4_gemm(a, w, s)
    out = mods.kernels.fp4_gemm(a.to(dev), w.to(dev), s.to(dev))
    assert rel_err(out, ref) < 2e-3
    s2 = torch.randint(120, 130, (N, K // 32), dtype=torch.uint8, generator=g)
    ref2 = oracle.fp4_gemm(a, w, s2)
    ge = torch.zeros(1, dtype=torch.int32, device=dev)
    gs = torch.tensor([0, M], dtype=torch.int32, device=dev)
    out2 = mods.cukern.grouped_fp4(a.to(dev), w.to(dev).unsqueeze(0), mods.synth.e8m0_to_bf16(s2).to(dev).unsqueeze(0), ge, gs, None, None, None, None, M)
    assert rel_err(out2, ref2) < 2e-3


def _experts(E, N, K, seed, lo=110, hi=135):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 256, (E, N, K // 2), dtype=torch.uint8, generator=g), torch.randint(lo, hi, (E, N, K // 32), dtype=torch.uint8, generator=g), g)


def test_fp4_gemv_pairs(mods, oracle, dev):
    E, N, K = 6, 512, 1024
    w, s, g = _experts(E, N, K, 11)
    x = torch.randn(4, K, generator=g).to(torch.bfloat16)
    P = 13
    row_in = torch.randint(0, 4, (P,), generator=g, dtype=torch.int32)
    expert = torch.randint(0, E, (P,), generator=g, dtype=torch.int32)
    wt = torch.rand(P, generator=g)
    ref = oracle.fp4_pairs(x, w, s, expert, row_in, torch.arange(P), wt, P)
    out = mods.cukern.fp4_gemv_pairs(x.to(dev), w.to(dev), s.to(dev), row_in.to(dev), expert.to(dev), wt.to(dev), P)
    assert rel_err(out, ref) < 2e-3


@pytest.mark.parametrize("G,M", [(1, 1), (1, 8), (1, 16), (6, 1), (6, 4), (3, 21)])
def test_fp4_gemm_tc_groups_and_shards(mods, oracle, dev, G, M):
    """Grouped form of dsv41/test_fp4_tc.py:31-41 plus the shard rule: foreign groups are skipped, zero_out zeroes their rows."""
    E, N, K = 8, 256, 1024
    w, s, g = _experts(E, N, K, 100 + G * 10 + M, 112, 128)
    x = oracle.fake_quant_fp8((torch.randn(M, K, generator=g) * 2).to(torch.bfloat16), 32)
    xp = mods.cukern.permute_x(x.to(dev))
    experts = torch.arange(G, dtype=torch.int32)
    grp_start = torch.arange(0, G * M + 1, M, dtype=torch.int32)
    pair_tok = torch.arange(M, dtype=torch.int32).repeat(G)
    P = G * M
    ref = oracle.fp4_pairs(x, w, s, experts.repeat_interleave(M), pair_tok, torch.arange(P), None, P)
    y = mods.cukern.fp4_gemm_tc(xp, w.to(dev), s.to(dev), experts.to(dev), grp_start.to(dev), pair_tok.to(dev), P, M)
    assert rel_err(y, ref) < 2e-3
    if G > 1:  # this GPU holds experts [2, 5): local tensors are w[2:5]
        out = torch.full((P, N), 7.0, device=dev)
        y = mods.cukern.fp4_gemm_tc(xp, w[2:5].to(dev), s[2:5].to(dev), experts.to(dev), grp_start.to(dev), pair_tok.to(dev), P, M, shard_start=2, shard_n=3,
                                    zero_out=True, out=out)
        mask = ((experts >= 2) & (experts < 5)).repeat_interleave(M)
        ref_sh = ref * mask[:, None]
        assert rel_err(y, ref_sh) < 2e-3
        assert (y.cpu()[~mask] == 0).all()
        out = torch.full((P, N), 7.0, device=dev)
        y = mods.cukern.fp4_gemm_tc(xp, w[2:5].to(dev), s[2:5].to(dev), experts.to(dev), grp_start.to(dev), pair_tok.to(dev), P, M, shard_start=2, shard_n=3,
                                    zero_out=False, out=out)
        assert (y.cpu()[~mask] == 7.0).all()


def test_grouped_pairs_matches_oracle_grouping(mods, oracle, dev):
    """The device bucketing against the checker's stable grouping: same order, same tiles (in expert order, at most block_m pairs each;
    the unused capacity of the tables carries expert -1 / count 0), ids outside the expert range dropped, make_p2 keeps the buckets."""
    g = torch.Generator().manual_seed(0)
    for n_pairs, E, bm in ((10, 16, 16), (400, 16, 64), (1000, 384, 64), (24576, 384, 64)):
        eid = torch.randint(0, E, (n_pairs,), generator=g)
        row = torch.randint(0, 1000, (n_pairs,), generator=g)
        wt = torch.rand(n_pairs, generator=g)
        gp = mods.moe_kernels.GroupedPairs(eid.to(dev), row.to(dev), row.clone().to(dev), wt.to(dev), bm, n_experts=E)
        assert gp.n_pairs == n_pairs and gp.block_m == bm
        order, counts = oracle.group_pairs(eid, E)
        assert torch.equal(gp.order.cpu(), order)
        assert torch.equal(gp.expert.cpu(), eid[order.long()].int())
        assert torch.equal(gp.row_in.cpu(), row[order.long()].int()) and torch.equal(gp.weight.cpu(), wt[order.long()])
        exp_tiles, start = [], 0
        for e in range(E):
            c = int(counts[e])
            for t0 in range(0, c, bm):
                exp_tiles.append((e, start + t0, min(bm, c - t0)))
            start += c
        n = int(gp.n_tiles.item())
        got = list(zip(gp.tile_expert.tolist(), gp.tile_start.tolist(), gp.tile_count.tolist()))
        assert n == len(exp_tiles) and got[:n] == exp_tiles
        assert all(t == (-1, 0, 0) for t in got[n:])
        row2 = torch.randint(0, 50, (n_pairs,), generator=g)
        p2 = gp.make_p2(row2.to(dev), row.to(dev), None)
        assert torch.equal(p2.row_in.cpu(), row2[order.long()].int()) and p2.tile_start is gp.tile_start and p2.weight is gp.weight
        w2 = torch.rand(n_pairs, generator=g)
        assert torch.equal(gp.make_p2(row.to(dev), row.to(dev), w2.to(dev)).weight.cpu(), w2[order.long()])
    # ids outside [0, E) are dropped
    eid = torch.tensor([3, -1, 2, 3, 99, 0])
    gp = mods.moe_kernels.GroupedPairs(eid.to(dev), torch.arange(6).to(dev), torch.arange(6).to(dev), torch.ones(6).to(dev), 4, n_experts=8)
    assert gp.order.cpu().tolist()[:4] == [5, 2, 0, 3] and int(gp.tile_count.sum()) == 4


def test_grouped_fp4_shard_zero_out_with_permuted_output_rows(mods, oracle, dev):
    """zero_out clears the rows the foreign pairs WRITE (pair_out), not the rows at their positions, and never a row beyond the
    output: output rows = tokens here (fewer than pairs), several pairs of a token would share a row, so each pair gets its own
    slot of a [T * topk] buffer addressed through pair_out."""
    E, N, K, T, topk = 8, 256, 512, 5, 3
    w, s, g = _experts(E, N, K, 321, 112, 128)
    x = oracle.fake_quant_fp8((torch.randn(T, K, generator=g) * 2).to(torch.bfloat16), 32)
    eid = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)])
    order = torch.argsort(eid.flatten(), stable=True)
    experts, counts = torch.unique(eid.flatten()[order], return_counts=True)
    grp_start = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)]).int()
    pair_tok, pair_out = (order // topk).int(), order.int()   # sorted position -> token row, -> original slot t * topk + j
    P = T * topk
    ref = oracle.fp4_pairs(x, w, s, eid.flatten()[order], pair_tok, pair_out, None, P)
    local = ((eid.flatten() >= 2) & (eid.flatten() < 5))     # by original slot
    for zero_out, fill in ((True, 0.0), (False, 7.0)):
        out = torch.full((P, N), 7.0, device=dev)
        y = mods.cukern.grouped_fp4(x.to(dev), w[2:5].to(dev), s[2:5].to(dev), experts.int().to(dev), grp_start.to(dev), None, pair_tok.to(dev), pair_out.to(dev),
                                    None, P, shard_start=2, shard_n=3, zero_out=zero_out, out=out).cpu()
        assert rel_err(y[local], ref[local]) < 2e-3
        assert (y[~local] == fill).all()
    assert mods.cukern.device_error(dev) == 0


@pytest.mark.parametrize("M,topk", [(1, 6), (5, 6), (64, 6), (100, 6)])
def test_grouped_fp4_gemm_scatter_add(mods, oracle, dev, M, topk):
    """dsv41/test_moe.py:21-36 at reduced size: out[row_out] += weight * a[row_in] @ W[expert]^T."""
    E, N, K = 16, 256, 512
    w, s, g = _experts(E, N, K, 200 + M)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    eid = torch.randint(0, E, (M, topk), generator=g)
    wt = torch.rand(M, topk, generator=g)
    row_in = torch.arange(M).repeat_interleave(topk)
    ref = oracle.fp4_pairs(a, w, s, eid.flatten(), row_in, row_in, wt.flatten(), M)
    pairs = mods.moe_kernels.GroupedPairs(eid.flatten().to(dev), row_in.to(dev), row_in.clone().to(dev), wt.flatten().to(dev), block_m=16 if M <= 16 else 64,
                                          n_experts=E)
    out = mods.moe_kernels.grouped_fp4_gemm(a.to(dev), w.to(dev), s.to(dev), pairs, M)
    assert rel_err(out, ref) < 2e-3
    out2 = mods.moe_kernels.grouped_fp4_gemm_chunked(a.to(dev), w.to(dev), s.to(dev), pairs, M, chunk_rows=32)
    assert rel_err(out2, ref) < 2e-3


def _rand_fp8(N, K, g, lo=110, hi=130):
    w = torch.randint(0, 256, (N, K), dtype=torch.uint8, generator=g)
    w[(w & 0x7F) == 0x7F] = 0  # no NaN codes (dsv41/test_fp8_tc.py:12-16)
    s = torch.randint(lo, hi, ((N + 31) // 32, K // 32), dtype=torch.uint8, generator=g)
    return w, s


@pytest.mark.parametrize("M,N,K", [(1, 512, 5120), (1, 1280, 5120), (6, 5120, 8192), (16, 4608, 5120), (1, 5120, 2304), (3, 4096, 1280), (8, 64, 64)])
def test_fp8_gemm_e8m0(mods, oracle, dev, M, N, K):
    g = torch.Generator().manual_seed(N + K + M)
    w, s = _rand_fp8(N, K, g)
    x = oracle.fake_quant_fp8((torch.randn(M, K, generator=g) * 2).to(torch.bfloat16), 32)
    ref = oracle.fp8_gemm(x, w, s)
    y = mods.cukern.fp8_gemm_tc(x.to(dev), mods.w8.permute_k(w).to(dev), s.to(dev), out_dtype=torch.float32)
    assert rel_err(y, ref) < 2e-3
    yb = mods.cukern.fp8_gemm_tc(x.to(dev), mods.w8.permute_k(w).to(dev), s.to(dev))
    assert yb.dtype == torch.bfloat16 and rel_err(yb, ref) < 1e-2
    if M == 1:
        y1 = mods.cukern.fp8_gemv(x.to(dev), w.to(dev), s.to(dev))
        assert y1.dtype == torch.float32 and rel_err(y1, ref) < 2e-3
        y2 = mods.cukern.fp8_gemv_m1(x.to(dev), mods.w8.permute_k(w).to(dev), s.to(dev))
        assert y2.dtype == torch.bfloat16 and rel_err(y2, ref) < 1e-2
    W = mods.w8.W8(w.to(dev), s.to(dev))
    yl = mods.w8.linear_w(x.to(dev), W)
    assert rel_err(yl, ref) < 1e-2
    assert rel_err(yl, torch.nn.functional.linear(x.to(dev), W.bf16())) < 1e-2


@pytest.mark.parametrize("M", [1, 2, 4, 8])
@pytest.mark.parametrize("N", [4096, 12288, 18432])
def test_fp8_gemv_f32_block_scales(mods, oracle, dev, M, N):
    """The 128x128 fp32-scaled format: weights N(0, 0.02) quantised per block with scale = blockmax/448."""
    K = 4096
    g = torch.Generator().manual_seed(N + M)
    wf = torch.randn(N, K, generator=g) * 0.02
    codes, scale = mods.synth.quantize_fp8_block(wf, "f32b")
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = oracle.fp8_gemm(x, codes, scale)
    y = mods.cukern.fp8_gemm_tc(x.to(dev), codes.to(dev), scale.to(dev), out_dtype=torch.float32, permuted=False)
    assert rel_err(y, ref) < 2e-3
    # the quantised matrix stays close to the fp32 one
    assert rel_err(ref, x.float() @ wf.T) < 0.1
    W = mods.w8.W8(codes.to(dev), scale.to(dev))
    assert rel_err(mods.w8.linear_w(x.to(dev), W), ref) < 1e-2


@pytest.mark.parametrize("M", [1, 2, 4, 8])
@pytest.mark.parametrize("N", [4096, 12288, 18432])
def test_fp8_gemv_e8m0_block_scales_at_benchmark_shapes(mods, oracle, dev, M, N):
    """The same N(0, 0.02) weights in the reference's own format (E8M0 per 32x32, scale 2^ceil(log2(blockmax/448))), K = 4096."""
    K = 4096
    g = torch.Generator().manual_seed(3 * N + M)
    codes, scale = mods.synth.quantize_fp8_block(torch.randn(N, K, generator=g) * 0.02, "e8m0")
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = oracle.fp8_gemm(x, codes, scale)
    y = mods.cukern.fp8_gemm_tc(x.to(dev), codes.to(dev), scale.to(dev), out_dtype=torch.float32, permuted=False)
    assert rel_err(y, ref) < 2e-3
    W = mods.w8.W8(codes.to(dev), scale.to(dev))
    assert rel_err(mods.w8.linear_w(x.to(dev), W), ref) < 1e-2


def test_p2p_sum_rows(mods, dev):
    src = torch.randn(3 * 6, 500, device=dev)
    dst = torch.zeros(3, 512, device=dev)
    mods.cukern.p2p_sum_rows(dst, src, dev, groups=3)
    assert torch.allclose(dst[:, :500], src.view(3, 6, 500).sum(1), atol=1e-5)


@pytest.mark.parametrize("dual", [True, False])
def test_scale_atoms_are_a_pure_relayout(mods, dev, dual):
    """The load-time re-layout of the scales (b200_scale_atoms): every byte of the result is the byte of the checkpoint-order tensor that the
    documented layout names; rows past the matrix read as 127 (scale 1)."""
    g = torch.Generator().manual_seed(9)
    E, K = 3, 512
    N = 2 * 160 if dual else 400     # inter = 160: the second tile of a gate | up matrix is ragged; 400 rows: the second 256-row tile is ragged
    s = torch.randint(1, 255, (E, N, K // 32), dtype=torch.uint8, generator=g)
    atoms = mods.cukern.scale_atoms(s.to(dev), N, K, dual).cpu()      # [E, tiles, K/128, 2, 512]
    tiles = atoms.shape[1]
    assert tiles == 2 and atoms.shape[2] == K // 128
    inter = N // 2
    for e in range(E):
        for t in range(tiles):
            for rb in range(2):
                for r in (0, 31, 32, 77, 127):
                    row, ok = ((rb * inter + t * 128 + r), t * 128 + r < inter) if dual else ((t * 256 + rb * 128 + r), t * 256 + rb * 128 + r < N)
                    for kb in range(K // 128):
                        got = atoms[e, t, kb, rb, (r % 32) * 16 + (r // 32) * 4:(r % 32) * 16 + (r // 32) * 4 + 4]
                        want = s[e, row, kb * 4:kb * 4 + 4] if ok else torch.full((4,), 127, dtype=torch.uint8)
                        assert torch.equal(got, want), (e, t, rb, r, kb)
    # the dense FP8 format (one scale per 32 rows x 32 k) expands every scale row to its 32 weight rows
    s8 = torch.randint(1, 255, ((N + 31) // 32, K // 32), dtype=torch.uint8, generator=g)
    a8 = mods.cukern.scale_atoms(s8.to(dev), N, K, dual).cpu()
    r = 45
    row = r if not dual else r
    assert torch.equal(a8[0, 0, 1, 0, (r % 32) * 16 + (r // 32) * 4:(r % 32) * 16 + (r // 32) * 4 + 4], s8[row // 32, 4:8])


def test_loader_relayout_and_layer_from_shard(mods, oracle, dev):
    """Loader end to end on the device: checkpoint-style tensors -> shard dict -> scale atoms -> layer; the layer's output matches the
    checker on the same weights."""
    import importlib
    load = importlib.import_module("dsv41_b200.load")
    E, D, I, topk, T = 8, 512, 256, 2, 5
    ex = mods.synth.make_experts(E, D, I, seed=5, scale_lo=116, scale_hi=122)
    ck = {}
    for e in range(E):
        q = f"layers.0.ffn.experts.{e}."
        ck[q + "w1.weight"], ck[q + "w3.weight"] = ex["w13"][e, :I], ex["w13"][e, I:]
        ck[q + "w1.scale"], ck[q + "w3.scale"] = ex["s13"][e, :I], ex["s13"][e, I:]
        ck[q + "w2.weight"], ck[q + "w2.scale"] = ex["w2"][e], ex["s2"][e]
    shard = load.relayout_scales(load.stack_experts(ck, "layers.0.", 2, 4, dev))
    assert torch.equal(shard["w13"].cpu(), ex["w13"][2:6]) and shard["s13_atoms"].shape[:3] == (4, I // 128, D // 128)
    layer = load.layer_from_shard(shard, E, topk=topk, swiglu_limit=10.0)
    x = mods.synth.make_tokens(T, D, 6)
    logits = mods.synth.make_logits(T, E, 7, topk=topk)
    routed = layer.forward(x.to(dev), logits.to(dev), final=False, want_routed=True)
    ref = oracle.moe_layer(x, logits.float(), None, ex["w13"][2:6], ex["s13"][2:6], ex["w2"][2:6], ex["s2"][2:6], None, topk=topk, shard=(2, 4), n_experts=E)
    assert rel_err(routed, ref["routed"]) <= 2e-3


@pytest.mark.parametrize("exact", [True, False])
def test_reference_named_launchers_choose_the_engine_on_the_device(mods, oracle, dev, exact):
    """grouped_fp4_gemm / fp4_gemm_tc / linear_w with an FP8-exact activation run the tcgen05 kernels, with any other bf16 activation the
    streaming kernels; both match the checker, and an inexact activation gives the streaming kernels' bits."""
    ck = mods.cukern
    E, N, K, M, topk = 8, 512, 1024, 300, 2
    w, s, g = _experts(E, N, K, 555, 112, 128)
    a = (torch.randn(M, K, generator=g) * 2).to(torch.bfloat16)
    if exact:
        a = oracle.fake_quant_fp8(a, 32)
    eid = torch.randint(0, E, (M, topk), generator=g)
    wt = torch.rand(M, topk, generator=g)
    row = torch.arange(M).repeat_interleave(topk)
    ref = oracle.fp4_pairs(a, w, s, eid.flatten(), row, row, wt.flatten(), M)
    pairs = mods.moe_kernels.GroupedPairs(eid.flatten().to(dev), row.to(dev), row.clone().to(dev), wt.flatten().to(dev), block_m=64, n_experts=E)
    got = mods.moe_kernels.grouped_fp4_gemm(a.to(dev), w.to(dev), s.to(dev), pairs, M)
    assert rel_err(got, ref) < 2e-3 and ck.device_error(dev) == 0
    ck.AUTO_ENGINE = False
    try:
        streaming = mods.moe_kernels.grouped_fp4_gemm(a.to(dev), w.to(dev), s.to(dev), pairs, M)
    finally:
        ck.AUTO_ENGINE = True
    assert rel_err(streaming, ref) < 2e-3
    # 8-k permuted activation (fp4_gemm_tc): one group per expert
    order = torch.argsort(eid[:, 0], stable=True)
    experts, counts = torch.unique(eid[order, 0], return_counts=True)
    gs = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)]).int()
    ref_tc = oracle.fp4_pairs(a, w, s, eid[order, 0], order, torch.arange(M), None, M)
    y = ck.fp4_gemm_tc(ck.permute_x(a.to(dev)), w.to(dev), s.to(dev), experts.int().to(dev), gs.to(dev), order.int().to(dev), M, 64)
    assert rel_err(y, ref_tc) < 2e-3
    # dense FP8, more than 8 rows
    w8, s8 = _rand_fp8(768, K, g)
    W = mods.w8.W8(w8.to(dev), s8.to(dev))
    ref8 = oracle.fp8_gemm(a, w8, s8)
    y8 = mods.w8.linear_w(a.to(dev), W)
    assert y8.shape == (M, 768) and rel_err(y8, ref8) < 1e-2
    ck.AUTO_ENGINE = False
    try:
        y8s = mods.w8.linear_w(a.to(dev), W)
    finally:
        ck.AUTO_ENGINE = True
    if not exact:  # nothing but the streaming kernel may have written the result
        assert torch.equal(got, streaming) and torch.equal(y8, y8s)
    assert ck.device_error(dev) == 0
