"""Whole-layer parity with the CPU oracle on identical seeded inputs: identical top-k expert indices, max relative error
<= 1e-2 on the bf16 output (relative to max |ref|), routing weights to 2e-5."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _layer(mods, dev, E, D, I, topk, seed, kind="e8m0", lo=123, hi=130, limit=10.0, shard=None, bf16_scales=False, engine=0):
    ex = mods.synth.make_experts(E, D, I, seed=seed, scale_lo=lo, scale_hi=hi)
    sh = mods.synth.make_shared(D, I, seed=seed + 1, kind=kind)
    start, n = shard or (0, E)
    sl = slice(start, start + n)
    conv = (lambda t: mods.synth.e8m0_to_bf16(t)) if bf16_scales else (lambda t: t)
    layer = mods.moe.MoELayer(ex["w13"][sl].to(dev), conv(ex["s13"][sl]).to(dev), ex["w2"][sl].to(dev), conv(ex["s2"][sl]).to(dev), n_experts=E, topk=topk,
                              sh_w13=mods.w8.W8(sh["w13"].to(dev), sh["s13"].to(dev)), sh_w2=mods.w8.W8(sh["w2"].to(dev), sh["s2"].to(dev)),
                              swiglu_limit=limit, shard_start=start, engine=engine)
    return ex, sh, layer


def _check(mods, oracle, dev, E, D, I, topk, T, seed, **kw):
    limit = kw.get("limit", 10.0)
    ex, sh, layer = _layer(mods, dev, E, D, I, topk, seed, **kw)
    x = mods.synth.make_tokens(T, D, seed + 2)
    logits = mods.synth.make_logits(T, E, seed + 3, topk=topk)
    ref = oracle.moe_layer(x, logits.float(), None, ex["w13"], ex["s13"], ex["w2"], ex["s2"], (sh["w13"], sh["s13"], sh["w2"], sh["s2"]), topk=topk,
                           limit=limit)
    out, routed, eid, wt = layer.forward(x.to(dev), logits.to(dev), want_routed=True, want_route=True)
    assert torch.equal(eid.cpu(), ref["eid"])
    assert torch.allclose(wt.cpu(), ref["wt"], rtol=2e-5, atol=1e-9)
    assert rel_err(routed, ref["routed"]) <= 1e-2
    assert rel_err(out, ref["out"]) <= 1e-2
    return rel_err(out, ref["out"])


@pytest.mark.parametrize("engine", [1, 2])
@pytest.mark.parametrize("T", [1, 2, 8, 9, 33, 64])
def test_layer_small_dims(mods, oracle, dev, T, engine):
    _check(mods, oracle, dev, E=16, D=512, I=256, topk=4, T=T, seed=10 + T, lo=116, hi=122, engine=engine)
    assert mods.cukern.device_error(dev) == 0


@pytest.mark.parametrize("T", [1, 8])
@pytest.mark.parametrize("setting", ["saturated", "unsaturated", "noclamp", "f32b"])
def test_layer_full_dims(mods, oracle, dev, T, setting):
    """Benchmark shapes (hidden 4096, expert width 2048, top-6 + shared) with 24 resident experts.  'saturated' uses the
    benchmark's scale bytes 123..129, where |gate|,|up| >> limit; 'unsaturated' uses 112..119 so that SiLU is exercised."""
    kw = {"saturated": dict(lo=123, hi=130), "unsaturated": dict(lo=112, hi=120), "noclamp": dict(lo=112, hi=120, limit=0.0),
          "f32b": dict(lo=112, hi=120, kind="f32b")}[setting]
    _check(mods, oracle, dev, E=24, D=4096, I=2048, topk=6, T=T, seed=50 + T, **kw)
    assert mods.cukern.device_error(dev) == 0
    if setting != "f32b":  # the streaming engine on the same inputs
        _check(mods, oracle, dev, E=24, D=4096, I=2048, topk=6, T=T, seed=50 + T, engine=1, **kw)


def test_layer_bf16_scales_equal_e8m0(mods, dev):
    T, E, D, I = 5, 8, 512, 256
    _, _, la = _layer(mods, dev, E, D, I, 3, 7, lo=118, hi=124)
    _, _, lb = _layer(mods, dev, E, D, I, 3, 7, lo=118, hi=124, bf16_scales=True)
    x = mods.synth.make_tokens(T, D, 1).to(dev)
    logits = mods.synth.make_logits(T, E, 2, topk=3).to(dev)
    assert torch.equal(la.forward(x, logits), lb.forward(x, logits))


def test_layer_is_deterministic(mods, dev):
    T, E, D, I = 17, 16, 512, 256
    _, _, layer = _layer(mods, dev, E, D, I, 4, 3, lo=116, hi=122)
    x = mods.synth.make_tokens(T, D, 1).to(dev)
    logits = mods.synth.make_logits(T, E, 2, topk=4).to(dev)
    a = layer.forward(x, logits).clone()
    for _ in range(3):
        assert torch.equal(a, layer.forward(x, logits))


def test_shard_partials_sum_to_full_layer(mods, oracle, dev):
    """Expert-shard contract (dsv41/ep.py:324-338): partial sums of disjoint shards add up to the unsharded routed sum."""
    T, E, D, I, topk = 12, 16, 512, 256, 4
    ex, sh, full = _layer(mods, dev, E, D, I, topk, 21, lo=116, hi=122)
    x = mods.synth.make_tokens(T, D, 22).to(dev)
    logits = mods.synth.make_logits(T, E, 23, topk=topk).to(dev)
    _, routed_full = full.forward(x, logits, want_routed=True)
    acc = torch.zeros_like(routed_full)
    for start, n in mods.ep.shard_ranges(E, 3):
        _, _, part = _layer(mods, dev, E, D, I, topk, 21, lo=116, hi=122, shard=(start, n))
        r = part.forward(x, logits, final=False, want_routed=True)
        ref = oracle.moe_layer(x.cpu(), logits.float().cpu(), None, ex["w13"][start:start + n], ex["s13"][start:start + n], ex["w2"][start:start + n],
                               ex["s2"][start:start + n], None, topk=topk, shard=(start, n), n_experts=E)
        assert rel_err(r, ref["routed"]) <= 1e-2
        acc += r
    assert rel_err(acc, routed_full) < 1e-5


@pytest.mark.parametrize("T", [100, 300, 800])
def test_layer_prefill_sized_batches(mods, oracle, dev, T):
    """More than 64 tokens run on the block-scaled tensor cores; more than 4096 pairs use the multi-block bucketing and the
    per-token accumulator (T = 800, top-6)."""
    topk = 4 if T < 800 else 6
    _check(mods, oracle, dev, E=16, D=512, I=256, topk=topk, T=T, seed=900 + T, lo=116, hi=122)
    assert mods.cukern.device_error(dev) == 0


def test_layer_prefill_shard(mods, oracle, dev):
    T, E, D, I, topk = 900, 16, 512, 256, 6
    ex, sh, part = _layer(mods, dev, E, D, I, topk, 31, lo=116, hi=122, shard=(4, 8))
    x = mods.synth.make_tokens(T, D, 32)
    logits = mods.synth.make_logits(T, E, 33, topk=topk)
    r = part.forward(x.to(dev), logits.to(dev), final=False, want_routed=True)
    ref = oracle.moe_layer(x, logits.float(), None, ex["w13"][4:12], ex["s13"][4:12], ex["w2"][4:12], ex["s2"][4:12], None, topk=topk, shard=(4, 8), n_experts=E)
    assert rel_err(r, ref["routed"]) <= 1e-2
    assert mods.cukern.device_error(dev) == 0


@pytest.mark.parametrize("T,engine", [(7, 1), (7, 2), (200, 0)])
def test_shared_expert_as_separate_output(mods, dev, T, engine):
    # what an expert-parallel caller uses: routed partial sum and the shared expert's own result from the same launches
    E, D, I, topk = 16, 512, 256, 4
    _, _, layer = _layer(mods, dev, E, D, I, topk, 31, engine=engine)
    x = mods.synth.make_tokens(T, D, 33).to(dev)
    logits = mods.synth.make_logits(T, E, 34, topk=topk).to(dev)
    out = layer.forward(x, logits)
    routed, ys = layer.forward(x, logits, final=False, want_routed=True, want_shared=True)
    assert ys.dtype == torch.bfloat16 and ys.shape == (T, D)
    assert torch.equal(mods.fused2.moe_combine(routed.unsqueeze(1), ys), out)
    assert rel_err(ys, layer.shared_expert(x)) < 1e-6
    assert mods.cukern.device_error(dev) == 0


@pytest.mark.parametrize("T,rows", [(300, (128, 75)), (900, (700, 200)), (900, (0, 900)), (40, (8, 8))])
def test_shared_expert_for_a_row_range_only(mods, dev, T, rows):
    # a rank of an expert-parallel group keeps its own token rows of the shared expert's result: those rows are the bits of the
    # full call, the routed sums are untouched
    E, D, I, topk = 16, 512, 256, 4
    _, _, layer = _layer(mods, dev, E, D, I, topk, 31)
    x = mods.synth.make_tokens(T, D, 35).to(dev)
    logits = mods.synth.make_logits(T, E, 36, topk=topk).to(dev)
    routed, ys = layer.forward(x, logits, final=False, want_routed=True, want_shared=True)
    ys2 = torch.full_like(ys, float("nan"))
    routed2 = layer.forward(x, logits, final=False, want_routed=True, want_shared=True, shared_out=ys2, shared_rows=rows)[0]
    a, n = rows
    assert torch.equal(ys2[a:a + n], ys[a:a + n]) and rel_err(routed2, routed) < 1e-5  # (the large batch adds with atomics)
    assert mods.cukern.device_error(dev) == 0
    with pytest.raises(AssertionError):
        layer.forward(x, logits, shared_rows=rows)  # only for calls that do not form the final output


@pytest.mark.parametrize("T", [1, 5, 40, 200])
def test_shard_that_no_token_routes_to(mods, dev, T):
    # a rank whose experts nobody chose: its routed partial sum is exactly zero, the shared expert still comes out right
    E, D, I, topk = 16, 512, 256, 4
    _, _, full = _layer(mods, dev, E, D, I, topk, 31)
    _, _, part = _layer(mods, dev, E, D, I, topk, 31, shard=(12, 4))
    x = mods.synth.make_tokens(T, D, 37).to(dev)
    logits = mods.synth.make_logits(T, E, 38, topk=topk).to(dev)
    logits[:, 12:] = -50.0  # experts 12..15 never make the top 4
    routed, ys = part.forward(x, logits, final=False, want_routed=True, want_shared=True)
    assert torch.count_nonzero(routed) == 0
    _, ys_full = full.forward(x, logits, final=False, want_routed=True, want_shared=True)
    assert torch.equal(ys, ys_full)
    assert mods.cukern.device_error(dev) == 0


def test_expert_parallel_layer_world_of_one_equals_layer(mods, dev):
    # the CUDA defaults of the expert-parallel wrapper (shared expert fused into the local launches) on a one-rank group
    import os
    import torch.distributed as dist
    if dist.is_initialized():
        pytest.skip("a process group already exists in this process")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        E, D, I, topk, T = 16, 512, 256, 4, 12
        _, _, layer = _layer(mods, dev, E, D, I, topk, 41)
        x = mods.synth.make_tokens(T, D, 43).to(dev)
        logits = mods.synth.make_logits(T, E, 44, topk=topk).to(dev)
        got = mods.ep.EPMoE(layer).forward(x, logits)
        assert torch.equal(got, layer.forward(x, logits))
    finally:
        dist.destroy_process_group()


# ------------------------------------------------------------------ edge cases
def test_layer_empty_batch(mods, dev):
    _, _, layer = _layer(mods, dev, 8, 256, 128, 2, 51)
    out = layer.forward(torch.empty(0, 256, dtype=torch.bfloat16, device=dev), torch.empty(0, 8, device=dev))
    assert out.shape == (0, 256)


def _skewed_logits(T, E, hot, topk):
    # every token ranks the `hot` experts first, in the same order: the worst imbalance the router can produce
    lg = torch.full((T, E), -30.0)
    for r, e in enumerate(hot[:topk]):
        lg[:, e] = 10.0 - r
    return lg


@pytest.mark.parametrize("T", [40, 128, 129, 300])
@pytest.mark.parametrize("engine", [0, 1])
def test_layer_all_tokens_on_the_same_experts(mods, oracle, dev, T, engine):
    # groups larger than a work (32 tokens in decode, 128 in prefill), exactly one tile, one tile plus one token
    if engine == 1 and T > 128:
        pytest.skip("the streaming kernels serve decode-sized batches")
    E, D, I, topk = 16, 512, 256, 2
    ex, sh, layer = _layer(mods, dev, E, D, I, topk, 61, engine=engine)
    x = mods.synth.make_tokens(T, D, 63)
    logits = _skewed_logits(T, E, [5, 11], topk)
    ref = oracle.moe_layer(x, logits, None, ex["w13"], ex["s13"], ex["w2"], ex["s2"], (sh["w13"], sh["s13"], sh["w2"], sh["s2"]), topk=topk, limit=10.0)
    out, eid, wt = layer.forward(x.to(dev), logits.to(dev), want_route=True)
    assert torch.equal(eid.cpu(), ref["eid"]) and set(eid.unique().tolist()) == {5, 11}
    assert rel_err(out, ref["out"]) <= 1e-2
    assert mods.cukern.device_error(dev) == 0


def test_layer_largest_router(mods, oracle, dev):
    # 1024 experts and 32 experts per token: the limits of the router and of the bucketing
    E, D, I, topk, T = 1024, 256, 128, 32, 5
    ex, sh, layer = _layer(mods, dev, E, D, I, topk, 71)
    x = mods.synth.make_tokens(T, D, 73)
    logits = mods.synth.make_logits(T, E, 74, topk=topk)
    ref = oracle.moe_layer(x, logits.float(), None, ex["w13"], ex["s13"], ex["w2"], ex["s2"], (sh["w13"], sh["s13"], sh["w2"], sh["s2"]), topk=topk, limit=10.0)
    out, eid, wt = layer.forward(x.to(dev), logits.to(dev), want_route=True)
    assert torch.equal(eid.cpu(), ref["eid"])
    assert torch.allclose(wt.cpu(), ref["wt"], rtol=2e-5, atol=1e-9)
    assert rel_err(out, ref["out"]) <= 1e-2


@pytest.mark.parametrize("engine,T", [(1, 6), (2, 6), (0, 150)])
def test_layer_reads_strided_rows(mods, dev, engine, T):
    # x and the logits as views into wider rows [x | logits], the layout of the packed expert-parallel exchange buffer
    E, D, I, topk = 16, 512, 256, 4
    _, _, layer = _layer(mods, dev, E, D, I, topk, 81, engine=engine)
    x = mods.synth.make_tokens(T, D, 83).to(dev)
    logits = mods.synth.make_logits(T, E, 84, topk=topk).to(dev).float()
    both = torch.zeros(T, D * 2 + E * 4, dtype=torch.uint8, device=dev)
    both[:, :D * 2].view(torch.bfloat16).copy_(x)
    both[:, D * 2:].view(torch.float32).copy_(logits)
    xv, lv = both[:, :D * 2].view(torch.bfloat16), both[:, D * 2:].view(torch.float32)
    assert not xv.is_contiguous() and xv.stride(0) == (D * 2 + E * 4) // 2
    assert torch.equal(layer.forward(xv, lv), layer.forward(x, logits))
    assert mods.cukern.device_error(dev) == 0


@pytest.mark.parametrize("T,use_xf", [(1, False), (5, True), (64, False), (200, True)])
def test_layer_starts_from_hidden_state(mods, dev, T, use_xf):
    # router projection inside the call (gate_w given, no logits) against the same layer fed with logits computed in float64
    E, D, I, topk = 48, 512, 256, 4
    ex, sh, _ = _layer(mods, dev, E, D, I, topk, 91)
    g = torch.Generator().manual_seed(92)
    gate_w = (torch.randn(E, D, generator=g) / D ** 0.5 * 3).float()
    layer = mods.moe.MoELayer(ex["w13"].to(dev), ex["s13"].to(dev), ex["w2"].to(dev), ex["s2"].to(dev), n_experts=E, topk=topk,
                              sh_w13=mods.w8.W8(sh["w13"].to(dev), sh["s13"].to(dev)), sh_w2=mods.w8.W8(sh["w2"].to(dev), sh["s2"].to(dev)),
                              gate_w=gate_w.to(dev))
    x = mods.synth.make_tokens(T, D, 93)
    xf = (x.float() + 1e-3 * torch.randn(T, D, generator=g)) if use_xf else None
    src = xf if use_xf else x.float()
    logits = (src.double() @ gate_w.double().T).float()
    want, eid_w, wt_w = layer.forward(x.to(dev), logits.to(dev), want_route=True)
    got, eid_g, wt_g = layer.forward(x.to(dev), None, xf=xf.to(dev) if use_xf else None, want_route=True)
    assert torch.equal(eid_g, eid_w)
    assert torch.allclose(wt_g, wt_w, rtol=1e-4, atol=1e-7)
    assert rel_err(got, want) < 1e-3
    again = layer.forward(x.to(dev), None, xf=xf.to(dev) if use_xf else None)
    assert torch.equal(again, got)  # the k-split sums are added in a fixed order: same logits, same routing, same output
    assert mods.cukern.device_error(dev) == 0


@pytest.mark.parametrize("with_shared", [True, False])
def test_expert_chain_entry_point(mods, oracle, dev, with_shared):
    """cukern.expert_chain with the reference's argument list (dsv41/cukern.py:504-547): one token, routing given as (eid, wt), one
    shard of the experts -> routed partial sum fp32 [dim] and the shared expert's result bf16 [dim]."""
    from types import SimpleNamespace
    E, D, I, topk, start, n = 16, 512, 256, 4, 4, 8
    ex = mods.synth.make_experts(E, D, I, seed=71, scale_lo=116, scale_hi=122)
    shd = mods.synth.make_shared(D, I, seed=72, kind="e8m0")
    x = mods.synth.make_tokens(1, D, 73)
    logits = mods.synth.make_logits(1, E, 74, topk=topk)
    eid, wt = oracle.gate_topk(logits.float(), None, 1.0, topk, 1.0, "softmax", True)
    xq = oracle.fake_quant_fp8(x, 32)
    sh = {"device": dev, "start": start, "n": n, **{k: ex[k][start:start + n].to(dev) for k in ("w13", "s13", "w2", "s2")}}
    moe = SimpleNamespace(n_experts=E, inter=I, swiglu_limit=10.0, sh_w13=mods.w8.W8(shd["w13"].to(dev), shd["s13"].to(dev)),
                          sh_w2=mods.w8.W8(shd["w2"].to(dev), shd["s2"].to(dev)))
    part = torch.full((D,), float("nan"), device=dev)
    ys = torch.empty(D, device=dev, dtype=torch.bfloat16) if with_shared else None
    xqd = xq[0].to(dev)
    for _ in range(2):  # the second call reuses the cached layer
        mods.cukern.expert_chain(mods.cukern.permute_x(xqd.view(1, -1))[0], xqd, eid[0].to(dev), wt[0].to(dev), (start, n), sh, moe, part, ys)
    assert mods.cukern.device_error(dev) == 0
    fetch = lambda ids: tuple(ex[k][ids] for k in ("w13", "s13", "w2", "s2"))
    ref = oracle.moe_rows(x, eid, wt, fetch, None, 10.0, shard=(start, n))
    assert rel_err(part.view(1, -1), ref["routed"]) <= 2e-3
    if with_shared:
        want = oracle.shared_expert(xq, shd["w13"], shd["s13"], shd["w2"], shd["s2"], 10.0)
        assert rel_err(ys.view(1, -1), want) <= 1e-2
