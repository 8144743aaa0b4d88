"""CPU: the plain-C oracle against the golden vectors produced from the reference (tests/golden/make_golden.py) and, when it
is available, against the reference's own compiled C++ library.  No GPU, no product code."""
import os

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
G = lambda name: torch.load(os.path.join(HERE, "golden", name), weights_only=False)


def _bits(t):
    return t.contiguous().view(torch.int16)


def test_fake_quant_fp8_bit_exact(oracle):
    q = G("quant.pt")
    assert torch.equal(_bits(oracle.fake_quant_fp8(q["x"], 32)), _bits(q["fake_quant_fp8"]))


def test_e2m1_table_and_e8m0():
    q = G("quant.pt")
    assert q["fp4_table"].tolist()[:8] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert q["fp4_table"].tolist()[8:] == [-0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    assert torch.equal(q["e8m0"], torch.exp2(torch.arange(100, 140).float() - 127))
    # ties-to-even examples of dsv41/test_kernels.py:51-54
    assert q["round_e2m1"].tolist() == [1.0, 1.0, 2.0, 2.0, 4.0, 4.0, -0.0, -4.0, 0.0, 6.0]


def test_fp4_gemm_matches_reference_dequant(oracle):
    q = G("quant.pt")
    out = oracle.fp4_gemm(q["a"], q["w4"], q["s4"])
    assert torch.allclose(out, q["fp4_gemm"], rtol=1e-5, atol=1e-5 * q["fp4_gemm"].abs().max().item())
    # the oracle's weight decode equals the reference's dequant_fp4 exactly: probe with one-hot activations
    K = q["w4"].shape[1] * 2
    eye = torch.eye(K).to(torch.bfloat16)
    assert torch.equal(oracle.fp4_gemm(eye, q["w4"], q["s4"]).T.to(torch.bfloat16), q["dequant_fp4"])


def test_fp8_gemm_matches_reference_dequant(oracle):
    q = G("quant.pt")
    out = oracle.fp8_gemm(q["a"][:, :96].contiguous(), q["w8"], q["s8"])
    assert torch.allclose(out, q["fp8_gemm"], rtol=1e-5, atol=1e-5 * q["fp8_gemm"].abs().max().item())
    eye = torch.eye(96).to(torch.bfloat16)
    assert torch.equal(oracle.fp8_gemm(eye, q["w8"], q["s8"]).T.to(torch.bfloat16), q["dequant_fp8_block"])


@pytest.mark.parametrize("func", ["softmax", "sigmoid", "sqrtsoftplus"])
@pytest.mark.parametrize("norm", [True, False])
def test_gate_matches_reference_moe_gate(oracle, func, norm):
    g = G("gate.pt")
    wts, idx = g["gates"][f"{func}_{int(norm)}"]
    eid, wt = oracle.gate_topk(g["scores"], g["bias"], g["temp"], g["topk"], g["route_scale"], func, norm)
    assert torch.equal(eid.long(), idx)
    assert torch.allclose(wt, wts, rtol=2e-5, atol=1e-9)


@pytest.mark.parametrize("limit", [10.0, 0.0])
def test_swiglu_quant_matches_reference_chain(oracle, limit):
    g = G("gate.pt")
    ref_w, ref_n = g["swiglu_quant"][f"w_{limit}"], g["swiglu_quant"][f"n_{limit}"]
    for ref, w in ((ref_w, g["wt"]), (ref_n, None)):
        h = oracle.swiglu_quant(g["gu"], w, 256, limit)
        same = (_bits(h) == _bits(ref)).float().mean().item()
        assert same >= 0.998, same  # (wt*silu)*u vs wt*(silu*u) may differ by one fp32 ulp before the bf16 cast
        assert (h.float() - ref.float()).abs().max() <= 0.07 * ref.float().abs().max()


def _routed(oracle, c, ids, wts, limit):
    import ctypes
    n = len(ids)
    P = ctypes.c_void_p * n
    out = torch.empty(c["w2"].shape[1])
    dim, inter = c["w2"].shape[1], c["w2"].shape[2] * 2
    oracle.lib().orc_routed_token(P(*[c["w13"][e].data_ptr() for e in ids]), P(*[c["s13"][e].data_ptr() for e in ids]), P(*[c["w2"][e].data_ptr() for e in ids]),
                                  P(*[c["s2"][e].data_ptr() for e in ids]), n, ctypes.c_void_p(c["xq"].data_ptr()), (ctypes.c_float * n)(*wts),
                                  ctypes.c_void_p(out.data_ptr()), dim, inter, dim, ctypes.c_float(limit))
    return out


def test_routed_chain_matches_reference_cpu_library_golden(oracle):
    """Stored outputs of the reference's C++ library (exact BF16 mode 0) on dsv41/test_cpumoe.py-style inputs."""
    c = G("cpumoe.pt")
    out = _routed(oracle, c, c["ids"], c["wts"], c["limit"])
    err = ((out - c["mode0"]).abs().max() / c["mode0"].abs().max()).item()
    assert err < 1e-5, err
    out2 = _routed(oracle, c, c["ids"][:2], c["wts"][:2], 0.0)
    err2 = ((out2 - c["mode0_nolimit_2experts"]).abs().max() / c["mode0_nolimit_2experts"].abs().max()).item()
    assert err2 < 1e-5, err2
    # the reference's int8 default (mode 2) is an approximation: it must be close to, but is not, the exact chain
    err_int8 = ((c["mode2"] - c["mode0"]).abs().max() / c["mode0"].abs().max()).item()
    assert 0 < err_int8 < 0.2


def test_routed_chain_matches_live_reference_library(oracle):
    """When the reference's library is built (oracle/_ref) and the host CPU can run it, compare live at another size."""
    try:
        R = oracle.RefCpuMoe(int8_mode=0)
    except RuntimeError as e:
        pytest.skip(str(e))
    g = torch.Generator().manual_seed(3)
    E, inter, dim = 6, 512, 384
    c = {"w13": torch.randint(0, 256, (E, 2 * inter, dim // 2), dtype=torch.uint8, generator=g), "s13": torch.randint(116, 126, (E, 2 * inter, dim // 32), dtype=torch.uint8, generator=g),
         "w2": torch.randint(0, 256, (E, dim, inter // 2), dtype=torch.uint8, generator=g), "s2": torch.randint(116, 126, (E, dim, inter // 32), dtype=torch.uint8, generator=g)}
    c["xq"] = oracle.fake_quant_fp8((torch.randn(1, dim, generator=g) * 2).to(torch.bfloat16), 32)
    ids, wts = [5, 1, 4], [0.5, 0.3, 0.2]
    ref = R.forward(c["xq"][0], c["w13"], c["s13"], c["w2"], c["s2"], ids, wts, 10.0)
    out = _routed(oracle, c, ids, wts, 10.0)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 1e-5


def test_moe_layer_composition(oracle):
    """orc_moe_layer = gate + fake quant + routed chain + shared expert + bf16 combine, composed from the pinned pieces."""
    g = torch.Generator().manual_seed(4)
    E, D, I, T, topk = 8, 256, 256, 3, 2
    w13 = torch.randint(0, 256, (E, 2 * I, D // 2), dtype=torch.uint8, generator=g)
    s13 = torch.randint(118, 124, (E, 2 * I, D // 32), dtype=torch.uint8, generator=g)
    w2 = torch.randint(0, 256, (E, D, I // 2), dtype=torch.uint8, generator=g)
    s2 = torch.randint(118, 124, (E, D, I // 32), dtype=torch.uint8, generator=g)
    sw13 = torch.randint(0, 120, (2 * I, D), dtype=torch.uint8, generator=g)
    ss13 = torch.randint(115, 120, (2 * I // 32, D // 32), dtype=torch.uint8, generator=g)
    sw2 = torch.randint(0, 120, (D, I), dtype=torch.uint8, generator=g)
    ss2 = torch.randint(115, 120, (D // 32, I // 32), dtype=torch.uint8, generator=g)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    r = oracle.moe_layer(x, logits, None, w13, s13, w2, s2, (sw13, ss13, sw2, ss2), topk=topk, limit=10.0)
    eid, wt = oracle.gate_topk(logits, None, 1.0, topk, 1.0, "softmax", True)
    assert torch.equal(eid, r["eid"]) and torch.equal(wt, r["wt"])
    xq = oracle.fake_quant_fp8(x, 32)
    ys = oracle.shared_expert(xq, sw13, ss13, sw2, ss2, 10.0)
    c = {"w13": w13, "s13": s13, "w2": w2, "s2": s2}
    for t in range(T):
        c["xq"] = xq[t:t + 1].contiguous()
        routed = _routed(oracle, c, eid[t].tolist(), wt[t].tolist(), 10.0)
        assert torch.equal(routed, r["routed"][t])
        assert torch.equal((routed + ys[t].float()).to(torch.bfloat16), r["out"][t])
    # shards partition the routed sum
    acc = torch.zeros(T, D)
    for start, n in ((0, 3), (3, 5)):
        acc += oracle.moe_layer(x, logits, None, w13[start:start + n], s13[start:start + n], w2[start:start + n], s2[start:start + n], None, topk=topk,
                                shard=(start, n), n_experts=E)["routed"]
    assert torch.allclose(acc, r["routed"], rtol=1e-6, atol=1e-6 * r["routed"].abs().max().item())


def test_moe_rows_equals_moe_layer(oracle):
    """`moe_rows` (the layer for selected rows with the experts fetched on demand, used at the benchmark's 384-expert size) is the
    same arithmetic as `moe_layer`, bit for bit, with and without a shard."""
    g = torch.Generator().manual_seed(4)
    E, D, I, T, topk = 8, 256, 256, 5, 3
    r8 = lambda lo, hi, *shape: torch.randint(lo, hi, shape, dtype=torch.uint8, generator=g)
    w13, s13, w2, s2 = r8(0, 256, E, 2 * I, D // 2), r8(118, 124, E, 2 * I, D // 32), r8(0, 256, E, D, I // 2), r8(118, 124, E, D, I // 32)
    sh = (r8(0, 120, 2 * I, D), r8(115, 120, 2 * I // 32, D // 32), r8(0, 120, D, I), r8(115, 120, D // 32, I // 32))
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    fetch = lambda ids: (w13[ids], s13[ids], w2[ids], s2[ids])
    full = oracle.moe_layer(x, logits, None, w13, s13, w2, s2, sh, topk=topk, limit=10.0)
    rows = oracle.moe_rows(x, full["eid"], full["wt"], fetch, sh, 10.0)
    assert torch.equal(rows["out"], full["out"]) and torch.equal(rows["routed"], full["routed"])
    part = oracle.moe_layer(x, logits, None, w13[2:5], s13[2:5], w2[2:5], s2[2:5], None, topk=topk, shard=(2, 3), n_experts=E)
    assert torch.equal(oracle.moe_rows(x, full["eid"], full["wt"], fetch, None, 10.0, shard=(2, 3))["routed"], part["routed"])


def test_hc_restatements_basic_properties():
    # dsv41/fused2.py:171-246, 505-558 restated on the CPU: identities that hold whatever the inputs
    import torch
    from oracle import oracle as O
    g = torch.Generator().manual_seed(3)
    B, hc, d = 2, 4, 128
    x = torch.randn(B, hc, d, generator=g).to(torch.bfloat16)
    w = torch.ones(d, dtype=torch.bfloat16)
    pre = torch.zeros(B, hc)
    pre[:, 2] = 1.0  # the pre-mix picks copy 2: y = rmsnorm(x[:, 2])
    y, yq, yqp = O.hc_pre_norm_quant2(x, pre, w, 0.0)
    t = x[:, 2].float()
    want = (t / t.pow(2).mean(dim=1, keepdim=True).sqrt()).to(torch.bfloat16)
    assert (y.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
    assert torch.equal(yq.view(torch.int16), O.fake_quant_fp8(y, 32).view(torch.int16))
    perm = [0, 4, 2, 6, 1, 5, 3, 7]
    assert all(torch.equal(yqp[:, j], yq[:, perm[j]]) for j in range(8))
    # post mix with post = 0 and comb = identity leaves the residual alone; with comb = 0 it broadcasts post * v
    eye = torch.eye(hc).repeat(B, 1, 1)
    assert torch.equal(O.hc_post2(x, torch.zeros(B, hc), eye, x=y), x)
    out = O.hc_post2(x, torch.ones(B, hc), torch.zeros(B, hc, hc), x=y)
    assert all(torch.equal(out[:, i], y) for i in range(hc))
    y2 = torch.randn(B, 3, d, generator=g)
    v = (y2.sum(dim=1) + y.float()).to(torch.bfloat16)
    assert (O.hc_post2(x, torch.ones(B, hc), torch.zeros(B, hc, hc), y2=y2, ys=y)[:, 0].float() - v.float()).abs().max() <= 2 ** -7 * v.float().abs().max()


def _bit_equal_share(a, b):
    return (a.view(torch.int16) == b.view(torch.int16)).float().mean().item()


def test_hc_restatements_match_the_reference_triton_kernels(oracle):
    """tests/golden/hc.pt holds outputs of the reference's own hc_pre_norm_quant2 / hc_post2_ (dsv41/fused2.py:213-246, 539-558) run on a
    B200 (tests/golden/make_hc_golden.py).  The pre-mix + rmsnorm + quantisation restatement reproduces them bit for bit; the post mix
    differs in isolated elements by a bf16 rounding (Triton contracts the multiply-adds of the mix)."""
    gold = G("hc.pt")
    for name, c in gold["cases"].items():
        y, yq, yqp = oracle.hc_pre_norm_quant2(c["x"][:, 0], c["pre"], c["w"], c["eps"])
        assert torch.equal(y, c["y"]) and torch.equal(yq, c["yq"]) and torch.equal(yqp, c["yqp"]), name
        assert torch.equal(c["yf"], c["y"].float())
        for got, want in ((oracle.hc_post2(c["res"][:, 0], c["post"], c["comb"], x=c["xin"]), c["res_after_x"][:, 0]),
                          (oracle.hc_post2(c["res"][:, 0], c["post"], c["comb"], y2=c["y2"], ys=c["ys"]), c["res_after_moe"][:, 0])):
            assert _bit_equal_share(got, want) >= 0.999, name
            assert ((got.float() - want.float()).abs().max() / want.float().abs().max()).item() < 4e-3, name  # at most one bf16 rounding of the largest element


def test_swiglu_and_gate_match_the_reference_triton_kernels(oracle):
    """Second pin of two steps on the path against the reference's Triton kernels (fused.swiglu_quant, fused2.gate_topk) run on a B200:
    expert indices identical, routing weights to 1e-6; SwiGLU bit-equal except where tl.sigmoid and 1 / (1 + exp(-g)) round apart (the
    difference the reference itself accepts between its Triton and CUDA / C++ forms, results/expert_chain_report.md:81-83)."""
    e = G("hc.pt")["extra"]
    for limit in (10.0, 0.0):
        h = oracle.swiglu_quant(e["gu"], e["wts"], e["inter"], limit)
        want = e[f"swiglu_limit{limit}"]
        assert _bit_equal_share(h, want) >= 0.995
        assert ((h.float() - want.float()).abs().max() / want.float().abs().max()).item() < 0.07  # a flipped e4m3 rounding at most
    for func in ("softmax", "sigmoid", "sqrtsoftplus"):
        eid, wt = oracle.gate_topk(e["scores"], e["bias"], 1.0, 6, 2.5, func, True)
        assert torch.equal(eid, e[f"gate_{func}"][0])
        assert torch.allclose(wt, e[f"gate_{func}"][1], rtol=2e-6, atol=1e-8)
