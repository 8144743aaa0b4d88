"""The steps either side of the MoE path (hyper-connection pre-mix + rmsnorm + FP8 fake quantisation, and the post mix that consumes
the layer's outputs) through the C ABI, against the CPU restatement of dsv41/fused2.py:171-246 and 505-558 and against
tests/golden/hc.pt, the outputs of the reference's own Triton kernels on a B200 (tests/golden/make_hc_golden.py)."""
import os
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _inputs(B, hc, d, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, 1, hc, d, generator=g).to(torch.bfloat16)
    pre = torch.rand(B, hc, generator=g) + 0.1
    w = (torch.rand(d, generator=g) + 0.5).to(torch.bfloat16)
    return g, x, pre, w


@pytest.mark.parametrize("B,d", [(1, 4096), (3, 512), (5, 2080)])
def test_hc_pre_norm_quant2(mods, oracle, dev, B, d):
    hc = 4
    g, x, pre, w = _inputs(B, hc, d, 7 * B + d)
    y_ref, yq_ref, yqp_ref = oracle.hc_pre_norm_quant2(x.view(B, hc, d), pre, w, 1e-6)
    y, yq, yf, yqp = mods.fused2.hc_pre_norm_quant2(x.to(dev), pre.to(dev), w.to(dev), 1e-6, want_f32=True, want_perm=True)
    # the row variance is a sum of d squares in another order: y may differ from the restatement by a bf16 rounding here and there
    assert rel_err(y, y_ref) < 1e-2 and (y.cpu() != y_ref).float().mean() < 0.01
    assert torch.equal(yf.cpu(), y.cpu().float())
    # the quantised copies are exact functions of y: checked bit for bit against the oracle applied to the kernel's own y
    assert torch.equal(yq.cpu().view(torch.int16), oracle.fake_quant_fp8(y.cpu(), 32).view(torch.int16))
    assert torch.equal(yqp.cpu(), mods.cukern.permute_x(yq).cpu())
    assert rel_err(yq, yq_ref) < 3e-2 and rel_err(yqp, yqp_ref) < 3e-2
    y2, yq2, yf2 = mods.fused2.hc_pre_norm_quant2(x.to(dev), pre.to(dev), w.float().to(dev), 1e-6)  # fp32 norm weight, no extras
    assert yf2 is None and torch.equal(y2, y) and torch.equal(yq2, yq)


@pytest.mark.parametrize("B,d,nsum", [(1, 4096, 6), (4, 512, 2), (2, 1024, 0)])
def test_hc_post2(mods, oracle, dev, B, d, nsum):
    hc = 4
    g, x, _, _ = _inputs(B, hc, d, 11 * B + d)
    res = x.view(B, hc, d).clone()
    post = torch.rand(B, hc, generator=g)
    comb = torch.rand(B, hc, hc, generator=g) - 0.3
    if nsum:
        y2 = torch.randn(B, nsum, d, generator=g)
        ys = torch.randn(B, d, generator=g).to(torch.bfloat16)
        ref = oracle.hc_post2(res, post, comb, y2=y2, ys=ys)
        r = x.clone().to(dev)
        out = mods.fused2.hc_post2_(None, r, post.to(dev), comb.to(dev), y2=y2.to(dev), ys=ys.to(dev))
        assert out.data_ptr() == r.data_ptr()  # in place
        # the layout with the sum index first (dsv41/fused2.py:549-551)
        r2 = x.clone().to(dev)
        mods.fused2.hc_post2_(None, r2, post.to(dev), comb.to(dev), y2=y2.transpose(0, 1).contiguous().to(dev), ys=ys.to(dev), y2_sum_first=True)
        assert torch.equal(r2, r)
    else:
        v = torch.randn(B, d, generator=g).to(torch.bfloat16)
        ref = oracle.hc_post2(res, post, comb, x=v)
        r = x.clone().to(dev)
        mods.fused2.hc_post2_(v.to(dev), r, post.to(dev), comb.to(dev))
    got = r.view(B, hc, d).cpu()
    # fused multiply-adds against separately rounded products: at most one bf16 step on isolated elements
    assert rel_err(got, ref) < 1e-2 and (got != ref).float().mean() < 0.02


def test_hc_steps_around_the_layer(mods, dev):
    # producer -> MoE layer -> consumer, the way the reference's decode loop strings them (dsv41/decode.py:446-464)
    E, D, I, topk, B, hc = 16, 512, 256, 4, 3, 4
    ex = mods.synth.make_experts(E, D, I, seed=5)
    sh = mods.synth.make_shared(D, I, seed=6, kind="e8m0")
    g = torch.Generator().manual_seed(9)
    gate_w = (torch.randn(E, D, generator=g) / D ** 0.5 * 3).float()
    layer = mods.moe.MoELayer(ex["w13"].to(dev), ex["s13"].to(dev), ex["w2"].to(dev), ex["s2"].to(dev), n_experts=E, topk=topk,
                              sh_w13=mods.w8.W8(sh["w13"].to(dev), sh["s13"].to(dev)), sh_w2=mods.w8.W8(sh["w2"].to(dev), sh["s2"].to(dev)),
                              gate_w=gate_w.to(dev))
    _, x, pre, w = _inputs(B, hc, D, 3)
    y, yq, yf = mods.fused2.hc_pre_norm_quant2(x.to(dev), pre.to(dev), w.to(dev), 1e-6, want_f32=True)
    routed, ys = layer.forward(y, None, xf=yf, final=False, want_routed=True, want_shared=True)
    res = x.clone().to(dev)
    post, comb = torch.rand(B, hc, generator=g).to(dev), torch.rand(B, hc, hc, generator=g).to(dev)
    mods.fused2.hc_post2_(None, res, post, comb, y2=routed.unsqueeze(1), ys=ys)
    # the same through the layer's own combine
    res2 = x.clone().to(dev)
    mods.fused2.hc_post2_(layer.forward(y, None, xf=yf), res2, post, comb)
    assert torch.equal(res, res2)
    assert mods.cukern.device_error(dev) == 0


def test_hc_kernels_match_the_reference_triton_outputs(mods, dev):
    """The CUDA kernels against what the reference's hc_pre_norm_quant2 / hc_post2_ produced for the same inputs: the pre-mix output may
    differ from Triton's by a bf16 rounding in isolated elements (the row variance is summed in another order), the quantised copies are
    exact functions of it, the post mix is equal up to one bf16 rounding."""
    gold = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hc.pt"), weights_only=False)
    same = lambda a, b: (a.view(torch.int16) == b.view(torch.int16)).float().mean().item()
    for name, c in gold["cases"].items():
        y, yq, yf, yqp = mods.fused2.hc_pre_norm_quant2(c["x"].to(dev), c["pre"].to(dev), c["w"].to(dev), c["eps"], want_f32=True, want_perm=True)
        assert same(y.cpu(), c["y"]) >= 0.995 and rel_err(y, c["y"]) < 1e-2, name
        assert same(yq.cpu(), c["yq"]) >= 0.99 and same(yqp.cpu(), c["yqp"]) >= 0.99, name
        r = mods.fused2.hc_post2_(c["xin"].to(dev), c["res"].clone().to(dev), c["post"].to(dev), c["comb"].to(dev)).cpu()
        assert same(r, c["res_after_x"]) >= 0.999 and rel_err(r, c["res_after_x"]) < 1e-2, name
        r = mods.fused2.hc_post2_(None, c["res"].clone().to(dev), c["post"].to(dev), c["comb"].to(dev), y2=c["y2"].to(dev), ys=c["ys"].to(dev)).cpu()
        assert same(r, c["res_after_moe"]) >= 0.999 and rel_err(r, c["res_after_moe"]) < 1e-2, name
