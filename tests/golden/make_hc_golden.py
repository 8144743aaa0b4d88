"""Golden vectors for the hyper-connection steps either side of the MoE path, produced by the REFERENCE's own Triton kernels
(dsv41/fused2.py: hc_pre_norm_quant2 :213-246, hc_post2_ :539-558; plus fused.swiglu_quant and fused2.gate_topk as a second pin).

Two steps, because the reference checkout and the GPU are on different machines:
  1. where the reference checkout is:   python tests/golden/make_hc_golden.py --stage <reference dir>
     copies dsv41/fused.py and dsv41/fused2.py (only these two, unmodified) into the git-ignored baseline/_ref/dsv41/
  2. on a machine with a CUDA GPU:       python tests/golden/make_hc_golden.py --run <output .pt>
     imports that copy (Triton compiles the kernels for the local GPU), runs them on small seeded inputs and saves inputs + outputs.
The committed tests/golden/hc.pt is the file step 2 wrote on a B200; tests compare the CPU restatement and the CUDA kernels with it."""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
STAGE = os.path.join(ROOT, "baseline", "_ref")


def stage(ref_dir: str) -> None:
    dst = os.path.join(STAGE, "dsv41")
    os.makedirs(dst, exist_ok=True)
    for name in ("fused.py", "fused2.py"):
        shutil.copyfile(os.path.join(ref_dir, "dsv41", name), os.path.join(dst, name))
    open(os.path.join(dst, "__init__.py"), "w").close()
    print("staged", dst)


def run(out_path: str) -> None:
    import torch
    sys.path.insert(0, STAGE)
    from dsv41 import fused, fused2  # the reference's modules
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(11)
    cases = {}
    for B, d in ((1, 512), (4, 512), (1, 4096), (4, 4096)):
        hc = 4
        x = torch.randn(B, 1, hc, d, generator=g).to(torch.bfloat16)
        pre = torch.rand(B, hc, generator=g) + 0.1
        w = (torch.rand(d, generator=g) + 0.5).to(torch.bfloat16)
        y, yq, yf, yqp = fused2.hc_pre_norm_quant2(x.to(dev), pre.to(dev), w.to(dev), 1e-6, want_f32=True, want_perm=True)
        post = torch.randn(B, hc, generator=g)
        comb = torch.randn(B, hc, hc, generator=g) * 0.5
        res = torch.randn(B, 1, hc, d, generator=g).to(torch.bfloat16)
        xin = torch.randn(B, d, generator=g).to(torch.bfloat16)
        r_x = fused2.hc_post2_(xin.to(dev), res.clone().to(dev), post.to(dev), comb.to(dev))
        nsum = 6
        y2 = torch.randn(B, nsum, d, generator=g) * 3
        ys = torch.randn(B, d, generator=g).to(torch.bfloat16)
        r_moe = fused2.hc_post2_(None, res.clone().to(dev), post.to(dev), comb.to(dev), y2=y2.to(dev), ys=ys.to(dev))
        cases[f"B{B}_d{d}"] = {"x": x, "pre": pre, "w": w, "eps": 1e-6, "y": y.cpu(), "yq": yq.cpu(), "yf": yf.cpu(), "yqp": yqp.cpu(),
                               "post": post, "comb": comb, "res": res, "xin": xin, "res_after_x": r_x.cpu(), "y2": y2, "ys": ys, "res_after_moe": r_moe.cpu()}
    # second pin: the Triton swiglu_quant and gate_topk
    inter = 256
    gu = torch.randn(12, 2 * inter, generator=g) * 4
    wts = torch.rand(12, generator=g)
    extra = {"gu": gu, "wts": wts, "inter": inter}
    for limit in (10.0, 0.0):
        extra[f"swiglu_limit{limit}"] = fused.swiglu_quant(gu.to(dev), wts.to(dev), inter, limit).cpu()
    scores = torch.randn(5, 384, generator=g)
    bias = torch.randn(384, generator=g) * 0.1
    for func in ("softmax", "sigmoid", "sqrtsoftplus"):
        eid, wt = fused2.gate_topk(scores.to(dev), bias.to(dev), 1.0, 6, 2.5, func, True)
        extra[f"gate_{func}"] = (eid.cpu(), wt.cpu())
    extra.update(scores=scores, bias=bias)
    torch.cuda.synchronize()
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    torch.save({"cases": cases, "extra": extra, "made_on": torch.cuda.get_device_name(0), "triton": __import__("triton").__version__}, out_path)
    print("wrote", out_path, "on", torch.cuda.get_device_name(0))


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--stage":
        stage(sys.argv[2])
    elif len(sys.argv) == 3 and sys.argv[1] == "--run":
        run(sys.argv[2])
    else:
        print(__doc__)
        sys.exit(2)
