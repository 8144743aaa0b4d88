"""Generate the golden vectors of tests/golden/*.pt from the reference checkout.

Run once where the reference checkout is at hand:

    python tests/golden/make_golden.py /path/to/reference

What is produced, and from which reference code:
  quant.pt   outputs of the reference's OWN torch definitions, imported from dsv41/quant.py: fake_quant_fp8 (:46-54),
             dequant_fp4 (:106-110), dequant_fp8_block (:90-95), round_e2m1 (:67-71), e8m0_to_float (:27-31), FP4_TABLE (:24)
  gate.pt    MoE.gate (dsv41/model.py:1614-1630) and _swiglu (dsv41/model.py:2337-2342): the function bodies are read from the
             reference file with `ast`, compiled and executed here (the module itself cannot be imported without a GPU driver),
             then the swiglu_quant chain of dsv41/test_fused.py:81-88 is formed with quant.fake_quant_fp8
  cpumoe.pt  outputs of the reference's C++ CPU MoE library (dsv41/cpu/moe_cpu.cpp compiled by oracle/build.py), mode 0 (exact
             BF16) and mode 2 (its int8 default), on the inputs of dsv41/test_cpumoe.py:9-17 at reduced size
Inputs are small seeded tensors stored next to the outputs so the tests need nothing but these files.
"""
import ast
import os
import sys
import types

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/reference")
REF = sys.argv[1]
sys.path.insert(0, REF)


def load_functions(path, wanted):
    """Compile the named top-level functions / class methods of a reference source file without importing the module."""
    tree = ast.parse(open(path).read())
    out = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in wanted and node.name not in out:
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"torch": torch, "F": F}
            exec(compile(mod, path, "exec"), ns)
            out[node.name] = ns[node.name]
    return out


def main():
    from dsv41 import quant  # the reference's own module (pure torch)
    g = torch.Generator().manual_seed(0)
    # ---------------------------------------------------------------- quant.pt
    x = (torch.randn(4, 256, generator=g) * 4).to(torch.bfloat16)
    x[0, :32] = 0
    x[1, :32] *= 1e-6
    x[2, :32] *= 3000
    w4 = torch.randint(0, 256, (24, 64), dtype=torch.uint8, generator=g)
    s4 = torch.randint(110, 135, (24, 4), dtype=torch.uint8, generator=g)
    w8 = torch.randint(0, 256, (64, 96), dtype=torch.uint8, generator=g)
    w8[(w8 & 0x7F) == 0x7F] = 0
    s8 = torch.randint(110, 130, (2, 3), dtype=torch.uint8, generator=g)
    a = torch.randn(3, 128, generator=g).to(torch.bfloat16)
    mids = torch.tensor([0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 0.24, 6.0])
    torch.save({
        "x": x, "fake_quant_fp8": quant.fake_quant_fp8(x, 32),
        "w4": w4, "s4": s4, "dequant_fp4": quant.dequant_fp4(w4, s4),
        "w8": w8, "s8": s8, "dequant_fp8_block": quant.dequant_fp8_block(w8.view(torch.float8_e4m3fn), s8),
        "a": a, "fp4_gemm": a.float() @ quant.dequant_fp4(w4, s4).float().T,
        "fp8_gemm": a[:, :96].float() @ quant.dequant_fp8_block(w8.view(torch.float8_e4m3fn), s8).float().T,
        "mids": mids, "round_e2m1": quant.round_e2m1(mids), "fp4_table": quant.FP4_TABLE.clone(),
        "e8m0": quant.e8m0_to_float(torch.arange(100, 140, dtype=torch.uint8)),
    }, os.path.join(HERE, "quant.pt"))
    # ---------------------------------------------------------------- gate.pt
    fns = load_functions(os.path.join(REF, "dsv41", "model.py"), {"gate", "_swiglu"})
    sc = torch.randn(5, 384, generator=g) * 2
    bias = torch.randn(384, generator=g) * 0.1
    gate_w = torch.eye(384)  # scores = F.linear(x, I) = x, so the logits are the input
    gates = {}
    for func in ("softmax", "sigmoid", "sqrtsoftplus"):
        for norm in (True, False):
            self = types.SimpleNamespace(gate_w=gate_w, gate_temp=1.3, score_func=func, gate_bias=bias, topk=6, norm_topk_prob=norm, route_scale=2.5)
            wts, idx = fns["gate"](self, sc)
            gates[f"{func}_{int(norm)}"] = (wts.clone(), idx.clone())
    gu = torch.randn(9, 2 * 256, generator=g) * 5
    wt = torch.rand(9, generator=g)
    sw = {}
    for limit in (10.0, 0.0):
        h = fns["_swiglu"](gu[:, :256], gu[:, 256:], limit)
        sw[f"w_{limit}"] = quant.fake_quant_fp8((wt[:, None] * h).to(torch.bfloat16), 32)
        sw[f"n_{limit}"] = quant.fake_quant_fp8(h.to(torch.bfloat16), 32)
    torch.save({"scores": sc, "bias": bias, "temp": 1.3, "route_scale": 2.5, "topk": 6, "gates": gates, "gu": gu, "wt": wt, "swiglu_quant": sw},
               os.path.join(HERE, "gate.pt"))
    # ---------------------------------------------------------------- cpumoe.pt
    from oracle import oracle as O
    E, inter, dim = 8, 256, 256
    w13 = torch.randint(0, 256, (E, 2 * inter, dim // 2), dtype=torch.uint8, generator=g)
    s13 = torch.randint(118, 128, (E, 2 * inter, dim // 32), dtype=torch.uint8, generator=g)
    w2 = torch.randint(0, 256, (E, dim, inter // 2), dtype=torch.uint8, generator=g)
    s2 = torch.randint(118, 128, (E, dim, inter // 32), dtype=torch.uint8, generator=g)
    xq = quant.fake_quant_fp8((torch.randn(1, dim, generator=g) * 2).to(torch.bfloat16), 32)
    ids, wts = [0, 2, 3, 5, 6, 7], [0.3, 0.2, 0.15, 0.15, 0.1, 0.1]
    R = O.RefCpuMoe(int8_mode=0)
    out0 = R.forward(xq[0], w13, s13, w2, s2, ids, wts, 10.0).clone()
    out0_nolimit = R.forward(xq[0], w13, s13, w2, s2, ids[:2], wts[:2], 0.0).clone()
    R.set_mode(2)
    out2 = R.forward(xq[0], w13, s13, w2, s2, ids, wts, 10.0).clone()
    torch.save({"w13": w13, "s13": s13, "w2": w2, "s2": s2, "xq": xq, "ids": ids, "wts": wts, "limit": 10.0, "mode0": out0, "mode2": out2,
                "mode0_nolimit_2experts": out0_nolimit}, os.path.join(HERE, "cpumoe.pt"))
    print("written:", [f for f in os.listdir(HERE) if f.endswith(".pt")])


if __name__ == "__main__":
    main()
