"""CPU: the shared library loads and exports every symbol the header declares; host-side bookkeeping (pair grouping, shard
ranges, synthetic generators, weight container) behaves like the reference's; the expert-parallel exchange is exercised with
two gloo ranks.  No compute call is made on the CUDA library."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(mods):
    header = open(os.path.join(ROOT, "include", "b200_moe.h")).read()
    declared = sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    L = ctypes.CDLL(mods.lib.LIB_PATH)
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/b200_moe.h but not exported"
    assert sorted(mods.lib.exported_symbols()) == [d for d in declared]
    assert mods.lib.lib().b200_version() >= 100
    assert b"workspace" in mods.lib.lib().b200_error_string(-4)


def test_moe_args_struct_matches_header(mods):
    header = open(os.path.join(ROOT, "include", "b200_moe.h")).read()
    body = header[header.index("typedef struct b200_moe_args {"):header.index("} b200_moe_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for stmt in body.split("{", 1)[1].split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        decl = re.sub(r"^(const\s+)?(void|float|int|size_t|long long)\s*\*?\s*", "", stmt)
        names += [n.strip().lstrip("*").strip() for n in decl.split(",")]
    assert names == [f[0] for f in mods.lib.MoeArgs._fields_]


def test_ep_peers_struct_matches_header(mods):
    header = open(os.path.join(ROOT, "include", "b200_moe.h")).read()
    body = header[header.index("typedef struct b200_ep_peers {"):header.index("} b200_ep_peers;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for stmt in body.split("{", 1)[1].split(";"):
        stmt = stmt.strip()
        if stmt:
            names += [re.sub(r".*[\s\*]", "", n.strip()) for n in stmt.split(",")]
    assert names == [f[0] for f in mods.lib.EpPeers._fields_]
    assert f"#define B200_EP_MAX_RANKS {mods.lib.EP_MAX_RANKS}" in header and f"#define B200_EP_HANDLE_BYTES {mods.lib.EP_HANDLE_BYTES}" in header


def test_peer_exchange_slab_layout():
    """Regions of a slab are 256-byte aligned, ordered and disjoint; the flag regions hold the largest supported world."""
    import __graft_entry__ as g
    ep, L = g._import("ep"), g._import("_lib")
    off = ep.PeerExchange.offsets(8, 64, 4096, 8192, 1536)
    order = ["fin", "fout", "x", "l", "part", "bytes"]
    assert all(off[k] % 256 == 0 for k in order) and [off[k] for k in order] == sorted(off[k] for k in order)
    assert off["fout"] - off["fin"] >= 4 * L.EP_MAX_RANKS and off["x"] - off["fout"] >= 4 * L.EP_MAX_RANKS
    assert off["l"] - off["x"] >= 64 * 8192 and off["part"] - off["l"] >= 64 * 1536 and off["bytes"] - off["part"] >= 64 * 8 * 4096 * 4


def test_operators_refuse_cpu_tensors(mods):
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mods.fused.fake_quant_fp8(x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mods.fused2.gate_topk(torch.zeros(1, 8), None, 1.0, 2, 1.0, "softmax", True)


def test_shard_ranges_and_token_split(mods):
    assert mods.ep.shard_ranges(384, 8) == [(48 * r, 48) for r in range(8)]
    assert mods.ep.shard_ranges(384, 2) == [(0, 192), (192, 192)]
    assert mods.ep.shard_ranges(10, 4) == [(0, 2), (2, 3), (5, 2), (7, 3)]  # boundaries at floor(10 r / 4), as dsv41/load.py:304-305
    assert mods.ep.split_tokens(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert sum(n for _, n in mods.ep.split_tokens(64, 3)) == 64


def test_loader_stacks_experts_and_shards(pkg):
    """Per-expert checkpoint tensors -> stacked tensors and shard dicts, bit for bit as the reference's loader lays them out
    (dsv41/load.py:213-249): w13 = [w1; w3] along the rows, shards hold contiguous global expert ranges."""
    import importlib
    load = importlib.import_module("dsv41_b200.load")
    g = torch.Generator().manual_seed(3)
    E, inter, dim, p = 6, 64, 128, "layers.3."
    ck = {}
    for e in range(E):
        q = f"{p}ffn.experts.{e}."
        for part, (n, k) in (("w1", (inter, dim)), ("w3", (inter, dim)), ("w2", (dim, inter))):
            ck[q + part + ".weight"] = torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, generator=g)   # any 1-byte dtype
            ck[q + part + ".scale"] = torch.randint(100, 140, (n, k // 32), dtype=torch.uint8, generator=g)
    ck[p + "ffn.gate.weight"] = torch.zeros(E, dim)
    assert load.expert_ids(ck.keys(), p) == list(range(E))
    full = load.load_experts(ck, p, "cpu")
    assert full["experts.w13"].shape == (E, 2 * inter, dim // 2) and full["experts.s2"].shape == (E, dim, inter // 32)
    for e in (0, 5):
        q = f"{p}ffn.experts.{e}."
        assert torch.equal(full["experts.w13"][e, :inter], ck[q + "w1.weight"].view(torch.uint8))
        assert torch.equal(full["experts.w13"][e, inter:], ck[q + "w3.weight"].view(torch.uint8))
        assert torch.equal(full["experts.s13"][e, inter:], ck[q + "w3.scale"]) and torch.equal(full["experts.w2"][e], ck[q + "w2.weight"].view(torch.uint8))
    assert load.shard_bounds(E, 4) == [(0, 1), (1, 2), (3, 1), (4, 2)] and load.shard_bounds(E, 3, [1, 2, 3]) == [(0, 1), (1, 2), (3, 3)]
    with pytest.raises(ValueError):
        load.shard_bounds(E, 3, [1, 2, 2])
    ep = [("cpu", s, n) for s, n in load.shard_bounds(E, 3)]
    sharded = load.load_experts(ck, p, "cpu", ep=ep)
    assert [(sh["start"], sh["n"]) for sh in sharded["experts.ep"]] == [(0, 2), (2, 2), (4, 2)]
    for sh in sharded["experts.ep"]:
        for k in ("w13", "s13", "w2", "s2"):
            assert torch.equal(sh[k], full["experts." + k][sh["start"]:sh["start"] + sh["n"]])
    assert sharded["experts.w13"] is sharded["experts.ep"][0]["w13"]


def test_w8_permutation_and_dequant(mods):
    g = torch.Generator().manual_seed(1)
    w = torch.randint(0, 120, (64, 128), dtype=torch.uint8, generator=g)
    s = torch.randint(115, 125, (2, 4), dtype=torch.uint8, generator=g)
    assert mods.w8.PERM_K == [0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15]
    assert torch.equal(mods.w8.unpermute_k(mods.w8.permute_k(w)), w)
    W = mods.w8.W8(w, s)
    assert W.shape == (64, 128) and torch.equal(W.bf16(), mods.quant.dequant_fp8_block(w.view(torch.float8_e4m3fn), s))
    both = mods.w8.W8.cat([W, W])
    assert both.shape == (128, 128) and both.s8.shape == (4, 4)


def test_quant_formats_and_torch_statement_of_the_activation_quantisation(mods, oracle):
    from oracle import torch_spec
    x = (torch.randn(3, 128) * 3).to(torch.bfloat16)
    assert torch.equal(torch_spec.fake_quant_fp8(x, 32).view(torch.int16), oracle.fake_quant_fp8(x, 32).view(torch.int16))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mods.quant.fake_quant_fp8(x, 32)  # the package has no CPU path
    assert mods.quant.round_e2m1(torch.tensor([0.75, 1.25, 2.5, 5.0, -0.25, 7.0, 0.2])).tolist() == [1.0, 1.0, 2.0, 4.0, -0.0, 6.0, 0.0]
    assert mods.quant.e8m0_to_float(torch.tensor([127, 123, 130, 1], dtype=torch.uint8)).tolist() == [1.0, 0.0625, 8.0, 2.0 ** -126]
    packed = torch.tensor([[0x21, 0xF8]], dtype=torch.uint8)
    assert mods.quant.unpack_fp4(packed).tolist() == [[0.5, 1.0, -0.0, -6.0]]
    g = torch.Generator().manual_seed(1)
    w = torch.randint(0, 256, (4, 32), dtype=torch.uint8, generator=g)
    s = torch.randint(120, 130, (4, 2), dtype=torch.uint8, generator=g)
    ref = oracle.fp4_gemm(torch.eye(64).to(torch.bfloat16), w, s).T  # rows of the dequantised matrix through the checker
    assert torch.equal(mods.quant.dequant_fp4(w, s).float(), ref)


def test_synthetic_generators(mods):
    sy = mods.synth
    ex = sy.make_experts(4, 256, 128, seed=1)
    assert ex["w13"].shape == (4, 256, 128) and ex["s13"].shape == (4, 256, 8) and ex["w2"].shape == (4, 256, 64) and ex["s2"].shape == (4, 256, 4)
    assert ex["s13"].min() >= 123 and ex["s13"].max() <= 129
    assert torch.equal(sy.make_experts(4, 256, 128, seed=1)["w2"], ex["w2"])
    assert sy.expert_bytes(4096, 2048) == 13369344 and sy.shared_bytes(4096, 2048, "e8m0") == 25190400
    logits = sy.make_logits(64, 384, seed=5)
    assert logits.dtype == torch.bfloat16
    top = logits.float().topk(7, dim=-1).values
    assert (top[:, 5] != top[:, 6]).all()
    # Zipf: the best-ranked experts dominate the selections
    b = sy.zipf_bias(384, 5)
    hot = set(b.topk(40).indices.tolist())
    sel = logits.float().topk(6, dim=-1).indices.flatten().tolist()
    assert sum(e in hot for e in sel) / len(sel) > 0.6
    assert torch.equal(torch.roll(b, 29), sy.zipf_bias(384, 5, rotate=29))
    w = torch.randn(256, 256) * 0.02
    for kind in ("f32b", "e8m0"):
        codes, scale = sy.quantize_fp8_block(w, kind)
        deq = mods.quant.dequant_fp8_f32block(codes.view(torch.float8_e4m3fn), scale) if kind == "f32b" else mods.quant.dequant_fp8_block(
            codes.view(torch.float8_e4m3fn), scale).float()
        assert (deq - w).abs().max() / w.abs().max() < 0.07
    assert torch.equal(sy.e8m0_to_bf16(torch.tensor([123, 127, 129], dtype=torch.uint8)).float(), torch.tensor([2.0 ** -4, 1.0, 4.0]))


EP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import __graft_entry__ as g
from oracle import oracle as O
ep = g._import("ep")
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
gen = torch.Generator().manual_seed(7)
E, D, I, T, topk = 8, 256, 256, 6, 2
w13 = torch.randint(0, 256, (E, 2 * I, D // 2), dtype=torch.uint8, generator=gen); s13 = torch.randint(118, 124, (E, 2 * I, D // 32), dtype=torch.uint8, generator=gen)
w2 = torch.randint(0, 256, (E, D, I // 2), dtype=torch.uint8, generator=gen); s2 = torch.randint(118, 124, (E, D, I // 32), dtype=torch.uint8, generator=gen)
sh = (torch.randint(0, 120, (2 * I, D), dtype=torch.uint8, generator=gen), torch.randint(115, 120, (2 * I // 32, D // 32), dtype=torch.uint8, generator=gen),
      torch.randint(0, 120, (D, I), dtype=torch.uint8, generator=gen), torch.randint(115, 120, (D // 32, I // 32), dtype=torch.uint8, generator=gen))
x = torch.randn(T, D, generator=gen).to(torch.bfloat16); logits = torch.randn(T, E, generator=gen)
start, n = ep.shard_ranges(E, world)[rank]
counts = [c for _, c in ep.split_tokens(T, world)]
first = sum(counts[:rank])
def partial(xa, la):   # this rank's experts over all tokens (CPU stand-in for the CUDA layer)
    return O.moe_layer(xa, la, None, w13[start:start+n], s13[start:start+n], w2[start:start+n], s2[start:start+n], None, topk=topk, shard=(start, n), n_experts=E)["routed"]
def shared(xl, routed):
    ys = O.shared_expert(O.fake_quant_fp8(xl, 32), *sh, 10.0)
    return (routed + ys.float()).to(torch.bfloat16)
layer = ep.EPMoE(partial_fn=partial, shared_fn=shared)
out = layer.forward(x[first:first + counts[rank]], logits[first:first + counts[rank]], counts)
ref = O.moe_layer(x, logits, None, w13, s13, w2, s2, sh, topk=topk)["out"][first:first + counts[rank]]
err = ((out.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
assert err < 1e-2, err
print(f"rank {rank} ok err {err:.2e}")
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_exchange_gloo(tmp_path, world):
    script = tmp_path / "ep_worker.py"
    script.write_text(EP_WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(29600 + world),
           str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count(" ok err ") == world
