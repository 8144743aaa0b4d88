"""Expert-parallel layer on two GPUs against the single-GPU layer (skipped on a one-GPU box).  One process per GPU, NCCL."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, T_total, out_path):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as g
    g.load_package()
    synth, moe, w8, ep = (g._import(n) for n in ("synth", "moe", "w8", "ep"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        E, D, I, topk = 16, 512, 256, 4
        ex = synth.make_experts(E, D, I, seed=5)
        sh = synth.make_shared(D, I, seed=6, kind="e8m0")
        x = synth.make_tokens(T_total, D, 7)
        logits = synth.make_logits(T_total, E, 8, topk=topk).float()

        def layer_for(start, n):
            sl = slice(start, start + n)
            return moe.MoELayer(ex["w13"][sl].to(dev), ex["s13"][sl].to(dev), ex["w2"][sl].to(dev), ex["s2"][sl].to(dev), n_experts=E, topk=topk,
                                sh_w13=w8.W8(sh["w13"].to(dev), sh["s13"].to(dev)), sh_w2=w8.W8(sh["w2"].to(dev), sh["s2"].to(dev)), swiglu_limit=10.0,
                                shard_start=start)

        start, n = ep.shard_ranges(E, world)[rank]
        counts = [c for _, c in ep.split_tokens(T_total, world)]
        first = sum(counts[:rank])
        got = ep.EPMoE(layer_for(start, n)).forward(x[first:first + counts[rank]].to(dev), logits[first:first + counts[rank]].to(dev), counts)
        want = layer_for(0, E).forward(x.to(dev), logits.to(dev))[first:first + counts[rank]]
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        torch.save({"err": err, "rows": got.shape[0]}, f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T_total", [8, 7, 300])
def test_expert_parallel_two_gpus_matches_one(tmp_path, T_total):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "ep")
    mp.spawn(_rank_main, args=(2, 29600 + T_total % 50, T_total, out), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(f"{out}.{r}")
        assert res["rows"] > 0 and res["err"] <= 1e-2  # bf16 rounding of a differently ordered fp32 sum
