"""The expert-parallel decode step over peer memory (csrc/epstep.cu, ep.PeerExchange).

On one GPU the ranks are emulated in ONE process and ONE stream: each "rank" has its own slab, and every phase is enqueued for all
ranks before the next phase (all dispatches, then all arrival waits, ...), so every flag a wait looks at has been published by a
kernel earlier in the stream and no kernel ever waits for a later one.  The two-GPU test runs the real thing: one process per GPU,
slabs mapped through CUDA IPC, no collective call in the step."""
import ctypes
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _layers(mods, dev, world, E=16, D=512, I=256, topk=4):
    synth, moe, w8, ep = mods.synth, mods.moe, mods.w8, mods.ep
    ex = synth.make_experts(E, D, I, seed=5)
    sh = synth.make_shared(D, I, seed=6, kind="e8m0")

    def layer_for(start, n):
        sl = slice(start, start + n)
        return moe.MoELayer(ex["w13"][sl].to(dev), ex["s13"][sl].to(dev), ex["w2"][sl].to(dev), ex["s2"][sl].to(dev), n_experts=E, topk=topk,
                            sh_w13=w8.W8(sh["w13"].to(dev), sh["s13"].to(dev)), sh_w2=w8.W8(sh["w2"].to(dev), sh["s2"].to(dev)), swiglu_limit=10.0,
                            shard_start=start)

    return layer_for(0, E), [layer_for(s, n) for s, n in ep.shard_ranges(E, world)]


@pytest.mark.parametrize("world,counts", [(1, [5]), (2, [4, 4]), (2, [3, 1]), (3, [2, 0, 5]), (4, [16, 16, 16, 16])])
def test_peer_exchange_step_emulated_ranks_match_single_layer(mods, dev, world, counts):
    ep, fused2 = mods.ep, mods.fused2
    E, D = 16, 512
    full, shards = _layers(mods, dev, world)
    T = sum(counts)
    xb, lb = D * 2, E * 4
    nbytes = ep.PeerExchange.offsets(world, 64, D, xb, lb)["bytes"]
    bases = [ep.PeerExchange.alloc_slab(nbytes, dev) for _ in range(world)]
    ranks = [ep.PeerExchange(r, world, bases, dev, 64, D, xb, lb, owned={"mine": bases[r], "opened": [], "group": None}) for r in range(world)]
    try:
        for step in range(3):  # the buffers and flags are reused, the step number advances
            x = mods.synth.make_tokens(T, D, 70 + step).to(dev)
            logits = mods.synth.make_logits(T, E, 80 + step, topk=4).float().to(dev)
            first = [sum(counts[:r]) for r in range(world)]
            for r, P in enumerate(ranks):
                P.dispatch(counts, x[first[r]:first[r] + counts[r]].contiguous(), logits[first[r]:first[r] + counts[r]].contiguous())
            for P in ranks:
                P.wait_arrival()
            for r, P in enumerate(ranks):
                x_all = P.x_all[:T * xb].view(torch.bfloat16).view(T, D)
                l_all = P.l_all[:T * lb].view(torch.float32).view(T, E)
                assert torch.equal(x_all, x) and torch.equal(l_all, logits)  # every rank holds every token row, bit for bit
                shards[r].forward(x_all, l_all, final=False, want_routed=True, routed_out=P.part[:T], want_shared=True, shared_out=P.ys[:T])
            for P in ranks:
                P.send_back(counts, P.part)
            for P in ranks:
                P.wait_return()
            outs = []
            for r, P in enumerate(ranks):
                n = counts[r]
                if n:
                    got_rows = P.partials[:n * world * D].view(n, world, D)
                    for q in range(world):  # the row rank q sent for token t is rank q's partial row of that token
                        assert torch.equal(got_rows[:, q], ranks[q].part[first[r]:first[r] + n])
                    outs.append(fused2.moe_combine(got_rows, P.ys[first[r]:first[r] + n]))
            got = torch.cat(outs)
            want = full.forward(x, logits)
            err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
            assert err <= 1e-2, (step, err)
            assert all(int(P.seq.item()) == step + 2 for P in ranks)
        code = ctypes.c_int(0)
        assert mods.lib.lib().b200_device_error(ctypes.byref(code), mods.lib.stream_of(dev)) == 0 and code.value == 0
    finally:
        torch.cuda.synchronize(dev)
        for P in ranks:
            P.close()


def test_peer_exchange_wait_gives_up_when_a_rank_never_sends(mods, dev):
    """A rank whose peer never dispatches: the arrival wait runs out of its (shortened) limit, stores 3003 and the stream stays usable."""
    ep, lib = mods.ep, mods.lib.lib()
    D, E = 512, 16
    nbytes = ep.PeerExchange.offsets(2, 64, D, D * 2, E * 4)["bytes"]
    bases = [ep.PeerExchange.alloc_slab(nbytes, dev) for _ in range(2)]
    P = ep.PeerExchange(0, 2, bases, dev, 64, D, D * 2, E * 4, owned={"mine": bases[0], "opened": [], "group": None})
    Q = ep.PeerExchange(1, 2, bases, dev, 64, D, D * 2, E * 4, owned={"mine": bases[1], "opened": [], "group": None})
    try:
        assert lib.b200_set_wait_limit_ns(2_000_000) == 0  # 2 ms
        x = mods.synth.make_tokens(2, D, 1).to(dev)
        logits = mods.synth.make_logits(2, E, 2, topk=4).float().to(dev)
        P.dispatch([2, 2], x, logits)  # rank 1 stays silent
        P.wait_arrival()
        code = ctypes.c_int(0)
        assert lib.b200_device_error(ctypes.byref(code), mods.lib.stream_of(dev)) == 0
        assert code.value == 3003
        y = torch.ones(8, device=dev) * 2  # the stream and the context still work
        assert float(y.sum()) == 16.0
        assert lib.b200_device_error(ctypes.byref(code), mods.lib.stream_of(dev)) == 0 and code.value == 0  # cleared by the read
    finally:
        lib.b200_set_wait_limit_ns(0)
        torch.cuda.synchronize(dev)
        P.close()
        Q.close()


def test_ep_entry_points_reject_bad_arguments(mods, dev):
    L, lib = mods.lib, mods.lib.lib()
    st = L.EpPeers()  # all null
    assert lib.b200_ep_dispatch(ctypes.byref(st), None, None, 0, L.stream_of(dev)) == -1
    assert lib.b200_ep_return(ctypes.byref(st), None, 1, L.stream_of(dev)) == -1
    assert lib.b200_ep_wait(None, 2, None, 0, 0, L.stream_of(dev)) == -1
    assert lib.b200_ep_alloc(0, None) == -1


def _rank_main(rank, world, port, counts, out_path):
    sys.path.insert(0, ROOT)
    import types
    import torch.distributed as dist
    import __graft_entry__ as g
    g.load_package()
    mods = types.SimpleNamespace(**{n: g._import(n) for n in ("synth", "moe", "w8", "ep", "fused2")}, lib=g._import("_lib"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {"err": None, "transport": None, "device_error": None}
    try:
        E, D = 16, 512
        full, shards = _layers(mods, dev, world)
        m = mods.ep.EPMoE(shards[rank])
        m.enable_peer_exchange(64, E)
        T = sum(counts)
        res["transport"] = m.transport(T)
        first = sum(counts[:rank])
        errs = []
        for step in range(4):
            x = mods.synth.make_tokens(T, D, 70 + step)
            logits = mods.synth.make_logits(T, E, 80 + step, topk=4).float()
            got = m.forward(x[first:first + counts[rank]].to(dev).contiguous(), logits[first:first + counts[rank]].to(dev).contiguous(), counts)
            if counts[rank]:
                want = full.forward(x.to(dev), logits.to(dev))[first:first + counts[rank]]
                errs.append(float((got.float() - want.float()).abs().max() / want.float().abs().max()))
        code = ctypes.c_int(0)
        mods.lib.lib().b200_device_error(ctypes.byref(code), mods.lib.stream_of(dev))
        res.update(err=max(errs) if errs else 0.0, device_error=code.value)
        torch.cuda.synchronize(dev)
        m.peer.close()
    finally:
        torch.save(res, f"{out_path}.{rank}")
        dist.destroy_process_group()


@pytest.mark.parametrize("counts", [[4, 4], [5, 2], [32, 32]])
def test_peer_exchange_two_gpus_matches_one(tmp_path, counts):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "epx")
    mp.spawn(_rank_main, args=(2, 29700 + sum(counts) % 50, counts, out), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(f"{out}.{r}")
        assert res["transport"].startswith("peer stores") and res["device_error"] == 0 and res["err"] <= 1e-2, res
