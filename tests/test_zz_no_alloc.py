"""The grouped FP4 expert GEMM with its scratch inside the library (b200_fp4_grouped_gemm_static) against the workspace form
(b200_fp4_grouped_gemm), both called through the C ABI.  Collected last on purpose (file name): it must pass alone and after
every other test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_p = ctypes.c_void_p
STATIC_MAX_PAIRS = 4096  # B200_STATIC_MAX_PAIRS of include/b200_moe.h


def _ptr(t):
    return c_p(t.data_ptr()) if t is not None else c_p(0)


def _problem(mods, dev, seed, E, N, K, counts):
    """Expert weights, activation rows and a group table with `counts[g]` pairs for expert g (0 = expert unused)."""
    g = torch.Generator().manual_seed(seed)
    ex = mods.synth.make_experts(E, K, N // 2, seed=seed)  # w13: [E, N, K/2] packed E2M1, s13: [E, N, K/32] E8M0 bytes
    w, s = ex["w13"], ex["s13"]
    n_pairs = int(sum(counts))
    rows = max(4, n_pairs // 2)
    x = (torch.randn(rows, K, generator=g) * 0.5).to(torch.bfloat16)
    experts = [e for e, c in enumerate(counts) if c > 0]
    starts, acc = [], 0
    for e in experts:
        starts.append(acc)
        acc += counts[e]
    starts.append(acc)
    pair_tok = torch.randint(0, rows, (n_pairs,), generator=g, dtype=torch.int32)
    pair_out = torch.randperm(n_pairs, generator=g).to(torch.int32)
    pair_w = torch.rand(n_pairs, generator=g) + 0.25
    t = lambda v: v.to(dev)
    return dict(x=t(x), w=t(w), s=t(s), ge=t(torch.tensor(experts, dtype=torch.int32)), gs=t(torch.tensor(starts, dtype=torch.int32)),
                pt=t(pair_tok), po=t(pair_out), pw=t(pair_w), n_pairs=n_pairs, E=E, N=N, K=K)


def _call(mods, p, static, out, shard=None, zero_out=0, accumulate=0, ws=None):
    """shard = (start, n): the weight tensors passed are the slice [start, start + n) of the problem's experts."""
    L = mods.lib
    lib = L.lib()
    dev = p["x"].device
    start, n = shard or (0, p["E"])
    w, s = p["w"][start:start + n], p["s"][start:start + n]
    fmt = L.FMT_FP4_E8M0 if s.dtype == torch.uint8 else L.FMT_FP4_BF16S
    head = [_ptr(p["x"]), p["x"].stride(0), 0, _ptr(w), w.stride(0), _ptr(s), s.stride(0) * s.element_size(), fmt, n, p["N"], p["K"],
            _ptr(p["ge"]), _ptr(p["gs"]), c_p(0), p["ge"].numel(), _ptr(p["pt"]), _ptr(p["po"]), _ptr(p["pw"]), p["n_pairs"], start, n, zero_out, accumulate,
            _ptr(out), out.stride(0)]
    stream = L.stream_of(dev)
    with torch.cuda.device(dev):
        if static:
            return lib.b200_fp4_grouped_gemm_static(*head, stream)
        if ws is None:
            ws = torch.empty(lib.b200_fp4_grouped_workspace_bytes(p["n_pairs"]) + 256, dtype=torch.uint8, device=dev)
        rc = lib.b200_fp4_grouped_gemm(*head, _ptr(ws), ws.numel(), stream)
        torch.cuda.synchronize(dev)  # ws must outlive the launch
        return rc


def test_static_scratch_matches_workspace_form_twice_in_a_row(mods, dev):
    # two different problems back to back on one stream: the second call reuses the array the first one filled, with more
    # works than the first (stale entries behind the first list) and then again with fewer
    problems = [_problem(mods, dev, 11, 8, 256, 512, [3, 0, 9, 1, 0, 17, 2, 5]),
                _problem(mods, dev, 12, 6, 128, 1024, [40, 1, 0, 8, 23, 2]),
                _problem(mods, dev, 13, 4, 256, 256, [1, 0, 0, 2])]
    want = []
    for p in problems:
        out = torch.full((p["n_pairs"], p["N"]), float("nan"), device=dev)
        assert _call(mods, p, False, out) == 0
        want.append(out)
    got = [torch.full((p["n_pairs"], p["N"]), float("nan"), device=dev) for p in problems]
    for p, out in zip(problems, got):  # no synchronisation in between
        assert _call(mods, p, True, out) == 0
    torch.cuda.synchronize(dev)
    for a, b in zip(got, want):
        assert torch.isfinite(b).all()
        assert torch.equal(a, b)  # same kernels on the same work list: bit-identical
    code = ctypes.c_int(0)
    assert mods.lib.lib().b200_device_error(ctypes.byref(code), mods.lib.stream_of(dev)) == 0 and code.value == 0


@pytest.mark.parametrize("mode", ["accumulate", "shard_zero_out", "shard_keep", "bf16_scales"])
def test_static_scratch_other_modes_equal_workspace_form(mods, dev, mode):
    """Scatter-add, an expert shard with and without zeroing of the foreign rows (permuted output rows), and bf16 scales: the
    static form gives the bits of the workspace form."""
    p = _problem(mods, dev, 21, 8, 256, 512, [5, 2, 0, 9, 1, 4, 0, 3])
    kw = {"accumulate": dict(accumulate=1), "shard_zero_out": dict(shard=(2, 4), zero_out=1), "shard_keep": dict(shard=(2, 4)), "bf16_scales": {}}[mode]
    if mode == "bf16_scales":
        p = dict(p, s=mods.synth.e8m0_to_bf16(p["s"].cpu()).to(dev))
    fill = 0.0 if mode == "accumulate" else 7.0
    want = torch.full((p["n_pairs"], p["N"]), fill, device=dev)
    got = torch.full((p["n_pairs"], p["N"]), fill, device=dev)
    assert _call(mods, p, False, want, **kw) == 0
    assert _call(mods, p, True, got, **kw) == 0
    torch.cuda.synchronize(dev)
    assert torch.equal(got, want)
    if mode.startswith("shard"):  # rows of the pairs of foreign experts: zeroed, or left as they were
        local = torch.zeros(p["n_pairs"], dtype=torch.bool)
        ge, gs = p["ge"].cpu().tolist(), p["gs"].cpu().tolist()
        for g, e in enumerate(ge):
            if 2 <= e < 6:
                local[gs[g]:gs[g + 1]] = True
        foreign_rows = p["po"].cpu()[~local].long()
        assert foreign_rows.numel() > 0
        assert (got.cpu()[foreign_rows] == (0.0 if mode == "shard_zero_out" else 7.0)).all()
        assert (got.cpu()[p["po"].cpu()[local].long()] != 7.0).any()


def test_static_scratch_calls_take_no_memory(mods, dev):
    """What the entry point is for: after the first (set-up) call, further calls neither reserve device memory nor touch torch's
    allocator, while the workspace form needs a buffer from its caller every time."""
    p = _problem(mods, dev, 31, 8, 256, 512, [3, 0, 9, 1, 0, 17, 2, 5])
    out = torch.empty(p["n_pairs"], p["N"], device=dev)
    assert _call(mods, p, True, out) == 0  # set-up call: symbol look-up, kernel attributes
    torch.cuda.synchronize(dev)
    free0, _ = torch.cuda.mem_get_info(dev)
    stats0 = torch.cuda.memory_stats(dev)
    for _ in range(100):
        assert _call(mods, p, True, out) == 0
    torch.cuda.synchronize(dev)
    free1, _ = torch.cuda.mem_get_info(dev)
    stats1 = torch.cuda.memory_stats(dev)
    assert free1 == free0  # nothing obtained from the driver (cudaMalloc would lower it)
    for key in ("allocation.all.allocated", "segment.all.allocated", "reserved_bytes.all.current"):
        assert stats1[key] == stats0[key], key  # nothing obtained from torch's caching allocator either


def test_static_scratch_rejects_more_pairs_than_it_holds(mods, dev):
    p = _problem(mods, dev, 14, 2, 128, 256, [2, 1])
    out = torch.zeros(4, p["N"], device=dev)
    p = dict(p, n_pairs=STATIC_MAX_PAIRS + 1)
    rc = _call(mods, p, True, out)
    assert rc == -6  # B200_ERR_TOO_LARGE, before any launch
    assert b"fixed maximum" in mods.lib.lib().b200_error_string(rc)
    torch.cuda.synchronize(dev)
    assert torch.count_nonzero(out) == 0
