"""Benchmark of the MoE-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode64|decode32|decode8|decode1|prefill4096|fp8_gemv] [--impl reference]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W      (N > 1: expert parallel)

A step = one pass of the whole MoE layer (router -> input FP8 fake quantisation -> routed FP4 experts -> FP8 shared
expert -> combine) over one batch of synthetic tokens.  Layer shapes: 384 experts, hidden 4096, expert width 2048,
top-6 + 1 shared expert; all 384 experts resident (N = 1) or range-sharded 384/N per GPU (N > 1).

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM; `e2e` = the same through the public API
with pinned HOST buffers (host->device and device->host copies inside the timed region); `roofline` = the dominant kernel
(the routed gate/up weight stream) timed live with CUDA events against the measured HBM peak; `cpu_baseline` = the
reference's own CPU expert chain timed on this box's host cores (N = 1 only).
`roofline.prefill4096` (tensor bound), `roofline.decode` (the other decode batch sizes) and `roofline.fp8_gemv` (the dense FP8
GEMV shapes M in {1,2,4,8} x N in {4096,12288,18432}, K = 4096) carry the other configurations of the same path; `parity` compares
rows of one step with the CPU checker outside every timed region.
`--impl reference` times only that CPU implementation, on the same workload and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

E, D, I, TOPK = 384, 4096, 2048, 6
WORKLOADS = {"decode64": 64, "decode32": 32, "decode8": 8, "decode1": 1, "prefill4096": 4096}   # + "fp8_gemv" (run_gpu)
POOL = 12             # distinct (tokens, logits) sets cycled over the steps
ROTATE = 29           # expert-id shift of the Zipf ranking between consecutive sets: hot experts change every step
SEED = 1234
METRIC = "MoE-layer tok/s (decode S=1..64, prefill 4K) at 1/2/4/8 B200; % HBM/TC roofline"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return float(j["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


def measured_tensor_sustained() -> float:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["bf16_tflops_sustained"])
    except Exception:
        return 1400.0


def measured_tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["bf16_tflops"]), "measured bf16 burst (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 1590.0, "fallback (1.59 PFLOP/s bf16)"


class ClockSampler:
    """SM clock and throttle-reason samples taken DURING the timed region: an in-process NVML thread (10 ms period; read-only
    queries), or an `nvidia-smi -lms` child when NVML cannot be imported."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, f"/tmp/b200_clocks_{os.getpid()}.csv"
        self.thread, self.stop_flag, self.sm, self.mx, self.reasons, self.power = None, False, [], [], set(), []

    def _nvml_loop(self, nv, h):
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in self.BITS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            import threading
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            if self.sm:
                out.update(sm_mhz=statistics.median(self.sm), sm_max_mhz=max(self.mx), reasons=sorted(self.reasons), samples=len(self.sm),
                           power_w=statistics.median(self.power), source="nvml")
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm), source="nvidia-smi")
        return out


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), world


# ----------------------------------------------------------------------------------------------------------------- CPU arm
def cpu_experts(n: int, seed: int):
    from __graft_entry__ import _import
    return _import("synth").make_experts(n, D, I, seed=seed)


def time_cpu_chain(tokens_per_step: int, steps: int, warmup: int, budget_s: float, n_resident: int = 48):
    """The reference's CPU implementation of the path: routed expert chain of one token at a time (the library does not
    batch), 6 experts per token, expert ids rotated so the weights stream from DRAM (method of dsv41/test_cpumoe.py:32-35).
    Returns (tokens/s, description dict).  Uses oracle/_ref (the reference's own C++ compiled from its sources) when the
    host CPU can run it, else this repository's C port."""
    from oracle import oracle as O
    from __graft_entry__ import _import
    synth = _import("synth")
    ex = cpu_experts(n_resident, SEED + 99)
    x = O.fake_quant_fp8(synth.make_tokens(1, D, SEED + 5), 32)[0]
    wts = [0.3, 0.2, 0.15, 0.15, 0.1, 0.1]
    kind, cores, mode_note = "port", os.cpu_count() or 1, ""
    ref = None
    try:
        ref = O.RefCpuMoe(int8_mode=2)  # the reference's production default (dsv41/cpumoe.py:36)
        kind, cores, mode_note = "reference", ref.threads, "int8 mode 2 (its default); "
    except Exception as e:  # no AVX-512 BF16 on this host, or library not built
        mode_note = f"C port ({type(e).__name__}); "
    import ctypes

    def one_token(i: int):
        ids = [(e * 7 + 6 * i) % n_resident for e in range(6)]
        if ref is not None:
            ref.forward(x, ex["w13"], ex["s13"], ex["w2"], ex["s2"], ids, wts, 10.0)
        else:
            P = ctypes.c_void_p * 6
            out = torch.empty(D)
            O.lib().orc_routed_token(P(*[ex["w13"][e].data_ptr() for e in ids]), P(*[ex["s13"][e].data_ptr() for e in ids]),
                                     P(*[ex["w2"][e].data_ptr() for e in ids]), P(*[ex["s2"][e].data_ptr() for e in ids]), 6,
                                     ctypes.c_void_p(x.data_ptr()), (ctypes.c_float * 6)(*wts), ctypes.c_void_p(out.data_ptr()), D, I, D, ctypes.c_float(10.0))

    n = 0
    for _ in range(max(1, warmup)):
        one_token(n)
        n += 1
    t0 = time.perf_counter()
    done_steps, done_tokens = 0, 0
    while done_steps < steps:
        for _ in range(tokens_per_step):
            one_token(n)
            n += 1
            done_tokens += 1
            if time.perf_counter() - t0 > budget_s:
                break
        else:
            done_steps += 1
            continue
        break
    dt = time.perf_counter() - t0
    tps = done_tokens / dt
    desc = {"kind": kind, "cores": cores,
            "sample": f"{mode_note}routed expert chain only (no router, no shared expert), one token per call, {done_tokens} tokens x 6 experts, "
                      f"ids rotated over {n_resident} resident experts, {dt:.1f} s"}
    return tps, dt, done_tokens, desc


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    S = WORKLOADS.get(args.workload, 64)
    tps, dt, done, desc = time_cpu_chain(S, args.steps, args.warmup, budget_s=120.0)
    steps_done = max(1, done // S)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * dt / max(done / S, 1e-9), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args.workload, args.gpus),
            "cpu_baseline": dict(value=tps, unit="tokens/s", **desc),
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "steps_completed": steps_done}
    print(json.dumps(line), flush=True)


def workload_config(name: str, gpus: int) -> dict:
    S = WORKLOADS.get(name, 64)
    kind = "decode" if S <= 64 else "prefill"
    return {"workload": f"moe_{name}: {S} {kind} tokens, 384 experts (FP4 e2m1 + E8M0/32), hidden 4096, inter 2048, top-6 Zipf(s=1) softmax routing, "
                        f"+1 FP8 (e4m3 + E8M0 32x32) shared expert", "tokens": S, "experts": E, "hidden": D, "inter": I, "topk": TOPK,
            "parallelism": "single GPU, all experts resident" if gpus == 1 else f"ep{gpus}: experts sharded {E // gpus}/GPU, tokens split {S}/{gpus}",
            "l2": f"inputs larger than L2: {pool_size(S)} token/logit sets cycle, Zipf ranking rotated by {ROTATE} experts per set over 5.13 GB of experts"}


# ----------------------------------------------------------------------------------------------------------------- GPU arm
def pool_size(S: int) -> int:
    return POOL if S <= 64 else 3


def build_inputs(synth, S: int, dev):
    xs, ls = [], []
    for i in range(pool_size(S)):
        xs.append(synth.make_tokens(S, D, SEED + 10 + i))
        ls.append(synth.make_logits(S, E, SEED + 3, topk=TOPK, rotate=ROTATE * i))
    return xs, ls


def time_steps(fn, steps: int, warmup: int, barrier, finish=None):
    """finish(): makes the current stream wait for work the steps put on other streams, so that the closing event covers it."""
    for i in range(warmup):
        fn(i)
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    if finish is not None:
        finish()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps  # ms per step


def kernel_pass(layer, xs, ls, out, n: int, warmup: int):
    """Separate short pass that times the dominant kernel alone: the library records a CUDA event pair around the routed gate/up
    launch of every step (events on the launching stream).  Kept out of the pass that measures `value`, where the two event records
    per step would sit between the chained launches.  Returns the mean launch duration in ms and the input set of every step."""
    prof = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n + warmup)]
    for a, b in prof:
        a.record()
        b.record()
    torch.cuda.synchronize()
    NP = len(xs)
    for i in range(n + warmup):
        layer.forward(xs[i % NP], ls[i % NP], out=out, prof_events=prof[i])
    torch.cuda.synchronize()
    durs = [prof[warmup + i][0].elapsed_time(prof[warmup + i][1]) for i in range(n)]
    return statistics.mean(durs), [(warmup + i) % NP for i in range(n)]


def parity_rows(layer_forward, synth, x_h, l_h, rows, fetch, shared, dev_rows_of):
    """Compare `rows` of one batch with the CPU checker (outside every timed region): expert indices of the rows must be identical,
    the bf16 output within 1e-2 of max |ref|.  layer_forward(x, logits) -> (out, eid) for the rows this rank holds; dev_rows_of maps
    batch rows to the rank's local rows."""
    from oracle import oracle as O
    out, eid = layer_forward()
    ref_eid, ref_wt = O.gate_topk(l_h[rows].float(), None, 1.0, TOPK, 1.0, "softmax", True)
    ref = O.moe_rows(x_h[rows], ref_eid, ref_wt, fetch, shared, 10.0)
    got = out[dev_rows_of].float().cpu()
    want = ref["out"].float()
    err = float((got - want).abs().max() / want.abs().max())
    eq = bool(torch.equal(eid[dev_rows_of].cpu(), ref_eid)) if eid is not None else None
    return {"max_rel_err": err, "eid_equal": eq, "tokens_checked": int(len(rows)), "tolerance": 1e-2, "ok": bool(err <= 1e-2 and eq is not False),
            "checker": "oracle/ CPU restatement (pinned against the reference's own CPU library and goldens), rows of one step, outside the timed regions"}


def bench_fp8_gemv(g, dev, steps: int, warmup: int, peak: float):
    """Dense block-scaled FP8 GEMV (x bf16 [M, 4096] against e4m3 [N, 4096] with one fp32 scale per 128 x 128 block, bf16 out):
    weights drawn as N(0, 0.02), quantised per block with scale = blockmax / 448.  Each shape cycles over enough weight copies to
    exceed L2 (method of dsv41/bench_gemv_m1.py:50-68), timed with CUDA events around `steps` launches.  Algorithmic bytes = N*K
    weight bytes + the scale bytes."""
    synth, cukern = g._import("synth"), g._import("cukern")
    K = 4096
    res = {}
    for N in (4096, 12288, 18432):
        gen = torch.Generator(device=dev).manual_seed(SEED + N)
        copies = max(3, -(-300_000_000 // (N * K)))
        wf = torch.randn(N, K, generator=gen, device=dev) * 0.02
        codes, scale = synth.quantize_fp8_block(wf, "f32b")
        ws = [codes] + [codes.roll(i + 1, 0).contiguous() for i in range(copies - 1)]
        del wf
        for M in (1, 2, 4, 8):
            x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            launch = lambda i: cukern.fp8_gemm_tc(x, ws[i % copies], scale, out_dtype=torch.bfloat16, permuted=False, out=out)
            # one launch lasts a few microseconds, less than Python needs to issue it: a CUDA graph of one pass over the weight copies is
            # replayed instead (the method of dsv41/bench_gemv_m1.py:50-68), so that the device time per launch is what is measured
            for i in range(copies):
                launch(i)
            torch.cuda.synchronize()
            per = copies
            try:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    for i in range(copies):
                        launch(i)
                ms = time_steps(lambda i: gr.replay(), max(3, steps // copies), warmup, lambda: None) / per
            except Exception:
                ms = time_steps(launch, steps, warmup, lambda: None)
            alg = N * K + scale.numel() * 4
            gbs = alg / (ms * 1e-3) / 1e9
            res[f"M{M}_N{N}"] = {"us": ms * 1e3, "gbs": gbs, "frac": gbs / peak, "algorithmic_bytes": alg, "weight_copies_cycled": copies}
        del ws, codes
        torch.cuda.empty_cache()
    fr = [v["frac"] for v in res.values()]
    return {"bound": "hbm", "unit": "GB/s", "peak": peak, "format": "e4m3 + fp32 scale per 128x128 block", "kernel": "skinny_kernel<FP8_F32B, STORE_BF16>",
            "frac_min": min(fr), "frac_max": max(fr), "frac_mean": statistics.mean(fr), "shapes": res}


def finish_ranks(graphs=None):
    """End of a multi-rank run: every rank has finished its work (barrier + synchronize), the captured graphs are released first, and
    the process leaves without tearing the communicator down (a teardown with NCCL work captured in live graphs can block for minutes)."""
    import torch.distributed as dist
    if graphs:
        graphs.clear()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def run_gpu(args):
    import __graft_entry__ as g
    rank, local_rank, world = dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    g.load_package()
    synth, moe, w8, ep, cukern = g._import("synth"), g._import("moe"), g._import("w8"), g._import("ep"), g._import("cukern")
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peak, peak_src = measured_peaks()
    tpeak, tsrc = measured_tensor_peak()
    if args.workload == "fp8_gemv":
        assert world == 1, "the FP8 GEMV workload is a single-GPU measurement"
        sampler = ClockSampler(local_rank)
        sampler.start()
        r = bench_fp8_gemv(g, dev, args.steps, args.warmup, peak)
        best = max(r["shapes"].values(), key=lambda v: v["gbs"])
        line = {"metric": "FP8 dense GEMV GB/s (config 1: M in {1,2,4,8}, N in {4096,12288,18432}, K=4096)", "value": r["frac_mean"] * peak, "unit": "GB/s",
                "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.mean(v["us"] for v in r["shapes"].values()) / 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "fp8_gemv: x bf16 [M,4096] @ e4m3 [N,4096] (fp32 scale per 128x128), mean over 12 shapes", "l2": "weight copies cycled past L2"},
                "clocks": sampler.stop(), "roofline": dict(r, achieved=best["gbs"], frac=best["frac"], traffic=None, peak_source=peak_src), "gpu_launches": 12 * args.steps}
        print(json.dumps(line), flush=True)
        return

    S = WORKLOADS[args.workload]
    start, n_local = ep.shard_ranges(E, world)[rank]
    # identical expert bits on every rank: the full layer is generated on the device from one seed, the rank keeps its slice
    ex = synth.make_experts(E, D, I, seed=SEED, device=dev)
    sh_h = synth.make_shared(D, I, seed=SEED + 1, kind="e8m0")
    xs_h, ls_h = build_inputs(synth, S, dev)
    counts = [c for _, c in ep.split_tokens(S, world)]
    first = sum(counts[:rank])
    T_r = counts[rank]
    # experts the parity rows (rank 0's first rows of input set 0) route to, fetched to the host before the layer is sliced
    n_check = min(8, T_r)
    par_fetch = None
    if rank == 0 and not args.no_parity:
        from oracle import oracle as O
        pe, _ = O.gate_topk(ls_h[0][:n_check].float(), None, 1.0, TOPK, 1.0, "softmax", True)
        ids = sorted(set(pe.reshape(-1).tolist()))
        host = {k: ex[k][torch.tensor(ids, device=dev)].cpu() for k in ("w13", "s13", "w2", "s2")}
        pos = {e: i for i, e in enumerate(ids)}
        par_fetch = lambda want: tuple(host[k][[pos[e] for e in want]] for k in ("w13", "s13", "w2", "s2"))
    if world > 1:
        ex = {k: v[start:start + n_local].clone() for k, v in ex.items()}
        torch.cuda.empty_cache()
    sh = {k: v.to(dev) for k, v in sh_h.items()}
    layer = moe.MoELayer(ex["w13"], ex["s13"], ex["w2"], ex["s2"], n_experts=E, topk=TOPK, sh_w13=w8.W8(sh["w13"], sh["s13"]), sh_w2=w8.W8(sh["w2"], sh["s2"]),
                         swiglu_limit=10.0, shard_start=start, engine=args.engine)
    xs = [x[first:first + T_r].to(dev) for x in xs_h]
    ls = [l[first:first + T_r].to(dev) for l in ls_h]
    out = torch.empty(T_r, D, device=dev, dtype=torch.bfloat16)
    epl = ep.EPMoE(layer) if world > 1 else None
    exchange_note = None
    if world > 1 and S <= 64 and args.exchange != "nccl":
        # decode steps exchange through this package's own kernels over peer memory; if the slabs cannot be mapped on this box every
        # rank learns of it together and the step keeps the NCCL collectives
        try:
            epl.enable_peer_exchange(64, E, xs[0].dtype, ls[0].dtype)
        except RuntimeError as e:
            exchange_note = str(e)[:300]

    # ---- parity of one step against the CPU checker (untimed)
    parity = None
    if world > 1 or not args.no_parity:
        def fwd():
            if world == 1:
                o, e_, _ = layer.forward(xs[0], ls[0], want_route=True)
                return o, e_
            return epl.forward(xs[0], ls[0], counts), None
        if rank == 0 and par_fetch is not None:
            parity = parity_rows(fwd, synth, xs_h[0], ls_h[0], torch.arange(n_check), par_fetch, tuple(sh_h[k] for k in ("w13", "s13", "w2", "s2")), torch.arange(n_check, device=dev))
        elif world > 1:
            fwd()  # the other ranks take part in the exchange of that step
        torch.cuda.synchronize()

    # unique experts touched per input set (bookkeeping for the byte counts; untimed): from the logits, on the host
    NP = pool_size(S)
    uniq = [int(torch.unique(l.float().topk(TOPK, dim=-1).indices).numel()) for l in ls_h]

    # Expert-parallel decode steps are replayed from CUDA graphs (one per input buffer): a step is a dozen small launches and two
    # collectives, and a serving loop would not pay their host-side launch cost every step either.  Every rank captures the same sequence.
    graphs = {}

    def graph_for(key, xin, lin, outbuf):
        if world == 1 or S > 64 or args.no_graph:
            return None
        if key not in graphs:
            try:
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    for _ in range(3):
                        epl.forward(xin, lin, counts, out=outbuf)
                torch.cuda.current_stream(dev).wait_stream(side)
                torch.cuda.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    epl.forward(xin, lin, counts, out=outbuf)
                graphs[key] = gr
            except Exception as e:  # capture refused: run the step eagerly and say so
                graphs[key] = None
                graphs["error"] = f"{type(e).__name__}: {e}"[:200]
        return graphs[key]

    x_static, l_static = torch.empty_like(xs[0]), torch.empty_like(ls[0])

    def step_resident(i):
        j = i % NP
        if world == 1:
            layer.forward(xs[j], ls[j], out=out)
            return
        gr = graph_for("resident", x_static, l_static, out)
        if gr is None:
            epl.forward(xs[j], ls[j], counts, out=out)
        else:
            x_static.copy_(xs[j])
            l_static.copy_(ls[j])
            gr.replay()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = max_over_ranks(time_steps(step_resident, args.steps, args.warmup, barrier))
    clocks = sampler.stop() if rank == 0 else {}
    value = S / (ms * 1e-3)

    # ---- e2e: host buffers, copies inside the timed region
    # a step's inputs (token rows + router logits) sit in ONE pinned host buffer, so that they cross PCIe in one copy
    nbx, nbl = xs[0].numel() * xs[0].element_size(), ls[0].numel() * ls[0].element_size()
    hb = []
    for x, l in zip(xs_h, ls_h):
        b = torch.empty(nbx + nbl, dtype=torch.uint8).pin_memory()
        b[:nbx].copy_(x[first:first + T_r].contiguous().view(torch.uint8).reshape(-1))
        b[nbx:].copy_(l[first:first + T_r].contiguous().view(torch.uint8).reshape(-1))
        hb.append(b)
    # Copies and compute are pipelined as a serving loop would: step i's inputs cross PCIe on a copy stream while step i-1 computes,
    # and step i-1's result goes back on a third stream; two sets of device and host buffers, ordered by events.  Every step still
    # pays its own host->device copy and its own device->host read inside the timed region.
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    oh = [torch.empty(T_r, D, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    db = [torch.empty(nbx + nbl, dtype=torch.uint8, device=dev) for _ in range(2)]
    xd = [b[:nbx].view(xs[0].dtype).view(xs[0].shape) for b in db]
    ld = [b[nbx:].view(ls[0].dtype).view(ls[0].shape) for b in db]
    outs = [torch.empty_like(out) for _ in range(2)]
    ev_in, ev_cmp, ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))
    for e in ev_in + ev_cmp + ev_out:
        e.record(cur)

    def step_e2e(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[b])       # the step before last has finished reading this input buffer
            db[b].copy_(hb[i % NP], non_blocking=True)
            ev_in[b].record(s_in)
        cur.wait_event(ev_in[b])
        cur.wait_event(ev_out[b])            # the step before last has left this output buffer
        if world == 1:
            layer.forward(xd[b], ld[b], out=outs[b])
        else:
            gr = graph_for(("e2e", b), xd[b], ld[b], outs[b])
            if gr is None:
                epl.forward(xd[b], ld[b], counts, out=outs[b])
            else:
                gr.replay()
        ev_cmp[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            oh[b].copy_(outs[b], non_blocking=True)
            ev_out[b].record(s_out)

    def finish_e2e():
        cur.wait_event(ev_out[0])
        cur.wait_event(ev_out[1])

    ms_e2e = max_over_ranks(time_steps(step_e2e, args.steps, args.warmup, barrier, finish_e2e))
    h2d = (nbx + nbl) * world
    d2h = T_r * D * 2 * world

    exp_b = synth.expert_bytes(D, I)
    sh_b = synth.shared_bytes(D, I, "e8m0")
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, world), "clocks": clocks,
            "e2e": {"value": S / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e},
            "gpu_launches": (layer.launches_per_step(T_r * world) + (4 if world > 1 and epl.peer is not None and S <= epl.peer.max_tokens else 0)) * args.steps}
    if parity is not None:
        line["parity"] = parity

    if world > 1:
        # ---- expert-parallel line: bytes of the rank that streams most, the exchange's share, and the prefill half of the configuration
        mine = [int(((torch.unique(l.float().topk(TOPK, dim=-1).indices) >= start) & (torch.unique(l.float().topk(TOPK, dim=-1).indices) < start + n_local)).sum())
                for l in ls_h]
        t = torch.tensor([statistics.mean(mine)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        max_rank_bytes = float(t.item()) * exp_b + epl.shared_bytes_per_rank(sh_b)
        phases = epl.time_phases(xs[0], ls[0], counts, reps=20) if hasattr(epl, "time_phases") else None
        if phases is not None:
            for k in list(phases):
                phases[k] = max_over_ranks(phases[k])
        pre = None
        if not args.no_sweep:
            Tp = 16384
            cp = [c for _, c in ep.split_tokens(Tp, world)]
            fp = sum(cp[:rank])
            xp = [synth.make_tokens(Tp, D, SEED + 40 + i)[fp:fp + cp[rank]].to(dev) for i in range(2)]
            lp = [synth.make_logits(Tp, E, SEED + 3, topk=TOPK, rotate=ROTATE * i)[fp:fp + cp[rank]].to(dev) for i in range(2)]
            op = torch.empty(cp[rank], D, device=dev, dtype=torch.bfloat16)
            msp = max_over_ranks(time_steps(lambda i: epl.forward(xp[i & 1], lp[i & 1], cp, out=op), 5, 3, barrier))
            fl = Tp * TOPK * (2.0 * D * 2 * I + 2.0 * I * D)
            pre = {"tokens": Tp, "ms_per_step": msp, "tokens_per_s": Tp / (msp * 1e-3), "routed_tflops_all_gpus": fl / (msp * 1e-3) / 1e12,
                   "frac_of_bf16_burst_per_gpu": fl / (msp * 1e-3) / 1e12 / world / tpeak}
            del xp, lp
        if rank == 0:
            gbs = max_rank_bytes / (ms * 1e-3) / 1e9
            line["config"]["cuda_graph"] = bool(graphs.get("resident")) if S <= 64 else False
            line["config"]["exchange"] = epl.transport(S)
            if exchange_note:
                line["config"]["exchange_note"] = exchange_note
            if "error" in graphs:
                line["config"]["cuda_graph_error"] = graphs["error"]
            line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None, "peak_source": peak_src,
                                "what": "whole step of the rank that streams most: (its distinct local experts x 13,369,344 B + its share of the shared expert) / max-over-ranks step time",
                                "max_rank_bytes_per_step": max_rank_bytes, "phases_ms": phases}
            if pre is not None:
                line["prefill16384"] = pre
            code = cukern.device_error(dev)
            line["device_error"] = code
            print(json.dumps(line), flush=True)
        finish_ranks(graphs)
        return

    # ---- single GPU: kernel-level roofline from a separate short pass with events around the dominant kernel
    n_k = min(args.steps, 60)
    avg_ms, sets = kernel_pass(layer, xs, ls, out, n_k, args.warmup)
    u_k = statistics.mean(uniq[j] for j in sets)
    u_all = statistics.mean(uniq[(args.warmup + i) % NP] for i in range(args.steps))
    layer_bytes = u_all * exp_b + sh_b
    exp_b13 = 2 * I * D // 2 + 2 * I * D // 32

    def prefill_roofline(ms_step: float, k_ms: float | None, u: float):
        fl_routed = S_PRE * TOPK * (2.0 * D * 2 * I + 2.0 * I * D)          # routed pairs only: pairs x 50,331,648
        fl_all = S_PRE * (TOPK + 1) * (2.0 * D * 2 * I + 2.0 * I * D)      # + the shared expert's rows
        ach = fl_routed / (ms_step * 1e-3) / 1e12
        r = {"bound": "tensor", "achieved": ach, "peak": tpeak, "unit": "TFLOP/s", "frac": ach / tpeak, "traffic": None, "peak_source": tsrc,
             "what": "whole layer step (route, bucketing, quantisation, both grouped GEMMs, combine); FLOPs = routed pairs x 50,331,648",
             "frac_of_sustained": ach / measured_tensor_sustained(), "ms_per_step": ms_step, "tokens_per_s": S_PRE / (ms_step * 1e-3),
             "with_shared_expert": {"achieved": fl_all / (ms_step * 1e-3) / 1e12, "frac": fl_all / (ms_step * 1e-3) / 1e12 / tpeak},
             "weight_stream_floor_ms": (u * exp_b + sh_b) / (peak * 1e9) * 1e3, "unique_experts_per_step": u}
        if k_ms is not None:
            f1 = S_PRE * (TOPK + 1) * 2.0 * D * 2 * I
            r["gate_up_kernel"] = {"kernel": "mx_gemm_kernel (gate/up grouped GEMM of routed + shared rows, tcgen05 kind::mxf8f6f4, + SwiGLU + FP8 quantisation)",
                                   "avg_launch_ms": k_ms, "achieved": f1 / (k_ms * 1e-3) / 1e12, "frac": f1 / (k_ms * 1e-3) / 1e12 / tpeak}
        return r

    S_PRE = WORKLOADS["prefill4096"]
    if S <= 64:
        mx = layer._use_mx(S)
        # the tensor-core launch streams the shared expert's gate/up matrix (FP8 + 32x32 scales) in the same kernel
        alg = u_k * exp_b13 + ((2 * I * D + 2 * I * D // 1024) if mx else 0)
        achieved = alg / (avg_ms * 1e-3) / 1e9
        # DRAM bytes per launch: (dram__bytes_read + dram__bytes_write) / algorithmic bytes of the same kernel in the committed ncu
        # capture of a smaller case, scaled to this launch by its algorithmic bytes (traffic grows with the experts streamed)
        ratio = layer.traffic_ratio(S)
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": alg * ratio,
                            "traffic_source": "ncu capture of a smaller case (profiles/), scaled by algorithmic bytes",
                            "kernel": layer.dominant_kernel(S),
                            "algorithmic_bytes_per_launch": alg, "avg_launch_ms": avg_ms, "peak_source": peak_src, "timed_in": f"separate pass of {n_k} steps with an event pair around the kernel",
                            "frac_of_8TBs_nominal": achieved / 8000.0, "unique_experts_per_step": u_k,
                            "whole_layer": {"bytes_per_step": layer_bytes, "achieved_gbs": layer_bytes / (ms * 1e-3) / 1e9,
                                            "frac": layer_bytes / (ms * 1e-3) / 1e9 / peak}}
    else:
        line["roofline"] = prefill_roofline(ms, avg_ms, u_all)
    # ---- the other batch sizes of the same configuration (short runs, same method), and the dense FP8 GEMV shapes
    if not args.no_sweep:
        dec = {}
        for name, s2 in WORKLOADS.items():
            if name == args.workload:
                continue
            xs2, ls2 = build_inputs(synth, s2, dev)
            u2 = statistics.mean(int(torch.unique(l.float().topk(TOPK, dim=-1).indices).numel()) for l in ls2)
            xs2, ls2 = [x.to(dev) for x in xs2], [l.to(dev) for l in ls2]
            o2 = torch.empty(s2, D, device=dev, dtype=torch.bfloat16)
            np2 = pool_size(s2)
            k2 = args.steps if s2 <= 64 else max(3, min(args.steps, 8))
            m2 = time_steps(lambda i: layer.forward(xs2[i % np2], ls2[i % np2], out=o2), k2, args.warmup, barrier)
            if s2 > 64:
                km, _ = kernel_pass(layer, xs2, ls2, o2, 3, 2)
                line["roofline"]["prefill4096"] = prefill_roofline(m2, km, u2)
            else:
                b2 = u2 * exp_b + sh_b
                dec[name] = {"bound": "hbm", "tokens_per_s": s2 / (m2 * 1e-3), "ms_per_step": m2, "unique_experts": u2, "achieved": b2 / (m2 * 1e-3) / 1e9, "unit": "GB/s",
                             "frac": b2 / (m2 * 1e-3) / 1e9 / peak, "what": "whole layer step: (distinct experts x 13,369,344 B + shared expert) / step time"}
            del xs2, ls2, o2
        line["roofline"]["decode"] = dec
        line["roofline"]["fp8_gemv"] = bench_fp8_gemv(g, dev, min(args.steps, 100), args.warmup, peak)
    line["device_error"] = cukern.device_error(dev)
    if not args.no_cpu:
        tps, dt, done, desc = time_cpu_chain(S, 10 ** 9, 1, budget_s=args.cpu_seconds)
        line["cpu_baseline"] = dict(value=tps, unit="tokens/s", **desc)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode64", choices=sorted(WORKLOADS) + ["fp8_gemv"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="expert-parallel decode: launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel decode: exchange through this package's kernels over peer memory (default), or NCCL all-gather + reduce-scatter")
    ap.add_argument("--engine", type=int, default=0, choices=[0, 1, 2], help="0 automatic, 1 weight-streaming kernels, 2 tcgen05 block-scaled kernels")
    ap.add_argument("--experts", type=int, default=E, help="expert count (smaller than the workload's 384 only for profiler captures)")
    ap.add_argument("--tokens", type=int, default=0, help="token count of the chosen workload (smaller than its own only for profiler captures)")
    args = ap.parse_args()
    globals()["E"] = args.experts
    if args.tokens > 0 and args.workload in WORKLOADS:
        WORKLOADS[args.workload] = args.tokens
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
