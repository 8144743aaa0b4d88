"""TEST INFRASTRUCTURE ONLY: Python bindings (ctypes, torch CPU tensors) for the CPU checkers.

  * `lib()`            -> this repository's plain-C oracle (oracle/moe_oracle.c)
  * `RefCpuMoe`        -> the reference's own CPU MoE library compiled from its sources (oracle/_ref), bound the way
                          the reference binds it (dsv41/cpumoe.py:15-58, 185-210), always in its exact BF16 mode 0.

Nothing in the product package imports this module.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

_lib = None
c_p = ctypes.c_void_p


def _ptr(t):
    return c_p(t.data_ptr()) if t is not None else c_p(0)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build_oracle())
    return _lib


def _u16(t: torch.Tensor) -> torch.Tensor:
    assert t.dtype == torch.bfloat16 and t.device.type == "cpu"
    return t.contiguous()


# ------------------------------------------------------------------ elementwise
def fake_quant_fp8(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    x = _u16(x)
    y = torch.empty_like(x)
    lib().orc_fake_quant_fp8(_ptr(x), _ptr(y), ctypes.c_long(x.numel()), ctypes.c_int(block))
    return y


def gate_topk(scores: torch.Tensor, bias, temp: float, topk: int, route_scale: float, score_func: str, norm: bool):
    scores = scores.float().contiguous()
    E = scores.shape[-1]
    B = scores.numel() // E
    mode = {"sqrtsoftplus": 0, "sigmoid": 1, "softmax": 2}[score_func]
    eid = torch.empty(B, topk, dtype=torch.int32)
    wt = torch.empty(B, topk, dtype=torch.float32)
    b = bias.float().contiguous() if bias is not None else None
    lib().orc_gate_topk(_ptr(scores), _ptr(b), B, E, ctypes.c_float(temp), topk, ctypes.c_float(route_scale), mode, int(bool(norm)), _ptr(eid), _ptr(wt))
    return eid, wt


def swiglu_quant(gu: torch.Tensor, weights, inter: int, limit: float, round_gu_bf16: bool = False) -> torch.Tensor:
    gu = gu.float().contiguous()
    rows = gu.shape[0]
    w = weights.float().contiguous() if weights is not None else None
    h = torch.empty(rows, inter, dtype=torch.bfloat16)
    lib().orc_swiglu_quant(_ptr(gu), _ptr(w), rows, inter, ctypes.c_float(limit), int(round_gu_bf16), _ptr(h))
    return h


# ------------------------------------------------------------------ FP4
def fp4_gemm(a: torch.Tensor, w: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    a, w, s = _u16(a), w.contiguous(), s.contiguous()
    M, K = a.shape
    N = w.shape[0]
    assert w.shape == (N, K // 2) and s.shape == (N, K // 32) and w.dtype == torch.uint8 and s.dtype == torch.uint8
    out = torch.empty(M, N, dtype=torch.float32)
    lib().orc_fp4_gemm(_ptr(a), ctypes.c_long(K), _ptr(w), _ptr(s), M, N, K, _ptr(out), ctypes.c_long(N))
    return out


def fp4_pairs(a, w, s, expert, row_in, row_out, weight, n_out_rows: int, out=None) -> torch.Tensor:
    a, w, s = _u16(a), w.contiguous(), s.contiguous()
    E, N, Kh = w.shape
    K = Kh * 2
    expert, row_in, row_out = (t.to(torch.int32).contiguous() for t in (expert, row_in, row_out))
    wt = weight.float().contiguous() if weight is not None else None
    if out is None:
        out = torch.zeros(n_out_rows, N, dtype=torch.float32)
    lib().orc_fp4_pairs(_ptr(a), ctypes.c_long(a.shape[1]), _ptr(w), ctypes.c_long(N * Kh), _ptr(s), ctypes.c_long(N * (K // 32)), _ptr(expert),
                        _ptr(row_in), _ptr(row_out), _ptr(wt), expert.numel(), N, K, _ptr(out), ctypes.c_long(N))
    return out


# ------------------------------------------------------------------ FP8 dense
def fp8_gemm(x: torch.Tensor, w8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x bf16 [M,K]; w8 uint8 e4m3 [N,K] natural k order; scale uint8 E8M0 [ceil(N/32),K/32] or fp32 [ceil(N/128),ceil(K/128)]."""
    x, w8, scale = _u16(x), w8.contiguous().view(torch.uint8), scale.contiguous()
    M, K = x.shape
    N = w8.shape[0]
    out = torch.empty(M, N, dtype=torch.float32)
    fn = lib().orc_fp8_gemm_e8m0 if scale.dtype == torch.uint8 else lib().orc_fp8_gemm_f32block
    assert scale.dtype in (torch.uint8, torch.float32)
    fn(_ptr(x), ctypes.c_long(K), _ptr(w8), _ptr(scale), scale.shape[1], M, N, K, _ptr(out), ctypes.c_long(N))
    return out


def shared_expert(xq, sh_w13, sh_s13, sh_w2, sh_s2, limit: float) -> torch.Tensor:
    xq = _u16(xq)
    T, dim = xq.shape
    inter = sh_w2.shape[1]
    fmt = 0 if sh_s13.dtype == torch.uint8 else 1
    ys = torch.empty(T, dim, dtype=torch.bfloat16)
    lib().orc_shared_expert(_ptr(xq), T, dim, inter, _ptr(sh_w13.contiguous()), _ptr(sh_s13.contiguous()), sh_s13.shape[1], _ptr(sh_w2.contiguous()),
                            _ptr(sh_s2.contiguous()), sh_s2.shape[1], fmt, ctypes.c_float(limit), _ptr(ys))
    return ys


# ------------------------------------------------------------------ whole layer
def moe_layer(x, logits, bias, w13, s13, w2, s2, shared, *, topk=6, temp=1.0, route_scale=1.0, score_func="softmax", norm=True, limit=10.0,
              shard=(0, 1 << 30), n_experts=None):
    """x bf16 [T,D] (not yet quantised), logits fp32 [T,E]; expert tensors in the stacked layout; shared = None or
    (sh_w13, sh_s13, sh_w2, sh_s2).  Returns dict(out bf16 [T,D], eid, wt, routed fp32 [T,D])."""
    x = _u16(x)
    T, D = x.shape
    logits = logits.float().contiguous()
    E = logits.shape[1] if n_experts is None else n_experts
    inter = w2.shape[2] * 2
    mode = {"sqrtsoftplus": 0, "sigmoid": 1, "softmax": 2}[score_func]
    out = torch.empty(T, D, dtype=torch.bfloat16)
    eid = torch.empty(T, topk, dtype=torch.int32)
    wt = torch.empty(T, topk, dtype=torch.float32)
    routed = torch.empty(T, D, dtype=torch.float32)
    b = bias.float().contiguous() if bias is not None else None
    if shared is not None:
        sw13, ss13, sw2, ss2 = (t.contiguous() for t in shared)
        fmt = 0 if ss13.dtype == torch.uint8 else 1
        sh = (1, _ptr(sw13), _ptr(ss13), ss13.shape[1], _ptr(sw2), _ptr(ss2), ss2.shape[1], fmt)
    else:
        sh = (0, c_p(0), c_p(0), 0, c_p(0), c_p(0), 0, 0)
    w13, s13, w2, s2 = (t.contiguous() for t in (w13, s13, w2, s2))
    start, n = shard
    n = min(n, w13.shape[0])
    lib().orc_moe_layer(_ptr(x), _ptr(logits), _ptr(b), T, E, topk, D, inter, ctypes.c_float(temp), ctypes.c_float(route_scale), mode, int(bool(norm)),
                        ctypes.c_float(limit), _ptr(w13), _ptr(s13), _ptr(w2), _ptr(s2), int(start), int(n), *sh, _ptr(out), _ptr(eid), _ptr(wt), _ptr(routed))
    return {"out": out, "eid": eid, "wt": wt, "routed": routed}


def moe_rows(x_rows, eid, wt, fetch_experts, shared, limit: float = 10.0, shard=(0, 1 << 30)):
    """The layer for a few token rows of a batch whose expert set is too large for the host (all 384 experts of the benchmark
    layer are 5.1 GB): the same steps as `moe_layer`, composed from the pinned pieces (fake quantisation -> gate/up pairs ->
    SwiGLU * weight + quantisation -> down pairs -> sum in slot order -> + shared expert -> bf16), on the experts the rows route to.
    x_rows bf16 [n, D]; eid int32 [n, topk] / wt fp32 [n, topk]: the routing of those rows (checked separately against
    `gate_topk`); fetch_experts(ids: list[int]) -> (w13, s13, w2, s2) CPU uint8 tensors stacked in the order of `ids`;
    shared = None or (sh_w13, sh_s13, sh_w2, sh_s2); shard = (start, n): only experts of that range contribute to `routed`.
    Returns dict(out bf16 [n, D], routed fp32 [n, D])."""
    x_rows = _u16(x_rows)
    n, D = x_rows.shape
    topk = eid.shape[1]
    xq = fake_quant_fp8(x_rows, 32)
    e = eid.to(torch.int64).reshape(-1)
    local = (e >= shard[0]) & (e < shard[0] + shard[1])
    ids = sorted(set(e[local].tolist()))
    routed = torch.zeros(n, D, dtype=torch.float32)
    if ids:
        w13, s13, w2, s2 = fetch_experts(ids)
        inter = w2.shape[2] * 2
        remap = {g: i for i, g in enumerate(ids)}
        sel = local.nonzero().flatten()
        P = sel.numel()
        ex = torch.tensor([remap[int(g)] for g in e[sel]], dtype=torch.int32)
        tok = (sel // topk).to(torch.int32)
        rows = torch.arange(P, dtype=torch.int32)
        gu = fp4_pairs(xq, w13, s13, ex, tok, rows, None, P)
        h = swiglu_quant(gu, wt.reshape(-1)[sel], inter, limit)
        y2 = fp4_pairs(h, w2, s2, ex, rows, rows, None, P)
        for p in range(P):  # slot order within a token, as y2.view(T, topk, D).sum(1)
            routed[int(tok[p])] += y2[p]
    out = routed
    if shared is not None:
        out = routed + shared_expert(xq, *shared, limit).float()
    return {"out": out.to(torch.bfloat16), "routed": routed}


def hc_pre_norm_quant2(x: torch.Tensor, pre: torch.Tensor, w: torch.Tensor, eps: float):
    """CPU restatement of the two passes of dsv41/fused2.py:171-211.  x bf16 [B, hc, d], pre fp32 [B, hc], w [d] -> (y bf16, yq bf16,
    yqp bf16): pass 1 t = bf16(sum_h pre[h] * x[h]) accumulated in h order in fp32, var = sum(t^2) / d; pass 2
    y = bf16(t * (1 / sqrt(var + eps)) * w), yq = per-32 FP8 fake quantisation, yqp = yq with every 8 k stored as 0,4,2,6,1,5,3,7."""
    B, hc, d = x.shape
    acc = torch.zeros(B, d, dtype=torch.float32)
    for h in range(hc):
        acc = acc + pre[:, h:h + 1].float() * x[:, h].float()
    t = acc.to(torch.bfloat16).float()
    var = (t.double() ** 2).sum(dim=1, keepdim=True).float() / d
    y = (t * (1.0 / torch.sqrt(var + eps)) * w.float()).to(torch.bfloat16)
    yq = fake_quant_fp8(y, 32)
    perm = torch.tensor([0, 4, 2, 6, 1, 5, 3, 7])
    yqp = yq.view(B, d // 8, 8)[:, :, perm].reshape(B, d)
    return y, yq, yqp


def hc_post2(residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor, x=None, y2=None, ys=None) -> torch.Tensor:
    """CPU restatement of dsv41/fused2.py:505-536.  residual bf16 [B, hc, d], post fp32 [B, hc], comb fp32 [B, hc, hc]; v = x bf16 [B, d]
    or bf16(sum_k y2[:, k] + ys) with y2 fp32 [B, nsum, d]; returns the new residual: out[i] = bf16(post[i] * v + sum_h comb[h][i] * r[h])."""
    B, hc, d = residual.shape
    if y2 is not None:
        v = torch.zeros(B, d, dtype=torch.float32)
        for k in range(y2.shape[1]):
            v = v + y2[:, k].float()
        if ys is not None:
            v = v + ys.float()
        v = v.to(torch.bfloat16).float()
    else:
        v = x.float()
    r = residual.float()
    out = torch.empty_like(residual)
    for i in range(hc):
        acc = post[:, i:i + 1].float() * v
        for h in range(hc):
            acc = acc + comb[:, h, i].float().unsqueeze(1) * r[:, h]
        out[:, i] = acc.to(torch.bfloat16)
    return out


def group_pairs(expert: torch.Tensor, n_experts: int):
    expert = expert.to(torch.int32).contiguous()
    order = torch.empty(int((expert >= 0).sum()), dtype=torch.int32)
    counts = torch.empty(n_experts, dtype=torch.int32)
    lib().orc_group_pairs(_ptr(expert), expert.numel(), n_experts, _ptr(order), _ptr(counts))
    return order, counts


# ------------------------------------------------------------------ the reference's own compiled library
def host_has_avx512_bf16() -> bool:
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        return False
    return all(f in flags for f in ("avx512_bf16", "avx512vbmi", "avx512_vnni", "avx512f"))


class RefCpuMoe:
    """The reference's CPU routed-expert chain (dsv41/cpu/moe_cpu.cpp), exact mode 0 unless `int8_mode` says otherwise.
    One token per call, at most 16 experts, inter % 256 == 0, K % 128 == 0, K <= 8192 (moe_cpu.cpp:394-397, 444)."""

    def __init__(self, threads: int | None = None, int8_mode: int = 0):
        so = _build.build_reference()
        if so is None or not os.path.exists(so):
            raise RuntimeError("reference library not built (no reference checkout and no prebuilt oracle/_ref)")
        if not host_has_avx512_bf16():
            raise RuntimeError("host CPU lacks AVX-512 BF16/VBMI/VNNI; the reference library cannot run here")
        L = ctypes.CDLL(so)
        L.cpumoe_forward.restype = ctypes.c_int
        cpus = sorted(os.sched_getaffinity(0))
        if threads is None:
            threads = max(1, len(cpus) - 1)  # the reference leaves one core to the caller (dsv41/cpumoe.py:72-107)
        cpus = cpus[:threads]
        arr = (ctypes.c_int * len(cpus))(*cpus)
        got = L.cpumoe_init_list(arr, len(cpus), len(cpus))  # one NUMA group: cores_per_node = threads
        self.threads = int(got)
        L.cpumoe_set_int8(int(int8_mode))
        L.cpumoe_set_chunks(96, 64)
        self.L = L
        self.mode = int8_mode

    def set_mode(self, mode: int):
        self.L.cpumoe_set_int8(int(mode))
        self.mode = mode

    def forward(self, x: torch.Tensor, w13, s13, w2, s2, ids, weights, limit: float) -> torch.Tensor:
        """x bf16 [K]; w13 [E,2I,K/2] ... stacked uint8 CPU tensors; ids/weights: python lists. Returns fp32 [dim]."""
        x = _u16(x).view(-1)
        n = len(ids)
        assert 0 < n <= 16
        K = x.numel()
        inter, dim = w2.shape[2] * 2, w2.shape[1]
        P = ctypes.c_void_p * n
        p13 = P(*[w13[e].data_ptr() for e in ids])
        ps13 = P(*[s13[e].data_ptr() for e in ids])
        p2 = P(*[w2[e].data_ptr() for e in ids])
        ps2 = P(*[s2[e].data_ptr() for e in ids])
        wts = (ctypes.c_float * n)(*[float(v) for v in weights])
        out = torch.empty(dim, dtype=torch.float32)
        gu = torch.empty(16 * 2 * inter, dtype=torch.float32)
        h = torch.empty(16 * inter, dtype=torch.bfloat16)
        r = self.L.cpumoe_forward(p13, ps13, p2, ps2, n, _ptr(x), wts, _ptr(out), K, inter, dim, ctypes.c_float(limit), _ptr(gu), _ptr(h))
        assert r == 0
        return out
