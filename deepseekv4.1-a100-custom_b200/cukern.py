"""Launchers of the CUDA kernels, with the names, argument order and dtypes of the reference's dsv41/cukern.py so that
its callers (decode.experts_tc, MoE.__call__, EPRuntime) can use them unchanged.  Every launcher allocates its own output
unless `out=` is given, launches on the current torch stream of the tensor's device and never synchronises.
"""
from __future__ import annotations

import torch

from . import _lib as L

_PERM8 = [0, 4, 2, 6, 1, 5, 3, 7]
FP4_W_MAX = 64  # tokens per group the reference's bucketing produces (dsv41/cukern.py:276-277); any size is accepted here
AUTO_ENGINE = True  # grouped FP4 / dense FP8 GEMMs pick the tensor-core kernel on the device when the activation is FP8-exact (tests switch it off)


def _i32(t: torch.Tensor | None, dev) -> torch.Tensor | None:
    if t is None:
        return None
    return t.to(device=dev, dtype=torch.int32).contiguous()


def _fp4_fmt(s: torch.Tensor) -> int:
    if s.dtype == torch.uint8:
        return L.FMT_FP4_E8M0
    if s.dtype == torch.bfloat16:
        return L.FMT_FP4_BF16S
    raise TypeError(f"expert scales must be uint8 (E8M0) or bfloat16, got {s.dtype}")


def grouped_fp4(x, w, s, grp_expert, grp_start, grp_count, pair_tok, pair_out, pair_w, n_pairs, *, x_perm8=False, shard_start=0,
                shard_n=1 << 30, zero_out=False, accumulate=False, out=None, n_out_rows=None):
    """Common launcher of b200_fp4_grouped_gemm (see include/b200_moe.h)."""
    dev = L.require_cuda(x, w, s, grp_expert, grp_start, out)
    E, N, Kh = w.shape
    K = Kh * 2
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1 and x.dim() == 2 and x.shape[1] == K
    assert w.dtype == torch.uint8 and w.is_contiguous() and s.is_contiguous() and s.shape == (E, N, K // 32)
    if out is None:
        rows = n_pairs if n_out_rows is None else n_out_rows
        out = (torch.zeros if accumulate else torch.empty)(rows, N, device=dev, dtype=torch.float32)
    assert out.dtype == torch.float32 and out.stride(-1) == 1
    ge, gs, gc = _i32(grp_expert, dev), _i32(grp_start, dev), _i32(grp_count, dev)
    pt, po = _i32(pair_tok, dev), _i32(pair_out, dev)
    pw = pair_w.to(device=dev, dtype=torch.float32).contiguous() if pair_w is not None else None
    G = ge.numel()
    assert gs.numel() >= (G if gc is not None else G + 1)
    lib = L.lib()
    fmt = _fp4_fmt(s)
    if fmt == L.FMT_FP4_E8M0 and K % 128 == 0 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0 and AUTO_ENGINE:
        # engine chosen on the device: the block-scaled tensor cores when the activation is FP8-exact (inside the MoE it always is), else
        # the weight-streaming kernel
        nbytes = lib.b200_fp4_grouped_auto_workspace_bytes(int(n_pairs), K)
        ws = L.workspace(dev, nbytes, "fp4_grouped_auto")
        with torch.cuda.device(dev):
            rc = lib.b200_fp4_grouped_gemm_auto(L.ptr(x), x.stride(0), int(bool(x_perm8)), L.ptr(w), w.stride(0) * w.element_size(), L.ptr(s), s.stride(0) * s.element_size(), E, N, K,
                                                L.ptr(ge), L.ptr(gs), L.ptr(gc), G, L.ptr(pt), L.ptr(po), L.ptr(pw), int(n_pairs), int(shard_start),
                                                int(min(shard_n, 1 << 30)), int(bool(zero_out)), int(bool(accumulate)), L.ptr(out), out.stride(0), L.ptr(ws),
                                                ws.numel(), L.stream_of(dev))
        L.check(rc, "b200_fp4_grouped_gemm_auto")
        return out
    nbytes = lib.b200_fp4_grouped_workspace_bytes(int(n_pairs))
    ws = L.workspace(dev, nbytes, "fp4_grouped")
    with torch.cuda.device(dev):
        rc = lib.b200_fp4_grouped_gemm(L.ptr(x), x.stride(0), int(bool(x_perm8)), L.ptr(w), w.stride(0) * w.element_size(), L.ptr(s),
                                       s.stride(0) * s.element_size(), fmt, E, N, K, L.ptr(ge), L.ptr(gs), L.ptr(gc), G, L.ptr(pt), L.ptr(po),
                                       L.ptr(pw), int(n_pairs), int(shard_start), int(min(shard_n, 1 << 30)), int(bool(zero_out)),
                                       int(bool(accumulate)), L.ptr(out), out.stride(0), L.ptr(ws), ws.numel(), L.stream_of(dev))
    L.check(rc, "b200_fp4_grouped_gemm")
    return out


_arange_cache: dict = {}


def _arange(n: int, dev) -> torch.Tensor:
    key = (n, dev)
    t = _arange_cache.get(key)
    if t is None:
        t = _arange_cache[key] = torch.arange(n, device=dev, dtype=torch.int32)
    return t


def fp4_gemv_pairs(x: torch.Tensor, w: torch.Tensor, s: torch.Tensor, row_in: torch.Tensor, expert: torch.Tensor, wt: torch.Tensor,
                   n_pairs: int) -> torch.Tensor:
    """x bf16 [rows_in, K]; w uint8 [E, N, K/2]; s uint8 [E, N, K/32]; row_in / expert int32 [pairs]; wt fp32 [pairs].
    Returns fp32 [pairs, N] = wt * x[row_in] @ W[expert]^T  (dsv41/cukern.py:60-77): one group per pair."""
    return grouped_fp4(x, w, s, expert, _arange(n_pairs + 1, x.device), None, row_in, None, wt, n_pairs)


def fp4_gemm_tc(xp: torch.Tensor, w: torch.Tensor, s: torch.Tensor, grp_expert: torch.Tensor, grp_start: torch.Tensor, pair_tok: torch.Tensor,
                n_pairs: int, max_tokens: int, shard_start: int = 0, shard_n: int = 1 << 30, zero_out: bool = False,
                out: torch.Tensor | None = None, min_tokens: int = 0) -> torch.Tensor:
    """xp: 8-k PERMUTED bf16 [rows, K] (permute_x); groups g: expert grp_expert[g] (global id, -1 = padding) with pairs
    grp_start[g] .. grp_start[g+1]-1, pair p reads x row pair_tok[p].  Returns fp32 [n_pairs, N].  Groups outside
    [shard_start, shard_start + shard_n) are skipped (zero_out: rows zeroed)  (dsv41/cukern.py:309-344).  max_tokens and
    min_tokens are accepted for compatibility; every group size runs on the same kernel."""
    assert xp.is_contiguous()
    return grouped_fp4(xp, w, s, grp_expert, grp_start, None, pair_tok, None, None, n_pairs, x_perm8=True, shard_start=shard_start, shard_n=shard_n,
                       zero_out=zero_out, out=out)


def fp4_gemv_m1(xp, w, s, grp_expert, grp_start, pair_tok, n_pairs, shard_start=0, shard_n=1 << 30, zero_out=False, out=None, kw=None, u=None):
    """One-token groups of a grouped expert GEMM (dsv41/cukern.py:286-306).  Same kernel as fp4_gemm_tc here; kw / u ignored."""
    return fp4_gemm_tc(xp, w, s, grp_expert, grp_start, pair_tok, n_pairs, 1, shard_start, shard_n, zero_out, out)


def permute_x(x: torch.Tensor) -> torch.Tensor:
    """bf16 [M, K] -> 8-k permuted copy (within every 8 k: 0,4,2,6,1,5,3,7)  (dsv41/cukern.py:270-273)."""
    dev = L.require_cuda(x)
    assert x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
    xc = x.contiguous()
    y = torch.empty_like(xc)
    with torch.cuda.device(dev):
        L.check(L.lib().b200_permute_x8(L.ptr(xc), L.ptr(y), xc.numel(), L.stream_of(dev)), "b200_permute_x8")
    return y


# --------------------------------------------------------------------------- FP8 dense
def _fp8(x, w8, s8, w_permk: bool, out_dtype, out=None):
    dev = L.require_cuda(x, w8, s8, out)
    M, K = x.shape
    N = w8.shape[0]
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and w8.is_contiguous() and s8.is_contiguous() and w8.shape[1] == K
    w8 = w8.view(torch.uint8)
    if s8.dtype == torch.uint8:
        fmt = L.FMT_FP8_E8M0
    elif s8.dtype == torch.float32:
        fmt = L.FMT_FP8_F32B
    else:
        raise TypeError(f"FP8 scales must be uint8 (E8M0 32x32) or float32 (128x128), got {s8.dtype}")
    assert out_dtype in (torch.bfloat16, torch.float32)
    if out is None:
        out = torch.empty(M, N, device=dev, dtype=out_dtype)
    assert out.dtype == out_dtype and out.stride(-1) == 1
    lib = L.lib()
    if fmt == L.FMT_FP8_E8M0 and M > 8 and K % 128 == 0 and AUTO_ENGINE and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0:
        # more than 8 rows: the tensor-core kernel reads the weights once (the streaming kernel once per 8 rows); it needs the weight bytes
        # in natural k order, kept beside a permuted tensor the first time it is used this way
        nat = w8 if not w_permk else _natural_copy(w8)
        ws = L.workspace(dev, lib.b200_fp8_gemm_auto_workspace_bytes(M, K), "fp8_auto")
        with torch.cuda.device(dev):
            rc = lib.b200_fp8_gemm_auto(L.ptr(x), x.stride(0), M, L.ptr(nat), L.ptr(w8) if w_permk else None, L.ptr(s8), s8.shape[1], N, K, L.ptr(out),
                                        int(out_dtype == torch.float32), out.stride(0), L.ptr(ws), ws.numel(), L.stream_of(dev))
        L.check(rc, "b200_fp8_gemm_auto")
        return out
    with torch.cuda.device(dev):
        rc = lib.b200_fp8_gemm(L.ptr(x), x.stride(0), M, L.ptr(w8), L.ptr(s8), fmt, s8.shape[1], int(bool(w_permk)), N, K, L.ptr(out),
                               int(out_dtype == torch.float32), out.stride(0), L.stream_of(dev))
    L.check(rc, "b200_fp8_gemm")
    return out


_natural: dict = {}


def _natural_copy(w8_permk: torch.Tensor) -> torch.Tensor:
    """Natural-k-order twin of a weight stored in the 16-k order of dsv41/w8.py:21-23 (made once per weight)."""
    key = (w8_permk.data_ptr(), tuple(w8_permk.shape), w8_permk.device)
    t = _natural.get(key)
    if t is None:
        from .w8 import unpermute_k
        t = _natural[key] = unpermute_k(w8_permk)
    return t


def fp8_gemv(x: torch.Tensor, w_fp8: torch.Tensor, s_u8: torch.Tensor) -> torch.Tensor:
    """x bf16 [1, K]; w_fp8 float8_e4m3fn/uint8 [N, K] in NATURAL k order; s_u8 uint8 [ceil(N/32), K/32] -> fp32 [1, N]
    (dsv41/cukern.py:80-96)."""
    return _fp8(x, w_fp8, s_u8, False, torch.float32)


def fp8_gemv_m1(x: torch.Tensor, w8: torch.Tensor, s8: torch.Tensor, group_cols: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """One-row FP8 GEMV, weights in the w8.PERM_K byte order -> bf16 [1, N]  (dsv41/cukern.py:116-133)."""
    if group_cols:
        raise NotImplementedError("block-diagonal use (attention o-projection) is outside the MoE path")
    return _fp8(x, w8, s8, True, torch.bfloat16, out)


def fp8_gemm_tc(x: torch.Tensor, w8: torch.Tensor, s8: torch.Tensor, group_cols: int = 0, out_dtype=torch.bfloat16, permuted: bool = True,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """x bf16 [M, K]; w8 uint8 e4m3 [N, K] in the w8.PERM_K byte order (permuted=False: natural order); s8 uint8 E8M0
    [ceil(N/32), K/32] or fp32 [ceil(N/128), ceil(K/128)].  Returns x @ dequant(w8, s8)^T as [M, N]  (dsv41/cukern.py:165-221)."""
    if group_cols:
        raise NotImplementedError("block-diagonal use (attention o-projection) is outside the MoE path")
    assert x.is_contiguous()
    return _fp8(x, w8, s8, permuted, out_dtype, out)


# --------------------------------------------------------------------------- device-side GPU messaging (expert parallelism)
# Same names and arguments as dsv41/cukern.py:348-434.  Every launcher enqueues on the current stream of `device`; destinations and
# flags may live on another GPU as long as this process can address them.  p2p_wait / p2p_wait_masked are bounded (see
# include/b200_moe.h): poll device_error() at the step's existing synchronisation point.
def _on(device, fn, what, *args):
    with torch.cuda.device(device):
        L.check(fn(*args, L.stream_of(device)), what)


def p2p_copy(dst: torch.Tensor, src: torch.Tensor, device: torch.device):
    """Copy src (contiguous, a multiple of 16 bytes) into dst with a kernel running on `device`."""
    n = src.numel() * src.element_size()
    assert src.is_contiguous() and n % 16 == 0 and dst.numel() * dst.element_size() >= n
    _on(device, L.lib().b200_p2p_copy, "b200_p2p_copy", L.ptr(dst), L.ptr(src), n)


def p2p_copy_row(dst_base: torch.Tensor, row_idx: torch.Tensor, src: torch.Tensor, device: torch.device, seq: torch.Tensor):
    """dst_base[seq[b], row_idx[b]] = src[b]; dst_base [S, rows, D], src [B, 1, D], row_idx / seq int64 [B]."""
    B = src.shape[0]
    row_bytes = src.numel() * src.element_size() // B
    assert src.is_contiguous() and src.shape[-1] == dst_base.shape[-1] and row_idx.dtype == torch.int64 and seq.dtype == torch.int64
    _on(device, L.lib().b200_p2p_copy_row, "b200_p2p_copy_row", L.ptr(dst_base), L.ptr(row_idx), L.ptr(src), row_bytes, B,
        dst_base.stride(0) * dst_base.element_size(), L.ptr(seq))


def p2p_sum_rows(dst: torch.Tensor, src: torch.Tensor, device: torch.device, groups: int = 1, dst_stride: int | None = None):
    """dst[g] = sum of the `rows` rows of group g of src fp32 [groups * rows, n]; dst rows `dst_stride` elements apart."""
    total, n = src.shape
    if dst_stride is None:
        dst_stride = dst.stride(0) if dst.dim() > 1 else n
    assert src.dtype == torch.float32 and dst.dtype == torch.float32 and src.is_contiguous()
    _on(device, L.lib().b200_sum_rows, "b200_sum_rows", L.ptr(dst), L.ptr(src), total // groups, n, groups, int(dst_stride))


def p2p_signal(flag_ptrs: torch.Tensor, seq: torch.Tensor, device: torch.device):
    """Set the int32 flags at the addresses in flag_ptrs (int64 tensor on `device`) to the value of seq (int32 scalar on `device`)."""
    assert flag_ptrs.dtype == torch.int64 and seq.dtype == torch.int32
    _on(device, L.lib().b200_p2p_signal, "b200_p2p_signal", L.ptr(flag_ptrs), flag_ptrs.numel(), L.ptr(seq))


def p2p_wait(flags: torch.Tensor, seq: torch.Tensor, device: torch.device):
    """Wait on the stream until all flags (int32 [n] on `device`) >= seq, or until the wait limit runs out (device_error() 3001)."""
    assert flags.dtype == torch.int32 and seq.dtype == torch.int32
    _on(device, L.lib().b200_p2p_wait, "b200_p2p_wait", L.ptr(flags), flags.numel(), L.ptr(seq), None)


def p2p_wait_masked(flags: torch.Tensor, seq: torch.Tensor, mask: torch.Tensor, device: torch.device):
    """The same for the flags whose mask entry (int32 [n], computed on the device) is non-zero."""
    assert flags.dtype == torch.int32 and seq.dtype == torch.int32 and mask.dtype == torch.int32 and mask.numel() == flags.numel()
    _on(device, L.lib().b200_p2p_wait, "b200_p2p_wait", L.ptr(flags), flags.numel(), L.ptr(seq), L.ptr(mask))


def p2p_seq_bump(seq: torch.Tensor, device: torch.device):
    _on(device, L.lib().b200_p2p_seq_bump, "b200_p2p_seq_bump", L.ptr(seq))


_counters: dict = {}


def p2p_multicast(dst_ptrs: torch.Tensor, src: torch.Tensor, flag_ptrs: torch.Tensor | None, seq: torch.Tensor, device: torch.device,
                  counter: torch.Tensor | None = None):
    """One launch: src into every destination address of dst_ptrs (int64 on `device`), then the flags at flag_ptrs get the value of seq."""
    n = src.numel() * src.element_size()
    assert src.is_contiguous() and n % 16 == 0 and dst_ptrs.dtype == torch.int64
    if flag_ptrs is not None and counter is None:
        counter = _counters.get(device)
        if counter is None:
            counter = _counters[device] = torch.zeros(1, dtype=torch.int32, device=device)
    _on(device, L.lib().b200_p2p_multicast, "b200_p2p_multicast", L.ptr(dst_ptrs), dst_ptrs.numel(), L.ptr(src), n, L.ptr(flag_ptrs), L.ptr(seq), L.ptr(counter))


def p2p_stamp(dst: torch.Tensor, device: torch.device):
    """The GPU's global nanosecond timer into dst (int64 scalar on `device`), stream-ordered."""
    _on(device, L.lib().b200_p2p_stamp, "b200_p2p_stamp", L.ptr(dst))


def memcpy_async(dst: torch.Tensor, src: torch.Tensor, device: torch.device, nbytes: int | None = None):
    """Copy-engine transfer on `device`'s current stream; dst may live on another GPU (dsv41/cukern.py:428-434)."""
    n = src.numel() * src.element_size() if nbytes is None else nbytes
    _on(device, L.lib().b200_memcpy_async, "b200_memcpy_async", L.ptr(dst), L.ptr(src), int(n))


def set_wait_limit_ns(ns: int):
    """Limit of the messaging waits on the current device (0: the 2 s default)."""
    L.check(L.lib().b200_set_wait_limit_ns(int(ns)), "b200_set_wait_limit_ns")


# --------------------------------------------------------------------------- the expert phase of one token in one call
_chain_layers: dict = {}


def expert_chain(xqp: torch.Tensor, xq: torch.Tensor, eid: torch.Tensor, wt: torch.Tensor, shard: tuple, sh: dict, moe, part: torch.Tensor,
                 ys: torch.Tensor | None, mode: int | None = None) -> None:
    """The whole expert phase of ONE token on this GPU (dsv41/cukern.py:504-547): the routed experts of the shard
    [shard[0], shard[0] + shard[1]) among the token's (eid, wt) pairs -> part fp32 [dim] (routing weights applied) and, when ys is
    given, the shared expert -> ys bf16 [dim].  xq: the token's FP8 fake-quantised activation bf16 [dim]; xqp (its 8-k permuted copy)
    and mode belong to the sm_80 kernels and are ignored.  sh: the shard dict {"w13","s13","w2","s2"}; moe: an object with n_experts
    (or n_routed_experts), inter, swiglu_limit, sh_w13, sh_w2 (W8 containers) as the reference's MoE.  Any dims with dim % 128 == 0 and
    inter % 128 == 0 (the reference's kernel exists for 5120 / 2304 only).  Runs the 4 launches of the decode path (routing copy +
    quantisation, gate/up GEMM with SwiGLU, down GEMM, combine)."""
    from .moe import MoELayer
    from .w8 import W8
    dev = L.require_cuda(xq, eid, wt, part, ys)
    key = (id(sh), id(moe), shard[0], ys is not None)
    layer = _chain_layers.get(key)
    if layer is None:
        def as_w8(w):
            return w if isinstance(w, W8) else W8(w.w8, w.s8, permuted=True)
        n_exp = getattr(moe, "n_experts", None) or getattr(moe, "n_routed_experts", None) or (shard[0] + shard[1])
        layer = _chain_layers[key] = MoELayer(sh["w13"], sh["s13"], sh["w2"], sh["s2"], n_experts=int(n_exp), topk=eid.numel(),
                                              sh_w13=as_w8(moe.sh_w13) if ys is not None else None, sh_w2=as_w8(moe.sh_w2) if ys is not None else None,
                                              swiglu_limit=float(moe.swiglu_limit), shard_start=int(shard[0]))
    x = xq.reshape(1, -1)
    assert x.shape[1] == layer.dim and part.dtype == torch.float32 and part.numel() == layer.dim and part.is_contiguous()
    layer.forward(x, None, eid=eid.reshape(1, -1), wt=wt.reshape(1, -1), final=False, want_routed=True, routed_out=part.view(1, -1), want_shared=ys is not None,
                  shared_out=ys.view(1, -1) if ys is not None else None)


# --------------------------------------------------------------------------- block-scaled tensor-core path (FP8 activations)
def mx_quantize_rows(x: torch.Tensor, src_row: torch.Tensor | None = None):
    """bf16 [rows_in, K] -> (q8 uint8 e4m3 [rows, K], sf uint8 E8M0 [rows, K/32]); src_row int32 [rows] gathers input rows.
    q8 * 2^(sf - 127) equals fake_quant_fp8(x) (dsv41/quant.py:46-64)."""
    dev = L.require_cuda(x, src_row)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 32 == 0
    K = x.shape[1]
    sr = _i32(src_row, dev)
    rows = sr.numel() if sr is not None else x.shape[0]
    q8 = torch.empty(rows + 128, K, device=dev, dtype=torch.uint8)[:rows]  # slack rows: tensor-map boxes may read past the last work
    sf = torch.empty(rows + 128, K // 32, device=dev, dtype=torch.uint8)[:rows]
    with torch.cuda.device(dev):
        L.check(L.lib().b200_mx_quantize_rows(L.ptr(x), x.stride(0), L.ptr(sr), rows, K, L.ptr(q8), L.ptr(sf), L.stream_of(dev)), "b200_mx_quantize_rows")
    return q8, sf


def mx_grouped(w, s, x8, xsf, grp_expert, grp_start, grp_count, pair_out, pair_w, n_rows, *, epilogue="f32", limit=0.0, round_gu_bf16=False,
               shard_start=0, shard_n=1 << 30, tokens_per_work=16, rows_per_tile=32, out=None, n_out_rows=None):
    """Launcher of b200_mx_grouped_gemm (include/b200_moe.h).  w uint8 [E, N, K/2] + s uint8 [E, N, K/32] (FP4) or w uint8 e4m3
    [N, K] natural k order + s uint8 [ceil(N/32), K/32] (FP8, grp_expert = None: every row against the one matrix)."""
    dev = L.require_cuda(w, s, x8, xsf, out)
    fp4 = w.dim() == 3
    if fp4:
        E, N, Kh = w.shape
        K = Kh * 2
        fmt, s_cols = L.FMT_FP4_E8M0, K // 32
        w_es, s_es = w.stride(0), s.stride(0)
    else:
        N, K = w.shape
        E, fmt, s_cols, w_es, s_es = 1, L.FMT_FP8_E8M0, s.shape[1], 0, 0
    assert w.is_contiguous() and s.is_contiguous() and x8.dtype == torch.uint8 and x8.shape[1] == K and x8.is_contiguous() and xsf.is_contiguous()
    epi = {"f32": 0, "swiglu_q8": 1, "bf16": 2}[epilogue]
    rows_out = n_rows if n_out_rows is None else n_out_rows
    out_sf = None
    if out is None:
        if epi == 1:
            out = torch.empty(rows_out + 128, N // 2, device=dev, dtype=torch.uint8)[:rows_out]
            out_sf = torch.empty(rows_out + 128, N // 64, device=dev, dtype=torch.uint8)[:rows_out]
        else:
            out = torch.empty(rows_out, N, device=dev, dtype=torch.float32 if epi == 0 else torch.bfloat16)
    elif epi == 1:
        out, out_sf = out
    ge, gs, gc = _i32(grp_expert, dev), _i32(grp_start, dev), _i32(grp_count, dev)
    po = _i32(pair_out, dev)
    pw = pair_w.to(device=dev, dtype=torch.float32).contiguous() if pair_w is not None else None
    lib = L.lib()
    ws = L.workspace(dev, lib.b200_mx_grouped_workspace_bytes(int(n_rows)), "mx_grouped")
    # the tensor map is bounded by the rows the underlying buffer really holds
    x8_rows = x8.untyped_storage().nbytes() // K if x8.storage_offset() == 0 else x8.shape[0]
    with torch.cuda.device(dev):
        rc = lib.b200_mx_grouped_gemm(L.ptr(w), w_es, L.ptr(s), s_es, s_cols, fmt, E, N, K, L.ptr(x8), x8_rows, L.ptr(xsf), L.ptr(ge), L.ptr(gs), L.ptr(gc),
                                      ge.numel() if ge is not None else 0, L.ptr(po), L.ptr(pw), int(n_rows), int(shard_start), int(min(shard_n, 1 << 30)), epi,
                                      float(limit), int(bool(round_gu_bf16)), L.ptr(out), out.stride(0), L.ptr(out_sf), int(tokens_per_work), int(rows_per_tile),
                                      L.ptr(ws), ws.numel(), L.stream_of(dev))
    L.check(rc, "b200_mx_grouped_gemm")
    return (out, out_sf) if epi == 1 else out


def scale_atoms(s: torch.Tensor, n_rows: int, K: int, dual: bool) -> torch.Tensor:
    """Load-time re-layout of E8M0 scales into the 512-byte atoms the tensor cores read (b200_scale_atoms, include/b200_moe.h).
    s uint8 [E, N, K/32] (expert scales, one row of scales per weight row) or [ceil(N/32), K/32] (dense FP8 format, 32x32 blocks);
    dual: a gate|up matrix (N = 2 * inter).  Returns uint8 [E, tiles, K/128, 2, 512]."""
    dev = L.require_cuda(s)
    assert s.dtype == torch.uint8 and s.is_contiguous() and K % 128 == 0
    lib = L.lib()
    if s.dim() == 3:
        E, fmt = s.shape[0], L.FMT_FP4_E8M0
        assert s.shape[1] == n_rows and s.shape[2] >= K // 32
    else:
        E, fmt = 1, L.FMT_FP8_E8M0
        assert s.shape[0] == (n_rows + 31) // 32 and s.shape[1] >= K // 32
    nbytes = lib.b200_scale_atoms_bytes(E, n_rows, K, int(dual))
    out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        L.check(lib.b200_scale_atoms(L.ptr(s), fmt, s.shape[-1], E, n_rows, K, int(dual), L.ptr(out), L.stream_of(dev)), "b200_scale_atoms")
    return out.view(E, -1, K // 128, 2, 512)


def device_error(device) -> int:
    """Synchronise the device's current stream and return (then clear) the device error word (0 = no bounded wait gave up)."""
    import ctypes
    code = ctypes.c_int(0)
    with torch.cuda.device(device):
        L.check(L.lib().b200_device_error(ctypes.byref(code), L.stream_of(device)), "b200_device_error")
    return code.value
