"""Router of the MoE layer (signature of the reference's dsv41/fused2.py:486-502) and the routed+shared combine."""
from __future__ import annotations

import torch

from . import _lib as L


def gate_topk(scores: torch.Tensor, bias: torch.Tensor | None, temp: float, topk: int, route_scale: float, score_func: str, norm: bool,
              eid: torch.Tensor | None = None, wt: torch.Tensor | None = None):
    """scores fp32 [B, E] -> (eid int32 [B, topk], wt fp32 [B, topk]); [topk] vectors when B == 1 and no buffers are given."""
    dev = L.require_cuda(scores, bias, eid, wt)
    E = scores.shape[-1]
    B = scores.numel() // E
    squeeze = B == 1 and eid is None and wt is None
    if eid is None:
        eid = torch.empty(B, topk, device=dev, dtype=torch.int32)
    if wt is None:
        wt = torch.empty(B, topk, device=dev, dtype=torch.float32)
    assert eid.dtype == torch.int32 and wt.dtype == torch.float32 and eid.is_contiguous() and wt.is_contiguous()
    s = scores.to(torch.float32).contiguous()
    b = bias.to(torch.float32).contiguous() if bias is not None else None
    with torch.cuda.device(dev):
        L.check(L.lib().b200_gate_topk(L.ptr(s), L.ptr(b), B, E, float(temp), int(topk), float(route_scale), L.SCORE_MODES[score_func], int(bool(norm)),
                                       L.ptr(eid), L.ptr(wt), L.stream_of(dev)), "b200_gate_topk")
    if squeeze:
        return eid.view(-1), wt.view(-1)
    return eid, wt


def moe_combine(y2: torch.Tensor, ys: torch.Tensor | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """The MoE branch of hc_post2_ (dsv41/fused2.py:518-523): bf16( sum over dim 1 of y2 fp32 [B, nsum, d] + ys bf16 [B, d] )."""
    dev = L.require_cuda(y2, ys, out)
    B, nsum, d = y2.shape
    y2c = y2.to(torch.float32).contiguous()
    ysc = ys.to(torch.bfloat16).contiguous() if ys is not None else None
    if out is None:
        out = torch.empty(B, d, device=dev, dtype=torch.bfloat16)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (B, d)
    with torch.cuda.device(dev):
        L.check(L.lib().b200_moe_combine(L.ptr(y2c), L.ptr(ysc), L.ptr(out), B, nsum, d, L.stream_of(dev)), "b200_moe_combine")
    return out


def hc_pre_norm_quant2(x, pre_in, w, eps, want_f32=False, out=None, want_perm=False):
    """x bf16 [B, 1, hc, d]; pre_in fp32 [B, hc] (or [hc] for B = 1); w [d] norm weight.  Returns (y, yq, yf | None[, yqp]) as the
    reference does (dsv41/fused2.py:213-246): y = rmsnorm of the hyper-connection pre-mix, yq its per-32 FP8 fake quantisation,
    yf = y in fp32, yqp = yq in the 8-k permuted order.  `out`: optional dict of persistent output buffers (keys y, yq, yf, yqp)."""
    dev = L.require_cuda(x, pre_in, w)
    hc, d = x.shape[-2], x.shape[-1]
    B = x.shape[0]
    out = out or {}
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and w.dtype in (torch.bfloat16, torch.float32) and w.numel() == d
    pre = pre_in.to(torch.float32).contiguous()
    assert pre.numel() == B * hc

    def buf(key, dtype):
        t = out.get(key)
        return t if t is not None else torch.empty(B, d, device=dev, dtype=dtype)

    y, yq = buf("y", torch.bfloat16), buf("yq", torch.bfloat16)
    yf = buf("yf", torch.float32) if want_f32 else None
    yqp = buf("yqp", torch.bfloat16) if want_perm else None
    with torch.cuda.device(dev):
        L.check(L.lib().b200_hc_pre_norm_quant2(L.ptr(x), L.ptr(pre), L.ptr(w.contiguous()), int(w.dtype == torch.float32), float(eps), B, hc, d, L.ptr(y),
                                                L.ptr(yq), L.ptr(yf), L.ptr(yqp), L.stream_of(dev)), "b200_hc_pre_norm_quant2")
    return (y, yq, yf, yqp) if want_perm else (y, yq, yf)


def hc_post2_(x, residual, post, comb, y2=None, ys=None, y2_sum_first=False):
    """In-place hyper-connection post mix (dsv41/fused2.py:539-558): residual [B, 1, hc, d] bf16 <- post * v + comb^T residual, with v = x
    (bf16 [B, d]) or the MoE pieces: y2 fp32 [B, nsum, d] (or [nsum, d] for B = 1, or [nsum, B, d] with y2_sum_first) summed, plus ys
    bf16 [B, d] (the shared expert), rounded to bf16.  post [B, hc], comb [B, hc, hc] fp32 (leading B optional when B = 1)."""
    dev = L.require_cuda(residual, x, y2, ys, post, comb)
    hc, d = residual.shape[-2], residual.shape[-1]
    B = residual.shape[0]
    assert residual.dtype == torch.bfloat16 and residual.is_contiguous()
    if y2 is None:
        assert x is not None and x.dtype == torch.bfloat16
        nsum, rs, ss = 0, 0, 0
        x = x.contiguous()
    elif y2_sum_first:
        y2 = y2.to(torch.float32).contiguous()
        nsum, rs, ss = y2.shape[0], d, y2.shape[1] * d
    else:
        y2 = y2.to(torch.float32).contiguous()
        nsum, rs, ss = y2.shape[-2], y2.shape[-2] * d, d
    ysc = ys.contiguous() if ys is not None else None
    with torch.cuda.device(dev):
        L.check(L.lib().b200_hc_post2(L.ptr(x if y2 is None else None), L.ptr(y2), L.ptr(ysc), rs, ss, nsum, L.ptr(residual),
                                      L.ptr(post.to(torch.float32).contiguous()), L.ptr(comb.to(torch.float32).contiguous()), B, hc, d, L.stream_of(dev)),
                "b200_hc_post2")
    return residual
