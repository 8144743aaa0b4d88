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


def moe_combine(y2: torch.Tensor, ys: torch.Tensor | None) -> torch.Tensor:
    """The MoE branch of hc_post2_ (dsv41/fused2.py:518-523): bf16( sum over dim 1 of y2 fp32 [B, nsum, d] + ys bf16 [B, d] )."""
    dev = L.require_cuda(y2, ys)
    B, nsum, d = y2.shape
    y2c = y2.to(torch.float32).contiguous()
    ysc = ys.to(torch.bfloat16).contiguous() if ys is not None else None
    out = torch.empty(B, d, device=dev, dtype=torch.bfloat16)
    with torch.cuda.device(dev):
        L.check(L.lib().b200_moe_combine(L.ptr(y2c), L.ptr(ysc), L.ptr(out), B, nsum, d, L.stream_of(dev)), "b200_moe_combine")
    return out
