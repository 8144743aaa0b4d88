"""Elementwise fusions on the MoE path, CUDA through the C-ABI.  Signatures of the reference's dsv41/fused.py."""
from __future__ import annotations

import torch

from . import _lib as L


def fake_quant_fp8(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Per-32 FP8 e4m3 quantise-dequantise with a power-of-two scale (dsv41/fused.py:72-83, MODE 0)."""
    assert block == 32 and x.dtype == torch.bfloat16, "the CUDA kernel handles bf16 with groups of 32"
    dev = L.require_cuda(x)
    xc = x.contiguous()
    y = torch.empty_like(xc)
    with torch.cuda.device(dev):
        L.check(L.lib().b200_fake_quant_fp8(L.ptr(xc), L.ptr(y), xc.numel(), L.stream_of(dev)), "b200_fake_quant_fp8")
    return y


def fake_quant_fp4(x, block=32, scale_e4m3=False):
    """FP4 activation quantisation (dsv41/fused.py:82-83) belongs to the attention indexer, which is outside this package."""
    raise NotImplementedError("fake_quant_fp4 is not on the MoE expert path")


def swiglu_quant(gu: torch.Tensor, weights: torch.Tensor | None, inter: int, limit: float, permute: bool = False) -> torch.Tensor:
    """gu fp32|bf16 [rows, 2*inter] (gate | up), weights fp32 [rows] or None -> bf16 [rows, inter], FP8-rounded per 32
    (dsv41/fused.py:309-316)."""
    dev = L.require_cuda(gu, weights)
    assert gu.dtype in (torch.float32, torch.bfloat16) and gu.shape[-1] == 2 * inter and inter % 32 == 0
    guc = gu.contiguous()
    rows = guc.numel() // (2 * inter)
    w = weights.to(torch.float32).contiguous() if weights is not None else None
    assert w is None or w.numel() == rows
    y = torch.empty(rows, inter, device=dev, dtype=torch.bfloat16)
    with torch.cuda.device(dev):
        L.check(L.lib().b200_swiglu_quant(L.ptr(guc), int(guc.dtype == torch.bfloat16), L.ptr(w), rows, inter, float(limit), int(bool(permute)),
                                          L.ptr(y), L.stream_of(dev)), "b200_swiglu_quant")
    return y
