"""Single-matrix FP4 x BF16 GEMM / GEMV with the signatures of the reference's dsv41/kernels.py:114-168."""
from __future__ import annotations

import torch

from . import cukern


def fp4_gemm(a: torch.Tensor, w_packed: torch.Tensor, w_scale: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """a bf16 [M, K]; w_packed uint8/int8 [N, K/2]; w_scale uint8 E8M0 [N, K/32] -> [M, N]."""
    assert a.dtype == torch.bfloat16 and a.is_contiguous()
    M, K = a.shape
    N = w_packed.shape[0]
    assert w_packed.shape[1] * 2 == K and w_scale.shape == (N, K // 32), (w_packed.shape, w_scale.shape, K)
    dev = a.device
    ge = torch.zeros(1, device=dev, dtype=torch.int32)
    gs = torch.tensor([0, M], device=dev, dtype=torch.int32)
    c = cukern.grouped_fp4(a, w_packed.view(torch.uint8).unsqueeze(0), w_scale.unsqueeze(0), ge, gs, None, None, None, None, M)
    return c if out_dtype == torch.float32 else c.to(out_dtype)


def fp4_gemv(a: torch.Tensor, w_packed: torch.Tensor, w_scale: torch.Tensor, block_n: int = 8, block_k: int = 256) -> torch.Tensor:
    """Small-M variant (dsv41/kernels.py:114-127); block_n / block_k are tuning knobs of the sm_80 kernel and are ignored."""
    return fp4_gemm(a, w_packed, w_scale)
