"""TEST INFRASTRUCTURE ONLY: torch statements of the activation quantisation, used to cross-check the C oracle and the CUDA kernels on
the CPU.  Follows dsv41/quant.py:34-54 (exact ceil(log2), power-of-two scale, clamp, e4m3 rounding)."""
from __future__ import annotations

import torch

FP8_MAX = 448.0


def ceil_log2(x: torch.Tensor) -> torch.Tensor:
    """exact ceil(log2 x) for x > 0, from the binary exponent (dsv41/quant.py:34-37)."""
    mant, exp = torch.frexp(x)          # x = mant * 2^exp, mant in [0.5, 1)
    return torch.where(mant == 0.5, exp - 1, exp)


def pow2_scale(amax: torch.Tensor, qmax: float) -> torch.Tensor:
    """2^ceil(log2(amax / qmax)) (dsv41/quant.py:40-42)."""
    return torch.ldexp(torch.ones_like(amax, dtype=torch.float32), ceil_log2(amax / qmax).to(torch.int32))


def fake_quant_fp8(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Per-`block` quantise-dequantise through float8_e4m3fn with the scale above; amax is floored at 1e-4 (dsv41/quant.py:46-54)."""
    groups = x.float().reshape(-1, block)
    scale = pow2_scale(groups.abs().amax(dim=1, keepdim=True).clamp_min(1e-4), FP8_MAX)
    codes = (groups / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return (codes.float() * scale).reshape(x.shape).to(x.dtype)
