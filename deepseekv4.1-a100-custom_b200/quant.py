"""Numeric formats of the checkpoint as plain torch definitions: E8M0 scales, FP8 e4m3 block weights, packed E2M1 expert
weights and the activation fake quantisation.  Same function names and semantics as the reference's dsv41/quant.py; these
are the specification helpers (weight dequantisation for tests and for `W8.bf16()`), not the hot path.  The hot-path
activation quantisation is `fused.fake_quant_fp8` (CUDA)."""
from __future__ import annotations

import torch

FP8_MAX = 448.0
FP4_MAX = 6.0
# E2M1 code -> value (dsv41/quant.py:24)
FP4_TABLE = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def e8m0_to_float(b: torch.Tensor) -> torch.Tensor:
    """uint8 scale byte -> fp32 2^(b-127)  (dsv41/quant.py:27-31)."""
    if b.dtype != torch.uint8:
        b = b.view(torch.uint8)
    return torch.exp2(b.to(torch.float32) - 127.0)


def ceil_log2(x: torch.Tensor) -> torch.Tensor:
    """exact ceil(log2 x), x > 0  (dsv41/quant.py:34-37)."""
    m, e = torch.frexp(x)
    return e - (m == 0.5).to(e.dtype)


def pow2_scale(amax: torch.Tensor, qmax: float) -> torch.Tensor:
    """2^ceil(log2(amax / qmax))  (dsv41/quant.py:40-42)."""
    return torch.exp2(ceil_log2(amax / qmax).to(torch.float32))


def fake_quant_fp8(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Per-`block` FP8 quantise-dequantise with a power-of-two scale (dsv41/quant.py:46-54).  CUDA tensors with
    block == 32 run the CUDA kernel; anything else evaluates the torch definition."""
    if x.is_cuda and block == 32 and x.dtype == torch.bfloat16:
        from .fused import fake_quant_fp8 as _fq
        return _fq(x, block)
    shape = x.shape
    xg = x.float().reshape(-1, block)
    amax = xg.abs().amax(dim=-1, keepdim=True).clamp_min(1e-4)
    s = pow2_scale(amax, FP8_MAX)
    q = (xg / s).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).float()
    return (q * s).reshape(shape).to(x.dtype)


def round_e2m1(v: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 grid value, ties to even, |v| <= 6  (dsv41/quant.py:67-71)."""
    a = v.abs()
    r = torch.where(a < 2.0, torch.round(a * 2.0) / 2.0, torch.where(a < 4.0, torch.round(a), torch.round(a / 2.0) * 2.0))
    return torch.copysign(r.clamp(max=FP4_MAX), v)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K/2] -> fp32 [N, K] unscaled E2M1 values; low nibble = even k  (dsv41/quant.py:98-103)."""
    p = packed.view(torch.uint8)
    tab = FP4_TABLE.to(p.device)
    return torch.stack([tab[(p & 0x0F).long()], tab[(p >> 4).long()]], dim=-1).flatten(-2)


def dequant_fp4(packed: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Slow reference dequantisation of one expert matrix -> bf16 [N, K]  (dsv41/quant.py:106-110)."""
    return (unpack_fp4(packed) * e8m0_to_float(scale).repeat_interleave(block, 1)).to(torch.bfloat16)


def dequant_fp8_block(w: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    """float8_e4m3fn [N, K] + E8M0 [ceil(N/block), ceil(K/block)] -> bf16 [N, K]  (dsv41/quant.py:90-95)."""
    n, k = w.shape
    s = e8m0_to_float(scale)[: (n + block - 1) // block, : (k + block - 1) // block]
    s = s.repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return (w.float() * s).to(torch.bfloat16)


def dequant_fp8_f32block(w: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    """float8_e4m3fn [N, K] + fp32 [ceil(N/128), ceil(K/128)] -> fp32 [N, K] (the 128x128 block-scale format; the reference
    has no counterpart)."""
    n, k = w.shape
    s = scale.float().repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return w.float() * s
