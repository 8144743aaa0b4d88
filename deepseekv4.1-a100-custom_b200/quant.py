"""Number formats of the checkpoint, with the function names of the reference's dsv41/quant.py.  The activation fake quantisation
runs on the GPU only (csrc/elementwise.cu); the weight-format helpers below are decoders used to build bf16 views of a weight
(`W8.bf16()`) and by tests: they work on whatever device the weight lives on and are not on the hot path.  A torch statement of the
activation quantisation, for checking, lives with the other checkers in oracle/."""
from __future__ import annotations

import torch

FP8_MAX = 448.0
FP4_MAX = 6.0
# E2M1 code -> value: bit 3 sign, bits 2-1 exponent, bit 0 mantissa (dsv41/quant.py:24)
FP4_TABLE = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def e8m0_to_float(b: torch.Tensor) -> torch.Tensor:
    """E8M0 scale byte b -> fp32 2^(b - 127)."""
    b = b if b.dtype == torch.uint8 else b.view(torch.uint8)
    return torch.ldexp(torch.ones(b.shape, dtype=torch.float32, device=b.device), b.to(torch.int32) - 127)


def fake_quant_fp8(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Per-32 FP8 e4m3 quantise-dequantise of a bf16 CUDA tensor with a power-of-two scale (semantics of dsv41/quant.py:46-54)."""
    if not x.is_cuda:
        raise RuntimeError("b200 operators run on CUDA tensors only (there is no CPU path)")
    from .fused import fake_quant_fp8 as on_gpu
    return on_gpu(x, block)


def round_e2m1(v: torch.Tensor) -> torch.Tensor:
    """Nearest value of the E2M1 grid {0, .5, 1, 1.5, 2, 3, 4, 6} with the sign of v; a value half way between two grid points goes to
    the one whose code is even (ties to even), magnitudes above 6 saturate."""
    grid = FP4_TABLE[:8].to(v.device, torch.float32)
    a = v.abs().float().clamp(max=FP4_MAX).unsqueeze(-1)
    d = (a - grid).abs()
    # prefer even codes on exact ties: penalise odd codes by less than any real distance difference
    code = (d + (torch.arange(8, device=v.device) % 2) * 1e-7).argmin(dim=-1)
    return torch.copysign(grid[code], v.float()).to(v.dtype)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., K/2] -> fp32 [..., K] unscaled E2M1 values; the low nibble of a byte is the even k (dsv41/quant.py:98-103)."""
    p = packed.view(torch.uint8).to(torch.int64)
    codes = torch.stack((p % 16, p // 16), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return FP4_TABLE.to(packed.device)[codes]


def _expand_blocks(scale: torch.Tensor, n: int, k: int, block: int) -> torch.Tensor:
    """[ceil(n/block), ceil(k/block)] per-block values -> [n, k] per-element values."""
    rows = torch.arange(n, device=scale.device) // block
    cols = torch.arange(k, device=scale.device) // block
    return scale[rows][:, cols]


def dequant_fp4(packed: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    """One expert matrix, packed E2M1 [N, K/2] + E8M0 [N, K/block] -> bf16 [N, K]."""
    vals = unpack_fp4(packed)
    n, k = vals.shape
    return (vals.view(n, k // block, block) * e8m0_to_float(scale)[:, : k // block, None]).view(n, k).to(torch.bfloat16)


def dequant_fp8_block(w: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    """float8_e4m3fn [N, K] + E8M0 bytes per block x block tile -> bf16 [N, K]."""
    n, k = w.shape
    return (w.float() * _expand_blocks(e8m0_to_float(scale), n, k, block)).to(torch.bfloat16)


def dequant_fp8_f32block(w: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    """float8_e4m3fn [N, K] + fp32 scale per 128 x 128 tile -> fp32 [N, K] (a format the reference does not have)."""
    n, k = w.shape
    return w.float() * _expand_blocks(scale.float(), n, k, block)
