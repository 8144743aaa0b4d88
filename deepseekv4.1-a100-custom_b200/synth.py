"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark configurations (they stand in
for the model checkpoint, which is not distributed with this package).  Everything is generated from `torch.Generator`
seeds so that the CUDA path and the CPU checker see identical bits when tensors are generated on the CPU and copied.

    experts   packed E2M1 nibbles uniform in 0..255 per byte; one E8M0 scale byte per (row, 32 k) uniform in
              [scale_lo, scale_hi) (123..129 = 2^-4 .. 2^2, log-uniform), also available as bf16 powers of two
    shared    e4m3 codes of N(0, 0.02) weights, block scaled: fp32 blockmax/448 per 128x128, or E8M0 per 32x32
    tokens    bf16 N(0, 1)
    logits    bf16( N(0,1) + b_e ),  b_e = -s * ln(rank_e) for a seeded random ranking of the experts (Zipf, s = 1);
              rows whose 6th and 7th largest logits are equal are redrawn so that the top-k set is unique
"""
from __future__ import annotations

import math

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def make_experts(n_experts: int, dim: int, inter: int, seed: int, device="cpu", scale_lo: int = 123, scale_hi: int = 130):
    """-> dict(w13 u8 [E,2I,D/2], s13 u8 [E,2I,D/32], w2 u8 [E,D,I/2], s2 u8 [E,D,I/32])  (layout of dsv41/load.py:237-249)."""
    g = _gen(seed, device)
    r = lambda lo, hi, *shape: torch.randint(lo, hi, shape, dtype=torch.uint8, device=device, generator=g)
    return {"w13": r(0, 256, n_experts, 2 * inter, dim // 2), "s13": r(scale_lo, scale_hi, n_experts, 2 * inter, dim // 32),
            "w2": r(0, 256, n_experts, dim, inter // 2), "s2": r(scale_lo, scale_hi, n_experts, dim, inter // 32)}


def e8m0_to_bf16(s: torch.Tensor) -> torch.Tensor:
    """E8M0 bytes -> the same powers of two as bf16 (the BF16-scale form of the expert format)."""
    return torch.exp2(s.to(torch.float32) - 127.0).to(torch.bfloat16)


def quantize_fp8_block(w: torch.Tensor, kind: str):
    """fp32 [N, K] -> (e4m3 codes uint8 [N, K] natural k order, scales).  kind 'f32b': fp32 [ceil(N/128), ceil(K/128)] =
    blockmax/448; kind 'e8m0': uint8 [ceil(N/32), ceil(K/32)], scale 2^ceil(log2(blockmax/448))."""
    blk = 128 if kind == "f32b" else 32
    n, k = w.shape
    nb, kb = (n + blk - 1) // blk, (k + blk - 1) // blk
    wp = torch.zeros(nb * blk, kb * blk, dtype=torch.float32, device=w.device)
    wp[:n, :k] = w
    amax = wp.view(nb, blk, kb, blk).abs().amax(dim=(1, 3)).clamp_min(1e-12)
    if kind == "f32b":
        scale = (amax / 448.0).to(torch.float32)
        sfull = scale
    else:
        m, e = torch.frexp(amax / 448.0)
        e = e - (m == 0.5).to(e.dtype)
        scale = (e + 127).clamp(1, 254).to(torch.uint8)
        sfull = torch.exp2(e.to(torch.float32))
    q = (wp.view(nb, blk, kb, blk) / sfull.view(nb, 1, kb, 1)).clamp(-448, 448).view(nb * blk, kb * blk)[:n, :k]
    codes = q.to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    return codes, scale.contiguous()


def make_shared(dim: int, inter: int, seed: int, kind: str = "e8m0", device="cpu", std: float = 0.02):
    """Shared expert: -> dict(w13 codes [2I, D], s13, w2 codes [D, I], s2), natural k order."""
    g = _gen(seed, device)
    w13 = torch.randn(2 * inter, dim, generator=g, device=device) * std
    w2 = torch.randn(dim, inter, generator=g, device=device) * std
    c13, s13 = quantize_fp8_block(w13, kind)
    c2, s2 = quantize_fp8_block(w2, kind)
    return {"w13": c13, "s13": s13, "w2": c2, "s2": s2}


def make_tokens(tokens: int, dim: int, seed: int, device="cpu") -> torch.Tensor:
    return torch.randn(tokens, dim, generator=_gen(seed, device), device=device).to(torch.bfloat16)


def zipf_bias(n_experts: int, seed: int, s: float = 1.0, rotate: int = 0) -> torch.Tensor:
    """b_e = -s * ln(rank_e) for a seeded random ranking; `rotate` shifts the ranking cyclically over the expert ids."""
    g = _gen(seed, "cpu")
    perm = torch.randperm(n_experts, generator=g)
    rank = torch.empty(n_experts, dtype=torch.float32)
    rank[perm] = torch.arange(1, n_experts + 1, dtype=torch.float32)
    if rotate:
        rank = torch.roll(rank, int(rotate) % n_experts)
    return -s * torch.log(rank)


def make_logits(tokens: int, n_experts: int, seed: int, topk: int = 6, s: float = 1.0, rotate: int = 0) -> torch.Tensor:
    """bf16 [tokens, E] router logits with the Zipf bias folded in (generated on the CPU; copy to the device)."""
    g = _gen(seed + 7919, "cpu")
    bias = zipf_bias(n_experts, seed, s, rotate)
    logits = (torch.randn(tokens, n_experts, generator=g) + bias).to(torch.bfloat16)
    for _ in range(64):
        top = logits.float().topk(topk + 1, dim=-1).values
        bad = (top[:, topk - 1] == top[:, topk]).nonzero().flatten()
        if bad.numel() == 0:
            break
        logits[bad] = (torch.randn(bad.numel(), n_experts, generator=g) + bias).to(torch.bfloat16)
    return logits


def expert_bytes(dim: int, inter: int, scale_bytes: int = 1) -> int:
    """Bytes of one routed expert: packed gate/up + down matrices and their scales (13,369,344 at 4096 / 2048)."""
    return 2 * inter * dim // 2 + dim * inter // 2 + (2 * inter * dim // 32 + dim * inter // 32) * scale_bytes


def shared_bytes(dim: int, inter: int, kind: str = "e8m0") -> int:
    blk, sb = (32, 1) if kind == "e8m0" else (128, 4)
    sc = (math.ceil(2 * inter / blk) * math.ceil(dim / blk) + math.ceil(dim / blk) * math.ceil(inter / blk)) * sb
    return 2 * inter * dim + dim * inter + sc
