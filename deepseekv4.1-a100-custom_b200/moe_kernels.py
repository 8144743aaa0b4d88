"""Grouped FP4 expert GEMM with the call surface of the reference's dsv41/moe_kernels.py: `GroupedPairs` (device-side
bucketing of (row, expert) pairs, no host synchronisation) and `grouped_fp4_gemm` (scatter-add of weight * a[row_in] @ W[expert]^T)."""
from __future__ import annotations

import os

import torch

from . import cukern


class GroupedPairs:
    """Pairs sorted by expert + tile table, built with torch ops on the device only (dsv41/moe_kernels.py:76-132).
    Fields: n_pairs, block_m, expert, row_in, row_out, weight, order (sorted case), tile_expert, tile_start, tile_count."""

    def __init__(self, expert_ids: torch.Tensor, row_in: torch.Tensor, row_out: torch.Tensor, weight: torch.Tensor, block_m: int, n_experts: int = 384):
        self.n_pairs = int(expert_ids.numel())
        self.block_m = block_m
        dev = expert_ids.device
        cast = lambda t, dt: t.to(device=dev, dtype=dt).contiguous()
        if self.n_pairs <= 64:  # decode: one tile per pair, unsorted
            self.expert, self.row_in, self.row_out = cast(expert_ids, torch.int32), cast(row_in, torch.int32), cast(row_out, torch.int32)
            self.weight = cast(weight, torch.float32)
            self.tile_expert = self.expert
            self.tile_start = torch.arange(self.n_pairs, dtype=torch.int32, device=dev)
            self.tile_count = torch.ones(self.n_pairs, dtype=torch.int32, device=dev)
            return
        order = torch.argsort(expert_ids, stable=True)
        self.order = order
        self.expert = cast(expert_ids[order], torch.int32)
        self.row_in, self.row_out = cast(row_in[order], torch.int32), cast(row_out[order], torch.int32)
        self.weight = cast(weight[order], torch.float32)
        counts = torch.bincount(self.expert.long(), minlength=n_experts)
        starts = torch.cumsum(counts, 0) - counts
        tiles_per = (counts + (block_m - 1)) // block_m
        self.tile_expert = torch.repeat_interleave(torch.arange(n_experts, dtype=torch.int32, device=dev), tiles_per)
        first_tile = torch.cumsum(tiles_per, 0) - tiles_per
        local = torch.arange(self.tile_expert.numel(), dtype=torch.int32, device=dev) - first_tile[self.tile_expert.long()].to(torch.int32)
        te = self.tile_expert.long()
        self.tile_start = (starts[te].to(torch.int32) + local * block_m).contiguous()
        self.tile_count = torch.clamp(counts[te].to(torch.int32) - local * block_m, min=0, max=block_m).contiguous()

    def make_p2(self, row_in: torch.Tensor, row_out: torch.Tensor, weight: torch.Tensor | None = None) -> "GroupedPairs":
        """Same sort order and tiles with new rows / weights (dsv41/moe_kernels.py:134-158)."""
        p2 = object.__new__(GroupedPairs)
        p2.n_pairs, p2.block_m, p2.expert = self.n_pairs, self.block_m, self.expert
        p2.order = getattr(self, "order", None)
        dev = self.expert.device
        sel = (lambda t: t[p2.order]) if p2.order is not None else (lambda t: t)
        p2.row_in = sel(row_in).to(device=dev, dtype=torch.int32).contiguous()
        p2.row_out = sel(row_out).to(device=dev, dtype=torch.int32).contiguous()
        p2.weight = self.weight if weight is None else sel(weight).to(device=dev, dtype=torch.float32).contiguous()
        p2.tile_expert, p2.tile_start, p2.tile_count = self.tile_expert, self.tile_start, self.tile_count
        return p2


def grouped_fp4_gemm(a: torch.Tensor, w: torch.Tensor, s: torch.Tensor, pairs: GroupedPairs, n_out_rows: int, out: torch.Tensor | None = None,
                     block_m: int | None = None) -> torch.Tensor:
    """a bf16 [rows_in, K]; w uint8 [E, N, K/2]; s uint8 [E, N, K/32] -> fp32 [n_out_rows, N] with
    out[row_out] += weight * a[row_in] @ W[expert]^T accumulated over the pairs (dsv41/moe_kernels.py:161-231)."""
    E, N = w.shape[0], w.shape[1]
    K = a.shape[1]
    if w.device != a.device or s.device != a.device:
        raise RuntimeError(f"grouped_fp4_gemm device mismatch: a={a.device} w={w.device} s={s.device}")
    assert s.shape == (E, N, K // 32)
    if out is None:
        out = torch.zeros(n_out_rows, N, device=a.device, dtype=torch.float32)
    if pairs.tile_expert.numel() == 0:
        return out
    return cukern.grouped_fp4(a, w, s, pairs.tile_expert, pairs.tile_start, pairs.tile_count, pairs.row_in, pairs.row_out, pairs.weight, pairs.n_pairs,
                              accumulate=True, out=out)


def grouped_fp4_gemm_chunked(a, w, s, pairs: GroupedPairs, n_out_rows: int, *, chunk_rows: int | None = None) -> torch.Tensor:
    """Output-row chunked variant for long prefill (dsv41/moe_kernels.py:234-338): bounds the fp32 temporary."""
    if chunk_rows is None:
        chunk_rows = int(os.environ.get("DSV41_MOE_OUT_CHUNK_ROWS", "4096"))
    if n_out_rows <= chunk_rows:
        return grouped_fp4_gemm(a, w, s, pairs, n_out_rows)
    outs = []
    for r0 in range(0, n_out_rows, chunk_rows):
        r1 = min(r0 + chunk_rows, n_out_rows)
        mask = (pairs.row_out >= r0) & (pairs.row_out < r1)
        cp = GroupedPairs(pairs.expert[mask], pairs.row_in[mask], pairs.row_out[mask] - r0, pairs.weight[mask], pairs.block_m, n_experts=w.shape[0])
        outs.append(grouped_fp4_gemm(a, w, s, cp, r1 - r0))
    return torch.cat(outs, dim=0)
