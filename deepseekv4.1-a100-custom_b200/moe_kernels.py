"""Grouped FP4 expert GEMM with the call surface of the reference's dsv41/moe_kernels.py: `GroupedPairs` (bucketing of (row, expert)
pairs on the device, no host synchronisation) and `grouped_fp4_gemm` (scatter-add of weight * a[row_in] @ W[expert]^T).  The bucketing
is the library's own counting sort (b200_group_pairs, csrc/pairs.cu); this module only allocates the tables and marshals pointers."""
from __future__ import annotations

import os

import torch

from . import _lib as L
from . import cukern


class GroupedPairs:
    """Pairs bucketed by expert (stable) and cut into tiles of at most `block_m` pairs of one expert.  Same attributes as the
    reference's class (dsv41/moe_kernels.py:76-132): n_pairs, block_m, expert, row_in, row_out, weight (all in sorted order), order
    (sorted position -> original pair), tile_expert, tile_start, tile_count.  The tile tables have a fixed capacity (experts +
    pairs // block_m); unused entries carry expert -1 and count 0 and are skipped by the kernels; `n_tiles` (int32 [1], on the
    device) holds the number in use."""

    def __init__(self, expert_ids: torch.Tensor, row_in: torch.Tensor, row_out: torch.Tensor, weight: torch.Tensor, block_m: int, n_experts: int = 384):
        dev = L.require_cuda(expert_ids, row_in, row_out, weight)
        P = int(expert_ids.numel())
        self.n_pairs, self.block_m, self.n_experts = P, int(block_m), int(n_experts)
        i32 = lambda t: t.reshape(-1).to(device=dev, dtype=torch.int32).contiguous()
        src = (i32(expert_ids), i32(row_in), i32(row_out), weight.reshape(-1).to(device=dev, dtype=torch.float32).contiguous())
        lib = L.lib()
        cap = lib.b200_group_pairs_max_tiles(P, self.n_experts, self.block_m)
        new_i = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
        self.order, self.expert, self.row_in, self.row_out = new_i(P), new_i(P), new_i(P), new_i(P)
        self.weight = torch.empty(P, dtype=torch.float32, device=dev)
        self.tile_expert, self.tile_start, self.tile_count, self.n_tiles = new_i(cap), new_i(cap), new_i(cap), new_i(1)
        ws = L.workspace(dev, lib.b200_group_pairs_workspace_bytes(self.n_experts), "group_pairs")
        with torch.cuda.device(dev):
            L.check(lib.b200_group_pairs(*(L.ptr(t) for t in src), P, self.n_experts, self.block_m, L.ptr(self.order), L.ptr(self.expert), L.ptr(self.row_in),
                                         L.ptr(self.row_out), L.ptr(self.weight), L.ptr(self.tile_expert), L.ptr(self.tile_start), L.ptr(self.tile_count),
                                         L.ptr(self.n_tiles), L.ptr(ws), ws.numel(), L.stream_of(dev)), "b200_group_pairs")

    def make_p2(self, row_in: torch.Tensor, row_out: torch.Tensor, weight: torch.Tensor | None = None) -> "GroupedPairs":
        """The same buckets and tiles for a second GEMM with other rows / weights (dsv41/moe_kernels.py:134-158): the new arrays are
        given in the ORIGINAL pair order and gathered into the sorted one; weight=None keeps this object's weights."""
        dev = self.order.device
        twin = GroupedPairs.__new__(GroupedPairs)
        twin.__dict__.update(self.__dict__)
        twin.row_in, twin.row_out = torch.empty_like(self.row_in), torch.empty_like(self.row_out)
        i32 = lambda t: t.reshape(-1).to(device=dev, dtype=torch.int32).contiguous()
        ri, ro = i32(row_in), i32(row_out)
        wsrc = None
        if weight is not None:
            wsrc = weight.reshape(-1).to(device=dev, dtype=torch.float32).contiguous()
            twin.weight = torch.empty_like(self.weight)
        with torch.cuda.device(dev):
            L.check(L.lib().b200_regroup_pairs(L.ptr(self.order), self.n_pairs, L.ptr(ri), L.ptr(ro), L.ptr(wsrc), L.ptr(twin.row_in), L.ptr(twin.row_out),
                                               L.ptr(twin.weight) if wsrc is not None else None, L.stream_of(dev)), "b200_regroup_pairs")
        return twin


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
    if pairs.n_pairs == 0:
        return out
    return cukern.grouped_fp4(a, w, s, pairs.tile_expert, pairs.tile_start, pairs.tile_count, pairs.row_in, pairs.row_out, pairs.weight, pairs.n_pairs,
                              accumulate=True, out=out)


def grouped_fp4_gemm_chunked(a, w, s, pairs: GroupedPairs, n_out_rows: int, *, chunk_rows: int | None = None) -> torch.Tensor:
    """Output-row chunked variant for long prefill (dsv41/moe_kernels.py:234-338): bounds the fp32 temporary.  Pairs whose output row
    falls outside a chunk are given the expert id -1, which the bucketing drops."""
    if chunk_rows is None:
        chunk_rows = int(os.environ.get("DSV41_MOE_OUT_CHUNK_ROWS", "4096"))
    if n_out_rows <= chunk_rows:
        return grouped_fp4_gemm(a, w, s, pairs, n_out_rows)
    outs = []
    for r0 in range(0, n_out_rows, chunk_rows):
        r1 = min(r0 + chunk_rows, n_out_rows)
        inside = (pairs.row_out >= r0) & (pairs.row_out < r1)
        part = GroupedPairs(torch.where(inside, pairs.expert, torch.full_like(pairs.expert, -1)), pairs.row_in, pairs.row_out - r0, pairs.weight, pairs.block_m,
                            n_experts=w.shape[0])
        outs.append(grouped_fp4_gemm(a, w, s, part, r1 - r0))
    return torch.cat(outs, dim=0)
