"""Expert parallelism over one node: the experts of a layer are range-sharded over the ranks exactly as the reference
shards them (contiguous global id ranges, dsv41/load.py:299-306, shard dict of dsv41/load.py:213-232), tokens are data
parallel, one process per GPU over torch.distributed.

Step for the rank's local tokens:
  dispatch   every rank receives all tokens' activations and router logits (all-gather; the reference's owner pushes the
             same packet [x | eid | wt] to every peer, dsv41/ep.py:69-80, 403-410)
  compute    each rank runs the chain over ITS experts only -> fp32 partial sum per token (the reference's
             _experts_shard + p2p_sum_rows, dsv41/ep.py:324-338, 431-435)
  combine    all-to-all of the partial rows back to each token's home rank, summed there in rank order (deterministic),
             plus the shared expert, which every rank computes for its own tokens, then the bf16 rounding
             (dsv41/ep.py:457-460, dsv41/fused2.py:518-523)
The collectives never give a peer's memory to a kernel; received data lands in local HBM first.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_ranges(n_experts: int, world: int) -> list[tuple[int, int]]:
    """(start, n) per rank: contiguous, as even as possible, first shards one larger (dsv41/load.py:299-306)."""
    base, rem = divmod(n_experts, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append((start, n))
        start += n
    return out


def make_shard(device, start: int, n: int, w13, s13, w2, s2) -> dict:
    """The reference's shard contract: tensors [n, ...] holding global experts [start, start + n)."""
    assert w13.shape[0] == n and s13.shape[0] == n and w2.shape[0] == n and s2.shape[0] == n
    return {"device": device, "start": start, "n": n, "w13": w13, "s13": s13, "w2": w2, "s2": s2}


def split_tokens(tokens: int, world: int) -> list[tuple[int, int]]:
    """(first, count) of the tokens each rank owns (even split, remainder to the first ranks)."""
    return shard_ranges(tokens, world)


class EPMoE:
    """Expert-parallel MoE layer.  `partial_fn(x_all, logits_all) -> fp32 [T, D]` computes this rank's routed partial sums,
    `shared_fn(x_local, routed_local) -> bf16 [T_loc, D]` adds the shared expert and rounds.  By default both come from a
    `moe.MoELayer` that holds this rank's shard (CUDA); tests inject CPU stand-ins to exercise the exchange on gloo."""

    def __init__(self, layer=None, group=None, partial_fn=None, shared_fn=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.layer = layer
        self.partial_fn = partial_fn or self._partial_cuda
        self.shared_fn = shared_fn or self._shared_cuda

    def shared_bytes_per_rank(self, shared_bytes: int) -> float:
        """Bytes of the shared expert one rank streams per step (every rank streams all of it)."""
        return float(shared_bytes)

    # ---- CUDA defaults
    def _partial_cuda(self, x_all, logits_all):
        return self.layer.forward(x_all, logits_all, final=False, want_routed=True)

    def _shared_cuda(self, x_local, routed_local):
        from .fused2 import moe_combine
        return moe_combine(routed_local.unsqueeze(1), self.layer.shared_expert(x_local))

    # ---- the exchange
    def forward(self, x_local: torch.Tensor, logits_local: torch.Tensor, counts: list[int] | None = None) -> torch.Tensor:
        """x_local bf16 [T_r, D], logits_local [T_r, E] -> bf16 [T_r, D].  counts = tokens per rank (default: all equal T_r)."""
        W = self.world
        T_r = x_local.shape[0]
        counts = counts or [T_r] * W
        assert counts[self.rank] == T_r
        T = sum(counts)
        even = all(c == counts[0] for c in counts)
        # dispatch: all tokens to all ranks.  With equal token counts the rows [x | logits] of this rank travel in ONE all-gather (the
        # exchange is latency-bound: one collective less is worth more than the two small packing copies); the layer reads x and the
        # logits as strided views of the gathered buffer.
        D, E = x_local.shape[1], logits_local.shape[1]
        xb, lb = D * x_local.element_size(), E * logits_local.element_size()
        if even and W > 1 and x_local.is_cuda and xb % 16 == 0 and lb % 16 == 0:
            mine = torch.empty(T_r, xb + lb, dtype=torch.uint8, device=x_local.device)
            mine[:, :xb].view(x_local.dtype).copy_(x_local)
            mine[:, xb:].view(logits_local.dtype).copy_(logits_local)
            both = torch.empty(T, xb + lb, dtype=torch.uint8, device=x_local.device)
            dist.all_gather_into_tensor(both, mine, group=self.group)
            x_all = both[:, :xb].view(x_local.dtype)
            l_all = both[:, xb:].view(logits_local.dtype)
        else:
            x_all = torch.empty(T, D, dtype=x_local.dtype, device=x_local.device)
            l_all = torch.empty(T, E, dtype=logits_local.dtype, device=logits_local.device)
            if even:
                dist.all_gather_into_tensor(x_all, x_local.contiguous(), group=self.group)
                dist.all_gather_into_tensor(l_all, logits_local.contiguous(), group=self.group)
            else:
                dist.all_gather(list(x_all.split(counts)), x_local.contiguous(), group=self.group)
                dist.all_gather(list(l_all.split(counts)), logits_local.contiguous(), group=self.group)
        fused = self.layer is not None and self.partial_fn == self._partial_cuda and self.shared_fn == self._shared_cuda
        if fused:
            # local experts over all tokens; the shared expert rides in the same launches (its weight stream costs the same for all
            # tokens as for this rank's), this rank keeps its own rows of the result
            part, ys_all = self.layer.forward(x_all, l_all, final=False, want_routed=True, want_shared=True)
        else:
            part = self.partial_fn(x_all, l_all)  # fp32 [T, D]
        # combine: rows of rank r's tokens go to rank r and are summed there
        if even and W > 1 and part.is_cuda:
            routed = torch.empty(T_r, part.shape[1], dtype=part.dtype, device=part.device)
            dist.reduce_scatter_tensor(routed, part.contiguous(), group=self.group)
        else:
            recv = torch.empty(W * T_r, part.shape[1], dtype=part.dtype, device=part.device)
            dist.all_to_all_single(recv, part.contiguous(), output_split_sizes=[T_r] * W, input_split_sizes=counts, group=self.group)
            routed = recv.view(W, T_r, -1).sum(dim=0) if W > 1 else recv  # summed in rank order
        if fused:
            from .fused2 import moe_combine
            first = sum(counts[:self.rank])
            return moe_combine(routed.unsqueeze(1), ys_all[first:first + T_r] if ys_all is not None else None)
        return self.shared_fn(x_local, routed)

    __call__ = forward
