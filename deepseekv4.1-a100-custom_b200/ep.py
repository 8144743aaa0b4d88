"""Expert parallelism over one node: the experts of a layer are range-sharded over the ranks exactly as the reference
shards them (contiguous global id ranges, dsv41/load.py:299-306, shard dict of dsv41/load.py:213-232), tokens are data
parallel, one process per GPU over torch.distributed.

Step for the rank's local tokens:
  dispatch   every rank receives all tokens' activations and router logits: ONE all-gather of rows [x | logits] (the reference's owner
             pushes the same packet [x | eid | wt] to every peer, dsv41/ep.py:69-80, 403-410)
  compute    each rank runs the chain over ITS experts only -> fp32 partial sum per token (the reference's
             _experts_shard + p2p_sum_rows, dsv41/ep.py:324-338, 431-435); the shared expert rides in the same launches
  combine    reduce-scatter of the partial rows to each token's home rank (NCCL adds them in an order its topology fixes; with uneven
             token counts an all-to-all and a sum in rank order instead), plus the shared expert's rows of this rank, then the bf16
             rounding (dsv41/ep.py:457-460, dsv41/fused2.py:518-523)
The collectives never give a peer's memory to a kernel; received data lands in local HBM first.  With equal token counts the step
uses persistent buffers only (no allocation, no host synchronisation), so a serving loop can capture it in a CUDA graph.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_ranges(n_experts: int, world: int) -> list[tuple[int, int]]:
    """(start, n) per rank: contiguous ranges with boundaries at floor(E * r / world), as the reference's loader cuts them
    (dsv41/load.py:299-306)."""
    from .load import shard_bounds
    return shard_bounds(n_experts, world)


def make_shard(device, start: int, n: int, w13, s13, w2, s2) -> dict:
    """The reference's shard contract: tensors [n, ...] holding global experts [start, start + n)."""
    assert w13.shape[0] == n and s13.shape[0] == n and w2.shape[0] == n and s2.shape[0] == n
    return {"device": device, "start": start, "n": n, "w13": w13, "s13": s13, "w2": w2, "s2": s2}


def split_tokens(tokens: int, world: int) -> list[tuple[int, int]]:
    """(first, count) of the tokens each rank owns: as even as possible, the first ranks take the remainder."""
    base, rem = divmod(tokens, world)
    out, first = [], 0
    for r in range(world):
        c = base + (1 if r < rem else 0)
        out.append((first, c))
        first += c
    return out


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
        self._bufs: dict = {}

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
    def _buffers(self, T_r: int, T: int, x_local: torch.Tensor, logits_local: torch.Tensor):
        """Persistent exchange buffers of the fused CUDA step, one set per (tokens, dtypes)."""
        D, E = x_local.shape[1], logits_local.shape[1]
        key = (T_r, T, D, E, x_local.dtype, logits_local.dtype)
        b = self._bufs.get(key)
        if b is None:
            dev = x_local.device
            xb, lb = D * x_local.element_size(), E * logits_local.element_size()
            b = {"xb": xb, "lb": lb,
                 "mine": torch.empty(T_r, xb + lb, dtype=torch.uint8, device=dev),
                 "both": torch.empty(T, xb + lb, dtype=torch.uint8, device=dev),
                 "part": torch.empty(T, D, dtype=torch.float32, device=dev),
                 "ys": torch.empty(T, D, dtype=torch.bfloat16, device=dev),
                 "routed": torch.empty(T_r, D, dtype=torch.float32, device=dev)}
            self._bufs[key] = b
        return b

    def forward(self, x_local: torch.Tensor, logits_local: torch.Tensor, counts: list[int] | None = None, out: torch.Tensor | None = None,
                events=None) -> torch.Tensor:
        """x_local bf16 [T_r, D], logits_local [T_r, E] -> bf16 [T_r, D].  counts = tokens per rank (default: all equal T_r); out: optional
        result buffer; events: optional list of 4 torch.cuda.Event recorded after the pack, the dispatch, the compute and the combine."""
        W = self.world
        T_r = x_local.shape[0]
        counts = counts or [T_r] * W
        assert counts[self.rank] == T_r
        T = sum(counts)
        even = all(c == counts[0] for c in counts)
        D, E = x_local.shape[1], logits_local.shape[1]
        xb, lb = D * x_local.element_size(), E * logits_local.element_size()
        fused = self.layer is not None and self.partial_fn == self._partial_cuda and self.shared_fn == self._shared_cuda
        mark = (lambda i: events[i].record()) if events is not None else (lambda i: None)
        if fused and even and W > 1 and xb % 16 == 0 and lb % 16 == 0:
            # ---- the fast path: persistent buffers, 2 packing copies + 1 all-gather + the layer's launches + 1 reduce-scatter + 1 combine
            from .fused2 import moe_combine
            b = self._buffers(T_r, T, x_local, logits_local)
            b["mine"][:, :xb].view(x_local.dtype).copy_(x_local)
            b["mine"][:, xb:].view(logits_local.dtype).copy_(logits_local)
            mark(0)
            dist.all_gather_into_tensor(b["both"], b["mine"], group=self.group)
            mark(1)
            x_all = b["both"][:, :xb].view(x_local.dtype)
            l_all = b["both"][:, xb:].view(logits_local.dtype)
            # local experts over all tokens; the shared expert rides in the same launches, this rank keeps its own rows of the result
            has_sh = self.layer.sh_w13 is not None
            self.layer.forward(x_all, l_all, final=False, want_routed=True, routed_out=b["part"], want_shared=has_sh, shared_out=b["ys"] if has_sh else None)
            mark(2)
            dist.reduce_scatter_tensor(b["routed"], b["part"], group=self.group)
            first = sum(counts[:self.rank])
            res = moe_combine(b["routed"].unsqueeze(1), b["ys"][first:first + T_r] if has_sh else None, out=out)
            mark(3)
            return res
        # ---- general path (uneven token counts, CPU stand-ins of the tests): separate gathers, all-to-all, sum in rank order
        x_all = torch.empty(T, D, dtype=x_local.dtype, device=x_local.device)
        l_all = torch.empty(T, E, dtype=logits_local.dtype, device=logits_local.device)
        if even:
            dist.all_gather_into_tensor(x_all, x_local.contiguous(), group=self.group)
            dist.all_gather_into_tensor(l_all, logits_local.contiguous(), group=self.group)
        else:
            dist.all_gather(list(x_all.split(counts)), x_local.contiguous(), group=self.group)
            dist.all_gather(list(l_all.split(counts)), logits_local.contiguous(), group=self.group)
        ys_all = None
        if fused:
            part, ys_all = self.layer.forward(x_all, l_all, final=False, want_routed=True, want_shared=True) if self.layer.sh_w13 is not None else \
                (self.layer.forward(x_all, l_all, final=False, want_routed=True), None)
        else:
            part = self.partial_fn(x_all, l_all)  # fp32 [T, D]
        recv = torch.empty(W * T_r, part.shape[1], dtype=part.dtype, device=part.device)
        dist.all_to_all_single(recv, part.contiguous(), output_split_sizes=[T_r] * W, input_split_sizes=counts, group=self.group)
        routed = recv.view(W, T_r, -1).sum(dim=0) if W > 1 else recv  # summed in rank order
        if fused:
            from .fused2 import moe_combine
            first = sum(counts[:self.rank])
            return moe_combine(routed.unsqueeze(1), ys_all[first:first + T_r] if ys_all is not None else None, out=out)
        res = self.shared_fn(x_local, routed)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def time_phases(self, x_local, logits_local, counts, reps: int = 20) -> dict | None:
        """Mean device time (ms) of the phases of the fused step over `reps` steps: pack, dispatch (all-gather), compute (the layer's
        launches), combine (reduce-scatter + final sum).  None when the step does not take the fused path."""
        if self.layer is None or self.world == 1 or not all(c == counts[0] for c in counts):
            return None
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(reps)]
        for r in range(reps + 3):
            e = ev[max(r - 3, 0)]
            e[0].record()
            self.forward(x_local, logits_local, counts, events=e[1:])
        torch.cuda.synchronize()
        names = ("pack", "dispatch", "compute", "combine")
        return {n: sum(e[i].elapsed_time(e[i + 1]) for e in ev) / reps for i, n in enumerate(names)}

    __call__ = forward
