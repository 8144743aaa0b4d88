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

Decode-sized steps (at most PeerExchange.max_tokens tokens over all ranks) can run WITHOUT collectives once `EPMoE.enable_peer_exchange`
has mapped every rank's exchange slab into every process (CUDA IPC): dispatch and return are kernels of this package that store
straight into the peers' slabs and publish flag words, the waits are bounded, the partial rows are summed in rank order (the
reference's protocol, dsv41/ep.py:356-525; kernels in csrc/epstep.cu).  Uneven token counts and ranks without tokens are handled by the
same kernels.
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


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerExchange:
    """One rank's view of the exchange slabs of all ranks: the addresses the kernels of csrc/epstep.cu store to, the local buffers the
    layer computes on, and the step counter.  `bases[p]` is the address of rank p's slab as THIS process sees it."""

    def __init__(self, rank: int, world: int, bases: list[int], device, max_tokens: int, dim: int, x_row_bytes: int, l_row_bytes: int, owned=None):
        from . import _lib as L
        assert 1 <= world <= L.EP_MAX_RANKS and len(bases) == world and x_row_bytes % 16 == 0 and l_row_bytes % 16 == 0 and dim % 4 == 0
        self.L, self.rank, self.world, self.device = L, rank, world, device
        self.max_tokens, self.dim, self.xb, self.lb = max_tokens, dim, x_row_bytes, l_row_bytes
        self.bases, self.owned = list(bases), owned
        off = self.offsets(world, max_tokens, dim, x_row_bytes, l_row_bytes)
        self.off = off
        i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=device)
        self.tab = {"inbox_x": i64([b + off["x"] for b in bases]), "inbox_l": i64([b + off["l"] for b in bases]),
                    "partials": i64([b + off["part"] for b in bases]),
                    "flags_in": i64([b + off["fin"] + 4 * rank for b in bases]), "flags_out": i64([b + off["fout"] + 4 * rank for b in bases])}
        self.seq = torch.ones(1, dtype=torch.int32, device=device)
        self.counter = torch.zeros(2, dtype=torch.int32, device=device)
        mine = bases[rank]
        self.flags_in_addr, self.flags_out_addr = mine + off["fin"], mine + off["fout"]
        self.x_all = L.tensor_over(mine + off["x"], max_tokens * x_row_bytes, device)
        self.l_all = L.tensor_over(mine + off["l"], max_tokens * l_row_bytes, device)
        self.partials = L.tensor_over(mine + off["part"], max_tokens * world * dim * 4, device).view(torch.float32)
        self.part = torch.empty(max_tokens, dim, dtype=torch.float32, device=device)
        self.ys = torch.empty(max_tokens, dim, dtype=torch.bfloat16, device=device)
        self._first: dict = {}

    @staticmethod
    def offsets(world: int, max_tokens: int, dim: int, xb: int, lb: int) -> dict:
        off, at = {}, 0
        for name, n in (("fin", 4 * 64), ("fout", 4 * 64), ("x", max_tokens * xb), ("l", max_tokens * lb), ("part", max_tokens * world * dim * 4)):
            off[name] = at
            at = _align(at + n)
        off["bytes"] = at
        return off

    @classmethod
    def alloc_slab(cls, nbytes: int, device) -> int:
        from . import _lib as L
        import ctypes
        p = ctypes.c_void_p(0)
        with torch.cuda.device(device):
            L.check(L.lib().b200_ep_alloc(nbytes, ctypes.byref(p)), "b200_ep_alloc")
        return int(p.value)

    @classmethod
    def over_ipc(cls, group, device, max_tokens: int, dim: int, x_row_bytes: int, l_row_bytes: int) -> "PeerExchange":
        """Allocate this rank's slab, exchange the 64-byte handles over the process group and map every peer's slab.  Collective: every
        rank of the group calls it; if one rank fails, all raise."""
        from . import _lib as L
        import ctypes
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        nbytes = cls.offsets(world, max_tokens, dim, x_row_bytes, l_row_bytes)["bytes"]
        lib = L.lib()
        err, mine, opened, bases = "", 0, [], [0] * world
        try:
            mine = cls.alloc_slab(nbytes, device)
            h = ctypes.create_string_buffer(L.EP_HANDLE_BYTES)
            with torch.cuda.device(device):
                L.check(lib.b200_ep_export(ctypes.c_void_p(mine), h), "b200_ep_export")
            handle = bytes(h.raw)
        except RuntimeError as e:
            err, handle = str(e), b""
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        if not err and all(handles):
            try:
                for p_, hp in enumerate(handles):
                    if p_ == rank:
                        bases[p_] = mine
                        continue
                    q = ctypes.c_void_p(0)
                    with torch.cuda.device(device):
                        L.check(lib.b200_ep_open(ctypes.create_string_buffer(hp, L.EP_HANDLE_BYTES), ctypes.byref(q)), "b200_ep_open")
                    bases[p_] = int(q.value)
                    opened.append(int(q.value))
            except RuntimeError as e:
                err = str(e)
        elif not err:
            err = "a peer could not export its slab"
        errs = [None] * world
        dist.all_gather_object(errs, err, group=group)
        if any(errs):
            with torch.cuda.device(device):
                for q in opened:
                    lib.b200_ep_close(ctypes.c_void_p(q))
            dist.barrier(group=group)
            if mine:
                with torch.cuda.device(device):
                    lib.b200_ep_free(ctypes.c_void_p(mine))
            raise RuntimeError("peer exchange unavailable: " + "; ".join(f"rank {i}: {e}" for i, e in enumerate(errs) if e))
        ex = cls(rank, world, bases, device, max_tokens, dim, x_row_bytes, l_row_bytes, owned={"mine": mine, "opened": opened, "group": group})
        dist.barrier(group=group)
        return ex

    def close(self) -> None:
        """Unmap the peers' slabs and free this rank's (collective when the slabs came from over_ipc): nobody frees memory a peer's kernels
        may still write."""
        import ctypes
        if not self.owned:
            return
        lib, o = self.L.lib(), self.owned
        torch.cuda.synchronize(self.device)
        if o.get("group") is not None:
            dist.barrier(group=o["group"])  # every rank's kernels have finished before anything is unmapped
        with torch.cuda.device(self.device):
            for q in o.get("opened", []):
                lib.b200_ep_close(ctypes.c_void_p(q))
        if o.get("group") is not None:
            dist.barrier(group=o["group"])
        with torch.cuda.device(self.device):
            if o.get("mine"):
                lib.b200_ep_free(ctypes.c_void_p(o["mine"]))
        self.owned = None

    def peers(self, counts: list[int]):
        """(struct b200_ep_peers, first-token table) for a split of the tokens over the ranks."""
        key = tuple(counts)
        hit = self._first.get(key)
        if hit is None:
            assert len(counts) == self.world and sum(counts) <= self.max_tokens
            first = [0]
            for c in counts:
                first.append(first[-1] + c)
            ft = torch.tensor(first, dtype=torch.int32, device=self.device)
            L = self.L
            st = L.EpPeers(self.rank, self.world, self.dim, self.xb, self.lb, L.ptr(ft), L.ptr(self.tab["inbox_x"]), L.ptr(self.tab["inbox_l"]),
                           L.ptr(self.tab["flags_in"]), L.ptr(self.tab["partials"]), L.ptr(self.tab["flags_out"]), L.ptr(self.seq), L.ptr(self.counter))
            hit = (st, ft, first)
            self._first[key] = hit
        return hit

    # ---- the four exchange launches of a step (csrc/epstep.cu); each enqueues on the current stream of the device
    def dispatch(self, counts, x_local, logits_local) -> None:
        import ctypes
        L, (st, _, _) = self.L, self.peers(counts)
        n = counts[self.rank]
        assert x_local.shape[0] == n and (n == 0 or (x_local.is_contiguous() and logits_local.is_contiguous()))
        assert n == 0 or (x_local.shape[1] * x_local.element_size() == self.xb and logits_local.shape[1] * logits_local.element_size() == self.lb)
        with torch.cuda.device(self.device):
            L.check(L.lib().b200_ep_dispatch(ctypes.byref(st), L.ptr(x_local) if n else None, L.ptr(logits_local) if n else None, n,
                                             L.stream_of(self.device)), "b200_ep_dispatch")

    def wait_arrival(self) -> None:
        L = self.L
        with torch.cuda.device(self.device):
            L.check(L.lib().b200_ep_wait(L.c_p(self.flags_in_addr), self.world, L.ptr(self.seq), 0, 0, L.stream_of(self.device)), "b200_ep_wait")

    def send_back(self, counts, part) -> None:
        import ctypes
        L, (st, _, first) = self.L, self.peers(counts)
        assert part.dtype == torch.float32 and part.is_contiguous() and part.shape[1] == self.dim and part.shape[0] >= first[-1]
        with torch.cuda.device(self.device):
            L.check(L.lib().b200_ep_return(ctypes.byref(st), L.ptr(part), first[-1], L.stream_of(self.device)), "b200_ep_return")

    def wait_return(self) -> None:
        L = self.L
        with torch.cuda.device(self.device):
            L.check(L.lib().b200_ep_wait(L.c_p(self.flags_out_addr), self.world, L.ptr(self.seq), 1, 1, L.stream_of(self.device)), "b200_ep_wait")


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
        self.peer: PeerExchange | None = None

    def enable_peer_exchange(self, max_tokens: int, n_experts: int, x_dtype=torch.bfloat16, logits_dtype=torch.float32) -> None:
        """Map the exchange slabs of all ranks (collective call).  Afterwards steps of at most `max_tokens` tokens over all ranks exchange
        through kernels of this package over peer memory instead of NCCL collectives.  Raises on every rank if any rank cannot."""
        assert self.layer is not None and self.world > 1
        D = self.layer.dim
        xb = D * torch.empty(0, dtype=x_dtype).element_size()
        lb = n_experts * torch.empty(0, dtype=logits_dtype).element_size()
        self.peer = PeerExchange.over_ipc(self.group, self.layer.device, max_tokens, D, xb, lb)

    def transport(self, total_tokens: int) -> str:
        return "peer stores + flag words (kernels of this package)" if self.peer is not None and total_tokens <= self.peer.max_tokens else \
            "NCCL all-gather + reduce-scatter"

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
        if fused and self.peer is not None and T <= self.peer.max_tokens and xb == self.peer.xb and lb == self.peer.lb:
            # ---- decode path over peer memory: dispatch kernel, bounded wait, the layer's launches, return kernel, bounded wait, combine
            from .fused2 import moe_combine
            P = self.peer
            first = sum(counts[:self.rank])
            P.dispatch(counts, x_local, logits_local)
            mark(0)
            P.wait_arrival()
            mark(1)
            x_all = P.x_all[:T * xb].view(x_local.dtype).view(T, D)
            l_all = P.l_all[:T * lb].view(logits_local.dtype).view(T, E)
            has_sh = self.layer.sh_w13 is not None
            self.layer.forward(x_all, l_all, final=False, want_routed=True, routed_out=P.part[:T], want_shared=has_sh, shared_out=P.ys[:T] if has_sh else None)
            mark(2)
            P.send_back(counts, P.part)
            P.wait_return()
            if out is None:
                out = torch.empty(T_r, D, dtype=torch.bfloat16, device=x_local.device)
            if T_r > 0:
                moe_combine(P.partials[:T_r * W * D].view(T_r, W, D), P.ys[first:first + T_r] if has_sh else None, out=out)
            mark(3)
            return out
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
            # local experts over all tokens; the shared expert rides in the same launches, for this rank's own token rows only
            has_sh = self.layer.sh_w13 is not None
            first = sum(counts[:self.rank])
            self.layer.forward(x_all, l_all, final=False, want_routed=True, routed_out=b["part"], want_shared=has_sh, shared_out=b["ys"] if has_sh else None,
                               shared_rows=(first, T_r) if has_sh else None)
            mark(2)
            dist.reduce_scatter_tensor(b["routed"], b["part"], group=self.group)
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
        launches), combine (reduce-scatter + final sum); over peer memory: pack = the dispatch kernel, dispatch = the wait for all ranks'
        rows, combine = return kernel + wait + final sum.  None when the step does not take the fused path."""
        if self.layer is None or self.world == 1 or (not all(c == counts[0] for c in counts) and self.peer is None):
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
