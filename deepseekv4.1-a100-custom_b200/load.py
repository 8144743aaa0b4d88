"""Expert loader: per-expert checkpoint tensors -> the stacked expert tensors and expert-parallel shard dicts the kernels take, plus
the load-time re-layout of the scales for B200.

Contract (what the reference's loader produces, dsv41/load.py:213-249): for a layer with E experts of width `inter` and hidden size
`dim`, `w13` uint8 [n, 2*inter, dim/2] (rows 0..inter-1 = w1 / gate, inter..2*inter-1 = w3 / up), `s13` uint8 [n, 2*inter, dim/32],
`w2` uint8 [n, dim, inter/2], `s2` uint8 [n, dim, inter/32]; a shard is the dict {"device", "start", "n", "w13", "s13", "w2", "s2"} holding
the global experts [start, start + n).  Checkpoint names: `<prefix>ffn.experts.<e>.{w1,w3,w2}.{weight,scale}`.

`tensors` is anything with `tensors[name] -> torch.Tensor` (a dict, or a lazy safetensors reader); only the experts of the requested range
are touched, one at a time, so a shard never needs more host memory than one expert."""
from __future__ import annotations

import re
from typing import Iterable, Mapping

import torch

_PARTS = (("w1", 0), ("w3", 1))  # halves of the gate | up matrix


def expert_ids(names: Iterable[str], prefix: str) -> list[int]:
    """Sorted expert numbers present under `<prefix>ffn.experts.`."""
    pat = re.compile(re.escape(prefix) + r"ffn\.experts\.(\d+)\.")
    return sorted({int(m.group(1)) for m in map(pat.match, names) if m})


def shard_bounds(n_experts: int, world: int, per_shard: list[int] | None = None) -> list[tuple[int, int]]:
    """(start, n) of every shard: `per_shard` experts each when given, else boundaries at floor(E * j / world)
    (dsv41/load.py:299-306)."""
    if per_shard is not None:
        if len(per_shard) != world or sum(per_shard) != n_experts:
            raise ValueError(f"per_shard must hold {world} counts summing to {n_experts}: {per_shard}")
        edges = [sum(per_shard[:j]) for j in range(world + 1)]
    else:
        edges = [n_experts * j // world for j in range(world + 1)]
    return [(edges[j], edges[j + 1] - edges[j]) for j in range(world)]


def stack_experts(tensors: Mapping[str, torch.Tensor], prefix: str, start: int, n: int, device, pin: bool = False) -> dict:
    """The shard dict of experts [start, start + n) on `device`."""
    def raw(name: str) -> torch.Tensor:
        t = tensors[name]
        return t.view(torch.uint8) if t.dtype != torch.uint8 else t

    probe_w1, probe_w2 = raw(f"{prefix}ffn.experts.{start}.w1.weight"), raw(f"{prefix}ffn.experts.{start}.w2.weight")
    inter, half_dim = probe_w1.shape
    dim = probe_w2.shape[0]
    if probe_w2.shape[1] * 2 != inter or half_dim * 2 != dim:
        raise ValueError(f"expert {start}: w1 {tuple(probe_w1.shape)} and w2 {tuple(probe_w2.shape)} do not describe one expert")
    new = (lambda *shape: torch.empty(*shape, dtype=torch.uint8, pin_memory=True)) if pin else (lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=device))
    out = {"device": device, "start": start, "n": n, "w13": new(n, 2 * inter, dim // 2), "s13": new(n, 2 * inter, dim // 32),
           "w2": new(n, dim, inter // 2), "s2": new(n, dim, inter // 32)}
    for j in range(n):
        q = f"{prefix}ffn.experts.{start + j}."
        for part, half in _PARTS:
            rows = slice(half * inter, (half + 1) * inter)
            out["w13"][j, rows].copy_(raw(q + part + ".weight"), non_blocking=True)
            out["s13"][j, rows].copy_(raw(q + part + ".scale"), non_blocking=True)
        out["w2"][j].copy_(raw(q + "w2.weight"), non_blocking=True)
        out["s2"][j].copy_(raw(q + "w2.scale"), non_blocking=True)
    return out


def load_experts(tensors: Mapping[str, torch.Tensor], prefix: str, device, ep: list[tuple] | None = None, names: Iterable[str] | None = None) -> dict:
    """All experts of a layer on `device`, or with `ep` = [(device, first_expert, n_experts), ...] one shard per entry.  Returns the keys
    the reference's layer dict carries: experts.w13 / s13 / w2 / s2 (this device's tensors) and, with ep, experts.ep (the shard list)."""
    if ep:
        shards = [stack_experts(tensors, prefix, s, n, d) for d, s, n in ep]
        mine = next((sh for sh in shards if torch.device(sh["device"]) == torch.device(device)), shards[0])
        layer = {"experts.ep": shards}
    else:
        ids = expert_ids(names if names is not None else tensors.keys(), prefix)
        if ids != list(range(len(ids))):
            raise ValueError(f"experts under {prefix} are not numbered 0..{len(ids) - 1}")
        mine = stack_experts(tensors, prefix, 0, len(ids), device)
        layer = {}
    layer.update({"experts.w13": mine["w13"], "experts.s13": mine["s13"], "experts.w2": mine["w2"], "experts.s2": mine["s2"], "experts.offload": False})
    for sh in ([mine] if not ep else layer["experts.ep"]):
        if torch.device(sh["device"]).type == "cuda":
            torch.cuda.synchronize(sh["device"])
    return layer


def relayout_scales(shard: dict) -> dict:
    """The optional load-time re-layout for B200: the E8M0 scales of a shard rewritten once into the 512-byte atoms the tensor cores
    read (adds "s13_atoms" and "s2_atoms" to the dict; the checkpoint-order scales stay, other kernels still read them).  1/16 of the
    weight bytes; afterwards the decode kernels fetch scales with bulk copies instead of gathering bytes."""
    from . import cukern
    n, two_inter, half_dim = shard["w13"].shape
    shard["s13_atoms"] = cukern.scale_atoms(shard["s13"], two_inter, half_dim * 2, True)
    shard["s2_atoms"] = cukern.scale_atoms(shard["s2"], half_dim * 2, two_inter // 2, False)
    return shard


def layer_from_shard(shard: dict, n_experts: int, **layer_kw):
    """moe.MoELayer over one shard dict (the layer builds the scale atoms itself)."""
    from .moe import MoELayer
    return MoELayer(shard["w13"], shard["s13"], shard["w2"], shard["s2"], n_experts=n_experts, shard_start=shard["start"], **layer_kw)
