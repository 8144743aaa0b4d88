"""ctypes binding of csrc/libb200moe.so (the C-ABI declared in include/b200_moe.h).

The library is the only compute path of this package: if it is missing the import of any operator fails loudly;
there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "csrc", "libb200moe.so")

FMT_FP4_E8M0, FMT_FP4_BF16S, FMT_FP8_E8M0, FMT_FP8_F32B = 0, 1, 2, 3
SCORE_MODES = {"sqrtsoftplus": 0, "sigmoid": 1, "softmax": 2}

c_p, c_i, c_ll, c_f, c_sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_size_t


class MoeArgs(ctypes.Structure):
    """struct b200_moe_args of include/b200_moe.h."""
    _fields_ = [("tokens", c_i), ("n_experts", c_i), ("topk", c_i), ("dim", c_i), ("inter", c_i),
                ("logits", c_p), ("logits_is_bf16", c_i), ("gate_bias", c_p), ("temp", c_f), ("route_scale", c_f),
                ("score_mode", c_i), ("norm", c_i),
                ("x", c_p), ("x_is_quantized", c_i),
                ("w13", c_p), ("s13", c_p), ("w2", c_p), ("s2", c_p), ("expert_fmt", c_i), ("shard_start", c_i), ("shard_n", c_i),
                ("has_shared", c_i), ("sh_w13", c_p), ("sh_s13", c_p), ("sh_w2", c_p), ("sh_s2", c_p),
                ("shared_fmt", c_i), ("sh_s13_cols", c_i), ("sh_s2_cols", c_i), ("sh_permk", c_i), ("swiglu_limit", c_f),
                ("out", c_p), ("routed_out", c_p), ("eid_out", c_p), ("wt_out", c_p), ("workspace", c_p), ("workspace_bytes", c_sz),
                ("prof_start", c_p), ("prof_stop", c_p), ("engine", c_i), ("shared_out", c_p), ("x_ld", c_ll), ("logits_ld", c_ll), ("gate_w", c_p), ("xf", c_p), ("xf_ld", c_ll),
                ("s13_atoms", c_p), ("s2_atoms", c_p), ("sh_s13_atoms", c_p), ("sh_s2_atoms", c_p), ("eid_in", c_p), ("wt_in", c_p), ("sh_first", c_i), ("sh_count", c_i)]


class EpPeers(ctypes.Structure):
    """struct b200_ep_peers of include/b200_moe.h."""
    _fields_ = [("rank", c_i), ("world", c_i), ("dim", c_i), ("x_row_bytes", c_i), ("l_row_bytes", c_i), ("first", c_p), ("inbox_x", c_p),
                ("inbox_l", c_p), ("flags_in", c_p), ("partials", c_p), ("flags_out", c_p), ("seq", c_p), ("counter", c_p)]


EP_MAX_RANKS, EP_HANDLE_BYTES = 16, 64

_SIGNATURES = {
    "b200_version": (c_i, []),
    "b200_error_string": (ctypes.c_char_p, [c_i]),
    "b200_sm_count": (c_i, []),
    "b200_fake_quant_fp8": (c_i, [c_p, c_p, c_ll, c_p]),
    "b200_gate_topk": (c_i, [c_p, c_p, c_i, c_i, c_f, c_i, c_f, c_i, c_i, c_p, c_p, c_p]),
    "b200_swiglu_quant": (c_i, [c_p, c_i, c_p, c_ll, c_i, c_f, c_i, c_p, c_p]),
    "b200_moe_combine": (c_i, [c_p, c_p, c_p, c_ll, c_i, c_i, c_p]),
    "b200_sum_rows": (c_i, [c_p, c_p, c_i, c_i, c_i, c_ll, c_p]),
    "b200_permute_x8": (c_i, [c_p, c_p, c_ll, c_p]),
    "b200_fp4_grouped_workspace_bytes": (c_sz, [c_i]),
    "b200_fp4_grouped_gemm": (c_i, [c_p, c_ll, c_i, c_p, c_ll, c_p, c_ll, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i,
                                    c_p, c_ll, c_p, c_sz, c_p]),
    "b200_fp4_grouped_gemm_static": (c_i, [c_p, c_ll, c_i, c_p, c_ll, c_p, c_ll, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_i, c_i, c_i,
                                           c_i, c_i, c_p, c_ll, c_p]),
    "b200_fp8_gemm": (c_i, [c_p, c_ll, c_i, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_i, c_ll, c_p]),
    "b200_moe_workspace_bytes": (c_sz, [c_i, c_i, c_i, c_i]),
    "b200_moe_forward": (c_i, [ctypes.POINTER(MoeArgs), c_p]),
    "b200_mx_quantize_rows": (c_i, [c_p, c_ll, c_p, c_i, c_i, c_p, c_p, c_p]),
    "b200_mx_grouped_workspace_bytes": (c_sz, [c_i]),
    "b200_mx_grouped_gemm": (c_i, [c_p, c_ll, c_p, c_ll, c_i, c_i, c_i, c_i, c_i, c_p, c_ll, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_i, c_i, c_i, c_i, c_f,
                                   c_i, c_p, c_ll, c_p, c_i, c_i, c_p, c_sz, c_p]),
    "b200_hc_pre_norm_quant2": (c_i, [c_p, c_p, c_p, c_i, c_f, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p]),
    "b200_hc_post2": (c_i, [c_p, c_p, c_p, c_ll, c_ll, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_p]),
    "b200_device_error": (c_i, [c_p, c_p]),
    "b200_fp8_gemm_auto_workspace_bytes": (c_sz, [c_i, c_i]),
    "b200_fp8_gemm_auto": (c_i, [c_p, c_ll, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_i, c_ll, c_p, c_sz, c_p]),
    "b200_fp4_grouped_auto_workspace_bytes": (c_sz, [c_i, c_i]),
    "b200_fp4_grouped_gemm_auto": (c_i, [c_p, c_ll, c_i, c_p, c_ll, c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_ll,
                                         c_p, c_sz, c_p]),
    "b200_p2p_copy": (c_i, [c_p, c_p, c_ll, c_p]),
    "b200_p2p_copy_row": (c_i, [c_p, c_p, c_p, c_ll, c_i, c_ll, c_p, c_p]),
    "b200_p2p_signal": (c_i, [c_p, c_i, c_p, c_p]),
    "b200_p2p_wait": (c_i, [c_p, c_i, c_p, c_p, c_p]),
    "b200_p2p_seq_bump": (c_i, [c_p, c_p]),
    "b200_p2p_multicast": (c_i, [c_p, c_i, c_p, c_ll, c_p, c_p, c_p, c_p]),
    "b200_p2p_stamp": (c_i, [c_p, c_p]),
    "b200_memcpy_async": (c_i, [c_p, c_p, c_ll, c_p]),
    "b200_set_wait_limit_ns": (c_i, [ctypes.c_ulonglong]),
    "b200_ep_dispatch": (c_i, [ctypes.POINTER(EpPeers), c_p, c_p, c_i, c_p]),
    "b200_ep_return": (c_i, [ctypes.POINTER(EpPeers), c_p, c_i, c_p]),
    "b200_ep_wait": (c_i, [c_p, c_i, c_p, c_i, c_i, c_p]),
    "b200_ep_alloc": (c_i, [c_sz, ctypes.POINTER(c_p)]),
    "b200_ep_free": (c_i, [c_p]),
    "b200_ep_export": (c_i, [c_p, c_p]),
    "b200_ep_open": (c_i, [c_p, ctypes.POINTER(c_p)]),
    "b200_ep_close": (c_i, [c_p]),
    "b200_group_pairs_max_tiles": (c_i, [c_i, c_i, c_i]),
    "b200_group_pairs_workspace_bytes": (c_sz, [c_i]),
    "b200_group_pairs": (c_i, [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "b200_regroup_pairs": (c_i, [c_p, c_i, c_p, c_p, c_p, c_p, c_p, c_p, c_p]),
    "b200_scale_atoms_bytes": (c_sz, [c_i, c_i, c_i, c_i]),
    "b200_scale_atoms": (c_i, [c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_p]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Every entry point this binding expects the shared library to export."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(this package has no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc: int, what: str) -> None:
    """Raise like the reference launcher does (dsv41/cukern.py:19-21) when a call reports an error."""
    if rc != 0:
        msg = lib().b200_error_string(rc).decode()
        raise RuntimeError(f"{what} failed with CUDA error {rc} ({msg})")


def ptr(t) -> ctypes.c_void_p:
    return c_p(t.data_ptr()) if t is not None else c_p(0)


class _RawDeviceMemory:
    """Array-interface view of device memory owned by the library (a slab of b200_ep_alloc), so torch can wrap it without copying."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}


def tensor_over(address: int, nbytes: int, device) -> torch.Tensor:
    """uint8 tensor over `nbytes` of device memory at `address`; the caller keeps the memory alive."""
    with torch.cuda.device(device):
        return torch.as_tensor(_RawDeviceMemory(address, nbytes), device=device)


def stream_of(device) -> ctypes.c_void_p:
    return c_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("b200 operators run on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"device mismatch: {t.device} vs {dev}")
    return dev


_workspaces: dict = {}


def workspace(device, nbytes: int, tag: str = "") -> torch.Tensor:
    """Per-device scratch, cached and grown on demand (the reference keeps its scratch the same way, dsv41/cukern.py:255-263)."""
    key = (device, tag)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        w = _workspaces[key] = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
    return w
