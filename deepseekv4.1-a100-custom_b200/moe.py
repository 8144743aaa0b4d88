"""The MoE layer as one object: routed FP4 experts (optionally one shard of them), the FP8 shared expert and the router
parameters, with `forward` = router -> input fake quantisation -> expert chain -> combine in a single C-ABI call
(b200_moe_forward).  Mirrors what the reference's MoE.__call__ (dsv41/model.py:2028-2233) and DecodeRuntime.moe2
(dsv41/decode.py:446-464) compute for a batch of tokens."""
from __future__ import annotations

import ctypes

import torch

from . import _lib as L
from .w8 import W8


class MoELayer:
    def __init__(self, w13: torch.Tensor, s13: torch.Tensor, w2: torch.Tensor, s2: torch.Tensor, *, n_experts: int | None = None, topk: int = 6,
                 sh_w13: W8 | None = None, sh_w2: W8 | None = None, gate_bias: torch.Tensor | None = None, gate_temp: float = 1.0,
                 route_scale: float = 1.0, score_func: str = "softmax", norm_topk_prob: bool = True, swiglu_limit: float = 10.0,
                 shard_start: int = 0, engine: int = 0, gate_w: torch.Tensor | None = None):
        """w13 uint8 [n, 2I, D/2], s13 [n, 2I, D/32] (uint8 E8M0 or bf16), w2 uint8 [n, D, I/2], s2 [n, D, I/32]: the n experts
        [shard_start, shard_start + n) of a layer with n_experts experts (shard dict of dsv41/load.py:213-232)."""
        dev = L.require_cuda(w13, s13, w2, s2, gate_bias)
        n, n13, dh = w13.shape
        self.dim, self.inter = dh * 2, n13 // 2
        self.n_local, self.shard_start = n, shard_start
        self.n_experts = n if n_experts is None else n_experts
        assert w2.shape == (n, self.dim, self.inter // 2) and s13.shape == (n, n13, self.dim // 32) and s2.shape == (n, self.dim, self.inter // 32)
        assert s13.dtype == s2.dtype and s13.dtype in (torch.uint8, torch.bfloat16)
        self.w13, self.s13, self.w2, self.s2 = (t.contiguous() for t in (w13, s13, w2, s2))
        self.expert_fmt = L.FMT_FP4_E8M0 if s13.dtype == torch.uint8 else L.FMT_FP4_BF16S
        assert (sh_w13 is None) == (sh_w2 is None)
        self.sh_w13, self.sh_w2 = sh_w13, sh_w2
        if sh_w13 is not None:
            assert sh_w13.shape == (2 * self.inter, self.dim) and sh_w2.shape == (self.dim, self.inter) and sh_w13.s8.dtype == sh_w2.s8.dtype
        self.topk, self.gate_bias, self.gate_temp, self.route_scale = topk, gate_bias, gate_temp, route_scale
        self.score_func, self.norm, self.swiglu_limit = score_func, norm_topk_prob and topk > 1, swiglu_limit
        self.device = dev
        # optional router matrix fp32 [n_experts, dim] (dsv41/model.py:1603): with it forward() can start from the hidden state
        self.gate_w = None
        if gate_w is not None:
            assert gate_w.shape == (self.n_experts, self.dim) and gate_w.dtype == torch.float32 and gate_w.is_cuda
            self.gate_w = gate_w.contiguous()
        # engine 0 = automatic (block-scaled tensor cores whenever the formats allow, else weight streaming), 1 = weight streaming with
        # in-register dequantisation, 2 = block-scaled tensor cores.  The tensor-core path reads the shared expert in natural k
        # order, so a natural-order copy is kept next to the W8 container.
        self.engine = engine
        self._mx_ok = (self.expert_fmt == L.FMT_FP4_E8M0 and (sh_w13 is None or sh_w13.s8.dtype == torch.uint8) and self.dim % 128 == 0 and self.inter % 128 == 0)
        if engine == 2 and not self._mx_ok:
            raise ValueError("engine 2 needs E8M0 scales for the experts and the shared expert and dims that are multiples of 128")
        self._sh_nat = None
        self._args: dict = {}  # (tokens, engine) -> (argument block, workspace bytes), see forward
        if self._mx_ok and engine != 1 and sh_w13 is not None:
            from .w8 import unpermute_k
            self._sh_nat = (unpermute_k(sh_w13.w8), unpermute_k(sh_w2.w8))
        # load-time re-layout of the scales (1/16 of the weight bytes): the decode kernels read them as ready-made tensor-core
        # scale atoms by bulk copy instead of gathering bytes in checkpoint order
        self._atoms = None
        if self._mx_ok and engine != 1:
            from . import cukern
            at = [cukern.scale_atoms(self.s13, 2 * self.inter, self.dim, True), cukern.scale_atoms(self.s2, self.dim, self.inter, False)]
            if sh_w13 is not None:
                at += [cukern.scale_atoms(sh_w13.s8, 2 * self.inter, self.dim, True), cukern.scale_atoms(sh_w2.s8, self.dim, self.inter, False)]
            self._atoms = at

    def _use_mx(self, tokens: int) -> bool:
        return self.engine == 2 or (self.engine == 0 and self._mx_ok and tokens > 0)

    # ---- facts about one forward() that a benchmark reports next to its timings
    def launches_per_step(self, tokens: int) -> int:
        """Kernels of this library one forward() launches for `tokens` tokens."""
        if tokens * self.topk > 4096:
            return 8   # route, histogram, scan, scatter, quantise, gate/up GEMM, down GEMM, finalise
        if self._use_mx(tokens) and self._atoms is not None and tokens <= 64:
            return 4 if tokens <= 16 else 5   # route + quantise, gate/up GEMM, (SwiGLU + quantise,) down GEMM, combine
        return 5 if self._use_mx(tokens) else (6 if self.sh_w13 is not None else 4)

    def dominant_kernel(self, tokens: int) -> str:
        if self._use_mx(tokens) and self._atoms is not None and tokens <= 64:
            return "wm_gemm_kernel (gate/up weight stream of the routed experts and the shared expert, tokens on the M side and 256 weight rows on the N side of tcgen05 kind::mxf8f6f4 tiles, the k blocks of all tiles cut evenly over the SMs)"
        if self._use_mx(tokens):
            return "mx_gemm_kernel (gate/up weight stream of the routed experts and the shared expert on tcgen05 kind::mxf8f6f4 + SwiGLU + FP8 quant)"
        return "skinny_kernel<FP4_E8M0, SWIGLU> (routed gate/up weight stream + SwiGLU + FP8 fake quant)"

    def traffic_ratio(self, tokens: int) -> float:
        """DRAM bytes (read + write) per algorithmic byte of the dominant kernel, from the profiler captures of a smaller case
        (profiles/wm_gemm_kernel_decode64_e96_ncu_full.md, profiles/skinny_fp4_decode8_ncu_full.md)."""
        return 1.057 if self._use_mx(tokens) else 1.075

    def shared_expert(self, x: torch.Tensor) -> torch.Tensor | None:
        """The shared expert alone: x bf16 [T, D] -> ys bf16 [T, D] (None without one); the values of dsv41/model.py:1635-1638 on FP8
        fake-quantised activations.  Tensor-core kernels when the layer would use them for T tokens, else the streaming ones."""
        if self.sh_w13 is None:
            return None
        T = x.shape[0]
        if self._use_mx(T) and self._sh_nat is not None:
            from . import cukern
            w13n, w2n = self._sh_nat
            tpw = 128 if T > 64 else 32
            works = (T + tpw - 1) // tpw
            rows1 = 128
            while rows1 > 32 and works * (self.inter // rows1) < 148:
                rows1 //= 2
            rows2 = 256
            while rows2 > 32 and works * (self.dim // rows2) < 148:
                rows2 //= 2
            q8, sf = cukern.mx_quantize_rows(x)
            h8, hsf = cukern.mx_grouped(w13n, self.sh_w13.s8, q8, sf, None, None, None, None, None, T, epilogue="swiglu_q8", limit=self.swiglu_limit,
                                        round_gu_bf16=True, tokens_per_work=tpw, rows_per_tile=rows1)
            return cukern.mx_grouped(w2n, self.sh_w2.s8, h8, hsf, None, None, None, None, None, T, epilogue="bf16", tokens_per_work=tpw, rows_per_tile=rows2)
        from .fused import fake_quant_fp8, swiglu_quant
        from .w8 import linear_w
        hs = swiglu_quant(linear_w(fake_quant_fp8(x, 32), self.sh_w13), None, self.inter, self.swiglu_limit)
        return linear_w(hs, self.sh_w2)

    def forward(self, x: torch.Tensor, logits: torch.Tensor | None = None, *, xf: torch.Tensor | None = None, out: torch.Tensor | None = None, want_routed: bool = False, want_route: bool = False,
                x_is_quantized: bool = False, with_shared: bool = True, final: bool = True, want_shared: bool = False, prof_events=None,
                eid: torch.Tensor | None = None, wt: torch.Tensor | None = None, shared_out: torch.Tensor | None = None, routed_out: torch.Tensor | None = None,
                shared_rows: tuple[int, int] | None = None):
        """x bf16 [T, D] (the hidden state before the per-32 FP8 fake quantisation), logits fp32|bf16 [T, E]; logits=None (the layer was
        built with gate_w): the router projection xf @ gate_w^T runs inside the call, xf fp32 [T, D] or None for x.float()
        (dsv41/decode.py:449, dsv41/model.py:1615).
        eid int32 / wt fp32 [T, topk]: routing decided by the caller instead of logits (at most 64 tokens, E8M0 formats).
        Returns out bf16 [T, D] = routed experts of this shard + shared expert; optionally also the fp32 routed partial sum
        and (eid, wt).  prof_events: a pair of torch.cuda.Event recorded around the routed gate/up kernel.  shared_out / routed_out:
        caller-provided buffers for the shared expert's result (bf16) and the routed sum (fp32) instead of fresh ones.  shared_rows =
        (first, count): the caller keeps only these rows of the shared expert's result (final=False), the others are unspecified."""
        dev = L.require_cuda(x, logits, out)
        # rows may be strided (views into a wider buffer), the elements of a row are contiguous
        assert dev == self.device and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == self.dim and x.stride(1) == 1
        assert (x.stride(0) * 2) % 16 == 0 and x.data_ptr() % 16 == 0
        T = x.shape[0]
        given = eid is not None
        if given:
            assert wt is not None and eid.dtype == torch.int32 and wt.dtype == torch.float32 and eid.is_contiguous() and wt.is_contiguous()
            assert eid.numel() == T * self.topk and wt.numel() == T * self.topk and T <= 64 and self._atoms is not None
        elif logits is None:
            assert self.gate_w is not None, "forward() without logits needs the layer's gate_w"
            assert xf is None or (xf.shape == (T, self.dim) and xf.dtype == torch.float32 and xf.stride(1) == 1 and xf.is_cuda)
        else:
            assert logits.shape == (T, self.n_experts) and logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(1) == 1
        lib = L.lib()
        mx = self._use_mx(T)
        if final and out is None:
            out = torch.empty(T, self.dim, device=dev, dtype=torch.bfloat16)
        routed = (routed_out if routed_out is not None else torch.empty(T, self.dim, device=dev, dtype=torch.float32)) if want_routed else None
        eid_o = torch.empty(T, self.topk, device=dev, dtype=torch.int32) if want_route else None
        wt_o = torch.empty(T, self.topk, device=dev, dtype=torch.float32) if want_route else None
        shared = with_shared and self.sh_w13 is not None and (final or want_shared)
        ys = (shared_out if shared_out is not None else torch.empty(T, self.dim, device=dev, dtype=torch.bfloat16)) if (want_shared and shared) else None
        # the argument block is kept per (token count, engine): a decode loop calls this tens of thousands of times per second, so
        # everything that does not change from call to call (weights, formats, router settings, workspace) is filled in once
        key = (T, mx)
        cached = self._args.get(key)
        if cached is None:
            a = L.MoeArgs()
            a.tokens, a.n_experts, a.topk, a.dim, a.inter = T, self.n_experts, self.topk, self.dim, self.inter
            a.gate_bias = self.gate_bias.data_ptr() if self.gate_bias is not None else None
            a.temp, a.route_scale = float(self.gate_temp), float(self.route_scale)
            a.score_mode, a.norm = L.SCORE_MODES[self.score_func], int(self.norm)
            a.w13, a.s13, a.w2, a.s2 = self.w13.data_ptr(), self.s13.data_ptr(), self.w2.data_ptr(), self.s2.data_ptr()
            a.expert_fmt, a.shard_start, a.shard_n = self.expert_fmt, self.shard_start, self.n_local
            if self.sh_w13 is not None:
                w13b, w2b = (self._sh_nat if mx else (self.sh_w13.w8, self.sh_w2.w8))
                a.sh_w13, a.sh_s13, a.sh_w2, a.sh_s2 = w13b.data_ptr(), self.sh_w13.s8.data_ptr(), w2b.data_ptr(), self.sh_w2.s8.data_ptr()
                a.shared_fmt = L.FMT_FP8_E8M0 if self.sh_w13.s8.dtype == torch.uint8 else L.FMT_FP8_F32B
                a.sh_s13_cols, a.sh_s2_cols, a.sh_permk = self.sh_w13.s8.shape[1], self.sh_w2.s8.shape[1], int(not mx)
            a.swiglu_limit = float(self.swiglu_limit)
            a.engine = 2 if mx else 1
            a.gate_w = self.gate_w.data_ptr() if self.gate_w is not None else None
            if mx and self._atoms is not None:
                a.s13_atoms, a.s2_atoms = self._atoms[0].data_ptr(), self._atoms[1].data_ptr()
                if len(self._atoms) == 4:
                    a.sh_s13_atoms, a.sh_s2_atoms = self._atoms[2].data_ptr(), self._atoms[3].data_ptr()
            nbytes = lib.b200_moe_workspace_bytes(T, self.topk, self.dim, self.inter)
            cached = self._args[key] = (a, nbytes)
        a, nbytes = cached
        ws = L.workspace(dev, nbytes, "moe")
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        a.logits = logits.data_ptr() if logits is not None else None
        a.logits_is_bf16 = int(logits is not None and logits.dtype == torch.bfloat16)
        a.xf, a.xf_ld = (xf.data_ptr(), xf.stride(0) if T > 1 else self.dim) if (logits is None and xf is not None) else (None, 0)
        a.x, a.x_is_quantized = x.data_ptr(), int(x_is_quantized)
        a.x_ld = x.stride(0) if T > 1 else self.dim
        a.logits_ld = logits.stride(0) if (logits is not None and T > 1) else self.n_experts
        a.has_shared = int(shared)
        a.out = out.data_ptr() if final else None
        a.routed_out = routed.data_ptr() if routed is not None else None
        a.shared_out = ys.data_ptr() if ys is not None else None
        a.eid_out = eid_o.data_ptr() if eid_o is not None else None
        a.wt_out = wt_o.data_ptr() if wt_o is not None else None
        a.eid_in, a.wt_in = (eid.data_ptr(), wt.data_ptr()) if given else (None, None)
        a.sh_first, a.sh_count = (0, 0)
        if shared_rows is not None:
            assert not final and 0 <= shared_rows[0] and shared_rows[0] + shared_rows[1] <= T
            a.sh_first, a.sh_count = int(shared_rows[0]), int(shared_rows[1])
        if prof_events is not None:  # (start, stop) torch.cuda.Event pair, already created (recorded once), timing enabled
            a.prof_start, a.prof_stop = prof_events[0].cuda_event, prof_events[1].cuda_event
        else:
            a.prof_start = a.prof_stop = None
        with torch.cuda.device(dev):
            L.check(lib.b200_moe_forward(ctypes.byref(a), L.stream_of(dev)), "b200_moe_forward")
        res = [out] if final else []
        if want_routed:
            res.append(routed)
        if want_route:
            res += [eid_o, wt_o]
        if want_shared:
            res.append(ys)
        return res[0] if len(res) == 1 else tuple(res)

    __call__ = forward
