/*
 * C-ABI of libb200moe: the sm_100a implementation of the packed-FP4 MoE expert chain and the block-scaled FP8
 * dense GEMV/GEMM of the DeepSeek-V4.1 A100 runtime, for NVIDIA B200.
 *
 * Conventions (the ones dsv41/cukern.py:1-57 sets for the reference's launchers):
 *   - every pointer is a DEVICE pointer on the current CUDA device unless the comment says "host";
 *   - every call that takes a `stream` only enqueues work on it and nothing allocates.  The one such call that synchronises is
 *     b200_device_error (it waits for `stream` and reads the device error word); the set-up calls without a stream argument
 *     (b200_ep_alloc / _free / _export / _open / _close, b200_set_wait_limit_ns) may allocate and synchronise.  Scratch memory is passed in
 *     by the caller (`workspace`), sized by the matching *_workspace_bytes function, except for
 *     b200_fp4_grouped_gemm_static, whose scratch is a fixed array inside the library;
 *   - b200_hc_post2 and b200_sum_rows put rows / groups on the grid's y dimension: at most 65,535 of them per call;
 *   - return value: 0 = ok; > 0 = the cudaError_t of a failed runtime call; < 0 = argument error
 *     (B200_ERR_* below) detected before anything was launched;
 *   - "bf16" = 16-bit bfloat, "e4m3" = float8_e4m3fn bit patterns, "E8M0" = one byte b meaning 2^(b-127),
 *     "E2M1" = 4-bit FP4 codes, two per byte, low nibble = even k (dsv41/quant.py:24-31, 98-103).
 *
 * The reference has no shared library for its GPU path: it launches cubin entry points through the driver API
 * from Python (dsv41/cukern.py:24-57).  Each function below names the reference launcher(s) it replaces.
 */
#ifndef B200_MOE_H
#define B200_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st* cudaStream_t;
#endif

#define B200_ERR_BAD_ARG (-1)
#define B200_ERR_BAD_SHAPE (-2)
#define B200_ERR_BAD_ALIGN (-3)
#define B200_ERR_WORKSPACE (-4)
#define B200_ERR_UNSUPPORTED (-5)
#define B200_ERR_TOO_LARGE (-6)

/* weight / scale formats */
#define B200_FMT_FP4_E8M0 0  /* E2M1 [.., N, K/2] + E8M0 byte per (row, 32 k)   : reference expert format   */
#define B200_FMT_FP4_BF16S 1 /* E2M1 [.., N, K/2] + bf16 power-of-two per (row, 32 k)                         */
#define B200_FMT_FP8_E8M0 2  /* e4m3 [N, K] + E8M0 byte per (32 rows, 32 k)      : reference dense format    */
#define B200_FMT_FP8_F32B 3  /* e4m3 [N, K] + fp32 per (128 rows, 128 k), scale = blockmax/448                */

/* router score functions (numbering of dsv41/fused2.py:497) */
#define B200_SCORE_SQRTSOFTPLUS 0
#define B200_SCORE_SIGMOID 1
#define B200_SCORE_SOFTMAX 2

int b200_version(void);
/* host string for a return code of this library (never NULL) */
const char* b200_error_string(int code);
/* number of SMs of the current device as the persistent kernels size their grids */
int b200_sm_count(void);

/* ---- activation FP8 fake quantisation.  Replaces dsv41/fused.py:72-83 (fake_quant_fp8; spec dsv41/quant.py:46-54).
 * x, y: bf16 [n_elems], n_elems % 32 == 0; groups of 32 along the flattened last dimension. */
int b200_fake_quant_fp8(const void* x, void* y, long long n_elems, cudaStream_t stream);

/* ---- router.  Replaces dsv41/fused2.py:486-502 (gate_topk; spec dsv41/model.py:1614-1630).
 * scores fp32 [rows, n_experts]; bias fp32 [n_experts] or NULL; eid int32 [rows, topk]; wt fp32 [rows, topk].
 * n_experts <= 1024, topk <= 32.  Equal keys select the lowest expert index. */
int b200_gate_topk(const float* scores, const float* bias, int rows, int n_experts, float temp, int topk, float route_scale,
                   int score_mode, int norm, int* eid, float* wt, cudaStream_t stream);

/* ---- SwiGLU (+ routing weight) + per-32 FP8 fake quantisation.  Replaces dsv41/fused.py:309-316 (swiglu_quant).
 * gu fp32 or bf16 [rows, 2*inter] (gate | up); weights fp32 [rows] or NULL; y bf16 [rows, inter]; inter % 32 == 0.
 * permute != 0 stores the 8-k permuted layout of dsv41/fused.py:303-305. */
int b200_swiglu_quant(const void* gu, int gu_is_bf16, const float* weights, long long rows, int inter, float limit, int permute, void* y,
                      cudaStream_t stream);

/* ---- routed + shared combine.  Replaces the NSUM branch of dsv41/fused2.py:518-523 and dsv41/model.py:2114-2118,2232.
 * out[t, :] = bf16( sum_j y2[t*nsum + j, :] + ys[t, :] ); y2 fp32 [tokens*nsum, dim]; ys bf16 [tokens, dim] or NULL. */
int b200_moe_combine(const float* y2, const void* ys, void* out, long long tokens, int nsum, int dim, cudaStream_t stream);

/* ---- per-token partial row sums.  Replaces p2p_sum_rows (dsv41/cuda/p2p.cu:21-28, dsv41/cukern.py:370-379).
 * dst[g*dst_stride + c] = sum_{r < rows} src[(g*rows + r)*n + c]; dst may be peer memory. */
int b200_sum_rows(float* dst, const float* src, int rows, int n, int groups, long long dst_stride, cudaStream_t stream);

/* ---- 8-k permuted copy of an activation.  Replaces dsv41/cukern.py:270-273 (permute_x).  bf16, n_elems % 8 == 0. */
int b200_permute_x8(const void* x, void* y, long long n_elems, cudaStream_t stream);

/* ---- grouped FP4 expert GEMM (decode form).  Replaces fp4_gemv_pairs (dsv41/cukern.py:60-77), fp4_gemv_m1
 * (dsv41/cukern.py:286-306) and fp4_gemm_tc (dsv41/cukern.py:309-344); with accumulate != 0 it has the scatter-add
 * contract of grouped_fp4_gemm (dsv41/moe_kernels.py:161-231).
 *   out[pair_out[p], :] (+)= pair_w[p] * x[pair_tok[p], :] @ W[grp_expert[g] - shard_start]^T   for p in group g
 *   x bf16 [rows, K] with row stride x_ld elements (x_perm8: the 8-k permuted layout); w uint8 [n_local_experts, N, K/2],
 *   s [n, N, K/32] (fmt B200_FMT_FP4_E8M0: bytes, B200_FMT_FP4_BF16S: bf16); w_estride / s_estride in BYTES;
 *   grp_expert int32 [n_groups] (global ids, -1 = padding); group g owns pairs grp_start[g] .. +count-1 with count =
 *   grp_count[g], or grp_start[g+1] - grp_start[g] when grp_count is NULL (then grp_start has n_groups+1 entries,
 *   dsv41/decode.py:431-432; the grp_count form is the tile table of dsv41/moe_kernels.py:118-132); pair_tok / pair_out int32
 *   [n_pairs] or NULL (= pair index), EVERY entry a valid row (also those of pairs no group covers: the auto form gathers them all); pair_w fp32 [n_pairs] or NULL; out fp32, row stride out_ld elements.
 *   Groups whose expert is outside [shard_start, shard_start + shard_n) are skipped; with zero_out their rows are
 *   zeroed (dsv41/cuda/fp4_tc.cu:66-72).  K % 128 == 0, N % 16 == 0, K <= 9088.  Groups of any size are accepted;
 *   more than 8 pairs re-read the expert once per 8.
 *   workspace: b200_fp4_grouped_workspace_bytes(n_pairs) bytes, 16-byte aligned. */
size_t b200_fp4_grouped_workspace_bytes(int n_pairs);
int b200_fp4_grouped_gemm(const void* x, long long x_ld, int x_perm8, const void* w, long long w_estride, const void* s, long long s_estride, int fmt,
                          int n_local_experts, int N, int K, const int* grp_expert, const int* grp_start, const int* grp_count, int n_groups, const int* pair_tok, const int* pair_out,
                          const float* pair_w, int n_pairs, int shard_start, int shard_n, int zero_out, int accumulate, float* out, long long out_ld,
                          void* workspace, size_t workspace_bytes, cudaStream_t stream);

/* ---- the same grouped FP4 expert GEMM with its scratch inside the library: no workspace argument, and the call obtains no
 * memory from the CUDA runtime or anyone else.  No counterpart in the reference.  Arguments, kernels and results are those of
 * b200_fp4_grouped_gemm.  The work list lives in one fixed array per device (66,048 bytes, part of the library's device
 * image), so n_pairs is limited to B200_STATIC_MAX_PAIRS; more returns B200_ERR_TOO_LARGE and launches nothing.
 *   - set-up: the first call on each device looks the array's address up (cudaGetSymbolAddress, result cached); make that
 *     call before any stream capture begins;
 *   - every call on a device shares the array.  Nothing in it has to start at zero or be cleared between calls: each call
 *     rewrites all it reads.  Calls on one stream are ordered and safe; calls that can overlap on the device (other
 *     streams) race on it and must be serialised by the caller, or use the workspace form above. */
#define B200_STATIC_MAX_PAIRS 4096
int b200_fp4_grouped_gemm_static(const void* x, long long x_ld, int x_perm8, const void* w, long long w_estride, const void* s, long long s_estride,
                                 int fmt, int n_local_experts, int N, int K, const int* grp_expert, const int* grp_start, const int* grp_count,
                                 int n_groups, const int* pair_tok, const int* pair_out, const float* pair_w, int n_pairs, int shard_start, int shard_n,
                                 int zero_out, int accumulate, float* out, long long out_ld, cudaStream_t stream);

/* ---- bucketing of (row, expert) pairs for the grouped GEMMs.  Replaces GroupedPairs (dsv41/moe_kernels.py:76-132: stable argsort by
 * expert, tile table of at most block_m pairs per tile) and GroupedPairs.make_p2 (dsv41/moe_kernels.py:134-158).
 *   expert int32 [n_pairs] (ids outside [0, n_experts) are dropped); row_in / row_out int32 [n_pairs] or NULL (= pair index); weight fp32
 *   [n_pairs] or NULL (= 1).  Outputs, all int32 / fp32 [n_pairs]: order (sorted position -> original pair, stable), s_expert, s_row_in,
 *   s_row_out, s_weight (the inputs in sorted order); tile_expert / tile_start / tile_count int32 [b200_group_pairs_max_tiles(...)] (tiles in
 *   expert order; unused entries: expert -1, count 0); n_tiles int32 [1].  n_experts <= 1024.  No host synchronisation.
 * b200_regroup_pairs gathers new rows / weights into an existing order: s_x[i] = x[order[i]]. */
int b200_group_pairs_max_tiles(int n_pairs, int n_experts, int block_m);
size_t b200_group_pairs_workspace_bytes(int n_experts);
int b200_group_pairs(const int* expert, const int* row_in, const int* row_out, const float* weight, int n_pairs, int n_experts, int block_m, int* order,
                     int* s_expert, int* s_row_in, int* s_row_out, float* s_weight, int* tile_expert, int* tile_start, int* tile_count, int* n_tiles,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream);
int b200_regroup_pairs(const int* order, int n_pairs, const int* row_in, const int* row_out, const float* weight, int* s_row_in, int* s_row_out,
                       float* s_weight, cudaStream_t stream);

/* ---- block-scaled FP8 dense GEMV / small-M GEMM.  Replaces fp8_gemv (dsv41/cukern.py:80-96), fp8_gemv_m1
 * (dsv41/cukern.py:116-133) and fp8_gemm_tc (dsv41/cukern.py:165-221, group_cols = 0).
 *   out[m, :] = x[m, :] @ dequant(w8, s)^T;  x bf16 [M, K] (row stride x_ld); w8 e4m3 [N, K];
 *   fmt B200_FMT_FP8_E8M0: s uint8 [ceil(N/32), s_cols]; B200_FMT_FP8_F32B: s fp32 [ceil(N/128), s_cols];
 *   w_permk != 0: weight bytes in the 16-k order of dsv41/w8.py:21-23 (what W8 holds);
 *   out bf16 (out_is_f32 = 0) or fp32, row stride out_ld.  K % 64 == 0, N % 16 == 0, K <= 9088.  Any M; the weights
 *   are read once per 8 rows. */
int b200_fp8_gemm(const void* x, long long x_ld, int M, const void* w8, const void* s, int fmt, int s_cols, int w_permk, int N, int K, void* out,
                  int out_is_f32, long long out_ld, cudaStream_t stream);

/* ---- the two GEMMs above with the engine chosen ON THE DEVICE.  The activation is quantised to FP8 (e4m3 + E8M0 per 32) and compared with
 * the original; if it is reproduced exactly (it always is inside the MoE layer, dsv41/model.py:2040, dsv41/fused.py:297-306) the
 * block-scaled tensor-core kernel (tcgen05) computes the result, otherwise the weight-streaming kernel does: both are launched, tied to the
 * outcome word, and one of them finds nothing to do.  Same results as the plain entry points, no host synchronisation, E8M0 scale formats.
 *   b200_fp8_gemm_auto: w8_natural = weight bytes in natural k order (needed by the tensor cores; NULL: streaming only), w8_permk = the same
 *   weights in the 16-k order of dsv41/w8.py:21-23 (or NULL); rows M <= 8 always stream.  Replaces linear_w / fp8_gemm_tc for any row
 *   count (dsv41/w8.py:64-83, dsv41/cukern.py:165-252): a 512-row call reads the weights once, not once per 8 rows.
 *   b200_fp4_grouped_gemm_auto: arguments of b200_fp4_grouped_gemm (E8M0 scales).  Replaces grouped_fp4_gemm
 *   (dsv41/moe_kernels.py:161-231) and fp4_gemv_pairs.  Workspaces: the *_workspace_bytes functions, 256-byte aligned. */
size_t b200_fp8_gemm_auto_workspace_bytes(int M, int K);
int b200_fp8_gemm_auto(const void* x, long long x_ld, int M, const void* w8_natural, const void* w8_permk, const void* s, int s_cols, int N, int K, void* out,
                       int out_is_f32, long long out_ld, void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t b200_fp4_grouped_auto_workspace_bytes(int n_pairs, int K);
int b200_fp4_grouped_gemm_auto(const void* x, long long x_ld, int x_perm8, const void* w, long long w_estride, const void* s, long long s_estride, int n_local_experts, int N,
                               int K, const int* grp_expert, const int* grp_start, const int* grp_count, int n_groups, const int* pair_tok, const int* pair_out,
                               const float* pair_w, int n_pairs, int shard_start, int shard_n, int zero_out, int accumulate, float* out, long long out_ld,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream);

/* ---- whole MoE layer for a decode batch: router -> input fake quantisation -> routed FP4 experts (gate/up, SwiGLU
 * with routing weight, FP8 fake quantisation, down) -> shared FP8 expert -> combine.  Replaces, in one call, the
 * chain dsv41/decode.py:446-464 (moe2 + experts_tc) + dsv41/fused2.py:518-523 and its fused single-token form
 * cukern.expert_chain (dsv41/cukern.py:504-547); with a shard it is EPRuntime._experts_shard (dsv41/ep.py:324-338). */
typedef struct b200_moe_args {
    int tokens, n_experts, topk, dim, inter;
    /* router: logits [tokens, n_experts] fp32 (logits_is_bf16 = 0) or bf16 (or NULL with gate_w, see below); bias fp32 [n_experts] or NULL */
    const void* logits;
    int logits_is_bf16;
    const float* gate_bias;
    float temp, route_scale;
    int score_mode, norm;
    /* input activation bf16 [tokens, dim]; x_is_quantized != 0 skips the per-32 FP8 fake quantisation */
    const void* x;
    int x_is_quantized;
    /* routed experts of this shard: w13 [shard_n, 2*inter, dim/2], s13 [shard_n, 2*inter, dim/32],
     * w2 [shard_n, dim, inter/2], s2 [shard_n, dim, inter/32]  (dsv41/load.py:213-249); expert_fmt = FP4_E8M0 or FP4_BF16S */
    const void *w13, *s13, *w2, *s2;
    int expert_fmt;
    int shard_start, shard_n;
    /* shared expert (FP8): sh_w13 e4m3 [2*inter, dim], sh_w2 e4m3 [dim, inter]; shared_fmt = FP8_E8M0 or FP8_F32B */
    int has_shared;
    const void *sh_w13, *sh_s13, *sh_w2, *sh_s2;
    int shared_fmt, sh_s13_cols, sh_s2_cols, sh_permk;
    float swiglu_limit;
    /* outputs: out bf16 [tokens, dim] (may be NULL); routed_out fp32 [tokens, dim] = this shard's routed sum without
     * the shared expert (may be NULL); eid_out int32 / wt_out fp32 [tokens, topk] (may be NULL) */
    void* out;
    float* routed_out;
    int* eid_out;
    float* wt_out;
    void* workspace;
    size_t workspace_bytes;
    /* optional cudaEvent_t pair recorded on `stream` right before and after the dominant kernel of the layer (the routed
     * gate/up weight stream), so that a benchmark can time that kernel alone; NULL = not recorded */
    void* prof_start;
    void* prof_stop;
    /* 0 = automatic, 1 = weight-streaming path with in-register dequantisation (any scale format), 2 = block-scaled
     * tensor-core path (tcgen05 kind::mxf8f6f4; needs E8M0 scales and the shared expert in natural k order, sh_permk = 0) */
    int engine;
    /* optional: the shared expert's own result, bf16 [tokens, dim] (NULL = not wanted).  With has_shared it is computed even when
     * `out` is NULL; an expert-parallel caller adds it to the routed sum it gets back from the exchange. */
    void* shared_out;
    /* row strides, in elements, of x and of the logits; 0 = dense (dim / n_experts).  Lets both live inside wider rows, e.g. the
     * rows [x | logits] of one exchange buffer.  x rows must stay 16-byte aligned. */
    long long x_ld, logits_ld;
    /* optional router projection, so that the layer starts from the hidden state instead of from logits (dsv41/model.py:1615,
     * dsv41/decode.py:449): with logits == NULL the layer computes logits = xf @ gate_w^T in fp32; gate_w fp32 [n_experts, dim];
     * xf fp32 [tokens, dim] with row stride xf_ld (0 = dim), or NULL to use x converted to fp32. */
    const void* gate_w;
    const void* xf;
    long long xf_ld;
    /* optional: the E8M0 scales re-laid-out once, at load time, into the 512-byte atoms the tensor cores read (b200_scale_atoms
     * below): s13_atoms of s13 (dual = 1), s2_atoms of s2 (dual = 0), sh_s13_atoms / sh_s2_atoms of the shared expert's 32x32 scales.
     * With all of them given (and E8M0 formats), batches of up to 64 tokens run on the weight-stream kernels: 4 launches per call, the
     * k range of every launch cut evenly over the SMs.  NULL: the kernels that read the scales in checkpoint order are used. */
    const void *s13_atoms, *s2_atoms, *sh_s13_atoms, *sh_s2_atoms;
    /* optional: routing decided by the caller, int32 / fp32 [tokens, topk] (the argument form of cukern.expert_chain,
     * dsv41/cukern.py:504-547): no router runs and `logits` may be NULL.  Needs the scale atoms above and at most 64 tokens. */
    const int* eid_in;
    const float* wt_in;
    /* optional: the shared expert for the token rows [sh_first, sh_first + sh_count) only (sh_count = 0: all tokens).  For callers that
     * keep only those rows of shared_out, as a rank of an expert-parallel group keeps its own tokens: in a prefill-sized call the shared
     * expert otherwise costs as much as all routed pairs of the rank together.  Needs out == NULL; rows of shared_out outside the range
     * are unspecified (calls that stream the shared expert's weights once for all tokens compute every row regardless). */
    int sh_first, sh_count;
} b200_moe_args;

size_t b200_moe_workspace_bytes(int tokens, int topk, int dim, int inter);
int b200_moe_forward(const b200_moe_args* args, cudaStream_t stream);

/* ---- load-time re-layout of E8M0 scales (the optional re-layout of the expert loader; the reference keeps checkpoint order,
 * dsv41/load.py:237-249, and gathers scale bytes in every kernel).  s: bytes [n_experts][N][K/32] (fmt B200_FMT_FP4_E8M0, s_cols = K/32)
 * or [ceil(N/32)][s_cols] (fmt B200_FMT_FP8_E8M0, n_experts = 1); dst: b200_scale_atoms_bytes(...) bytes, 16-byte aligned, laid out
 * [expert][tile of 256 rows][K/128][2][512]: byte (r % 32) * 16 + (r / 32) * 4 + g of an atom = scale of row r (of the 128 of its row
 * block), 32-group g of the 128-wide k block.  dual = 1 for a gate|up matrix (N = 2 * inter): tile t = gate rows 128 t .. and up rows
 * inter + 128 t ..; dual = 0: rows 256 t ...  K % 128 == 0. */
size_t b200_scale_atoms_bytes(int n_experts, int N, int K, int dual);
int b200_scale_atoms(const void* s, int fmt, int s_cols, int n_experts, int N, int K, int dual, void* dst, cudaStream_t stream);

/* ---- FP8 quantisation of activation rows kept in quantised form: q8 e4m3 [rows, K], sf E8M0 bytes [rows, K/32], the
 * values of quant_fp8 (dsv41/quant.py:57-64).  src_row int32 [rows] gathers input rows (NULL = identity). */
int b200_mx_quantize_rows(const void* x, long long x_ld, const int* src_row, int rows, int K, void* q8, void* sf, cudaStream_t stream);

/* ---- grouped expert GEMM on the block-scaled tensor cores (tcgen05.mma kind::mxf8f6f4, TMA, TMEM).  Same group / shard
 * contract as b200_fp4_grouped_gemm, but the activation arrives FP8-quantised (x8 e4m3 [x8_rows, K] + xsf E8M0 [x8_rows, K/32];
 * row p of x8 is pair p, i.e. already gathered into pair order), which is what the MoE layer feeds its experts
 * (dsv41/model.py:2040, dsv41/fused.py:297-306).  Replaces grouped_fp4_gemm (dsv41/moe_kernels.py:161-231) and fp4_gemm_tc
 * (dsv41/cukern.py:309-344) on that path, and linear_w (dsv41/w8.py:64-83) for the shared expert (fmt B200_FMT_FP8_E8M0, weight
 * bytes in NATURAL k order, n_groups = 0: every row of x8 against the single matrix).
 *   epilogue 0: out fp32 [.., N] = rows of x8 @ W^T (times pair_w);  2: the same rounded to bf16;
 *   epilogue 1: N = 2*inter, out e4m3 [.., inter] + out_sf E8M0 [.., inter/32] = FP8 quantisation of
 *               bf16(pair_w * silu(min(g, limit)) * clamp(u, +-limit)), g = rows 0..inter-1, u = rows inter..2*inter-1
 *               (dsv41/fused.py:285-306); round_gu_bf16 rounds g, u to bf16 first (shared expert).
 *   tokens_per_work: 16..128, multiple of 16 (the tokens are the M side of the tensor-core tile); rows_per_tile: weight rows per
 *   tile on the N side: 32, 64, 128 or (epilogues 0, 2) 256; epilogue 1 pairs rows_per_tile gate rows with as many up rows.
 *   K % 128 == 0; w 32-byte aligned; workspace b200_mx_grouped_workspace_bytes(n_rows) bytes when groups are given. */
size_t b200_mx_grouped_workspace_bytes(int n_rows);
int b200_mx_grouped_gemm(const void* w, long long w_estride, const void* s, long long s_estride, int s_cols, int fmt, int n_local_experts, int N, int K,
                         const void* x8, long long x8_rows, const void* xsf, const int* grp_expert, const int* grp_start, const int* grp_count,
                         int n_groups, const int* pair_out, const float* pair_w, int n_rows, int shard_start, int shard_n, int epilogue, float limit,
                         int round_gu_bf16, void* out, long long out_ld, void* out_sf, int tokens_per_work, int rows_per_tile, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream);

/* ---- the steps either side of the MoE path in the reference's decode loop (hyper-connection mixes).
 * b200_hc_pre_norm_quant2 replaces hc_pre_norm_quant2 (dsv41/fused2.py:171-246): x bf16 [rows, hc, dim], pre fp32 [rows, hc], norm weight
 *   w [dim] (bf16, or fp32 with w_is_f32);  t = bf16(sum_h pre[h] * x[h]);  y = bf16(t / sqrt(mean(t^2) + eps) * w) bf16 [rows, dim];
 *   yq = per-32 FP8 fake quantisation of y;  yf = y as fp32 (or NULL);  yqp = yq in the 8-k permuted order (or NULL).
 *   dim % 32 == 0, hc <= 8, 16-byte aligned buffers.
 * b200_hc_post2 replaces hc_post2_ (dsv41/fused2.py:505-558): residual bf16 [rows, hc, dim] is updated in place,
 *   residual[i] <- bf16(post[i] * v + sum_h comb[h][i] * residual[h]),  post fp32 [rows, hc], comb fp32 [rows, hc, hc];
 *   v = x bf16 [rows, dim] (nsum = 0) or bf16(sum_k y2[k] + ys): y2 fp32, element (row, k, c) at y2[row * y2_row_stride +
 *   k * y2_sum_stride + c], ys bf16 [rows, dim] or NULL.  dim % 8 == 0. */
int b200_hc_pre_norm_quant2(const void* x, const float* pre, const void* w, int w_is_f32, float eps, int rows, int hc, int dim, void* y, void* yq,
                            float* yf, void* yqp, cudaStream_t stream);
int b200_hc_post2(const void* x, const float* y2, const void* ys, long long y2_row_stride, long long y2_sum_stride, int nsum, void* residual,
                  const float* post, const float* comb, int rows, int hc, int dim, cudaStream_t stream);

/* ---- device-side messaging between GPUs for the expert-parallel decode protocol.  Replace the kernels of dsv41/cuda/p2p.cu behind
 * dsv41/cukern.py:348-434 (p2p_copy, p2p_copy_row, p2p_signal, p2p_wait, p2p_wait_masked, p2p_seq_bump, p2p_multicast, p2p_stamp) and
 * memcpy_async.  Destinations and flags may be local memory or any memory of another GPU that the calling context can address; fan-out is
 * a loop of ordinary stores (no multicast objects).  Sizes are multiples of 16 bytes, pointers 16-byte aligned.
 *   flag_ptrs / dst_ptrs: DEVICE arrays of addresses; seq: device int32 holding the step number that signal publishes and wait expects
 *   (flags count upwards, a wait is satisfied by flag >= *seq); mask: device int32 [n] or NULL, zero entries are not waited for;
 *   counter: device uint32, zero before the first use, resets itself.
 * b200_p2p_wait is BOUNDED, unlike the reference's: after the limit (2 s; b200_set_wait_limit_ns changes it, 0 restores the default) it
 * stores 3001 (3002 with a mask) in the device error word and returns, leaving the stream usable. */
int b200_p2p_copy(void* dst, const void* src, long long nbytes, cudaStream_t stream);
int b200_p2p_copy_row(void* dst_base, const long long* row_idx, const void* src, long long row_bytes, int n_rows, long long batch_stride_bytes,
                      const long long* seq, cudaStream_t stream);
int b200_p2p_signal(int* const* flag_ptrs, int n, const int* seq, cudaStream_t stream);
int b200_p2p_wait(const int* flags, int n, const int* seq, const int* mask, cudaStream_t stream);
int b200_p2p_seq_bump(int* seq, cudaStream_t stream);
int b200_p2p_multicast(void* const* dst_ptrs, int n_dst, const void* src, long long nbytes, int* const* flag_ptrs, const int* seq, unsigned int* counter,
                       cudaStream_t stream);
int b200_p2p_stamp(long long* dst, cudaStream_t stream);
int b200_memcpy_async(void* dst, const void* src, long long nbytes, cudaStream_t stream);
int b200_set_wait_limit_ns(unsigned long long ns);

/* ---- expert-parallel decode step over peer memory: the dispatch / return exchange of one MoE layer step among the GPUs of a node as
 * three stream-ordered kernels with ordinary peer stores and flag words.  Replaces, as ONE protocol, what the reference's decode
 * runtime assembles from p2p_copy_row / p2p_multicast / p2p_signal / p2p_wait / p2p_sum_rows per layer (dsv41/ep.py:69-80, 356-525).
 * Every rank owns one slab that all ranks can address; `b200_ep_peers` holds, per rank p, the addresses inside p's slab:
 *   inbox_x[p]   [tokens][x_row_bytes]       activation rows of all ranks in global token order
 *   inbox_l[p]   [tokens][l_row_bytes]       router logits rows
 *   partials[p]  [tokens of p][world][dim]   fp32 partial sums of p's own tokens, one row per contributing rank
 *   flags_in[p]  address of flags_in[rank] in p's slab;  flags_out[p]  address of flags_out[rank] in p's slab
 * (all five: DEVICE arrays of `world` addresses), plus local words: first = device int32 [world + 1], first global token of each rank
 * (first[world] = all tokens); seq = device int32, the step number, starts at 1 with all flags 0; counter = device uint32 [2], zero.
 * Step on every rank, one stream:  b200_ep_dispatch -> b200_ep_wait(own flags_in, world, seq, 0, 0) -> compute partial fp32 [tokens][dim]
 * over the rows of the own inbox -> b200_ep_return -> b200_ep_wait(own flags_out, world, seq, 1, 1) -> sum partials[rank] over ranks.
 * The waits are bounded (b200_set_wait_limit_ns): a wait that gives up stores 3003 (arrival) / 3004 (return) in the device error word
 * and the step runs on.  Each rank must run on its own GPU (kernels of two ranks that wait for each other cannot share one). */
#define B200_EP_MAX_RANKS 16
#define B200_EP_HANDLE_BYTES 64
typedef struct b200_ep_peers {
    int rank, world;
    int dim;                    /* values of a partial row */
    int x_row_bytes, l_row_bytes; /* multiples of 16 */
    const int* first;
    void* const* inbox_x;
    void* const* inbox_l;
    int* const* flags_in;
    float* const* partials;
    int* const* flags_out;
    int* seq;
    unsigned int* counter;
} b200_ep_peers;
int b200_ep_dispatch(const b200_ep_peers* peers, const void* x_local, const void* logits_local, int local_tokens, cudaStream_t stream);
int b200_ep_return(const b200_ep_peers* peers, const float* partial, int tokens, cudaStream_t stream);
/* waits for flags[0 .. n) >= *seq; advance != 0: then *seq += 1; which: 0 = arrival (code 3003), 1 = return (code 3004) */
int b200_ep_wait(const int* flags, int n, int* seq, int advance, int which, cudaStream_t stream);
/* Set-up calls, NOT stream-ordered (they allocate, synchronise the device, map memory): a zero-filled slab of device memory that other
 * processes may map, its 64-byte handle (CUDA IPC), and the mapping of another process's slab into this one. */
int b200_ep_alloc(size_t bytes, void** ptr);
int b200_ep_free(void* ptr);
int b200_ep_export(const void* ptr, void* handle /* B200_EP_HANDLE_BYTES */);
int b200_ep_open(const void* handle, void** ptr);
int b200_ep_close(void* ptr);

/* ---- device error word.  Every device-side wait of this library is bounded; one that runs out of time stores a non-zero
 * code instead of hanging.  Synchronises `stream`, returns the code in *code (0 = none) and clears it. */
int b200_device_error(int* code, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MOE_H */
