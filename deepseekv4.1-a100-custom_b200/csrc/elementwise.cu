// Small per-token kernels on the MoE path: activation FP8 fake quantisation, router (score / top-k / renormalise),
// SwiGLU + fake quantisation, routed + shared combine, per-token partial row sums, 8-k activation permutation.
// All are HBM/latency bound; one warp per 32-element group or one block per token row.
#include "common.cuh"
#include "router.cuh"
#include "b200_moe.h"

namespace b200 {

// ------------------------------------------------------------------ fake_quant_fp8  (dsv41/quant.py:46-54, dsv41/fused.py:48-79 MODE 0)
// one warp per group of 32, lane = element.  x,y bf16 [n_groups*32].
__global__ void fake_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long n_groups) {
    long g = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (g >= n_groups) return;
    float v = __bfloat162float(x[g * 32 + lane]);
    float s = fp8_group_scale(warp_max(fabsf(v)));
    y[g * 32 + lane] = __float2bfloat16_rn(fp8_fake_quant_value(v, s));
}

__global__ void __launch_bounds__(32 * GATE_ROWS_PER_BLOCK) gate_topk_kernel(const float* __restrict__ scores, const float* __restrict__ bias, int rows,
                                                                             int E, float temp, int topk, float route_scale, int mode, int norm,
                                                                             int* __restrict__ eid, float* __restrict__ wt) {
    extern __shared__ float gate_smem[];  // per warp: E scores + E keys
    const int warp = threadIdx.x >> 5;
    const long row = (long)blockIdx.x * GATE_ROWS_PER_BLOCK + warp;
    if (row >= rows) return;
    float* s_val = gate_smem + (size_t)warp * 2 * E;
    gate_topk_warp(scores + row * E, nullptr, bias, E, temp, topk, route_scale, mode, norm, eid + row * topk, wt + row * topk, s_val, s_val + E);
}

// ------------------------------------------------------------------ swiglu_quant  (dsv41/fused.py:285-316)
// one warp per (row, group of 32 columns).  GU fp32 or bf16 [rows, 2*inter]; Y bf16 [rows, inter].
template <typename TIn>
__global__ void swiglu_quant_kernel(const TIn* __restrict__ gu, const float* __restrict__ weights, __nv_bfloat16* __restrict__ y, long rows, int inter,
                                    float limit, int permute) {
    long gid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    int gpr = inter >> 5;
    if (gid >= rows * gpr) return;
    long row = gid / gpr;
    int col = (int)(gid % gpr) * 32 + lane;
    float g = (float)gu[row * 2 * inter + col];
    float u = (float)gu[row * 2 * inter + inter + col];
    float h = swiglu_bf16(g, u, weights ? weights[row] : 1.f, limit);
    float s = fp8_group_scale(warp_max(fabsf(h)));
    float q = fp8_fake_quant_value(h, s);
    if (permute) {  // 8-k permuted store (bit reversal of the low 3 column bits), dsv41/fused.py:303-305
        int j = col & 7;
        col = (col & ~7) | ((j & 1) << 2) | (j & 2) | (j >> 2);
    }
    y[row * inter + col] = __float2bfloat16_rn(q);
}

// ------------------------------------------------------------------ combine  (dsv41/fused2.py:518-523 NSUM branch; dsv41/model.py:2114-2118, 2232)
// out[t, n] = bf16( sum_j y2[t*nsum + j, n] + float(ys[t, n]) ), fp32 sum in slot order.
__global__ void combine_kernel(const float* __restrict__ y2, const __nv_bfloat16* __restrict__ ys, __nv_bfloat16* __restrict__ out, long T, int nsum,
                               int dim) {
    long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * dim) return;
    long t = i / dim;
    int n = (int)(i % dim);
    float acc = 0.f;
    for (int j = 0; j < nsum; ++j) acc += y2[(t * nsum + j) * dim + n];
    if (ys) acc += __bfloat162float(ys[i]);
    out[i] = __float2bfloat16_rn(acc);
}

// ------------------------------------------------------------------ sum_rows  (dsv41/cuda/p2p.cu:21-28 via dsv41/cukern.py:370-379)
// dst[g*dst_stride + c] = sum_{r<rows} src[(g*rows + r)*n + c]
__global__ void sum_rows_kernel(float* __restrict__ dst, const float* __restrict__ src, int rows, int n, int groups, long dst_stride) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    int g = blockIdx.y;
    if (c >= n) return;
    float acc = 0.f;
    for (int r = 0; r < rows; ++r) acc += src[((long)g * rows + r) * n + c];
    dst[(long)g * dst_stride + c] = acc;
}

// ------------------------------------------------------------------ permute_x  (dsv41/cukern.py:267-273)
__global__ void permute8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long n) {
    long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int j = (int)(i & 7);
    long src = (i & ~7L) | ((j & 1) << 2) | (j & 2) | (j >> 2);  // stored slot j holds k = bitrev3(j)
    y[i] = x[src];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_fake_quant_fp8(const void* x, void* y, long long n_elems, cudaStream_t stream) {
    if (!x || !y || n_elems < 0) return ERR_BAD_ARG;
    if (n_elems % 32) return ERR_BAD_SHAPE;
    if (n_elems == 0) return 0;
    long groups = n_elems / 32;
    int wpb = 8;
    fake_quant_fp8_kernel<<<(unsigned)((groups + wpb - 1) / wpb), wpb * 32, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, groups);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_gate_topk(const float* scores, const float* bias, int rows, int n_experts, float temp, int topk, float route_scale,
                              int score_mode, int norm, int* eid, float* wt, cudaStream_t stream) {
    if (!scores || !eid || !wt || rows < 0) return ERR_BAD_ARG;
    if (n_experts < 1 || n_experts > GATE_MAX_EXPERTS || topk < 1 || topk > n_experts || topk > 32) return ERR_BAD_SHAPE;
    if (score_mode < 0 || score_mode > 2) return ERR_UNSUPPORTED;
    if (rows == 0) return 0;
    const size_t smem = (size_t)GATE_ROWS_PER_BLOCK * 2 * n_experts * sizeof(float);
    gate_topk_kernel<<<(rows + GATE_ROWS_PER_BLOCK - 1) / GATE_ROWS_PER_BLOCK, 32 * GATE_ROWS_PER_BLOCK, smem, stream>>>(scores, bias, rows, n_experts, temp, topk,
                                                                                                                  route_scale, score_mode, norm, eid, wt);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_swiglu_quant(const void* gu, int gu_is_bf16, const float* weights, long long rows, int inter, float limit, int permute, void* y,
                                 cudaStream_t stream) {
    if (!gu || !y || rows < 0) return ERR_BAD_ARG;
    if (inter <= 0 || inter % 32) return ERR_BAD_SHAPE;
    if (rows == 0) return 0;
    long warps = rows * (inter / 32);
    int wpb = 8;
    unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
    if (gu_is_bf16)
        swiglu_quant_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, stream>>>((const __nv_bfloat16*)gu, weights, (__nv_bfloat16*)y, rows, inter, limit, permute);
    else
        swiglu_quant_kernel<float><<<grid, wpb * 32, 0, stream>>>((const float*)gu, weights, (__nv_bfloat16*)y, rows, inter, limit, permute);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_moe_combine(const float* y2, const void* ys, void* out, long long tokens, int nsum, int dim, cudaStream_t stream) {
    if (!y2 || !out || tokens < 0 || nsum < 0 || dim <= 0) return ERR_BAD_ARG;
    if (tokens == 0) return 0;
    long n = tokens * dim;
    combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(y2, (const __nv_bfloat16*)ys, (__nv_bfloat16*)out, tokens, nsum, dim);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_sum_rows(float* dst, const float* src, int rows, int n, int groups, long long dst_stride, cudaStream_t stream) {
    if (!dst || !src || rows < 0 || n <= 0 || groups < 0) return ERR_BAD_ARG;
    if (groups == 0) return 0;
    dim3 grid((n + 255) / 256, groups);
    sum_rows_kernel<<<grid, 256, 0, stream>>>(dst, src, rows, n, groups, dst_stride);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_permute_x8(const void* x, void* y, long long n_elems, cudaStream_t stream) {
    if (!x || !y || n_elems < 0) return ERR_BAD_ARG;
    if (n_elems % 8) return ERR_BAD_SHAPE;
    if (n_elems == 0) return 0;
    permute8_kernel<<<(unsigned)((n_elems + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n_elems);
    B200_CHECK_LAUNCH();
    return 0;
}
