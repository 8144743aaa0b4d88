// Router of the MoE layer as a block-level device routine (128 threads route one token row), shared by the stand-alone
// gate_topk kernel and the fused routing kernel of the decode layer.
#pragma once
#include "common.cuh"

namespace b200 {

// ------------------------------------------------------------------ router  (dsv41/model.py:1614-1630, dsv41/fused2.py:451-483)
// one block (128 threads) per token row.  mode 0 sqrt(softplus), 1 sigmoid, 2 softmax.
constexpr int GATE_THREADS = 128;
constexpr int GATE_MAX_PER_THREAD = 8;  // E <= 1024

__device__ __forceinline__ float block_max_128(float v, float* sh) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum_128(float v, float* sh) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = (sh[0] + sh[1]) + (sh[2] + sh[3]);
    __syncthreads();
    return r;
}

// Device routine shared with the fused decode prologue: the calling block (128 threads) routes one row.
__device__ inline void gate_topk_row(const float* __restrict__ srow, const __nv_bfloat16* __restrict__ srow_bf16, const float* __restrict__ bias, int E,
                              float temp, int topk, float route_scale, int mode, int norm, int* __restrict__ eid, float* __restrict__ wt,
                              float* sh_f, int* sh_i) {
    const int tid = threadIdx.x;
    float s[GATE_MAX_PER_THREAD], key[GATE_MAX_PER_THREAD];
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) {
        int e = tid + i * GATE_THREADS;
        float v = -INFINITY;
        if (e < E) v = __fdiv_rn(srow ? srow[e] : __bfloat162float(srow_bf16[e]), temp);
        s[i] = v;
    }
    if (mode == 2) {
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) mx = fmaxf(mx, s[i]);
        mx = block_max_128(mx, sh_f);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) {
            int e = tid + i * GATE_THREADS;
            s[i] = e < E ? expf(s[i] - mx) : 0.f;
            sum += s[i];
        }
        sum = block_sum_128(sum, sh_f);
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) s[i] = __fdiv_rn(s[i], sum);
    } else if (mode == 1) {
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) s[i] = __fdiv_rn(1.f, 1.f + expf(-s[i]));
    } else {
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) s[i] = sqrtf(s[i] > 20.f ? s[i] : log1pf(expf(s[i])));
    }
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) {
        int e = tid + i * GATE_THREADS;
        key[i] = e < E ? s[i] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    float wsum = 0.f;
    for (int k = 0; k < topk; ++k) {
        // block arg-max with the lowest index on equal keys
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        float bs = 0.f;
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i) {
            int e = tid + i * GATE_THREADS;
            if (e < E && (key[i] > bv || (key[i] == bv && e < bi))) { bv = key[i]; bi = e; bs = s[i]; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            float os = __shfl_xor_sync(0xffffffffu, bs, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
        }
        if ((tid & 31) == 0) { sh_f[tid >> 5] = bv; sh_i[tid >> 5] = bi; sh_f[4 + (tid >> 5)] = bs; }
        __syncthreads();
        bv = sh_f[0]; bi = sh_i[0]; bs = sh_f[4];
#pragma unroll
        for (int w = 1; w < 4; ++w) {
            float ov = sh_f[w]; int oi = sh_i[w];
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = sh_f[4 + w]; }
        }
        __syncthreads();
        if (tid == 0) { eid[k] = bi; wt[k] = bs; }
        wsum += bs;
#pragma unroll
        for (int i = 0; i < GATE_MAX_PER_THREAD; ++i)
            if (tid + i * GATE_THREADS == bi) key[i] = -INFINITY;
    }
    __syncthreads();
    if (tid < topk) {
        float w = wt[tid];
        if (norm) w = __fdiv_rn(w, wsum + 1e-20f);
        wt[tid] = w * route_scale;
    }
}


}  // namespace b200
