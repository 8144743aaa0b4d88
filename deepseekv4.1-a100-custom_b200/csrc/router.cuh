// Router of the MoE layer as a warp-level device routine (one warp routes one token row), shared by the stand-alone
// gate_topk kernel and the fused routing kernel of the layer.
#pragma once
#include "common.cuh"

namespace b200 {

// ------------------------------------------------------------------ router  (dsv41/model.py:1614-1630, dsv41/fused2.py:451-483)
// mode 0 sqrt(softplus), 1 sigmoid, 2 softmax.  One warp per row keeps the whole selection free of block barriers: the
// scores and the selection keys of the row live in shared memory (E floats each), lane l owns the experts l, l + 32, ...
constexpr int GATE_MAX_EXPERTS = 1024;
constexpr int GATE_ROWS_PER_BLOCK = 4;  // of the stand-alone kernel

// Called by all 32 lanes of one warp.  s_val / s_key: shared-memory scratch of E floats each, private to the warp.
__device__ inline void gate_topk_warp(const float* __restrict__ srow, const __nv_bfloat16* __restrict__ srow_bf16, const float* __restrict__ bias, int E,
                                      float temp, int topk, float route_scale, int mode, int norm, int* __restrict__ eid, float* __restrict__ wt,
                                      float* s_val, float* s_key) {
    const int lane = threadIdx.x & 31;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) {
        const float raw = srow ? srow[e] : __bfloat162float(srow_bf16[e]);
        const float v = __fdiv_rn(raw, temp);
        s_val[e] = v;
        mx = fmaxf(mx, v);
    }
    if (mode == 2) {
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float ex = expf(s_val[e] - mx);
            s_val[e] = ex;
            sum += ex;
        }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) s_val[e] = __fdiv_rn(s_val[e], sum);
    } else if (mode == 1) {
        for (int e = lane; e < E; e += 32) s_val[e] = __fdiv_rn(1.f, 1.f + expf(-s_val[e]));
    } else {
        for (int e = lane; e < E; e += 32) {
            const float v = s_val[e];
            s_val[e] = sqrtf(v > 20.f ? v : log1pf(expf(v)));
        }
    }
    for (int e = lane; e < E; e += 32) s_key[e] = s_val[e] + (bias ? bias[e] : 0.f);
    __syncwarp();
    float wsum = 0.f, mine = 0.f;
    for (int k = 0; k < topk; ++k) {
        // warp arg-max with the lowest index on equal keys
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float kv = s_key[e];
            if (kv > bv || (kv == bv && e < bi)) { bv = kv; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= E) bi = 0;  // every key NaN: nothing compares; keep the indices in range
        const float bs = s_val[bi];
        if (lane == 0) eid[k] = bi;
        if (lane == k) mine = bs;
        wsum += bs;
        if (lane == (bi & 31)) s_key[bi] = -INFINITY;
        __syncwarp();
    }
    if (lane < topk) {
        float w = mine;
        if (norm) w = __fdiv_rn(w, wsum + 1e-20f);
        wt[lane] = w * route_scale;
    }
}

}  // namespace b200
