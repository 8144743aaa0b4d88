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

// Called by all 32 lanes of one warp.  The scores and the selection keys of the row live in REGISTERS: lane l owns the experts
// l, l + 32, ... (at most GATE_MAX_EXPERTS / 32 = 32 of them, fully unrolled so that the exponentials, the divisions and the per-lane
// maxima of different experts overlap); shared memory is not used (s_val / s_key are accepted for the callers' sake).
template <int PER>
__device__ __forceinline__ void gate_topk_regs(const float* __restrict__ srow, const __nv_bfloat16* __restrict__ srow_bf16, const float* __restrict__ bias, int E,
                                               float temp, int topk, float route_scale, int mode, int norm, int* __restrict__ eid, float* __restrict__ wt) {
    const int lane = threadIdx.x & 31;
    float val[PER], key[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        float v = -INFINITY;
        if (e < E) v = __fdiv_rn(srow ? srow[e] : __bfloat162float(srow_bf16[e]), temp);
        val[i] = v;
        mx = fmaxf(mx, v);
    }
    if (mode == 2) {
        mx = warp_max(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if (i * 32 < E) {  // lanes past E hold -inf: exp gives 0
                val[i] = i * 32 + lane < E ? expf(val[i] - mx) : 0.f;
                sum += val[i];
            }
        }
        sum = warp_sum(sum);
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 < E) val[i] = __fdiv_rn(val[i], sum);
    } else if (mode == 1) {
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 < E) val[i] = __fdiv_rn(1.f, 1.f + expf(-val[i]));
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 < E) { const float v = val[i]; val[i] = sqrtf(v > 20.f ? v : log1pf(expf(v))); }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        key[i] = e < E ? val[i] + (bias ? bias[e] : 0.f) : -INFINITY;
        if (e >= E) key[i] = -INFINITY;
    }
    float wsum = 0.f, mine = 0.f;
    for (int k = 0; k < topk; ++k) {
        // warp arg-max with the lowest index on equal keys; a lane's experts are in increasing index order, so `>` keeps its lowest
        float bv = -INFINITY, bs = 0.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if (i * 32 < E) {
                const int e = i * 32 + lane;
                if (e < E && (key[i] > bv || (key[i] == bv && e < bi))) { bv = key[i]; bi = e; bs = val[i]; }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
        }
        if (bi >= E) {  // every key NaN: nothing compares; keep the indices in range
            bi = 0;
            bs = __shfl_sync(0xffffffffu, val[0], 0);
        }
        if (lane == 0) eid[k] = bi;
        if (lane == k) mine = bs;
        wsum += bs;
        // the owner lane retires the expert
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 < E && i * 32 + lane == bi) key[i] = -INFINITY;
    }
    if (lane < topk) {
        float w = mine;
        if (norm) w = __fdiv_rn(w, wsum + 1e-20f);
        wt[lane] = w * route_scale;
    }
}

// the unrolled body is instantiated for a few expert counts so that a 384-expert router does not carry 1024 experts' worth of code
__device__ inline void gate_topk_warp(const float* __restrict__ srow, const __nv_bfloat16* __restrict__ srow_bf16, const float* __restrict__ bias, int E,
                                      float temp, int topk, float route_scale, int mode, int norm, int* __restrict__ eid, float* __restrict__ wt,
                                      float* /*s_val*/, float* /*s_key*/) {
    if (E <= 128) gate_topk_regs<4>(srow, srow_bf16, bias, E, temp, topk, route_scale, mode, norm, eid, wt);
    else if (E <= 384) gate_topk_regs<12>(srow, srow_bf16, bias, E, temp, topk, route_scale, mode, norm, eid, wt);
    else gate_topk_regs<GATE_MAX_EXPERTS / 32>(srow, srow_bf16, bias, E, temp, topk, route_scale, mode, norm, eid, wt);
}

// ------------------------------------------------------------------ the same router by a whole block of 128 threads (one token row)
// Thread t owns the experts t, t + 128, ...; maxima, sums and the arg-max of every selection round are reduced inside the warps by
// shuffles and across the four warps through a few words of shared memory (one block barrier per reduction).  Four times fewer
// experts per thread than the warp form and four times the instruction-level parallelism: the routing of a decode step drops from
// about 9 us to about 2.  Results are those of gate_topk_warp except for the order in which the softmax sum is added up.
constexpr int GATE_BLOCK_THREADS = 128;
struct GateBlockSmem {
    float red[2][4];     // max / sum reductions
    float bv[2][4], bs[2][4];
    int bi[2][4];        // per-warp candidates of a selection round, double-buffered by round parity
};

template <int PER>
__device__ __forceinline__ void gate_topk_block_regs(const float* __restrict__ srow, const __nv_bfloat16* __restrict__ srow_bf16, const float* __restrict__ bias,
                                                     int E, float temp, int topk, float route_scale, int mode, int norm, int* __restrict__ eid,
                                                     float* __restrict__ wt, GateBlockSmem& sm) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float val[PER], key[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * GATE_BLOCK_THREADS + tid;
        float v = -INFINITY;
        if (e < E) v = __fdiv_rn(srow ? srow[e] : __bfloat162float(srow_bf16[e]), temp);
        val[i] = v;
        mx = fmaxf(mx, v);
    }
    if (mode == 2) {
        mx = warp_max(mx);
        if (lane == 0) sm.red[0][warp] = mx;
        __syncthreads();
        mx = fmaxf(fmaxf(sm.red[0][0], sm.red[0][1]), fmaxf(sm.red[0][2], sm.red[0][3]));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            val[i] = i * GATE_BLOCK_THREADS + tid < E ? expf(val[i] - mx) : 0.f;
            sum += val[i];
        }
        sum = warp_sum(sum);
        if (lane == 0) sm.red[1][warp] = sum;
        __syncthreads();
        sum = (sm.red[1][0] + sm.red[1][1]) + (sm.red[1][2] + sm.red[1][3]);
#pragma unroll
        for (int i = 0; i < PER; ++i) val[i] = __fdiv_rn(val[i], sum);
    } else if (mode == 1) {
#pragma unroll
        for (int i = 0; i < PER; ++i) val[i] = __fdiv_rn(1.f, 1.f + expf(-val[i]));
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) { const float v = val[i]; val[i] = sqrtf(v > 20.f ? v : log1pf(expf(v))); }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * GATE_BLOCK_THREADS + tid;
        key[i] = e < E ? val[i] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    const float val0 = val[0];  // thread 0: expert 0 (the fallback when every key is NaN)
    float wsum = 0.f, mine = 0.f;
    for (int k = 0; k < topk; ++k) {
        // arg-max with the lowest index on equal keys: per thread (increasing index order), per warp (shuffles), per block (shared memory)
        float bv = -INFINITY, bs = 0.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * GATE_BLOCK_THREADS + tid;
            if (e < E && (key[i] > bv || (key[i] == bv && e < bi))) { bv = key[i]; bi = e; bs = val[i]; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
        }
        const int pb = k & 1;
        if (lane == 0) { sm.bv[pb][warp] = bv; sm.bi[pb][warp] = bi; sm.bs[pb][warp] = bs; }
        if (k == 0 && tid == 0) sm.red[0][0] = val0;
        __syncthreads();
        bv = sm.bv[pb][0]; bi = sm.bi[pb][0]; bs = sm.bs[pb][0];
#pragma unroll
        for (int w = 1; w < 4; ++w) {
            const float ov = sm.bv[pb][w];
            const int oi = sm.bi[pb][w];
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = sm.bs[pb][w]; }
        }
        if (bi >= E) { bi = 0; bs = sm.red[0][0]; }  // every key NaN: nothing compares; keep the indices in range
        if (tid == 0) eid[k] = bi;
        if (tid == k) mine = bs;
        wsum += bs;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * GATE_BLOCK_THREADS + tid == bi) key[i] = -INFINITY;  // the owner retires the expert
    }
    if (tid < topk) {
        float w = mine;
        if (norm) w = __fdiv_rn(w, wsum + 1e-20f);
        wt[tid] = w * route_scale;
    }
}

// Called by all GATE_BLOCK_THREADS threads of a block (contains block barriers).
__device__ inline void gate_topk_block(const float* __restrict__ srow, const __nv_bfloat16* __restrict__ srow_bf16, const float* __restrict__ bias, int E,
                                       float temp, int topk, float route_scale, int mode, int norm, int* __restrict__ eid, float* __restrict__ wt,
                                       GateBlockSmem& sm) {
    if (E <= 384) gate_topk_block_regs<3>(srow, srow_bf16, bias, E, temp, topk, route_scale, mode, norm, eid, wt, sm);
    else gate_topk_block_regs<GATE_MAX_EXPERTS / GATE_BLOCK_THREADS>(srow, srow_bf16, bias, E, temp, topk, route_scale, mode, norm, eid, wt, sm);
}

}  // namespace b200
