// MoE layer (any batch size) and the C-ABI entry points of the grouped FP4 / dense FP8 GEMMs.
//
// Layer = one routing kernel (router, bucketing of the (token, expert) pairs by expert, work list; for the streaming engine also
// the input fake quantisation), then either the block-scaled tensor-core GEMMs (mxgemm.cu: one quantisation launch, gate/up GEMM and
// down GEMM, each carrying the routed experts and the shared expert) or the weight-streaming GEMMs (skinny.cu), then a combine.
#include <cuda_fp8.h>

#include "common.cuh"
#include "skinny.cuh"
#include "mxgemm.cuh"
#include "wmgemm.cuh"
#include "gate_gemm.cuh"
#include "router.cuh"
#include "b200_moe.h"

namespace b200 {

int p2p_device_error(int* out);  // p2p.cu

constexpr int ROUTE_THREADS = 128;
static_assert(ROUTE_THREADS == GATE_BLOCK_THREADS, "the block router is written for the routing kernels' block size");
constexpr int ROUTE_MAX_PAIRS = 4096;   // pairs the single-block bucketing handles
constexpr int ROUTE_MAX_EXPERTS = 1024;
constexpr int MX_AUTO_MIN_TOKENS = 0;   // automatic engine choice: the tensor-core kernels serve every batch size whose formats they accept
constexpr int MX_ND_DECODE = 32;        // tokens per work of the block-scaled tensor-core path

struct RouteArgs {
    int tokens, E, topk, dim;
    const float* logits_f32;
    const __nv_bfloat16* logits_bf16;
    const float* bias;
    float temp, route_scale;
    int mode, norm;
    const __nv_bfloat16* x;
    __nv_bfloat16* xq;  // nullptr: x is already quantised
    long long x_ld, logits_ld;  // row strides (elements) of x and of the logits
    int logit_parts;            // > 0: logits_f32 holds that many partial-sum slabs [tokens, E], logit_part_stride floats apart
    long long logit_part_stride;
    int shard_start, shard_n;
    int tpw;            // pairs per work
    int* eid;           // [tokens, topk]
    float* wt;          // [tokens, topk]
    int* pair_tok;      // sorted position -> token
    int* pair_out;      // sorted position -> original pair index t*topk + j
    float* pair_w;      // sorted position -> routing weight
    int4* work;
    int* n_work;
    unsigned int* counter;
    int no_bucket;      // 1: only quantise + route; the pairs are bucketed by the multi-block kernels below
};

// One block per token: fake-quantise the token's activation (dsv41/quant.py:46-54; one thread per group of 32, four 16-byte
// loads in flight) and route it (dsv41/model.py:1614-1630).  The last block to finish buckets all pairs by expert (the
// grouping of dsv41/moe_kernels.py:111-116 and dsv41/decode.py:417-433; the order inside an expert is free) and emits the work list of
// the shard's experts.
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(const RouteArgs a) {
    __shared__ float s_val[ROUTE_MAX_EXPERTS], s_key[ROUTE_MAX_EXPERTS];  // router scratch of warp 0
    __shared__ float s_raw[ROUTE_MAX_EXPERTS];                            // logits of the token when they arrive as k-split partial sums
    __shared__ int is_last;
    __shared__ int s_eid[ROUTE_MAX_PAIRS];
    __shared__ int s_cnt[ROUTE_MAX_EXPERTS];
    __shared__ int s_start[ROUTE_MAX_EXPERTS];
    __shared__ int s_woff[ROUTE_MAX_EXPERTS];
    __shared__ int s_cur[ROUTE_MAX_EXPERTS];
    __shared__ int s_wtot[2][ROUTE_THREADS / 32];
    const int tok = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();  // the next kernel may be placed early; it waits for this one to complete before it reads anything

    if (a.xq) {
        const int groups = a.dim >> 5;
        for (int gi = tid; gi < groups; gi += ROUTE_THREADS) {
            const uint4* src = reinterpret_cast<const uint4*>(a.x + (long)tok * a.x_ld + gi * 32);
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = src[j];
            const uint32_t* w = reinterpret_cast<const uint32_t*>(v);
            float f[32], amax = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                f[2 * j] = bf16_bits_to_f32(w[j] & 0xFFFFu);
                f[2 * j + 1] = bf16_bits_to_f32(w[j] >> 16);
                amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
            }
            const float s = fp8_group_scale(amax);
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
                o[j] = f32_to_bf16_bits(fp8_fake_quant_value(f[2 * j], s)) | (f32_to_bf16_bits(fp8_fake_quant_value(f[2 * j + 1], s)) << 16);
            uint4* dst = reinterpret_cast<uint4*>(a.xq + (long)tok * a.dim + gi * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        }
    }
    if (a.logit_parts > 0) {
        // the fused router projection leaves k-split partial sums: the whole block adds them, in split order, before warp 0 routes
        const float* base = a.logits_f32 + (long)tok * a.E;
        for (int e = tid; e < a.E; e += ROUTE_THREADS) {
            float v = 0.f;
#pragma unroll 4
            for (int p = 0; p < a.logit_parts; ++p) v += __ldg(base + (long long)p * a.logit_part_stride + e);
            s_raw[e] = v;
        }
        __syncthreads();
    }
    if (warp == 0) {
        const float* row_f32 = a.logit_parts > 0 ? s_raw : (a.logits_f32 ? a.logits_f32 + (long)tok * a.logits_ld : nullptr);
        gate_topk_warp(row_f32, a.logits_bf16 ? a.logits_bf16 + (long)tok * a.logits_ld : nullptr, a.bias, a.E, a.temp, a.topk, a.route_scale, a.mode, a.norm,
                       a.eid + (long)tok * a.topk, a.wt + (long)tok * a.topk, s_val, s_key);
    }
    if (a.no_bucket) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = (atomicInc(a.counter, gridDim.x - 1) == gridDim.x - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    const int P = a.tokens * a.topk, E = a.E;
    for (int e = tid; e < E; e += ROUTE_THREADS) s_cnt[e] = 0;
    __syncthreads();
    for (int p = tid; p < P; p += ROUTE_THREADS) {
        const int e = __ldcg(a.eid + p);
        s_eid[p] = e;
        atomicAdd(&s_cnt[e], 1);
    }
    __syncthreads();
    // exclusive scans over experts: pair offsets (all experts) and work offsets (this shard's experts); thread t owns the
    // experts [t*per, t*per + per)
    const int per = (E + ROUTE_THREADS - 1) / ROUTE_THREADS;
    int loc_p = 0, loc_w = 0;
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e < E) {
            loc_p += s_cnt[e];
            if (e >= a.shard_start && e < a.shard_start + a.shard_n) loc_w += (s_cnt[e] + a.tpw - 1) / a.tpw;
        }
    }
    int inc_p = loc_p, inc_w = loc_w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int vp = __shfl_up_sync(0xffffffffu, inc_p, o), vw = __shfl_up_sync(0xffffffffu, inc_w, o);
        if (lane >= o) { inc_p += vp; inc_w += vw; }
    }
    if (lane == 31) { s_wtot[0][warp] = inc_p; s_wtot[1][warp] = inc_w; }
    __syncthreads();
    int run_p = inc_p - loc_p, run_w = inc_w - loc_w, tot_w = 0;
    for (int w = 0; w < ROUTE_THREADS / 32; ++w) {
        if (w < warp) { run_p += s_wtot[0][w]; run_w += s_wtot[1][w]; }
        tot_w += s_wtot[1][w];
    }
    if (tid == 0) *a.n_work = tot_w;
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e < E) {
            s_start[e] = run_p;
            s_woff[e] = run_w;
            run_p += s_cnt[e];
            if (e >= a.shard_start && e < a.shard_start + a.shard_n) run_w += (s_cnt[e] + a.tpw - 1) / a.tpw;
        }
    }
    __syncthreads();
    // works of this shard's experts, then the placement of the pairs through one cursor per expert.  The order of the pairs
    // inside an expert is whatever the atomics give: every pair is computed on its own and lands in its own output slot, so
    // the order does not reach the results.
    for (int e = tid; e < E; e += ROUTE_THREADS) {
        const int cnt = s_cnt[e];
        s_cur[e] = s_start[e];
        if (cnt > 0 && e >= a.shard_start && e < a.shard_start + a.shard_n) {
            const int nsub = (cnt + a.tpw - 1) / a.tpw;
            for (int i = 0; i < nsub; ++i) {
                const int rem = cnt - i * a.tpw;
                a.work[s_woff[e] + i] = make_int4(e - a.shard_start, s_start[e] + i * a.tpw, rem < a.tpw ? rem : a.tpw, e);
            }
        }
    }
    __syncthreads();
    for (int p = tid; p < P; p += ROUTE_THREADS) {
        const int o = atomicAdd(&s_cur[s_eid[p]], 1);
        a.pair_tok[o] = p / a.topk;
        a.pair_out[o] = p;
        a.pair_w[o] = __ldcg(a.wt + p);
    }
}

// Router alone for prefill-sized batches whose pairs are bucketed by the multi-block kernels below: one WARP per token, eight tokens per
// block, scratch of 3 E floats per warp.  (moe_route_kernel keeps 50 KB of bucketing tables per block, which leaves four one-warp
// routers per SM: 70 us for 4096 tokens.)
constexpr int ROUTE_ROWS_PER_BLOCK = 8;
__global__ void __launch_bounds__(32 * ROUTE_ROWS_PER_BLOCK) route_rows_kernel(const RouteArgs a) {
    extern __shared__ float route_smem[];  // per warp: E scores, E keys, E raw logits
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long tok = (long)blockIdx.x * ROUTE_ROWS_PER_BLOCK + warp;
    if (tok >= a.tokens) return;
    float* s_val = route_smem + (size_t)warp * 3 * a.E;
    float* s_key = s_val + a.E;
    float* s_raw = s_key + a.E;
    const float* row_f32 = a.logits_f32 ? a.logits_f32 + tok * a.logits_ld : nullptr;
    if (a.logit_parts > 0) {  // k-split partial sums of the fused router projection, added in split order
        const float* base = a.logits_f32 + tok * a.E;
        for (int e = lane; e < a.E; e += 32) {
            float v = 0.f;
#pragma unroll 4
            for (int p = 0; p < a.logit_parts; ++p) v += __ldg(base + (long long)p * a.logit_part_stride + e);
            s_raw[e] = v;
        }
        __syncwarp();
        row_f32 = s_raw;
    }
    gate_topk_warp(row_f32, a.logits_bf16 ? a.logits_bf16 + tok * a.logits_ld : nullptr, a.bias, a.E, a.temp, a.topk, a.route_scale, a.mode, a.norm,
                   a.eid + tok * a.topk, a.wt + tok * a.topk, s_val, s_key);
}

// ------------------------------------------------------------------ decode-sized batches (at most 64 tokens) on the weight-stream kernels
// One block per token: FP8 quantisation of the token's activation kept in quantised form (e4m3 bytes + the E8M0 scale bytes written
// straight into the 512-byte atoms the tensor cores read, see wmgemm.cu), and the router.  The last block to finish lists the
// distinct experts of this shard that any token chose (one work each, in expert order) and fills, per work, a table over the tokens:
// slot[w][t] = 1 + the top-k slot of expert w in token t's selection (0: t did not choose it), wtab[w][t] = its routing weight.
// Nothing is sorted or gathered: every work multiplies its expert with all tokens and the epilogues keep the chosen pairs.
struct DqRouteArgs {
    int tokens, E, topk, dim, NT;
    const float* logits_f32;
    const __nv_bfloat16* logits_bf16;
    const float* bias;
    float temp, route_scale;
    int mode, norm;
    const __nv_bfloat16* x;
    long long x_ld, logits_ld;
    int logit_parts;
    long long logit_part_stride;
    int shard_start, shard_n;
    int* eid;
    float* wt;
    const int* eid_in;  // routing decided by the caller (then no router runs): [tokens][topk], with wt_in
    const float* wt_in;
    uint8_t* x8;        // [NT][dim]
    uint8_t* x_atoms;   // [dim / 128][512]
    int* work;
    int* n_work;
    uint8_t* slot;      // [works][NT]
    int* pair_work;     // [tokens * topk]: work of the pair's expert, -1 when the expert is not in this shard
    unsigned int* counter;
    int* flags;         // flag words of the split-k exchange of the two GEMM launches that follow: cleared here
    int n_flags;
};

__global__ void __launch_bounds__(ROUTE_THREADS) dq_route_kernel(const DqRouteArgs a) {
    __shared__ GateBlockSmem s_gate;
    __shared__ float s_raw[ROUTE_MAX_EXPERTS];
    __shared__ int s_widx[ROUTE_MAX_EXPERTS];
    __shared__ int s_wtot[ROUTE_THREADS / 32];
    __shared__ int is_last;
    const int tok = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    if (blockIdx.x == 0)
        for (int i = tid; i < a.n_flags; i += ROUTE_THREADS) a.flags[i] = 0;

    const int groups = a.dim >> 5;
    for (int gi = tid; gi < groups; gi += ROUTE_THREADS) {
        const uint4* src = reinterpret_cast<const uint4*>(a.x + (long)tok * a.x_ld + gi * 32);
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __ldg(src + j);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(v);
        float f[32], amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            f[2 * j] = bf16_bits_to_f32(w[j] & 0xFFFFu);
            f[2 * j + 1] = bf16_bits_to_f32(w[j] >> 16);
            amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
        }
        const float sc = fp8_group_scale_bf16(amax);  // the inputs are bf16 values
        const uint32_t sb = (f32_as_u32(sc) >> 23) & 0xFFu;
        const float inv = u32_as_f32((254u - sb) << 23);  // 1 / sc, exact
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t q = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float qv = fminf(fmaxf(f[4 * j + e] * inv, -448.f), 448.f);
                q |= (uint32_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3) << (8 * e);
            }
            o[j] = q;
        }
        uint4* dst = reinterpret_cast<uint4*>(a.x8 + (long)tok * a.dim + gi * 32);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        a.x_atoms[(size_t)(gi >> 2) * 512 + (tok & 31) * 16 + (tok >> 5) * 4 + (gi & 3)] = (uint8_t)sb;
    }
    if (a.logit_parts > 0) {
        const float* base = a.logits_f32 + (long)tok * a.E;
        for (int e = tid; e < a.E; e += ROUTE_THREADS) {
            float v = 0.f;
#pragma unroll 4
            for (int p = 0; p < a.logit_parts; ++p) v += __ldg(base + (long long)p * a.logit_part_stride + e);
            s_raw[e] = v;
        }
        __syncthreads();
    }
    if (a.eid_in) {
        if (tid < a.topk) {
            a.eid[(long)tok * a.topk + tid] = __ldg(a.eid_in + (long)tok * a.topk + tid);
            a.wt[(long)tok * a.topk + tid] = __ldg(a.wt_in + (long)tok * a.topk + tid);
        }
    } else {
        const float* row_f32 = a.logit_parts > 0 ? s_raw : (a.logits_f32 ? a.logits_f32 + (long)tok * a.logits_ld : nullptr);
        gate_topk_block(row_f32, a.logits_bf16 ? a.logits_bf16 + (long)tok * a.logits_ld : nullptr, a.bias, a.E, a.temp, a.topk, a.route_scale, a.mode, a.norm,
                        a.eid + (long)tok * a.topk, a.wt + (long)tok * a.topk, s_gate);
    }
    __threadfence();
    __syncthreads();
    if (gridDim.x > 1) {  // a single token needs no election (and the host skips clearing the counter)
        if (tid == 0) is_last = (atomicInc(a.counter, gridDim.x - 1) == gridDim.x - 1);
        __syncthreads();
        if (!is_last) return;
        __threadfence();
    }

    const int P = a.tokens * a.topk, E = a.E;
    for (int e = tid; e < E; e += ROUTE_THREADS) s_widx[e] = 0;
    __syncthreads();
    for (int p = tid; p < P; p += ROUTE_THREADS) {
        const int e = __ldcg(a.eid + p);
        if (e >= a.shard_start && e < a.shard_start + a.shard_n) s_widx[e] = 1;  // every writer stores the same value
    }
    __syncthreads();
    const int per = (E + ROUTE_THREADS - 1) / ROUTE_THREADS;
    int loc = 0;
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e < E) loc += s_widx[e];
    }
    int inc = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) s_wtot[warp] = inc;
    __syncthreads();
    int run = inc - loc, total = 0;
    for (int w = 0; w < ROUTE_THREADS / 32; ++w) {
        if (w < warp) run += s_wtot[w];
        total += s_wtot[w];
    }
    if (tid == 0) *a.n_work = total;
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e < E) {
            if (s_widx[e]) {
                a.work[run] = e - a.shard_start;
                s_widx[e] = run++;
            } else {
                s_widx[e] = -1;
            }
        }
    }
    uint32_t* slot32 = reinterpret_cast<uint32_t*>(a.slot);
    for (int i = tid; i < total * (a.NT >> 2); i += ROUTE_THREADS) slot32[i] = 0;
    __syncthreads();
    for (int p = tid; p < P; p += ROUTE_THREADS) {
        const int e = __ldcg(a.eid + p);
        if (e < a.shard_start || e >= a.shard_start + a.shard_n) { a.pair_work[p] = -1; continue; }
        const int w = s_widx[e], t = p / a.topk, j = p - t * a.topk;
        a.slot[(size_t)w * a.NT + t] = (uint8_t)(j + 1);
        a.pair_work[p] = w;
    }
}

// SwiGLU (+ routing weight) + FP8 quantisation between the two GEMMs of a decode-sized batch (dsv41/fused.py:285-306): one block per
// (token, expert) pair and one per token for the shared expert; a warp per group of 32 columns.  Reads the fp32 gate | up rows the first
// GEMM stored, writes e4m3 bytes into the rows the second GEMM reads (row = work * NT + token) and the E8M0 scale bytes straight into
// the 512-byte atoms its tensor cores take (wmgemm.cu).
struct DqSwigluArgs {
    const float* gu;       // [pairs][2 inter]
    const float* gus;      // [tokens][2 inter] (shared expert; nullptr: none)
    int pairs, tokens, topk, inter, NT;
    const float* wt;       // [pairs]
    const int* pair_work;  // [pairs]
    float limit;
    uint8_t *h8, *h_atoms, *hs8, *hs_atoms;
};

__global__ void __launch_bounds__(256) dq_swiglu_kernel(const DqSwigluArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, I = a.inter;
    const float* src;
    uint8_t *out, *atoms;
    float w = 1.f;
    int t, round_gu = 0;
    if (b < a.pairs) {
        const int wk = __ldg(a.pair_work + b);
        if (wk < 0) return;
        t = b / a.topk;
        w = __ldg(a.wt + b);
        src = a.gu + (size_t)b * 2 * I;
        out = a.h8 + ((size_t)wk * a.NT + t) * I;
        atoms = a.h_atoms + (size_t)wk * (I >> 7) * 512;
    } else {
        t = b - a.pairs;
        src = a.gus + (size_t)t * 2 * I;
        out = a.hs8 + (size_t)t * I;
        atoms = a.hs_atoms;
        round_gu = 1;  // the shared expert's gate / up values pass through bf16 (dsv41/model.py:1635-1638)
    }
    for (int g0 = warp; g0 < (I >> 5); g0 += 64) {  // eight groups per warp and pass, their 16 loads in flight together
        float gt[8], up[8], h[8], amax[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int g = g0 + 8 * u;
            gt[u] = up[u] = 0.f;
            if (g < (I >> 5)) { gt[u] = __ldcg(src + g * 32 + lane); up[u] = __ldcg(src + I + g * 32 + lane); }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (round_gu) { gt[u] = round_bf16(gt[u]); up[u] = round_bf16(up[u]); }
            h[u] = swiglu_bf16(gt[u], up[u], w, a.limit);
            amax[u] = fabsf(h[u]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < 8; ++u) amax[u] = fmaxf(amax[u], __shfl_xor_sync(0xffffffffu, amax[u], o));
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int g = g0 + 8 * u;
            if (g >= (I >> 5)) continue;
            const uint32_t sb = (f32_as_u32(fp8_group_scale_bf16(amax[u])) >> 23) & 0xFFu;
            const float qv = fminf(fmaxf(h[u] * u32_as_f32((254u - sb) << 23), -448.f), 448.f);
            out[g * 32 + lane] = (uint8_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3);
            if (lane == 0) atoms[(size_t)(g >> 2) * 512 + (t & 31) * 16 + (t >> 5) * 4 + (g & 3)] = (uint8_t)sb;
        }
    }
}

// ------------------------------------------------------------------ bucketing of many pairs (prefill): histogram, scan + work list, scatter.
// The order of the pairs inside an expert is whatever the atomic cursors give: every pair is computed independently and the
// per-token sum is formed elsewhere, so the order does not reach the results.
__global__ void pair_hist_kernel(const int* __restrict__ eid, int P, int* __restrict__ cnt) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p < P) atomicAdd(cnt + eid[p], 1);
}

__global__ void __launch_bounds__(1024) pair_scan_kernel(const int* __restrict__ cnt, int E, int shard_start, int shard_n, int tpw, int* __restrict__ cursor,
                                                         int4* __restrict__ work, int* __restrict__ n_work) {
    __shared__ int wp[32], ww[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = tid < E ? cnt[tid] : 0;
    const bool mine = tid < E && tid >= shard_start && tid < shard_start + shard_n;
    const int nw = mine ? (c + tpw - 1) / tpw : 0;
    int ip = c, iw = nw;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int vp = __shfl_up_sync(0xffffffffu, ip, o), vw = __shfl_up_sync(0xffffffffu, iw, o);
        if (lane >= o) { ip += vp; iw += vw; }
    }
    if (lane == 31) { wp[warp] = ip; ww[warp] = iw; }
    __syncthreads();
    int bp = ip - c, bw = iw - nw, tw = 0;
    for (int w = 0; w < 32; ++w) {
        if (w < warp) { bp += wp[w]; bw += ww[w]; }
        tw += ww[w];
    }
    if (tid < E) {
        cursor[tid] = bp;
        for (int i = 0; i < nw; ++i) {
            const int rem = c - i * tpw;
            work[bw + i] = make_int4(tid - shard_start, bp + i * tpw, rem < tpw ? rem : tpw, tid);
        }
    }
    if (tid == 0) *n_work = tw;
}

__global__ void pair_scatter_kernel(const int* __restrict__ eid, const float* __restrict__ wt, int P, int topk, int* __restrict__ cursor,
                                    int* __restrict__ pair_tok, int* __restrict__ pair_out, float* __restrict__ pair_w, int out_is_token) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int pos = atomicAdd(cursor + eid[p], 1);
    pair_tok[pos] = p / topk;
    pair_out[pos] = out_is_token ? p / topk : p;
    pair_w[pos] = wt[p];
}

// out[t, n] = bf16(acc[t, n] + float(ys[t, n]))
__global__ void moe_finalize_kernel(const float* __restrict__ acc, const __nv_bfloat16* __restrict__ ys, __nv_bfloat16* __restrict__ out, long n) {
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(acc[i] + (ys ? __bfloat162float(ys[i]) : 0.f));
}
// the same, eight values per thread with 16-byte accesses (all three pointers 16-byte aligned, n a multiple of 8)
__global__ void moe_finalize_vec_kernel(const float4* __restrict__ acc, const uint4* __restrict__ ys, uint4* __restrict__ out, long n8) {
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const float4 a0 = acc[2 * i], a1 = acc[2 * i + 1];
    const uint4 y = ys ? ys[i] : make_uint4(0, 0, 0, 0);
    const float f[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t yw[4] = {y.x, y.y, y.z, y.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = f32_to_bf16_bits(f[2 * j] + bf16_bits_to_f32(yw[j] & 0xFFFFu)) | (f32_to_bf16_bits(f[2 * j + 1] + bf16_bits_to_f32(yw[j] >> 16)) << 16);
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// out[t, n] = bf16( sum over the token's LOCAL experts of y2[t*topk + j, n] + float(ys[t, n]) )  (dsv41/fused2.py:518-523);
// routed[t, n] (optional) = the fp32 routed sum alone (what an expert-parallel rank sends back, dsv41/ep.py:431-435).
__global__ void moe_combine_kernel(const float* __restrict__ y2, const int* __restrict__ eid, const __nv_bfloat16* __restrict__ ys,
                                   __nv_bfloat16* __restrict__ out, float* __restrict__ routed, int tokens, int topk, int dim, int shard_start,
                                   int shard_n) {
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)tokens * dim) return;
    const int t = (int)(i / dim), n = (int)(i % dim);
    float acc = 0.f;
    for (int j = 0; j < topk; ++j) {
        const int e = eid[t * topk + j];
        if (e >= shard_start && e < shard_start + shard_n) acc += y2[((long)t * topk + j) * dim + n];
    }
    if (routed) routed[i] = acc;
    if (out) out[i] = __float2bfloat16_rn(acc + (ys ? __bfloat162float(ys[i]) : 0.f));
}

// the same with four columns per thread: the top-k slots of a token are read with all their loads in flight (dim % 4 == 0, topk <= 8,
// 16-byte aligned rows); the order of the additions is that of the scalar kernel (slot order)
__global__ void moe_combine_vec_kernel(const float* __restrict__ y2, const int* __restrict__ eid, const __nv_bfloat16* __restrict__ ys,
                                       __nv_bfloat16* __restrict__ out, float* __restrict__ routed, int tokens, int topk, int dim, int shard_start,
                                       int shard_n) {
    pdl_wait();
    const int d4 = dim >> 2;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)tokens * d4) return;
    const int t = (int)(i / d4), n = (int)(i - (long)t * d4) * 4;
    float4 v[8];
    bool on[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        on[j] = false;
        if (j < topk) {
            const int e = __ldg(eid + t * topk + j);
            on[j] = e >= shard_start && e < shard_start + shard_n;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
        v[j] = on[j] ? __ldcg(reinterpret_cast<const float4*>(y2 + ((long)t * topk + j) * dim + n)) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (on[j]) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    if (routed) *reinterpret_cast<float4*>(routed + (long)t * dim + n) = acc;
    if (out) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        if (ys) {
            const uint2 y = *reinterpret_cast<const uint2*>(ys + (long)t * dim + n);
            s0 = bf16_bits_to_f32(y.x & 0xFFFFu); s1 = bf16_bits_to_f32(y.x >> 16); s2 = bf16_bits_to_f32(y.y & 0xFFFFu); s3 = bf16_bits_to_f32(y.y >> 16);
        }
        *reinterpret_cast<uint2*>(out + (long)t * dim + n) = make_uint2(f32_to_bf16_bits(acc.x + s0) | (f32_to_bf16_bits(acc.y + s1) << 16),
                                                                        f32_to_bf16_bits(acc.z + s2) | (f32_to_bf16_bits(acc.w + s3) << 16));
    }
}

static cudaError_t launch_combine(const float* y2, const int* eid, const __nv_bfloat16* ys, __nv_bfloat16* out, float* routed, int tokens, int topk, int dim,
                                  int shard_start, int shard_n, cudaStream_t stream) {
    const long n = (long)tokens * dim;
    if (dim % 4 == 0 && topk <= 8 && !(((uintptr_t)y2 | (uintptr_t)routed) & 15) && !(((uintptr_t)ys | (uintptr_t)out) & 7))
        return launch_pdl(moe_combine_vec_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, y2, eid, ys, out, routed, tokens, topk, dim,
                          shard_start, shard_n);
    return launch_pdl(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, y2, eid, ys, out, routed, tokens, topk, dim, shard_start,
                      shard_n);
}

struct Carver {
    char* p;
    size_t left;
    bool ok = true;
    template <typename T>
    T* take(size_t n) {
        size_t bytes = (n * sizeof(T) + 255) & ~(size_t)255;
        if (bytes > left) { ok = false; return nullptr; }
        T* r = reinterpret_cast<T*>(p);
        p += bytes;
        left -= bytes;
        return r;
    }
};

static size_t rnd256(size_t b) { return (b + 255) & ~(size_t)255; }

}  // namespace b200

using namespace b200;

extern "C" int b200_version(void) { return 100; }

extern "C" int b200_sm_count(void) { return sm_count(); }

extern "C" const char* b200_error_string(int code) {
    switch (code) {
        case 0: return "ok";
        case ERR_BAD_ARG: return "b200: bad argument (null pointer or non-positive size)";
        case ERR_BAD_SHAPE: return "b200: shape violates a divisibility or range rule";
        case ERR_BAD_ALIGN: return "b200: pointer or stride misaligned";
        case ERR_WORKSPACE: return "b200: workspace too small";
        case ERR_UNSUPPORTED: return "b200: unsupported format or mode";
        case ERR_TOO_LARGE: return "b200: size beyond the fixed maximum of this entry point";
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "b200: unknown error";
}

// ------------------------------------------------------------------ grouped FP4 GEMM
extern "C" size_t b200_fp4_grouped_workspace_bytes(int n_pairs) {
    if (n_pairs < 0) n_pairs = 0;
    return rnd256((size_t)(n_pairs + 1) * sizeof(int4)) + 256;
}

extern "C" int b200_fp4_grouped_gemm(const void* x, long long x_ld, int x_perm8, const void* w, long long w_estride, const void* s,
                                     long long s_estride, int fmt, int n_local_experts, int N, int K, const int* grp_expert, const int* grp_start,
                                     const int* grp_count, int n_groups, const int* pair_tok, const int* pair_out, const float* pair_w, int n_pairs, int shard_start, int shard_n,
                                     int zero_out, int accumulate, float* out, long long out_ld, void* workspace, size_t workspace_bytes,
                                     cudaStream_t stream) {
    if (!x || !w || !s || !grp_expert || !grp_start || !out || !workspace || n_groups < 0 || n_pairs < 0 || n_local_experts < 1) return ERR_BAD_ARG;
    if (fmt != SK_FMT_FP4_E8M0 && fmt != SK_FMT_FP4_BF16S) return ERR_UNSUPPORTED;
    if (workspace_bytes < b200_fp4_grouped_workspace_bytes(n_pairs) || ((uintptr_t)workspace & 15)) return ERR_WORKSPACE;
    if (n_pairs == 0 || n_groups == 0) return 0;
    Carver cv{(char*)workspace, workspace_bytes};
    int4* work = cv.take<int4>((size_t)n_pairs + 1);
    int* n_work = cv.take<int>(1);
    if (!cv.ok) return ERR_WORKSPACE;
    SkinnyArgs a{};
    a.w = (const uint8_t*)w; a.w_estride = w_estride; a.n_experts = n_local_experts;
    a.s = (const uint8_t*)s; a.s_estride = s_estride;
    a.s_rstride = (K / 32) * (fmt == SK_FMT_FP4_BF16S ? 2 : 1);
    a.N = N; a.K = K;
    a.x = (const __nv_bfloat16*)x; a.x_ld = x_ld; a.x_perm8 = x_perm8;
    a.work = work; a.n_work = n_work;
    a.pair_tok = pair_tok; a.pair_out = pair_out; a.pair_w = pair_w;
    a.out = out; a.out_ld = out_ld;
    const int epi = accumulate ? SK_EPI_ATOMIC_F32 : SK_EPI_STORE_F32;
    int rc = skinny_check(a, fmt, epi);
    if (rc) return rc;
    if (shard_n > n_local_experts) shard_n = n_local_experts;
    rc = skinny_plan(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, work, n_work, n_pairs, stream);
    if (rc) return rc;
    if (zero_out && !accumulate) {
        rc = skinny_zero_foreign(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, pair_out, out, out_ld, N, stream);
        if (rc) return rc;
    }
    return skinny_launch(a, fmt, epi, stream);
}

// ------------------------------------------------------------------ dense FP8
extern "C" int b200_fp8_gemm(const void* x, long long x_ld, int M, const void* w8, const void* s, int fmt, int s_cols, int w_permk, int N, int K,
                             void* out, int out_is_f32, long long out_ld, cudaStream_t stream) {
    if (!x || !w8 || !s || !out || M < 0 || s_cols <= 0) return ERR_BAD_ARG;
    if (fmt != SK_FMT_FP8_E8M0 && fmt != SK_FMT_FP8_F32B) return ERR_UNSUPPORTED;
    if (fmt == SK_FMT_FP8_E8M0 ? s_cols < K / 32 : s_cols < (K + 127) / 128) return ERR_BAD_SHAPE;
    if (M == 0) return 0;
    SkinnyArgs a{};
    a.w = (const uint8_t*)w8; a.w_estride = 0;
    a.s = (const uint8_t*)s; a.s_estride = 0;
    a.s_rstride = fmt == SK_FMT_FP8_E8M0 ? s_cols : s_cols * 4;
    a.N = N; a.K = K;
    a.x = (const __nv_bfloat16*)x; a.x_ld = x_ld; a.w_permk = w_permk;
    a.work = nullptr; a.dense_rows = M; a.n_work = nullptr; a.n_work_host = (M + SK_TOK - 1) / SK_TOK;
    a.out = out; a.out_ld = out_ld;
    return skinny_launch(a, fmt, out_is_f32 ? SK_EPI_STORE_F32 : SK_EPI_STORE_BF16, stream);
}

// ------------------------------------------------------------------ whole layer
// Workspace of one layer call, carved identically by b200_moe_workspace_bytes and b200_moe_forward.
struct MoeWs {
    __nv_bfloat16* xq; int* eid; float* wt; int* pair_tok; int* pair_out; float* pair_w; int4* work; int* n_work; unsigned int* counter;
    int* cnt; int* cursor; __nv_bfloat16* hq; __nv_bfloat16* hs; float* y2; float* acc; __nv_bfloat16* ys;
    uint8_t *x8s, *xsfs, *x8t, *xsft, *hq8, *hsf, *hs8, *hssf;
    float* logit_parts;  // k-split partial logits of the fused router projection: [GATE_MAX_SPLITS or fewer][T][E]
    // decode-sized batches on the weight-stream kernels (wmgemm.cu)
    uint8_t *dq_x_atoms, *dq_h8, *dq_h_atoms, *dq_hs_atoms, *dq_slot;
    float *dq_gu, *dq_gus, *dq_partial;
    int *dq_work, *dq_pair_work, *dq_flags;
};

constexpr int DQ_MAX_TOKENS = WM_NT_MAX;   // batches up to this size take the weight-stream kernels
constexpr int DQ_FUSE_SWIGLU_TOKENS = 16;  // up to this many tokens SwiGLU runs in the gate/up GEMM's epilogue
constexpr int DQ_MAX_CTAS = 192;           // CTAs the split-k exchange buffers are sized for
static int dq_nt(int T) { return T <= 16 ? 16 : (T <= 32 ? 32 : 64); }
static size_t dq_max_works(size_t P) { return P < (size_t)ROUTE_MAX_EXPERTS ? P : (size_t)ROUTE_MAX_EXPERTS; }

static bool carve_moe(Carver& cv, MoeWs& w, int T, int topk, int D, int I) {
    const size_t P = (size_t)T * topk;
    const bool small = P <= (size_t)ROUTE_MAX_PAIRS;  // decode-sized batches keep bf16 intermediates for the streaming engine
    w.xq = cv.take<__nv_bfloat16>(small ? (size_t)T * D : 0);
    w.eid = cv.take<int>(P);
    w.wt = cv.take<float>(P);
    w.pair_tok = cv.take<int>(P);
    w.pair_out = cv.take<int>(P);
    w.pair_w = cv.take<float>(P);
    w.work = cv.take<int4>(P + 1);
    w.n_work = cv.take<int>(1);
    w.counter = cv.take<unsigned int>(1);
    w.cnt = cv.take<int>(ROUTE_MAX_EXPERTS);
    w.cursor = cv.take<int>(ROUTE_MAX_EXPERTS);
    w.hq = cv.take<__nv_bfloat16>(small ? P * I : 0);
    w.hs = cv.take<__nv_bfloat16>(small ? (size_t)T * I : 0);
    w.y2 = cv.take<float>(small ? P * D : 0);          // per-pair results (summed in slot order: deterministic)
    w.acc = cv.take<float>(small ? 0 : (size_t)T * D);  // per-token accumulator of the prefill path
    w.ys = cv.take<__nv_bfloat16>((size_t)T * D);
    // activations as e4m3 bytes + E8M0 scale bytes; 128 slack rows: tensor-map boxes of the last work may read past the end
    w.x8s = cv.take<uint8_t>((P + 128) * D);
    w.xsfs = cv.take<uint8_t>((P + 128) * (D / 32));
    w.x8t = cv.take<uint8_t>(((size_t)T + 128) * D);
    w.xsft = cv.take<uint8_t>(((size_t)T + 128) * (D / 32));
    w.hq8 = cv.take<uint8_t>((P + 128) * I);
    w.hsf = cv.take<uint8_t>((P + 128) * (I / 32));
    w.hs8 = cv.take<uint8_t>(((size_t)T + 128) * I);
    w.hssf = cv.take<uint8_t>(((size_t)T + 128) * (I / 32));
    size_t lp = 0;  // the fused router projection: room for any expert count up to the router's maximum
    for (int e = 64; e <= ROUTE_MAX_EXPERTS; e += 64) {
        const size_t need = (size_t)gate_gemm_splits(T, e, D) * T * e;
        if (need > lp) lp = need;
    }
    w.logit_parts = cv.take<float>(lp);
    const bool dq = T > 0 && T <= DQ_MAX_TOKENS && D % 128 == 0 && I % 128 == 0;
    const size_t NT = dq_nt(T), MW = dq_max_works(P);
    w.dq_x_atoms = cv.take<uint8_t>(dq ? (size_t)(D / 128) * 512 : 0);
    w.dq_h8 = cv.take<uint8_t>(dq ? (MW * NT + 128) * I : 0);          // SwiGLU outputs of work w: rows [w * NT, w * NT + NT)
    w.dq_h_atoms = cv.take<uint8_t>(dq ? MW * (I / 128) * 512 : 0);
    w.dq_hs_atoms = cv.take<uint8_t>(dq ? (size_t)(I / 128) * 512 : 0);
    w.dq_slot = cv.take<uint8_t>(dq ? MW * NT : 0);
    w.dq_gu = cv.take<float>(dq ? P * 2 * I : 0);                       // gate | up of every (token, expert) pair, row = token * topk + slot
    w.dq_gus = cv.take<float>(dq ? (size_t)T * 2 * I : 0);              // gate | up of the shared expert
    w.dq_work = cv.take<int>(dq ? MW : 0);
    w.dq_pair_work = cv.take<int>(dq ? P : 0);
    w.dq_partial = cv.take<float>(dq ? (size_t)DQ_MAX_CTAS * (WM_PARTIAL_BYTES / sizeof(float)) : 0);
    w.dq_flags = cv.take<int>(dq ? 2 * DQ_MAX_CTAS : 0);
    return cv.ok;
}

extern "C" size_t b200_moe_workspace_bytes(int tokens, int topk, int dim, int inter) {
    if (tokens < 0 || topk < 0 || dim < 0 || inter < 0) return 0;
    Carver cv{nullptr, (size_t)1 << 62};
    MoeWs w;
    carve_moe(cv, w, tokens, topk, dim, inter);
    return (size_t)(cv.p - (char*)nullptr) + 256;
}

extern "C" int b200_moe_forward(const b200_moe_args* m, cudaStream_t stream) {
    if (!m) return ERR_BAD_ARG;
    if (m->tokens < 0 || m->topk < 1 || m->n_experts < 1 || m->dim < 1 || m->inter < 1) return ERR_BAD_ARG;
    if ((m->x_ld > 0 && m->x_ld < m->dim) || (m->logits_ld > 0 && m->logits_ld < m->n_experts)) return ERR_BAD_ARG;
    if (m->tokens == 0) return 0;  // an empty batch is not an error; its (empty) buffers may be null
    if (m->eid_in && (!m->wt_in || m->tokens > DQ_MAX_TOKENS || !m->s13_atoms)) return ERR_UNSUPPORTED;  // given routing: decode-sized batches only
    if ((!m->logits && !m->gate_w && !m->eid_in) || !m->x || !m->w13 || !m->s13 || !m->w2 || !m->s2 || !m->workspace) return ERR_BAD_ARG;
    if (m->has_shared && (!m->sh_w13 || !m->sh_s13 || !m->sh_w2 || !m->sh_s2)) return ERR_BAD_ARG;
    if (m->sh_count < 0 || m->sh_first < 0 || (m->sh_count > 0 && (m->out || m->sh_first + m->sh_count > m->tokens))) return ERR_BAD_ARG;
    const int T = m->tokens, topk = m->topk, D = m->dim, I = m->inter, E = m->n_experts;
    const long P = (long)T * topk;
    if (P > (1L << 30) || E > ROUTE_MAX_EXPERTS || topk > 32 || topk > E) return ERR_BAD_SHAPE;
    if (D % 128 || I % 128) return ERR_BAD_SHAPE;
    if (m->expert_fmt != SK_FMT_FP4_E8M0 && m->expert_fmt != SK_FMT_FP4_BF16S) return ERR_UNSUPPORTED;
    if (m->has_shared && m->shared_fmt != SK_FMT_FP8_E8M0 && m->shared_fmt != SK_FMT_FP8_F32B) return ERR_UNSUPPORTED;
    if (m->score_mode < 0 || m->score_mode > 2) return ERR_UNSUPPORTED;
    if (m->workspace_bytes < b200_moe_workspace_bytes(T, topk, D, I) || ((uintptr_t)m->workspace & 255)) return ERR_WORKSPACE;
    const int shard_n = m->shard_n;  // = number of experts the shard tensors hold
    if (m->shard_start < 0 || shard_n < 1 || shard_n > E) return ERR_BAD_ARG;

    Carver cv{(char*)m->workspace, m->workspace_bytes};
    MoeWs w;
    if (!carve_moe(cv, w, T, topk, D, I)) return ERR_WORKSPACE;
    const bool small = P <= ROUTE_MAX_PAIRS;
    // engine: 1 = weight streaming with in-register dequantisation (any scale format, decode-sized batches only),
    //         2 = block-scaled tensor cores (E8M0 scales, natural k order of the shared expert), 0 = automatic:
    //         tensor cores whenever the formats allow (measured faster from one token up), else streaming
    const bool mx_ok = m->expert_fmt == SK_FMT_FP4_E8M0 && (!m->has_shared || (m->shared_fmt == SK_FMT_FP8_E8M0 && !m->sh_permk));
    if ((m->engine == 2 || !small) && !mx_ok) return ERR_UNSUPPORTED;
    if (m->engine == 1 && !small) return ERR_UNSUPPORTED;
    const bool use_mx = m->engine == 2 || !small || (m->engine == 0 && mx_ok && T > MX_AUTO_MIN_TOKENS);
    const bool shared = m->has_shared && (m->out || m->shared_out);
    __nv_bfloat16* const ys_buf = m->shared_out ? (__nv_bfloat16*)m->shared_out : w.ys;  // the shared expert's result
    cudaError_t ce;
    int rc;

    // ---- decode-sized batches: the weight-stream kernels (wmgemm.cu), 4 launches: route + quantise, gate/up, down, combine
    const bool dq_shared_ok = !m->has_shared || (m->sh_s13_atoms && m->sh_s2_atoms);
    if (T <= DQ_MAX_TOKENS && mx_ok && m->engine != 1 && m->s13_atoms && m->s2_atoms && dq_shared_ok && !m->x_is_quantized) {
        const int NT = dq_nt(T);
        DqRouteArgs r{};
        r.tokens = T; r.E = E; r.topk = topk; r.dim = D; r.NT = NT;
        r.logits_f32 = m->logits_is_bf16 ? nullptr : (const float*)m->logits;
        r.logits_bf16 = m->logits_is_bf16 ? (const __nv_bfloat16*)m->logits : nullptr;
        r.eid_in = m->eid_in; r.wt_in = m->wt_in;
        if (!m->logits && !m->eid_in) {
            const int splits = gate_gemm_splits(T, E, D);
            if ((rc = gate_gemm((const float*)m->xf, m->xf_ld > 0 ? m->xf_ld : D, m->xf ? nullptr : (const __nv_bfloat16*)m->x, m->x_ld > 0 ? m->x_ld : D,
                                (const float*)m->gate_w, T, E, D, splits, w.logit_parts, stream)))
                return rc;
            r.logits_f32 = w.logit_parts; r.logits_bf16 = nullptr;
            r.logit_parts = splits; r.logit_part_stride = (long long)T * E;
        }
        r.bias = m->gate_bias; r.temp = m->temp; r.route_scale = m->route_scale; r.mode = m->score_mode; r.norm = m->norm;
        r.x = (const __nv_bfloat16*)m->x; r.x_ld = m->x_ld > 0 ? m->x_ld : D; r.logits_ld = (m->logits && m->logits_ld > 0) ? m->logits_ld : E;
        r.shard_start = m->shard_start; r.shard_n = shard_n;
        r.eid = w.eid; r.wt = w.wt; r.x8 = w.x8t; r.x_atoms = w.dq_x_atoms; r.work = w.dq_work; r.n_work = w.n_work; r.slot = w.dq_slot; r.pair_work = w.dq_pair_work;
        r.counter = w.counter; r.flags = w.dq_flags; r.n_flags = 2 * DQ_MAX_CTAS;
        if (T > 1 && (ce = cudaMemsetAsync(w.counter, 0, sizeof(unsigned int), stream)) != cudaSuccess) return (int)ce;
        dq_route_kernel<<<T, ROUTE_THREADS, 0, stream>>>(r);
        B200_CHECK_LAUNCH();
        const long long MW = (long long)dq_max_works((size_t)P);
        // SwiGLU + quantisation: in the epilogue of the gate/up GEMM for the smallest batches (a handful of rows per tile), in a kernel of
        // its own between the GEMMs otherwise (a hot expert's tile carries dozens of rows, which would hold up the CTA that gets it)
        const bool fuse_swiglu = T <= DQ_FUSE_SWIGLU_TOKENS;
        WmArgs g1{};
        g1.n_prob = shared ? 2 : 1;
        g1.K = D; g1.NT = NT; g1.dual = 1; g1.inter = I; g1.limit = m->swiglu_limit;
        g1.split_k = 1; g1.partial = w.dq_partial; g1.flags = w.dq_flags; g1.flag_value = 1; g1.max_ctas = DQ_MAX_CTAS;
        {
            WmProb& q = g1.p[0];
            q.w = m->w13; q.w_estride = (long long)2 * I * (D / 2); q.n_experts = shard_n; q.a_fmt = MX_A_E2M1;
            q.w_atoms = (const uint8_t*)m->s13_atoms; q.atoms_estride = (long long)scale_atoms_bytes(1, 2 * I, D, 1);
            q.N = 2 * I; q.x8 = w.x8t; q.x8_rows = T + 128; q.x_atoms = w.dq_x_atoms; q.x_per_work = 0;
            q.work = w.dq_work; q.n_work = w.n_work; q.slot = w.dq_slot; q.tokens = T; q.topk = topk;
            if (fuse_swiglu) { q.epi = WM_EPI_SWIGLU_Q8; q.out = w.dq_h8; q.out_ld = I; q.out_atoms = w.dq_h_atoms; q.pair_w = w.wt; }
            else { q.epi = WM_EPI_STORE_F32; q.out = w.dq_gu; q.out_ld = 2 * I; }
        }
        if (shared) {
            WmProb& q = g1.p[1];
            q.w = m->sh_w13; q.n_experts = 1; q.a_fmt = MX_A_E4M3;
            q.w_atoms = (const uint8_t*)m->sh_s13_atoms; q.N = 2 * I; q.x8 = w.x8t; q.x8_rows = T + 128; q.x_atoms = w.dq_x_atoms; q.x_per_work = 0;
            q.work = nullptr; q.n_work_host = 1; q.tokens = T; q.topk = topk;
            if (fuse_swiglu) { q.epi = WM_EPI_SWIGLU_Q8; q.out = w.hs8; q.out_ld = I; q.out_atoms = w.dq_hs_atoms; q.round_gu_bf16 = 1; }
            else { q.epi = WM_EPI_STORE_F32; q.out = w.dq_gus; q.out_ld = 2 * I; }
        }
        if (m->prof_start && (ce = cudaEventRecord((cudaEvent_t)m->prof_start, stream)) != cudaSuccess) return (int)ce;
        if ((rc = wm_launch(g1, stream))) return rc;
        if (m->prof_stop && (ce = cudaEventRecord((cudaEvent_t)m->prof_stop, stream)) != cudaSuccess) return (int)ce;
        DqSwigluArgs sq{};
        sq.gu = w.dq_gu; sq.gus = shared ? w.dq_gus : nullptr; sq.pairs = (int)P; sq.tokens = T; sq.topk = topk; sq.inter = I; sq.NT = NT;
        sq.wt = w.wt; sq.pair_work = w.dq_pair_work; sq.limit = m->swiglu_limit;
        sq.h8 = w.dq_h8; sq.h_atoms = w.dq_h_atoms; sq.hs8 = w.hs8; sq.hs_atoms = w.dq_hs_atoms;
        if (!fuse_swiglu && (ce = launch_pdl(dq_swiglu_kernel, dim3((unsigned)(P + (shared ? T : 0))), dim3(256), 0, stream, sq)) != cudaSuccess) return (int)ce;
        WmArgs g2{};
        g2.n_prob = shared ? 2 : 1;
        g2.K = I; g2.NT = NT; g2.dual = 0;
        g2.split_k = 1; g2.partial = w.dq_partial; g2.flags = w.dq_flags + DQ_MAX_CTAS; g2.flag_value = 1; g2.max_ctas = DQ_MAX_CTAS;
        {
            WmProb& q = g2.p[0];
            q.w = m->w2; q.w_estride = (long long)D * (I / 2); q.n_experts = shard_n; q.a_fmt = MX_A_E2M1;
            q.w_atoms = (const uint8_t*)m->s2_atoms; q.atoms_estride = (long long)scale_atoms_bytes(1, D, I, 0);
            q.N = D; q.x8 = w.dq_h8; q.x8_rows = MW * NT + 128; q.x_atoms = w.dq_h_atoms; q.x_per_work = 1;
            q.work = w.dq_work; q.n_work = w.n_work; q.slot = w.dq_slot; q.tokens = T; q.topk = topk;
            q.epi = WM_EPI_STORE_F32; q.out = w.y2; q.out_ld = D;
        }
        if (shared) {
            WmProb& q = g2.p[1];
            q.w = m->sh_w2; q.n_experts = 1; q.a_fmt = MX_A_E4M3;
            q.w_atoms = (const uint8_t*)m->sh_s2_atoms; q.N = D; q.x8 = w.hs8; q.x8_rows = T + 128; q.x_atoms = w.dq_hs_atoms; q.x_per_work = 0;
            q.work = nullptr; q.n_work_host = 1; q.tokens = T; q.topk = topk;
            q.epi = WM_EPI_STORE_BF16; q.out = ys_buf; q.out_ld = D;
        }
        if ((rc = wm_launch(g2, stream))) return rc;
        if ((ce = launch_combine((const float*)w.y2, (const int*)w.eid, (const __nv_bfloat16*)(shared ? ys_buf : nullptr), (__nv_bfloat16*)m->out, m->routed_out,
                                 T, topk, D, m->shard_start, shard_n, stream)) != cudaSuccess)
            return (int)ce;
        if (m->eid_out && (ce = cudaMemcpyAsync(m->eid_out, w.eid, P * sizeof(int), cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) return (int)ce;
        if (m->wt_out && (ce = cudaMemcpyAsync(m->wt_out, w.wt, P * sizeof(float), cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) return (int)ce;
        return 0;
    }

    // ---- routing (+ bf16 fake quantisation of the input for the streaming engine)
    RouteArgs r{};
    r.tokens = T; r.E = E; r.topk = topk; r.dim = D;
    r.logits_f32 = m->logits_is_bf16 ? nullptr : (const float*)m->logits;
    r.logits_bf16 = m->logits_is_bf16 ? (const __nv_bfloat16*)m->logits : nullptr;
    if (!m->logits) {
        // the path starts from the hidden state: router projection x @ gate_w^T in fp32 (dsv41/model.py:1615), left as k-split
        // partial sums that the router adds in order
        const int splits = gate_gemm_splits(T, E, D);
        if ((rc = gate_gemm((const float*)m->xf, m->xf_ld > 0 ? m->xf_ld : D, m->xf ? nullptr : (const __nv_bfloat16*)m->x, m->x_ld > 0 ? m->x_ld : D,
                            (const float*)m->gate_w, T, E, D, splits, w.logit_parts, stream)))
            return rc;
        r.logits_f32 = w.logit_parts; r.logits_bf16 = nullptr;
        r.logit_parts = splits; r.logit_part_stride = (long long)T * E;
    }
    r.bias = m->gate_bias; r.temp = m->temp; r.route_scale = m->route_scale; r.mode = m->score_mode; r.norm = m->norm;
    r.x = (const __nv_bfloat16*)m->x; r.xq = (m->x_is_quantized || use_mx) ? nullptr : w.xq;
    const long long x_ld = m->x_ld > 0 ? m->x_ld : D;  // rows of x / logits may sit inside wider rows (a packed exchange buffer)
    r.x_ld = x_ld; r.logits_ld = (m->logits && m->logits_ld > 0) ? m->logits_ld : E;
    r.shard_start = m->shard_start; r.shard_n = shard_n;
    const int nd = small ? MX_ND_DECODE : 128;  // tokens per work of the tensor-core path
    r.tpw = use_mx ? nd : SK_TOK;
    r.eid = w.eid; r.wt = w.wt; r.pair_tok = w.pair_tok; r.pair_out = w.pair_out; r.pair_w = w.pair_w; r.work = w.work; r.n_work = w.n_work;
    r.counter = w.counter; r.no_bucket = small ? 0 : 1;
    if (small) {  // the counter of the "last block" election starts at zero and resets itself after every launch
        if ((ce = cudaMemsetAsync(w.counter, 0, sizeof(unsigned int), stream)) != cudaSuccess) return (int)ce;
    }
    if (r.no_bucket && !r.xq && (size_t)ROUTE_ROWS_PER_BLOCK * 3 * E * sizeof(float) <= 48 * 1024) {
        route_rows_kernel<<<(T + ROUTE_ROWS_PER_BLOCK - 1) / ROUTE_ROWS_PER_BLOCK, 32 * ROUTE_ROWS_PER_BLOCK, (size_t)ROUTE_ROWS_PER_BLOCK * 3 * E * sizeof(float), stream>>>(r);
    } else {
        moe_route_kernel<<<T, ROUTE_THREADS, 0, stream>>>(r);
    }
    B200_CHECK_LAUNCH();
    if (!small) {  // many pairs: multi-block histogram / scan / scatter; GEMM-2 adds into a per-token accumulator
        if ((ce = cudaMemsetAsync(w.cnt, 0, sizeof(int) * ROUTE_MAX_EXPERTS, stream)) != cudaSuccess) return (int)ce;
        if ((ce = cudaMemsetAsync(w.acc, 0, sizeof(float) * (size_t)T * D, stream)) != cudaSuccess) return (int)ce;
        pair_hist_kernel<<<(unsigned)((P + 255) / 256), 256, 0, stream>>>(w.eid, (int)P, w.cnt);
        B200_CHECK_LAUNCH();
        pair_scan_kernel<<<1, 1024, 0, stream>>>(w.cnt, E, m->shard_start, shard_n, nd, w.cursor, w.work, w.n_work);
        B200_CHECK_LAUNCH();
        pair_scatter_kernel<<<(unsigned)((P + 255) / 256), 256, 0, stream>>>(w.eid, w.wt, (int)P, topk, w.cursor, w.pair_tok, w.pair_out, w.pair_w, 1);
        B200_CHECK_LAUNCH();
    }

    if (use_mx) {
        // activations -> e4m3 + E8M0 (the FP8 fake quantisation kept in quantised form), gathered into pair-sorted order
        // (and, for the shared expert, in token order: one launch for both)
        if ((rc = mx_quantize_rows((const __nv_bfloat16*)m->x, x_ld, w.pair_tok, (int)P, D, w.x8s, w.xsfs, stream, shared ? T : 0, w.x8t, w.xsft))) return rc;
        // always the widest tiles (256 weight rows per MMA): even when that leaves fewer (work, tile) items than SMs, as for a single
        // token (6 works x 16 tiles), the wide tiles stream faster than more, narrower ones (measured 83 us against 136 us per step)
        const int rows1 = 128, rows2 = 256;
        // the shared expert's rows: all tokens, or the sub-range the caller keeps
        const int sh_first = m->sh_count > 0 ? m->sh_first : 0, sh_rows = m->sh_count > 0 ? m->sh_count : T;
        // each GEMM launch carries the routed experts (problem 0) and, behind them in the same item list, the shared expert
        // (problem 1: one FP8 matrix against all tokens)
        MxArgs g1{};
        g1.n_prob = shared ? 2 : 1;
        g1.K = D; g1.nd = nd; g1.rows_a = rows1; g1.dual = 1; g1.kb = 4; g1.limit = m->swiglu_limit; g1.inter = I;
        {
            MxProb& q = g1.p[0];
            q.w = m->w13; q.w_estride = (long long)2 * I * (D / 2); q.n_experts = shard_n; q.a_fmt = MX_A_E2M1;
            q.s = (const uint8_t*)m->s13; q.s_estride = (long long)2 * I * (D / 32); q.s_rstride = D / 32; q.s_row_shift = 0;
            q.N = 2 * I; q.x8 = w.x8s; q.x8_rows = P + 128; q.xsf = w.xsfs; q.xsf_ld = D / 32;
            q.work = w.work; q.n_work = w.n_work; q.epi = MX_EPI_SWIGLU_Q8;
            q.pair_w = w.pair_w; q.out = w.hq8; q.out_ld = I; q.out_sf = w.hsf; q.out_sf_ld = I / 32;
        }
        if (shared) {
            MxProb& q = g1.p[1];
            q.w = m->sh_w13; q.n_experts = 1; q.a_fmt = MX_A_E4M3;
            q.s = (const uint8_t*)m->sh_s13; q.s_rstride = m->sh_s13_cols; q.s_row_shift = 5;
            q.N = 2 * I; q.x8 = w.x8t + (size_t)sh_first * D; q.x8_rows = T + 128 - sh_first; q.xsf = w.xsft + (size_t)sh_first * (D / 32); q.xsf_ld = D / 32;
            q.work = nullptr; q.dense_rows = sh_rows; q.n_work_host = (sh_rows + nd - 1) / nd; q.epi = MX_EPI_SWIGLU_Q8;
            q.out = w.hs8; q.out_ld = I; q.out_sf = w.hssf; q.out_sf_ld = I / 32; q.round_gu_bf16 = 1;  // rows 0 .. sh_rows-1 of hs8
        }
        if (m->prof_start && (ce = cudaEventRecord((cudaEvent_t)m->prof_start, stream)) != cudaSuccess) return (int)ce;
        if ((rc = mx_launch(g1, stream))) return rc;
        if (m->prof_stop && (ce = cudaEventRecord((cudaEvent_t)m->prof_stop, stream)) != cudaSuccess) return (int)ce;
        MxArgs g2{};
        g2.n_prob = shared ? 2 : 1;
        g2.K = I; g2.nd = nd; g2.rows_a = rows2; g2.dual = 0; g2.kb = 4;
        {
            MxProb& q = g2.p[0];
            q.w = m->w2; q.w_estride = (long long)D * (I / 2); q.n_experts = shard_n; q.a_fmt = MX_A_E2M1;
            q.s = (const uint8_t*)m->s2; q.s_estride = (long long)D * (I / 32); q.s_rstride = I / 32; q.s_row_shift = 0;
            q.N = D; q.x8 = w.hq8; q.x8_rows = P + 128; q.xsf = w.hsf; q.xsf_ld = I / 32;
            q.work = w.work; q.n_work = w.n_work;
            q.epi = small ? MX_EPI_STORE_F32 : MX_EPI_ATOMIC_F32;
            q.pair_out = w.pair_out; q.out = small ? w.y2 : w.acc; q.out_ld = D;
        }
        if (shared) {
            MxProb& q = g2.p[1];
            q.w = m->sh_w2; q.n_experts = 1; q.a_fmt = MX_A_E4M3;
            q.s = (const uint8_t*)m->sh_s2; q.s_rstride = m->sh_s2_cols; q.s_row_shift = 5;
            q.N = D; q.x8 = w.hs8; q.x8_rows = T + 128; q.xsf = w.hssf; q.xsf_ld = I / 32;
            q.work = nullptr; q.dense_rows = sh_rows; q.n_work_host = (sh_rows + nd - 1) / nd; q.epi = MX_EPI_STORE_BF16;
            q.out = ys_buf + (size_t)sh_first * D; q.out_ld = D;
        }
        if ((rc = mx_launch(g2, stream))) return rc;
    } else {
        const __nv_bfloat16* xin = m->x_is_quantized ? (const __nv_bfloat16*)m->x : w.xq;
        const int sbytes = m->expert_fmt == SK_FMT_FP4_BF16S ? 2 : 1;
        // routed gate/up + SwiGLU * weight + fake quant -> hq [sorted pair, inter]
        SkinnyArgs a{};
        a.w = (const uint8_t*)m->w13; a.w_estride = (long long)2 * I * (D / 2); a.n_experts = shard_n;
        a.s = (const uint8_t*)m->s13; a.s_estride = (long long)2 * I * (D / 32) * sbytes; a.s_rstride = (D / 32) * sbytes;
        const long long xin_ld = m->x_is_quantized ? x_ld : D;
        a.N = 2 * I; a.K = D; a.x = xin; a.x_ld = xin_ld;
        a.work = w.work; a.n_work = w.n_work; a.pair_tok = w.pair_tok; a.pair_out = nullptr; a.pair_w = w.pair_w;
        a.out = w.hq; a.out_ld = I; a.limit = m->swiglu_limit; a.inter = I;
        if (m->prof_start && (ce = cudaEventRecord((cudaEvent_t)m->prof_start, stream)) != cudaSuccess) return (int)ce;
        if ((rc = skinny_launch(a, m->expert_fmt, SK_EPI_SWIGLU, stream))) return rc;
        if (m->prof_stop && (ce = cudaEventRecord((cudaEvent_t)m->prof_stop, stream)) != cudaSuccess) return (int)ce;
        // routed down -> y2 [original pair, dim] fp32
        SkinnyArgs b{};
        b.w = (const uint8_t*)m->w2; b.w_estride = (long long)D * (I / 2); b.n_experts = shard_n;
        b.s = (const uint8_t*)m->s2; b.s_estride = (long long)D * (I / 32) * sbytes; b.s_rstride = (I / 32) * sbytes;
        b.N = D; b.K = I; b.x = w.hq; b.x_ld = I;
        b.work = w.work; b.n_work = w.n_work; b.pair_tok = nullptr; b.pair_out = w.pair_out; b.pair_w = nullptr;
        b.out = w.y2; b.out_ld = D;
        if ((rc = skinny_launch(b, m->expert_fmt, SK_EPI_STORE_F32, stream))) return rc;
        if (shared) {
            // shared expert: gu rounded to bf16, SwiGLU without weight, fake quant, down projection rounded to bf16 (dsv41/decode.py:461-463)
            SkinnyArgs c{};
            c.w = (const uint8_t*)m->sh_w13; c.s = (const uint8_t*)m->sh_s13;
            c.s_rstride = m->shared_fmt == SK_FMT_FP8_E8M0 ? m->sh_s13_cols : m->sh_s13_cols * 4;
            c.N = 2 * I; c.K = D; c.x = xin; c.x_ld = xin_ld; c.w_permk = m->sh_permk;
            c.work = nullptr; c.dense_rows = T; c.n_work_host = (T + SK_TOK - 1) / SK_TOK;
            c.out = w.hs; c.out_ld = I; c.limit = m->swiglu_limit; c.inter = I; c.round_gu_bf16 = 1;
            if ((rc = skinny_launch(c, m->shared_fmt, SK_EPI_SWIGLU, stream))) return rc;
            SkinnyArgs d{};
            d.w = (const uint8_t*)m->sh_w2; d.s = (const uint8_t*)m->sh_s2;
            d.s_rstride = m->shared_fmt == SK_FMT_FP8_E8M0 ? m->sh_s2_cols : m->sh_s2_cols * 4;
            d.N = D; d.K = I; d.x = w.hs; d.x_ld = I; d.w_permk = m->sh_permk;
            d.work = nullptr; d.dense_rows = T; d.n_work_host = (T + SK_TOK - 1) / SK_TOK;
            d.out = ys_buf; d.out_ld = D;
            if ((rc = skinny_launch(d, m->shared_fmt, SK_EPI_STORE_BF16, stream))) return rc;
        }
    }
    // ---- combine: routed sum (+ shared expert) -> bf16
    const long n = (long)T * D;
    if (small) {
        if ((ce = launch_combine((const float*)w.y2, (const int*)w.eid, (const __nv_bfloat16*)(shared ? ys_buf : nullptr), (__nv_bfloat16*)m->out, m->routed_out,
                                 T, topk, D, m->shard_start, shard_n, stream)) != cudaSuccess)
            return (int)ce;
    } else {
        if (m->out) {
            const __nv_bfloat16* ysp = shared ? ys_buf : nullptr;
            if (n % 8 == 0 && !(((uintptr_t)w.acc | (uintptr_t)ysp | (uintptr_t)m->out) & 15)) {
                if ((ce = launch_pdl(moe_finalize_vec_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (const float4*)w.acc, (const uint4*)ysp,
                                     (uint4*)m->out, n / 8)) != cudaSuccess)
                    return (int)ce;
            } else if ((ce = launch_pdl(moe_finalize_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float*)w.acc, ysp,
                                        (__nv_bfloat16*)m->out, n)) != cudaSuccess)
                return (int)ce;
        }
        if (m->routed_out && (ce = cudaMemcpyAsync(m->routed_out, w.acc, sizeof(float) * n, cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) return (int)ce;
    }
    if (m->eid_out && (ce = cudaMemcpyAsync(m->eid_out, w.eid, P * sizeof(int), cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) return (int)ce;
    if (m->wt_out && (ce = cudaMemcpyAsync(m->wt_out, w.wt, P * sizeof(float), cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) return (int)ce;
    return 0;
}

// ------------------------------------------------------------------ the reference-named GEMMs on the block-scaled tensor cores when that is exact
// The reference's launchers take a bf16 activation.  Inside the MoE layer that tensor is always an FP8 fake-quantised one, i.e. exactly
// e4m3 values times a power of two per group of 32, which is what the block-scaled tensor cores multiply; elsewhere it need not be.
// The *_auto entry points find out ON THE DEVICE: they quantise the activation, compare it with the original, and launch the tensor-core
// kernel and the weight-streaming kernel both tied to the outcome, so exactly one of them does the work.  No host synchronisation; the
// result is the reference's in either case.
extern "C" size_t b200_fp8_gemm_auto_workspace_bytes(int M, int K) {
    if (M < 0 || K < 0) return 0;
    return rnd256((size_t)(M + 128) * K) + rnd256((size_t)(M + 128) * (K / 32)) + 512;
}

extern "C" int b200_fp8_gemm_auto(const void* x, long long x_ld, int M, const void* w8_natural, const void* w8_permk, const void* s, int s_cols, int N, int K,
                                  void* out, int out_is_f32, long long out_ld, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!x || (!w8_natural && !w8_permk) || !s || !out || M < 0) return ERR_BAD_ARG;
    if (M == 0) return 0;
    const bool mx_ok = w8_natural && K % 128 == 0 && M > SK_TOK && workspace && !((uintptr_t)workspace & 255) &&
                       workspace_bytes >= b200_fp8_gemm_auto_workspace_bytes(M, K) && !((uintptr_t)x & 15) && x_ld % 8 == 0;
    const void* wstream = w8_permk ? w8_permk : w8_natural;
    if (!mx_ok) return b200_fp8_gemm(x, x_ld, M, wstream, s, SK_FMT_FP8_E8M0, s_cols, w8_permk ? 1 : 0, N, K, out, out_is_f32, out_ld, stream);
    Carver cv{(char*)workspace, workspace_bytes};
    uint8_t* q8 = cv.take<uint8_t>((size_t)(M + 128) * K);
    uint8_t* sf = cv.take<uint8_t>((size_t)(M + 128) * (K / 32));
    int* exact = cv.take<int>(1);
    if (!cv.ok) return ERR_WORKSPACE;
    int rc = mx_quantize_rows_check((const __nv_bfloat16*)x, x_ld, nullptr, M, K, q8, sf, exact, stream);
    if (rc) return rc;
    MxArgs a{};
    MxProb& q = a.p[0];
    a.n_prob = 1;
    q.w = w8_natural; q.n_experts = 1; q.a_fmt = MX_A_E4M3;
    q.s = (const uint8_t*)s; q.s_rstride = s_cols; q.s_row_shift = 5;
    q.N = N; a.K = K; q.x8 = q8; q.x8_rows = M + 128; q.xsf = sf; q.xsf_ld = K / 32;
    a.nd = M > 64 ? 128 : 64; a.rows_a = 256; a.kb = 4;
    q.epi = out_is_f32 ? MX_EPI_STORE_F32 : MX_EPI_STORE_BF16; q.out = out; q.out_ld = out_ld;
    q.work = nullptr; q.dense_rows = M; q.n_work_host = (M + a.nd - 1) / a.nd;
    a.run_if = exact; a.run_if_nonzero = 1;
    if ((rc = mx_launch(a, stream))) return rc;
    SkinnyArgs k{};
    k.w = (const uint8_t*)wstream; k.s = (const uint8_t*)s; k.s_rstride = s_cols;
    k.N = N; k.K = K; k.x = (const __nv_bfloat16*)x; k.x_ld = x_ld; k.w_permk = w8_permk ? 1 : 0;
    k.work = nullptr; k.dense_rows = M; k.n_work_host = (M + SK_TOK - 1) / SK_TOK;
    k.out = out; k.out_ld = out_ld;
    k.run_if = exact; k.run_if_nonzero = 0;
    return skinny_launch(k, SK_FMT_FP8_E8M0, out_is_f32 ? SK_EPI_STORE_F32 : SK_EPI_STORE_BF16, stream);
}

extern "C" size_t b200_fp4_grouped_auto_workspace_bytes(int n_pairs, int K) {
    if (n_pairs < 0 || K < 0) return 0;
    return 2 * rnd256((size_t)(n_pairs + 1) * sizeof(int4)) + rnd256((size_t)(n_pairs + 128) * K) + rnd256((size_t)(n_pairs + 128) * (K / 32)) + 1024;
}

extern "C" int b200_fp4_grouped_gemm_auto(const void* x, long long x_ld, int x_perm8, const void* w, long long w_estride, const void* s, long long s_estride, int n_local_experts,
                                          int N, int K, const int* grp_expert, const int* grp_start, const int* grp_count, int n_groups, const int* pair_tok,
                                          const int* pair_out, const float* pair_w, int n_pairs, int shard_start, int shard_n, int zero_out, int accumulate,
                                          float* out, long long out_ld, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!x || !w || !s || !grp_expert || !grp_start || !out || !workspace || n_groups < 0 || n_pairs < 0 || n_local_experts < 1) return ERR_BAD_ARG;
    if (workspace_bytes < b200_fp4_grouped_auto_workspace_bytes(n_pairs, K) || ((uintptr_t)workspace & 255)) return ERR_WORKSPACE;
    if (K % 128 || ((uintptr_t)x & 15) || x_ld % 8 || ((uintptr_t)w & 31) || (w_estride & 31)) return ERR_BAD_ALIGN;
    if (n_pairs == 0 || n_groups == 0) return 0;
    Carver cv{(char*)workspace, workspace_bytes};
    int4* work_mx = cv.take<int4>((size_t)n_pairs + 1);
    int4* work_sk = cv.take<int4>((size_t)n_pairs + 1);
    uint8_t* q8 = cv.take<uint8_t>((size_t)(n_pairs + 128) * K);
    uint8_t* sf = cv.take<uint8_t>((size_t)(n_pairs + 128) * (K / 32));
    int* n_work_mx = cv.take<int>(1);
    int* n_work_sk = cv.take<int>(1);
    int* exact = cv.take<int>(1);
    if (!cv.ok) return ERR_WORKSPACE;
    if (shard_n > n_local_experts) shard_n = n_local_experts;
    int rc;
    if (zero_out && !accumulate &&
        (rc = skinny_zero_foreign(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, pair_out, out, out_ld, N, stream)))
        return rc;
    // activation rows gathered into pair order, quantised, checked
    if ((rc = mx_quantize_rows_check((const __nv_bfloat16*)x, x_ld, pair_tok, n_pairs, K, q8, sf, exact, stream, x_perm8))) return rc;
    // ---- tensor-core kernel, if the activation was FP8-exact
    const int nd = 64;
    if ((rc = skinny_plan(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, work_mx, n_work_mx, n_pairs, stream, nd))) return rc;
    MxArgs a{};
    MxProb& q = a.p[0];
    a.n_prob = 1;
    q.w = w; q.w_estride = w_estride; q.n_experts = n_local_experts; q.a_fmt = MX_A_E2M1;
    q.s = (const uint8_t*)s; q.s_estride = s_estride; q.s_rstride = K / 32; q.s_row_shift = 0;
    q.N = N; a.K = K; q.x8 = q8; q.x8_rows = n_pairs + 128; q.xsf = sf; q.xsf_ld = K / 32;
    a.nd = nd; a.rows_a = 256; a.kb = 4;
    q.epi = accumulate ? MX_EPI_ATOMIC_F32 : MX_EPI_STORE_F32;
    q.pair_out = pair_out; q.pair_w = pair_w; q.out = out; q.out_ld = out_ld;
    q.work = work_mx; q.n_work = n_work_mx;
    a.run_if = exact; a.run_if_nonzero = 1;
    if ((rc = mx_launch(a, stream))) return rc;
    // ---- weight-streaming kernel otherwise
    SkinnyArgs k{};
    k.w = (const uint8_t*)w; k.w_estride = w_estride; k.n_experts = n_local_experts;
    k.s = (const uint8_t*)s; k.s_estride = s_estride; k.s_rstride = K / 32;
    k.N = N; k.K = K; k.x = (const __nv_bfloat16*)x; k.x_ld = x_ld; k.x_perm8 = x_perm8;
    k.work = work_sk; k.n_work = n_work_sk; k.pair_tok = pair_tok; k.pair_out = pair_out; k.pair_w = pair_w;
    k.out = out; k.out_ld = out_ld;
    k.run_if = exact; k.run_if_nonzero = 0;
    const int epi = accumulate ? SK_EPI_ATOMIC_F32 : SK_EPI_STORE_F32;
    if ((rc = skinny_check(k, SK_FMT_FP4_E8M0, epi))) return rc;
    if ((rc = skinny_plan(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, work_sk, n_work_sk, n_pairs, stream))) return rc;
    return skinny_launch(k, SK_FMT_FP4_E8M0, epi, stream);
}

// ------------------------------------------------------------------ load-time re-layout of the scales
extern "C" size_t b200_scale_atoms_bytes(int n_experts, int N, int K, int dual) { return scale_atoms_bytes(n_experts, N, K, dual); }

extern "C" int b200_scale_atoms(const void* s, int fmt, int s_cols, int n_experts, int N, int K, int dual, void* dst, cudaStream_t stream) {
    if (fmt != SK_FMT_FP4_E8M0 && fmt != SK_FMT_FP8_E8M0) return ERR_UNSUPPORTED;
    return scale_atoms((const uint8_t*)s, fmt == SK_FMT_FP8_E8M0 ? 5 : 0, s_cols, n_experts, N, K, dual, (uint8_t*)dst, stream);
}

// ------------------------------------------------------------------ block-scaled tensor-core GEMM, stand-alone entry points
extern "C" int b200_mx_quantize_rows(const void* x, long long x_ld, const int* src_row, int rows, int K, void* q8, void* sf, cudaStream_t stream) {
    return mx_quantize_rows((const __nv_bfloat16*)x, x_ld, src_row, rows, K, (uint8_t*)q8, (uint8_t*)sf, stream);
}

extern "C" int b200_device_error(int* code, cudaStream_t stream) {
    if (!code) return ERR_BAD_ARG;
    int mx = 0, sk = 0;
    int rc = mx_device_error(&mx, stream);  // synchronises the stream
    if (rc) return rc;
    if ((rc = skinny_device_error(&sk))) return rc;
    int wm = 0, pp = 0;
    if ((rc = wm_device_error(&wm))) return rc;
    if ((rc = p2p_device_error(&pp))) return rc;
    // prefill tensor-core kernel 11..41, streaming kernels 1001..1091, decode weight-stream kernel 2011..2042, messaging waits 3001..3004
    *code = mx ? mx : (sk ? 1000 + sk : (wm ? 2000 + wm : (pp ? 3000 + pp : 0)));
    return 0;
}

extern "C" size_t b200_mx_grouped_workspace_bytes(int n_rows) {
    if (n_rows < 0) n_rows = 0;
    return rnd256((size_t)(n_rows + 1) * sizeof(int4)) + 256;
}

extern "C" int b200_mx_grouped_gemm(const void* w, long long w_estride, const void* s, long long s_estride, int s_cols, int fmt, int n_local_experts, int N,
                                    int K, const void* x8, long long x8_rows, const void* xsf, const int* grp_expert, const int* grp_start,
                                    const int* grp_count, int n_groups, const int* pair_out, const float* pair_w, int n_rows, int shard_start,
                                    int shard_n, int epilogue, float limit, int round_gu_bf16, void* out, long long out_ld, void* out_sf,
                                    int tokens_per_work, int rows_per_tile, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!w || !s || !x8 || !xsf || !out || n_rows < 0 || n_local_experts < 1) return ERR_BAD_ARG;
    if (fmt != SK_FMT_FP4_E8M0 && fmt != SK_FMT_FP8_E8M0) return ERR_UNSUPPORTED;
    if (n_rows == 0) return 0;
    MxArgs a{};
    MxProb& q = a.p[0];
    a.n_prob = 1;
    q.w = w; q.w_estride = w_estride; q.n_experts = n_local_experts; q.a_fmt = fmt == SK_FMT_FP4_E8M0 ? MX_A_E2M1 : MX_A_E4M3;
    q.s = (const uint8_t*)s; q.s_estride = s_estride;
    q.s_rstride = fmt == SK_FMT_FP4_E8M0 ? K / 32 : s_cols; q.s_row_shift = fmt == SK_FMT_FP4_E8M0 ? 0 : 5;
    q.N = N; a.K = K; q.x8 = (const uint8_t*)x8; q.x8_rows = x8_rows; q.xsf = (const uint8_t*)xsf; q.xsf_ld = K / 32;
    a.nd = tokens_per_work; a.rows_a = rows_per_tile; a.kb = 4;
    q.epi = epilogue; a.dual = epilogue == MX_EPI_SWIGLU_Q8; a.inter = a.dual ? N / 2 : 0; a.limit = limit; q.round_gu_bf16 = round_gu_bf16;
    q.pair_out = pair_out; q.pair_w = pair_w; q.out = out; q.out_ld = out_ld; q.out_sf = (uint8_t*)out_sf; q.out_sf_ld = a.dual ? N / 2 / 32 : 0;
    if (grp_expert && n_groups > 0) {
        if (!grp_start || !workspace || workspace_bytes < b200_mx_grouped_workspace_bytes(n_rows) || ((uintptr_t)workspace & 15)) return ERR_WORKSPACE;
        Carver cv{(char*)workspace, workspace_bytes};
        int4* work = cv.take<int4>((size_t)n_rows + 1);
        int* n_work = cv.take<int>(1);
        if (!cv.ok) return ERR_WORKSPACE;
        if (shard_n > n_local_experts) shard_n = n_local_experts;
        int rc = skinny_plan(grp_expert, grp_start, grp_count, n_groups, n_rows, shard_start, shard_n, work, n_work, n_rows, stream, tokens_per_work);
        if (rc) return rc;
        q.work = work; q.n_work = n_work;
    } else {
        q.work = nullptr; q.dense_rows = n_rows; q.n_work_host = (n_rows + tokens_per_work - 1) / tokens_per_work;
    }
    return mx_launch(a, stream);
}
