/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the packed-FP4 MoE expert chain and the block-scaled FP8
 * dense GEMV/GEMM around it.  Only tests, the smoke check and the CPU-baseline leg of the benchmark may
 * load this library; the product path never does.
 *
 * It is a plain-C restatement (own code, scalar loops, double accumulation) of the arithmetic defined by
 * the reference runtime.  Each function names the reference lines it follows (paths are relative to the
 * reference project root):
 *   number formats ........ dsv41/quant.py:24-110
 *   router ................ dsv41/model.py:1614-1630, tie rule dsv41/fused2.py:470-477
 *   SwiGLU + fake quant ... dsv41/fused.py:285-306, dsv41/cpu/moe_cpu.cpp:336-377
 *   routed expert chain ... dsv41/cpu/moe_cpu.cpp:386-503 (mode 0, the exact BF16 path)
 *   shared expert ......... dsv41/decode.py:461-463, dsv41/w8.py:64-83
 *   final combine ......... dsv41/fused2.py:518-523, dsv41/model.py:2232-2233
 *
 * Pinned against (a) the reference's own C++ library compiled from its sources (oracle/_ref, mode 0) and
 * (b) golden vectors produced by importing the reference's dsv41/quant.py (tests/golden/make_golden.py).
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC -o oracle/_build/libmoe_oracle.so oracle/moe_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ scalar formats */
static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round to nearest even, as torch .to(bfloat16) and moe_cpu.cpp:336-340 */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN stays NaN */
    uint32_t r = u + 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(r >> 16);
}

/* E2M1 code -> value, quant.py:24 */
static const float E2M1_VALUE[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

/* E8M0 byte -> 2^(b-127), quant.py:27-31.  Byte 0 is treated as 0 like the kernels do
 * (moe_cpu.cpp:190, moe_kernels.py:22). */
static inline double e8m0_value(uint8_t b) { return b == 0 ? 0.0 : ldexp(1.0, (int)b - 127); }

/* float8_e4m3fn bit pattern -> value (NaN codes S.1111.111 decode to NaN) */
static inline float e4m3_value(uint8_t b) {
    int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.f + (float)m / 8.f, e - 7);
    return s ? -v : v;
}

/* nearest e4m3 value of v, |v| <= 448, ties to even; fused.py:25-34, moe_cpu.cpp:341-350 */
static inline float round_e4m3(float v) {
    float a = fabsf(v);
    if (a == 0.f) return v;
    int e;
    frexpf(a, &e);
    e -= 1; /* floor(log2 a) */
    if (e < -6) e = -6;
    float ulp = ldexpf(1.f, e - 3);
    float r = rintf(a / ulp) * ulp;
    if (r > 448.f) r = 448.f;
    return v < 0 ? -r : r;
}

/* 2^ceil(log2 a), a > 0; quant.py:34-42, moe_cpu.cpp:351-355 */
static inline float pow2_ceil(float a) {
    int e;
    float m = frexpf(a, &e);
    if (m == 0.5f) e -= 1;
    return ldexpf(1.f, e);
}

/* ------------------------------------------------------------------ activation fake quantisation */
/* quant.py:46-54 -- per group of `block` along the last dim: amax clamp 1e-4, power-of-two scale,
 * e4m3 round, dequantise, cast back to bf16.  n must be a multiple of block. */
ORC_API void orc_fake_quant_fp8(const uint16_t* x, uint16_t* y, long n, int block) {
#pragma omp parallel for schedule(static)
    for (long g = 0; g < n / block; ++g) {
        const uint16_t* xg = x + g * block;
        float amax = 0.f;
        for (int j = 0; j < block; ++j) {
            float a = fabsf(bf16_to_f32(xg[j]));
            if (a > amax) amax = a;
        }
        if (!(amax >= 1e-4f)) amax = 1e-4f;
        float s = pow2_ceil(amax / 448.f);
        for (int j = 0; j < block; ++j) {
            float q = bf16_to_f32(xg[j]) / s;
            q = fminf(fmaxf(q, -448.f), 448.f);
            y[g * block + j] = f32_to_bf16(round_e4m3(q) * s);
        }
    }
}

/* ------------------------------------------------------------------ router */
/* model.py:1614-1630.  scores: fp32 [B,E] gate logits; mode 0 = sqrt(softplus), 1 = sigmoid, 2 = softmax
 * (numbering of fused2.py:497).  Selection uses score + bias, the weight is the unbiased score;
 * equal keys pick the lowest index (fused2.py:471-472).  Output order = selection order. */
ORC_API void orc_gate_topk(const float* scores, const float* bias, int B, int E, float temp, int topk, float route_scale,
                           int mode, int norm, int32_t* eid, float* wt) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b) {
        double* s = (double*)malloc(sizeof(double) * E);
        double* key = (double*)malloc(sizeof(double) * E);
        const float* row = scores + (long)b * E;
        if (mode == 2) {
            float mx = -INFINITY;
            for (int e = 0; e < E; ++e) {
                float v = row[e] / temp;
                if (v > mx) mx = v;
            }
            double sum = 0;
            for (int e = 0; e < E; ++e) {
                s[e] = exp((double)(row[e] / temp) - (double)mx);
                sum += s[e];
            }
            for (int e = 0; e < E; ++e) s[e] = (double)(float)(s[e] / sum);
        } else if (mode == 1) {
            for (int e = 0; e < E; ++e) s[e] = (double)(float)(1.0 / (1.0 + exp(-(double)(row[e] / temp))));
        } else {
            for (int e = 0; e < E; ++e) {
                double v = (double)(row[e] / temp);
                double sp = v > 20.0 ? v : log1p(exp(v));
                s[e] = (double)(float)sqrt((double)(float)sp);
            }
        }
        for (int e = 0; e < E; ++e) key[e] = (double)((float)s[e] + (bias ? bias[e] : 0.f));
        float wsum = 0.f;
        for (int k = 0; k < topk; ++k) {
            int best = 0;
            for (int e = 1; e < E; ++e)
                if (key[e] > key[best]) best = e;
            eid[(long)b * topk + k] = best;
            wt[(long)b * topk + k] = (float)s[best];
            wsum += (float)s[best];
            key[best] = -INFINITY;
        }
        for (int k = 0; k < topk; ++k) {
            float w = wt[(long)b * topk + k];
            if (norm) w = w / (wsum + 1e-20f);
            wt[(long)b * topk + k] = w * route_scale;
        }
        free(s);
        free(key);
    }
}

/* ------------------------------------------------------------------ FP4 dot products */
/* quant.py:98-110: packed byte holds k even in the low nibble, k odd in the high nibble; one E8M0 byte per
 * 32 k.  Products bf16 x (E2M1 * 2^s) are exact in double; the sum is rounded once to fp32. */
static inline double fp4_row_dot(const uint8_t* w, const uint8_t* s, const uint16_t* x, int K) {
    double acc = 0;
    for (int g = 0; g < K / 32; ++g) {
        double sc = e8m0_value(s[g]);
        double part = 0;
        for (int j = 0; j < 16; ++j) {
            uint8_t p = w[g * 16 + j];
            part += (double)E2M1_VALUE[p & 15] * (double)bf16_to_f32(x[g * 32 + 2 * j]);
            part += (double)E2M1_VALUE[p >> 4] * (double)bf16_to_f32(x[g * 32 + 2 * j + 1]);
        }
        acc += sc * part;
    }
    return acc;
}

/* out[m,n] = sum_k a[m,k] * dequant_fp4(w,s)[n,k]  (kernels.py:145-168 contract, test_kernels.py:12-19) */
ORC_API void orc_fp4_gemm(const uint16_t* a, long lda, const uint8_t* w, const uint8_t* s, int M, int N, int K, float* out, long ldo) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m)
            out[(long)m * ldo + n] = (float)fp4_row_dot(w + (long)n * (K / 2), s + (long)n * (K / 32), a + (long)m * lda, K);
}

/* out[row_out[p]] += weight[p] * a[row_in[p]] @ W[expert[p]]^T   (moe_kernels.py:161-163; cukern.py:60-63 with
 * row_out = p).  out must be initialised by the caller.  Pairs are applied in index order. */
ORC_API void orc_fp4_pairs(const uint16_t* a, long lda, const uint8_t* w, long w_estride, const uint8_t* s, long s_estride,
                           const int32_t* expert, const int32_t* row_in, const int32_t* row_out, const float* weight, int n_pairs,
                           int N, int K, float* out, long ldo) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int p = 0; p < n_pairs; ++p) {
            int e = expert[p];
            if (e < 0) continue;
            double d = fp4_row_dot(w + (long)e * w_estride + (long)n * (K / 2), s + (long)e * s_estride + (long)n * (K / 32),
                                   a + (long)row_in[p] * lda, K);
            float v = (float)d;
            if (weight) v *= weight[p];
            out[(long)row_out[p] * ldo + n] += v;
        }
}

/* ------------------------------------------------------------------ SwiGLU + per-32 FP8 fake quant */
/* fused.py:285-306 / moe_cpu.cpp:359-377: clamp, silu(g)*u (times the routing weight), bf16 cast, then the
 * per-32 fake quantisation; gu fp32 [rows, 2*inter] (gate | up) -> h bf16 [rows, inter].
 * round_gu_bf16 != 0 first rounds gate/up to bf16 (the shared expert's GEMM returns bf16, decode.py:461-462). */
ORC_API void orc_swiglu_quant(const float* gu, const float* weights, int rows, int inter, float limit, int round_gu_bf16, uint16_t* h) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)rows * (inter / 32); ++i) {
        int r = (int)(i / (inter / 32)), b = (int)(i % (inter / 32)) * 32;
        const float* row = gu + (long)r * 2 * inter;
        float wt = weights ? weights[r] : 1.f;
        float tmp[32], amax = 1e-4f;
        for (int j = 0; j < 32; ++j) {
            float g = row[b + j], u = row[inter + b + j];
            if (round_gu_bf16) {
                g = bf16_to_f32(f32_to_bf16(g));
                u = bf16_to_f32(f32_to_bf16(u));
            }
            if (limit > 0) {
                u = fminf(fmaxf(u, -limit), limit);
                g = fminf(g, limit);
            }
            float v = wt * (g / (1.f + expf(-g))) * u;
            v = bf16_to_f32(f32_to_bf16(v));
            tmp[j] = v;
            if (fabsf(v) > amax) amax = fabsf(v);
        }
        float sc = pow2_ceil(amax / 448.f);
        for (int j = 0; j < 32; ++j) {
            float q = fminf(fmaxf(tmp[j] / sc, -448.f), 448.f);
            h[(long)r * inter + b + j] = f32_to_bf16(round_e4m3(q) * sc);
        }
    }
}

/* ------------------------------------------------------------------ routed experts of one token */
/* moe_cpu.cpp:386-503 (mode 0): stage 1 gu[e] = W13[e] x, stage 2 h[e] = swiglu_quant(gu[e]) * wt[e],
 * stage 3 out[n] = sum_e W2[e][n] . h[e].  Pointers per selected expert. */
ORC_API void orc_routed_token(const uint8_t* const* w13, const uint8_t* const* s13, const uint8_t* const* w2, const uint8_t* const* s2, int E,
                              const uint16_t* x, const float* wts, float* out, int K, int inter, int dim, float limit) {
    float* gu = (float*)malloc(sizeof(float) * (size_t)E * 2 * inter);
    uint16_t* h = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)E * inter);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)E * 2 * inter; ++i) {
        int e = (int)(i / (2 * inter)), n = (int)(i % (2 * inter));
        gu[i] = (float)fp4_row_dot(w13[e] + (long)n * (K / 2), s13[e] + (long)n * (K / 32), x, K);
    }
    orc_swiglu_quant(gu, wts, E, inter, limit, 0, h);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < dim; ++n) {
        float acc = 0.f; /* fp32 sum over experts in list order, as moe_cpu.cpp:481-485 */
        for (int e = 0; e < E; ++e)
            acc += (float)fp4_row_dot(w2[e] + (long)n * (inter / 2), s2[e] + (long)n * (inter / 32), h + (long)e * inter, inter);
        out[n] = acc;
    }
    free(gu);
    free(h);
}

/* ------------------------------------------------------------------ FP8 dense */
/* Reference format (quant.py:90-95, w8.py:39-61): e4m3 bytes [N,K] in natural k order + E8M0 byte per 32x32
 * block [ceil(N/32), scols].  y = x @ dequant^T with the sum rounded once to fp32. */
ORC_API void orc_fp8_gemm_e8m0(const uint16_t* x, long ldx, const uint8_t* w, const uint8_t* s, int scols, int M, int N, int K,
                               float* out, long ldo) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
            double acc = 0;
            for (int g = 0; g < K / 32; ++g) {
                double sc = ldexp(1.0, (int)s[(long)(n / 32) * scols + g] - 127);
                double part = 0;
                for (int j = 0; j < 32; ++j)
                    part += (double)e4m3_value(w[(long)n * K + g * 32 + j]) * (double)bf16_to_f32(x[(long)m * ldx + g * 32 + j]);
                acc += sc * part;
            }
            out[(long)m * ldo + n] = (float)acc;
        }
}

/* The other on-disk format this build accepts: e4m3 [N,K] + one FP32 scale per 128x128 block
 * [ceil(N/128), ceil(K/128)]; y = sum_blocks scale_b * sum_{k in b} x_k w_k.  The reference has no code for
 * this variant (parity for it is pinned only by this restatement of the published block-scale recipe). */
ORC_API void orc_fp8_gemm_f32block(const uint16_t* x, long ldx, const uint8_t* w, const float* s, int scols, int M, int N, int K,
                                   float* out, long ldo) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
            double acc = 0;
            for (int k0 = 0; k0 < K; k0 += 128) {
                double part = 0;
                int k1 = k0 + 128 < K ? k0 + 128 : K;
                for (int k = k0; k < k1; ++k) part += (double)e4m3_value(w[(long)n * K + k]) * (double)bf16_to_f32(x[(long)m * ldx + k]);
                acc += (double)s[(long)(n / 128) * scols + k0 / 128] * part;
            }
            out[(long)m * ldo + n] = (float)acc;
        }
}

/* Shared expert, decode.py:461-463: gu = bf16(W13s xq); hs = swiglu_quant(gu, no weight); ys = bf16(W2s hs).
 * fmt 0: E8M0 32x32 scales (uint8), fmt 1: FP32 128x128 scales.  xq bf16 [T,dim] -> ys bf16 [T,dim]. */
ORC_API void orc_shared_expert(const uint16_t* xq, int T, int dim, int inter, const uint8_t* w13, const void* s13, int s13cols,
                               const uint8_t* w2, const void* s2, int s2cols, int fmt, float limit, uint16_t* ys) {
    float* gu = (float*)malloc(sizeof(float) * (size_t)T * 2 * inter);
    uint16_t* h = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)T * inter);
    float* y = (float*)malloc(sizeof(float) * (size_t)T * dim);
    if (fmt == 0) orc_fp8_gemm_e8m0(xq, dim, w13, (const uint8_t*)s13, s13cols, T, 2 * inter, dim, gu, 2 * inter);
    else orc_fp8_gemm_f32block(xq, dim, w13, (const float*)s13, s13cols, T, 2 * inter, dim, gu, 2 * inter);
    orc_swiglu_quant(gu, NULL, T, inter, limit, 1, h);
    if (fmt == 0) orc_fp8_gemm_e8m0(h, inter, w2, (const uint8_t*)s2, s2cols, T, dim, inter, y, dim);
    else orc_fp8_gemm_f32block(h, inter, w2, (const float*)s2, s2cols, T, dim, inter, y, dim);
    for (long i = 0; i < (long)T * dim; ++i) ys[i] = f32_to_bf16(y[i]);
    free(gu);
    free(h);
    free(y);
}

/* ------------------------------------------------------------------ whole MoE layer */
/* model.py:2028-2233 / decode.py:446-464 + fused2.py:518-523 for T tokens:
 *   eid, wt = gate(logits);  xq = fake_quant_fp8(x);  y[t] = sum_j routed(xq[t], eid[t,j], wt[t,j]) (fp32)
 *   out[t] = bf16(y[t] + float(shared(xq[t]))).
 * Expert tensors in the stacked layout of load.py:237-249: w13 [E,2I,D/2], s13 [E,2I,D/32], w2 [E,D,I/2],
 * s2 [E,D,I/32].  Experts outside [shard_start, shard_start+shard_n) contribute nothing (ep.py:324-338);
 * has_shared = 0 skips the shared expert.  eid_out/wt_out (may be NULL) receive the routing.
 * routed_out (may be NULL) receives the fp32 routed sum [T,dim] before the shared expert is added. */
ORC_API void orc_moe_layer(const uint16_t* x, const float* logits, const float* bias, int T, int E, int topk, int dim, int inter,
                           float temp, float route_scale, int score_mode, int norm, float limit, const uint8_t* w13, const uint8_t* s13,
                           const uint8_t* w2, const uint8_t* s2, int shard_start, int shard_n, int has_shared, const uint8_t* sh_w13,
                           const void* sh_s13, int sh_s13cols, const uint8_t* sh_w2, const void* sh_s2, int sh_s2cols, int sh_fmt,
                           uint16_t* out, int32_t* eid_out, float* wt_out, float* routed_out) {
    int32_t* eid = (int32_t*)malloc(sizeof(int32_t) * (size_t)T * topk);
    float* wt = (float*)malloc(sizeof(float) * (size_t)T * topk);
    uint16_t* xq = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)T * dim);
    uint16_t* ys = (uint16_t*)calloc((size_t)T * dim, sizeof(uint16_t));
    float* y = (float*)calloc((size_t)T * dim, sizeof(float));
    orc_gate_topk(logits, bias, T, E, temp, topk, route_scale, score_mode, norm, eid, wt);
    orc_fake_quant_fp8(x, xq, (long)T * dim, 32);
    const size_t b13 = (size_t)2 * inter * (dim / 2), bs13 = (size_t)2 * inter * (dim / 32);
    const size_t b2 = (size_t)dim * (inter / 2), bs2 = (size_t)dim * (inter / 32);
    for (int t = 0; t < T; ++t) {
        const uint8_t *p13[64], *ps13[64], *p2[64], *ps2[64];
        float w[64];
        int n = 0;
        for (int j = 0; j < topk && n < 64; ++j) {
            int e = eid[(long)t * topk + j];
            if (e < shard_start || e >= shard_start + shard_n) continue;
            int le = e - shard_start; /* shard tensors hold [n, ...] for global experts [start, start+n) */
            p13[n] = w13 + le * b13;
            ps13[n] = s13 + le * bs13;
            p2[n] = w2 + le * b2;
            ps2[n] = s2 + le * bs2;
            w[n++] = wt[(long)t * topk + j];
        }
        if (n) orc_routed_token(p13, ps13, p2, ps2, n, xq + (long)t * dim, w, y + (long)t * dim, dim, inter, dim, limit);
    }
    if (has_shared) orc_shared_expert(xq, T, dim, inter, sh_w13, sh_s13, sh_s13cols, sh_w2, sh_s2, sh_s2cols, sh_fmt, limit, ys);
    for (long i = 0; i < (long)T * dim; ++i) out[i] = f32_to_bf16(y[i] + bf16_to_f32(ys[i]));
    if (eid_out) memcpy(eid_out, eid, sizeof(int32_t) * (size_t)T * topk);
    if (wt_out) memcpy(wt_out, wt, sizeof(float) * (size_t)T * topk);
    if (routed_out) memcpy(routed_out, y, sizeof(float) * (size_t)T * dim);
    free(eid);
    free(wt);
    free(xq);
    free(ys);
    free(y);
}

/* Stable grouping of pairs by expert: the integer bookkeeping of moe_kernels.py:111-132.
 * order[i] = index of the i-th pair after a stable sort by expert id; counts[e] = pairs of expert e. */
ORC_API void orc_group_pairs(const int32_t* expert, int n_pairs, int n_experts, int32_t* order, int32_t* counts) {
    memset(counts, 0, sizeof(int32_t) * (size_t)n_experts);
    for (int p = 0; p < n_pairs; ++p)
        if (expert[p] >= 0 && expert[p] < n_experts) counts[expert[p]]++;
    int32_t* pos = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_experts + 1));
    pos[0] = 0;
    for (int e = 0; e < n_experts; ++e) pos[e + 1] = pos[e] + counts[e];
    for (int p = 0; p < n_pairs; ++p)
        if (expert[p] >= 0 && expert[p] < n_experts) order[pos[expert[p]]++] = p;
    free(pos);
}
