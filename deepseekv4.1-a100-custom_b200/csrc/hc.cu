// The two steps either side of the MoE path in the reference's decode loop (hyper-connection mixes):
//   hc_pre_norm_quant2 (dsv41/fused2.py:171-246): y = rmsnorm(bf16(sum_h pre[h] * x[h])) * w, its FP8 fake-quantised copy, optionally
//     y as fp32 and the 8-k permuted copy -- the producer of the layer's inputs xq / xf / xqp;
//   hc_post2_ (dsv41/fused2.py:505-558): residual[i] <- post[i] * x + sum_h comb[h][i] * residual[h], where x is either given or
//     assembled from the MoE pieces bf16(sum_k y2[k] + ys) -- the consumer of the layer's outputs.
// Both are bandwidth-trivial row kernels: one block per token row, 8 contiguous columns per thread.
#include "b200_moe.h"
#include "common.cuh"

namespace b200 {

constexpr int HC_THREADS = 256;
constexpr int HC_MAX = 8;  // hyper-connection copies per token the kernels accept (the reference uses 4)

__device__ __forceinline__ void unpack8(const uint4& r, float (&v)[8]) {
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = bf16_bits_to_f32(u[i] & 0xFFFFu);
        v[2 * i + 1] = bf16_bits_to_f32(u[i] >> 16);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) u[i] = f32_to_bf16_bits(v[2 * i]) | (f32_to_bf16_bits(v[2 * i + 1]) << 16);
    return make_uint4(u[0], u[1], u[2], u[3]);
}

// x bf16 [B, hc, D]; pre fp32 [B, hc]; w bf16 or fp32 [D]; outputs y, yq bf16 [B, D], yf fp32 [B, D] or null, yqp bf16 [B, D] or null.
// D % 32 == 0.  Phase 1 leaves bf16(sum_h pre[h] x[h]) in y and the row's sum of squares in shared memory; phase 2 re-reads it
// (same thread, same columns), normalises, and quantises per group of 32 (4 threads).
template <typename TW>
__global__ void __launch_bounds__(HC_THREADS) hc_pre_norm_quant_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ pre,
                                                                       const TW* __restrict__ w, float eps, int hc, int D, __nv_bfloat16* __restrict__ y,
                                                                       __nv_bfloat16* __restrict__ yq, float* __restrict__ yf, __nv_bfloat16* __restrict__ yqp) {
    __shared__ float red[HC_THREADS / 32];
    __shared__ float s_rinv;
    const long row = blockIdx.x;
    const int tid = threadIdx.x;
    float p[HC_MAX];
    for (int h = 0; h < hc; ++h) p[h] = pre[row * hc + h];
    float ss = 0.f;
    for (int c = tid * 8; c < D; c += HC_THREADS * 8) {
        float acc[8] = {};
        for (int h = 0; h < hc; ++h) {  // in h order, as the reference accumulates
            float v[8];
            unpack8(*reinterpret_cast<const uint4*>(x + (row * hc + h) * D + c), v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(p[h], v[i], acc[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[i] = round_bf16(acc[i]);
            ss += acc[i] * acc[i];
        }
        *reinterpret_cast<uint4*>(y + row * D + c) = pack8(acc);
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int i = 0; i < HC_THREADS / 32; ++i) t += red[i];
        s_rinv = __fdiv_rn(1.f, sqrtf(__fdiv_rn(t, (float)D) + eps));
    }
    __syncthreads();
    const float rinv = s_rinv;
    for (int base = 0; base < D; base += HC_THREADS * 8) {  // uniform trip count: the shuffles below need the whole warp
        const int c = base + tid * 8;
        const bool on = c < D;  // D % 32 == 0: the 4 threads of a group are on or off together
        float v[8] = {}, amax = 0.f;
        if (on) unpack8(*reinterpret_cast<const uint4*>(y + row * D + c), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = on ? round_bf16(v[i] * rinv * (float)w[c + i]) : 0.f;
            amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        if (!on) continue;
        *reinterpret_cast<uint4*>(y + row * D + c) = pack8(v);
        if (yf) {
            float4* o = reinterpret_cast<float4*>(yf + row * D + c);
            o[0] = make_float4(v[0], v[1], v[2], v[3]);
            o[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
        // group of 32 = this thread and its 3 neighbours (c is a multiple of 8, groups start at multiples of 32): amax above
        const float s = fp8_group_scale_bf16(amax);
        float q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = fp8_fake_quant_value(v[i], s);
        *reinterpret_cast<uint4*>(yq + row * D + c) = pack8(q);
        if (yqp) {  // stored order inside every 8 k: 0,4,2,6,1,5,3,7 (dsv41/cukern.py:267-273): position j holds element perm[j]
            const float qp[8] = {q[0], q[4], q[2], q[6], q[1], q[5], q[3], q[7]};
            *reinterpret_cast<uint4*>(yqp + row * D + c) = pack8(qp);
        }
    }
}

// residual bf16 [B, hc, D] (in place); post fp32 [B, hc]; comb fp32 [B, hc, hc]; x bf16 [B, D] or null; y2 fp32 (nsum rows per token,
// element (b, k, c) at y2[b * y2_row_stride + k * y2_sum_stride + c]) + ys bf16 [B, D] or null.
__global__ void __launch_bounds__(HC_THREADS) hc_post_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ y2,
                                                             const __nv_bfloat16* __restrict__ ys, long long y2_row_stride, long long y2_sum_stride,
                                                             int nsum, __nv_bfloat16* __restrict__ residual, const float* __restrict__ post,
                                                             const float* __restrict__ comb, int hc, int D) {
    pdl_wait();
    const long row = blockIdx.y;
    const int c = (blockIdx.x * HC_THREADS + threadIdx.x) * 8;
    if (c >= D) return;
    float xv[8];
    if (nsum > 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = 0.f;
        for (int k = 0; k < nsum; ++k) {  // in slot order, as the reference adds them
            const float4* p = reinterpret_cast<const float4*>(y2 + row * y2_row_stride + (long long)k * y2_sum_stride + c);
            const float4 a = p[0], b = p[1];
            xv[0] += a.x; xv[1] += a.y; xv[2] += a.z; xv[3] += a.w; xv[4] += b.x; xv[5] += b.y; xv[6] += b.z; xv[7] += b.w;
        }
        if (ys) {
            float sv[8];
            unpack8(*reinterpret_cast<const uint4*>(ys + row * D + c), sv);
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[i] += sv[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = round_bf16(xv[i]);
    } else {
        unpack8(*reinterpret_cast<const uint4*>(x + row * D + c), xv);
    }
    float r[HC_MAX][8];
    for (int h = 0; h < hc; ++h) unpack8(*reinterpret_cast<const uint4*>(residual + (row * hc + h) * D + c), r[h]);
    for (int i = 0; i < hc; ++i) {
        float acc[8];
        const float pi = post[row * hc + i];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = pi * xv[e];
        for (int h = 0; h < hc; ++h) {
            const float ch = comb[(row * hc + h) * hc + i];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(ch, r[h][e], acc[e]);
        }
        *reinterpret_cast<uint4*>(residual + (row * hc + i) * D + c) = pack8(acc);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_hc_pre_norm_quant2(const void* x, const float* pre, const void* w, int w_is_f32, float eps, int rows, int hc, int dim, void* y, void* yq,
                                       float* yf, void* yqp, cudaStream_t stream) {
    if (!x || !pre || !w || !y || !yq || rows < 0 || hc < 1 || hc > HC_MAX || dim <= 0) return ERR_BAD_ARG;
    if (dim % 32) return ERR_BAD_SHAPE;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)yq | (uintptr_t)yf | (uintptr_t)yqp) & 15) return ERR_BAD_ALIGN;
    if (rows == 0) return 0;
    if (w_is_f32)
        hc_pre_norm_quant_kernel<float><<<rows, HC_THREADS, 0, stream>>>((const __nv_bfloat16*)x, pre, (const float*)w, eps, hc, dim, (__nv_bfloat16*)y,
                                                                         (__nv_bfloat16*)yq, yf, (__nv_bfloat16*)yqp);
    else
        hc_pre_norm_quant_kernel<__nv_bfloat16><<<rows, HC_THREADS, 0, stream>>>((const __nv_bfloat16*)x, pre, (const __nv_bfloat16*)w, eps, hc, dim,
                                                                                 (__nv_bfloat16*)y, (__nv_bfloat16*)yq, yf, (__nv_bfloat16*)yqp);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_hc_post2(const void* x, const float* y2, const void* ys, long long y2_row_stride, long long y2_sum_stride, int nsum, void* residual,
                             const float* post, const float* comb, int rows, int hc, int dim, cudaStream_t stream) {
    if (!residual || !post || !comb || rows < 0 || hc < 1 || hc > HC_MAX || dim <= 0 || nsum < 0) return ERR_BAD_ARG;
    if (nsum == 0 ? !x : !y2) return ERR_BAD_ARG;
    if (dim % 8) return ERR_BAD_SHAPE;
    if (((uintptr_t)x | (uintptr_t)ys | (uintptr_t)residual) & 15) return ERR_BAD_ALIGN;
    if (nsum > 0 && (((uintptr_t)y2 & 15) || (y2_row_stride & 3) || (y2_sum_stride & 3))) return ERR_BAD_ALIGN;
    if (rows == 0) return 0;
    const dim3 grid((dim / 8 + HC_THREADS - 1) / HC_THREADS, rows);
    const cudaError_t e = launch_pdl(hc_post_kernel, grid, dim3(HC_THREADS), 0, stream, (const __nv_bfloat16*)x, y2, (const __nv_bfloat16*)ys, y2_row_stride,
                                     y2_sum_stride, nsum, (__nv_bfloat16*)residual, post, comb, hc, dim);
    return e == cudaSuccess ? 0 : (int)e;
}
