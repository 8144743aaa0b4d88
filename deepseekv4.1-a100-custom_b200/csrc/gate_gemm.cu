// Router projection: logits[t, e] = sum_k x[t, k] * gate_w[e, k] in fp32 (dsv41/model.py:1615, dsv41/decode.py:449), so that the
// MoE layer can start from the hidden state instead of from logits.
//
// A small fp32 GEMM (tokens x experts x dim; 64 x 384 x 4096 in decode).  128 x 64 output tiles, 256 threads, an 8 x 4 register
// tile per thread, operands staged through shared memory 16 k at a time.  With few tokens there are only a handful of tiles, so
// the k range is split over `splits` blocks per tile; every split writes its partial tile to its own slab and the router adds
// the slabs in split order: no atomics, the logits (and with them the routing) are the same from run to run.
#include "common.cuh"
#include "gate_gemm.cuh"

namespace b200 {

constexpr int GG_TT = 128, GG_TE = 64, GG_KSTEP = 16, GG_THREADS = 256;  // tile: 128 tokens x 64 experts, 16 k per step

// x: fp32 [T, x_ld] (xf) or bf16 [T, xb_ld] (converted on load); w fp32 [E, D]; out fp32 [splits][T][E].
// A thread owns an 8 x 4 block of the tile (tokens 8 tr .., experts 4 tc ..); the global loads of step i + 1 are in flight while
// step i is computed from shared memory.
__global__ void __launch_bounds__(GG_THREADS) gate_gemm_kernel(const float* __restrict__ xf, long long xf_ld, const __nv_bfloat16* __restrict__ xb,
                                                               long long xb_ld, const float* __restrict__ w, int T, int E, int D, int k_per_split,
                                                               float* __restrict__ out) {
    __shared__ __align__(16) float xs[GG_KSTEP][GG_TT + 4], ws[GG_KSTEP][GG_TE + 4];
    const int t0 = blockIdx.x * GG_TT, e0 = blockIdx.y * GG_TE, split = blockIdx.z;
    const int k_lo = split * k_per_split, k_hi = min(D, k_lo + k_per_split);
    const int tid = threadIdx.x, tr = tid >> 4, tc = tid & 15;
    // loaders: x tile 128 rows x 16 k = 512 float4 (two per thread: rows lr and lr + 64), w tile 64 rows x 16 k = 256 float4
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[8][4] = {};
    float xv[2][4], wv[4];
    auto fetch = [&](int k0) {
        const int k = k0 + lk;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int t = t0 + lr + 64 * h;
            xv[h][0] = xv[h][1] = xv[h][2] = xv[h][3] = 0.f;
            if (t < T && k < k_hi) {  // D % 4 == 0: the 4 values are all inside or all outside
                if (xf) {
                    const float4 v = *reinterpret_cast<const float4*>(xf + (long long)t * xf_ld + k);
                    xv[h][0] = v.x; xv[h][1] = v.y; xv[h][2] = v.z; xv[h][3] = v.w;
                } else {
                    const uint2 v = *reinterpret_cast<const uint2*>(xb + (long long)t * xb_ld + k);
                    xv[h][0] = bf16_bits_to_f32(v.x & 0xFFFFu); xv[h][1] = bf16_bits_to_f32(v.x >> 16);
                    xv[h][2] = bf16_bits_to_f32(v.y & 0xFFFFu); xv[h][3] = bf16_bits_to_f32(v.y >> 16);
                }
            }
        }
        wv[0] = wv[1] = wv[2] = wv[3] = 0.f;
        if (e0 + lr < E && k < k_hi) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(w + (long long)(e0 + lr) * D + k));
            wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
        }
    };
    if (k_lo < k_hi) fetch(k_lo);
    for (int k0 = k_lo; k0 < k_hi; k0 += GG_KSTEP) {
        __syncthreads();  // the previous step's tiles have been read
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            xs[lk + i][lr] = xv[0][i];
            xs[lk + i][lr + 64] = xv[1][i];
            ws[lk + i][lr] = wv[i];
        }
        __syncthreads();
        if (k0 + GG_KSTEP < k_hi) fetch(k0 + GG_KSTEP);  // in flight during the arithmetic below
#pragma unroll
        for (int kk = 0; kk < GG_KSTEP; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&xs[kk][tr * 8]);
            const float4 a1 = *reinterpret_cast<const float4*>(&xs[kk][tr * 8 + 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[kk][tc * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    float* o = out + (size_t)split * T * E;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int t = t0 + tr * 8 + i;
        if (t >= T) continue;
        const int e = e0 + tc * 4;
        if (e + 3 < E && (E & 3) == 0) {
            *reinterpret_cast<float4*>(o + (size_t)t * E + e) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (e + j < E) o[(size_t)t * E + e + j] = acc[i][j];
        }
    }
}

int gate_gemm_splits(int T, int E, int D) {
    const int tiles = ((T + GG_TT - 1) / GG_TT) * ((E + GG_TE - 1) / GG_TE);
    if (tiles < 1) return 1;  // empty batch
    int splits = (148 + tiles - 1) / tiles;  // about one block per SM in all
    const int max_splits = D / 128 > 0 ? D / 128 : 1;  // at least 128 k per split
    if (splits > max_splits) splits = max_splits;
    if (splits > GATE_MAX_SPLITS) splits = GATE_MAX_SPLITS;
    return splits < 1 ? 1 : splits;
}

int gate_gemm(const float* xf, long long xf_ld, const __nv_bfloat16* xb, long long xb_ld, const float* w, int T, int E, int D, int splits, float* out,
              cudaStream_t stream) {
    if ((!xf && !xb) || !w || !out || T <= 0 || E <= 0 || D <= 0 || D % 4 || splits < 1) return ERR_BAD_ARG;
    if (xf ? (((uintptr_t)xf & 15) || (xf_ld & 3)) : (((uintptr_t)xb & 7) || (xb_ld & 3))) return ERR_BAD_ALIGN;
    if ((uintptr_t)w & 15) return ERR_BAD_ALIGN;
    int kps = (D + splits - 1) / splits;
    kps = (kps + GG_KSTEP - 1) / GG_KSTEP * GG_KSTEP;
    const dim3 grid((T + GG_TT - 1) / GG_TT, (E + GG_TE - 1) / GG_TE, splits);
    // plain launch: the first kernel of a layer step, nothing to overlap with
    gate_gemm_kernel<<<grid, GG_THREADS, 0, stream>>>(xf, xf_ld, xb, xb_ld, w, T, E, D, kps, out);
    B200_CHECK_LAUNCH();
    return 0;
}

}  // namespace b200
