// Weight-streaming grouped "skinny" GEMM for decode: out[pair, n] = sum_k x[tok(pair), k] * W[expert][n, k] for groups
// of at most 8 tokens per expert (larger groups are cut into 8-token works that re-read the expert).
//
// HBM-bound by design: every weight byte is read exactly once per work with 128-bit streaming loads straight into
// registers (8 loads of 16 B in flight per lane, 64 KB per SM), dequantised in registers to packed bf16 with the
// block scale folded into the exponent, and contracted against the (<= 8) token columns with warp-level 16x8x16
// tensor-core tiles that accumulate in fp32.  One CTA = 16 warps = 4 row blocks of 16 weight rows x 4 splits of K;
// the K splits are summed through shared memory.  Activations of the work's tokens sit in shared memory in the
// fragment order of the tile, pre-scaled by 2^ACT_SHIFT.
//
// Replaces, for the sm_100a build, the reference's sm_80 kernels fp4_gemv_pairs (dsv41/cuda/fp4_gemv.cu:15),
// fp4_gemv_m1 (dsv41/cuda/fp4_gemv_m1.cu:57), fp4_gemm_tc8/16 (dsv41/cuda/fp4_tc.cu:52), fp8_gemv_m1
// (dsv41/cuda/fp8_gemv_m1.cu:55) and fp8_gemm_tc8/16 (dsv41/cuda/fp8_tc.cu:53) with one kernel template.
#include "common.cuh"
#include "skinny.cuh"

namespace b200 {

// ------------------------------------------------------------------ in-register dequantisation
// FP4: eight E2M1 codes of one 32-bit word -> four bf16x2 registers; register j holds codes (j, j+4) in its
// (low, high) halves.  A code `s e1 e0 m` placed at bf16 bits [15 | 8:6] is the bf16 number value * 2^-126
// (the sub-normal case e = 0 included), so one packed multiply by 2^(scale_byte - 1 - ACT_SHIFT) yields the
// exact scaled weight (times 2^-ACT_SHIFT).  Same values as dsv41/quant.py:24,98-110.
__device__ __forceinline__ void dequant_fp4_word(uint32_t w, uint32_t mult, uint32_t (&r)[4]) {
    uint32_t m0 = ((w << 6) & 0x01C001C0u) | ((w << 12) & 0x80008000u);
    uint32_t m1 = ((w << 2) & 0x01C001C0u) | ((w << 8) & 0x80008000u);
    uint32_t m2 = ((w >> 2) & 0x01C001C0u) | ((w << 4) & 0x80008000u);
    uint32_t m3 = ((w >> 6) & 0x01C001C0u) | (w & 0x80008000u);
    r[0] = mul_bf16x2(m0, mult);
    r[1] = mul_bf16x2(m1, mult);
    r[2] = mul_bf16x2(m2, mult);
    r[3] = mul_bf16x2(m3, mult);
}

// FP8 e4m3: four codes of one word -> two bf16x2 registers; r[0] holds bytes (0, 2), r[1] bytes (1, 3).
// A code `s eeee mmm` placed at bf16 bits [15 | 10:4] is value * 2^-120 (sub-normals included).
__device__ __forceinline__ void dequant_fp8_word(uint32_t w, uint32_t mult, uint32_t (&r)[2]) {
    uint32_t m0 = ((w << 4) & 0x07F007F0u) | ((w << 8) & 0x80008000u);
    uint32_t m1 = ((w >> 4) & 0x07F007F0u) | (w & 0x80008000u);
    r[0] = mul_bf16x2(m0, mult);
    r[1] = mul_bf16x2(m1, mult);
}

__device__ __forceinline__ uint32_t bf16x2_pow2(int field) {  // both halves = 2^(field - 127), field in [1, 254]
    uint32_t m = (uint32_t)field << 7;
    return m | (m << 16);
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

__device__ __forceinline__ uint4 lds128(const uint4* p) { return *p; }

// byte order of every 16-k block of the reference's FP8 weight container (dsv41/w8.py:21-23)
__constant__ int PERM_K16[16] = {0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15};

template <int FMT>
struct FmtTraits {
    static constexpr bool FP4 = (FMT == SK_FMT_FP4_E8M0 || FMT == SK_FMT_FP4_BF16S);
    static constexpr int CK = FP4 ? 128 : 64;  // k covered by one 16-byte load of each of the 4 lanes of a quad
};

// ------------------------------------------------------------------ activation tile
// Fill the shared-memory activation tile for the tokens of one work.  16-byte unit u = ((c*A + i)*4 + t)*8 + g holds,
// for token column g, the eight activations lane (g, t) needs for the two (FP4: word i of chunk c) or two (FP8: words
// 2i, 2i+1) tensor-core steps, in (b0.lo, b0.hi, b1.lo, b1.hi) x 2 order.
template <int FMT>
__device__ void fill_act_tile(uint4* xs, const SkinnyArgs& a, int first, int ntok) {
    constexpr bool FP4 = FmtTraits<FMT>::FP4;
    const int K = a.K;
    const float up = u32_as_f32((uint32_t)(127 + ACT_SHIFT) << 23);
    for (int u = threadIdx.x; u < K; u += blockDim.x) {
        const int g = u & 7, t = (u >> 3) & 3;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < ntok) {
            const int pair = first + g;
            const long row = a.pair_tok ? a.pair_tok[pair] : pair;
            const __nv_bfloat16* xr = a.x + row * a.x_ld;
            float f[8];
            if (FP4) {
                const int i = (u >> 5) & 3, c = u >> 7;
                const int k0 = c * 128 + t * 32 + i * 8;
                uint4 raw = *reinterpret_cast<const uint4*>(xr + k0);
                uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
                float e[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = bf16_bits_to_f32((rw[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu);
                if (a.x_perm8) {  // stored slot j holds k = bitrev3(j) (dsv41/cukern.py:267-273); the map is its own inverse
                    float n[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) n[j] = e[((j & 1) << 2) | (j & 2) | (j >> 2)];
#pragma unroll
                    for (int j = 0; j < 8; ++j) e[j] = n[j];
                }
                // slot order 0,4,1,5,2,6,3,7: registers (x0,x4) (x1,x5) | (x2,x6) (x3,x7)
                f[0] = e[0]; f[1] = e[4]; f[2] = e[1]; f[3] = e[5]; f[4] = e[2]; f[5] = e[6]; f[6] = e[3]; f[7] = e[7];
            } else {
                const int h = (u >> 5) & 1, c = u >> 6;
                const int kb = c * 64 + t * 16;
#pragma unroll
                for (int sl = 0; sl < 8; ++sl) {
                    const int i = 2 * h + (sl >> 2);
                    const int q = ((sl & 1) << 1) | ((sl >> 1) & 1);  // slot order 0,2,1,3 within a word
                    const int p = 4 * i + q;
                    const int k = kb + (a.w_permk ? PERM_K16[p] : p);
                    f[sl] = __bfloat162float(xr[k]);
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f32_to_bf16_bits(f[2 * j] * up) | (f32_to_bf16_bits(f[2 * j + 1] * up) << 16);
            v = make_uint4(o[0], o[1], o[2], o[3]);
        }
        xs[u] = v;
    }
}

// ------------------------------------------------------------------ the kernel
constexpr int U = SK_CHUNKS_PER_BATCH;

struct Batch {
    uint4 wq[2][U];     // 16 weight bytes of rows g and g+8 for each chunk
    uint32_t sc[2][U];  // raw scale bits for those loads
};

template <int FMT, int EPI>
__global__ void __launch_bounds__(SK_THREADS, 1) skinny_kernel(const SkinnyArgs a) {
    using T = FmtTraits<FMT>;
    constexpr bool FP4 = T::FP4;
    constexpr int CK = T::CK;
    extern __shared__ uint4 smem[];
    uint4* xs = smem;                                       // K units of 16 B
    float* red = reinterpret_cast<float*>(smem + a.K);      // [2][4 kq][4 rb][16][8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rb = warp & 3, kq = warp >> 2;
    const int K = a.K, N = a.N;
    const int nchunks = K / CK;
    const int nbat = (nchunks + U - 1) / U;
    const int b0 = kq * nbat / 4, b1 = (kq + 1) * nbat / 4;
    const int ipw = (EPI == SK_EPI_SWIGLU) ? (a.inter >> 5) : ((N + SK_ROWS - 1) / SK_ROWS);
    const int n_work = a.n_work ? *a.n_work : a.n_work_host;
    const long total = (long)n_work * ipw;
    const long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    const long wrow_bytes = FP4 ? (K >> 1) : K;

    // dense mode (no work list): work wk = rows [8 wk, 8 wk + 8) of x against expert 0
    auto get_work = [&](int wk) -> int4 {
        if (a.work) return __ldg(a.work + wk);
        const int rem = a.dense_rows - wk * SK_TOK;
        return make_int4(0, wk * SK_TOK, rem < SK_TOK ? rem : SK_TOK, 0);
    };
    auto row_base = [&](int it) -> int {
        if (EPI == SK_EPI_SWIGLU) return (rb < 2) ? it * 32 + rb * 16 : a.inter + it * 32 + (rb - 2) * 16;
        return it * SK_ROWS + rb * 16;
    };

    auto issue = [&](long item, int b, Batch& L) {
        const int wk = (int)(item / ipw), it = (int)(item % ipw);
        const int4 wrk = get_work(wk);
        const int r0 = row_base(it);
        const bool rows_ok = r0 < N;
        const uint8_t* w0 = a.w + (long long)wrk.x * a.w_estride + (long)(r0 + g) * wrow_bytes + t * 16;
        const uint8_t* w1 = w0 + 8 * wrow_bytes;
        const uint8_t* sbase = a.s + (long long)wrk.x * a.s_estride;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = b * U + u;
            if (rows_ok && c < nchunks) {
                L.wq[0][u] = ldg_stream16(w0 + c * 64);
                L.wq[1][u] = ldg_stream16(w1 + c * 64);
                if (FMT == SK_FMT_FP4_E8M0) {  // one byte per (row, 32 k): the chunk's four bytes, lane t uses byte t
                    L.sc[0][u] = ldg_stream4(sbase + (long)(r0 + g) * a.s_rstride + 4 * c);
                    L.sc[1][u] = ldg_stream4(sbase + (long)(r0 + g + 8) * a.s_rstride + 4 * c);
                } else if (FMT == SK_FMT_FP4_BF16S) {  // one bf16 per (row, 32 k)
                    L.sc[0][u] = *reinterpret_cast<const unsigned short*>(sbase + (long)(r0 + g) * a.s_rstride + 2 * (4 * c + t));
                    L.sc[1][u] = *reinterpret_cast<const unsigned short*>(sbase + (long)(r0 + g + 8) * a.s_rstride + 2 * (4 * c + t));
                } else if (FMT == SK_FMT_FP8_E8M0) {  // one byte per (32 rows, 32 k); rows g and g+8 share it
                    L.sc[0][u] = *(sbase + (long)(r0 >> 5) * a.s_rstride + 2 * c + (t >> 1));
                } else {  // one fp32 per (128 rows, 128 k)
                    L.sc[0][u] = ldg_stream4(sbase + (long)(r0 >> 7) * a.s_rstride + 4 * (c >> 1));
                }
            } else {
                L.wq[0][u] = make_uint4(0, 0, 0, 0);
                L.wq[1][u] = make_uint4(0, 0, 0, 0);
                L.sc[0][u] = 0;
                L.sc[1][u] = 0;
            }
        }
    };

    float acc[4];
    auto compute = [&](int b, const Batch& L) {
        float blk[4] = {0.f, 0.f, 0.f, 0.f};  // FP8 / fp32 block scales: partial sum of one 128-k block
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = b * U + u;
            if (c >= nchunks) break;
            if (FP4) {
                uint32_t m0, m1;
                if (FMT == SK_FMT_FP4_E8M0) {
                    const uint32_t s0 = (L.sc[0][u] >> (8 * t)) & 0xFFu, s1 = (L.sc[1][u] >> (8 * t)) & 0xFFu;
                    m0 = s0 ? bf16x2_pow2((int)s0 + 126 - ACT_SHIFT) : 0u;  // 2^(s - 127) * 2^126 * 2^-ACT_SHIFT
                    m1 = s1 ? bf16x2_pow2((int)s1 + 126 - ACT_SHIFT) : 0u;
                } else {
                    const float up = u32_as_f32((uint32_t)(127 + 126 - ACT_SHIFT) << 23);
                    uint32_t h0 = f32_to_bf16_bits(bf16_bits_to_f32(L.sc[0][u]) * up), h1 = f32_to_bf16_bits(bf16_bits_to_f32(L.sc[1][u]) * up);
                    m0 = h0 | (h0 << 16);
                    m1 = h1 | (h1 << 16);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t p[4], q[4];
                    dequant_fp4_word(word_of(L.wq[0][u], i), m0, p);
                    dequant_fp4_word(word_of(L.wq[1][u], i), m1, q);
                    const uint4 bv = lds128(xs + (((c * 4 + i) * 4 + t) * 8 + g));
                    mma_bf16_16816(acc, p[0], q[0], p[1], q[1], bv.x, bv.y);
                    mma_bf16_16816(acc, p[2], q[2], p[3], q[3], bv.z, bv.w);
                }
            } else {
                uint32_t m;
                if (FMT == SK_FMT_FP8_E8M0) {
                    const uint32_t s0 = L.sc[0][u] & 0xFFu;
                    m = s0 ? bf16x2_pow2((int)s0 + 120 - ACT_SHIFT) : 0u;  // 2^(s - 127) * 2^120 * 2^-ACT_SHIFT
                } else {
                    m = bf16x2_pow2(127 + 120 - ACT_SHIFT);
                }
                float* dst = (FMT == SK_FMT_FP8_F32B) ? blk : acc;
                float (&d)[4] = *reinterpret_cast<float (*)[4]>(dst);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 bv = lds128(xs + (((c * 2 + h) * 4 + t) * 8 + g));
                    uint32_t p[2], q[2];
                    dequant_fp8_word(word_of(L.wq[0][u], 2 * h), m, p);
                    dequant_fp8_word(word_of(L.wq[1][u], 2 * h), m, q);
                    mma_bf16_16816(d, p[0], q[0], p[1], q[1], bv.x, bv.y);
                    dequant_fp8_word(word_of(L.wq[0][u], 2 * h + 1), m, p);
                    dequant_fp8_word(word_of(L.wq[1][u], 2 * h + 1), m, q);
                    mma_bf16_16816(d, p[0], q[0], p[1], q[1], bv.z, bv.w);
                }
                if (FMT == SK_FMT_FP8_F32B && ((c & 1) || c + 1 == nchunks)) {
                    const float sc = u32_as_f32(L.sc[0][u]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) { acc[j] = fmaf(sc, blk[j], acc[j]); blk[j] = 0.f; }
                }
            }
        }
    };

    Batch cur, nxt;
    const bool has_k = b0 < b1;
    if (lo < hi && has_k) issue(lo, b0, cur);
    int cur_wk = -1, buf = 0;
    int4 wrk = make_int4(0, 0, 0, 0);
    for (long item = lo; item < hi; ++item) {
        const int wk = (int)(item / ipw), it = (int)(item % ipw);
        if (wk != cur_wk) {  // new work: the token columns change
            __syncthreads();
            wrk = get_work(wk);
            fill_act_tile<FMT>(xs, a, wrk.y, wrk.z);
            __syncthreads();
            cur_wk = wk;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = 0.f;
        for (int b = b0; b < b1; ++b) {
            const bool more = b + 1 < b1;
            if (more) issue(item, b + 1, nxt);
            else if (item + 1 < hi) issue(item + 1, b0, nxt);
            compute(b, cur);
            cur = nxt;
        }
        // partial sums of the 4 K splits -> shared memory
        float* rp = red + ((((buf * 4 + kq) * 4 + rb) * 16) * 8);
        *reinterpret_cast<float2*>(rp + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(rp + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
        __syncthreads();
        const float* rbuf = red + buf * (4 * 4 * 16 * 8);
        const int ntok = wrk.z, first = wrk.y;
        if (EPI == SK_EPI_SWIGLU) {
            // warp = token column, lane = column of the 32-wide quantisation group (dsv41/fused.py:285-306)
            if (warp < ntok) {
                const int rg = lane >> 4, row = lane & 15;
                float gt = 0.f, up = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    gt += rbuf[(((q * 4 + rg) * 16) + row) * 8 + warp];
                    up += rbuf[(((q * 4 + 2 + rg) * 16) + row) * 8 + warp];
                }
                if (a.round_gu_bf16) { gt = round_bf16(gt); up = round_bf16(up); }
                const int pair = first + warp;
                const float h = swiglu_bf16(gt, up, a.pair_w ? a.pair_w[pair] : 1.f, a.limit);
                const float s = fp8_group_scale(warp_max(fabsf(h)));
                const long orow = a.pair_out ? a.pair_out[pair] : pair;
                reinterpret_cast<__nv_bfloat16*>(a.out)[orow * a.out_ld + it * 32 + lane] = __float2bfloat16_rn(fp8_fake_quant_value(h, s));
            }
        } else {
            const int col = tid >> 6, rr = tid & 63;
            const int n = it * SK_ROWS + rr;
            if (col < ntok && n < N) {
                float v = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) v += rbuf[(((q * 4 + (rr >> 4)) * 16) + (rr & 15)) * 8 + col];
                const int pair = first + col;
                if (a.pair_w) v *= a.pair_w[pair];
                const long orow = a.pair_out ? a.pair_out[pair] : pair;
                if (EPI == SK_EPI_STORE_F32) reinterpret_cast<float*>(a.out)[orow * a.out_ld + n] = v;
                else if (EPI == SK_EPI_ATOMIC_F32) atomicAdd(reinterpret_cast<float*>(a.out) + orow * a.out_ld + n, v);
                else reinterpret_cast<__nv_bfloat16*>(a.out)[orow * a.out_ld + n] = __float2bfloat16_rn(v);
            }
        }
        buf ^= 1;
    }
}

// ------------------------------------------------------------------ work list
// One block.  Groups g (expert grp_expert[g], pairs grp_start[g] .. grp_start[g+1]-1) that belong to this shard are cut
// into works of at most 8 pairs: work = {local expert, first pair, n pairs, group}.  Groups of other shards (and padded
// groups, expert -1) get their output rows zeroed when zero_out is set, as dsv41/cuda/fp4_tc.cu:66-72 does.
__global__ void __launch_bounds__(1024) skinny_plan_kernel(const int* __restrict__ grp_expert, const int* __restrict__ grp_start,
                                                           const int* __restrict__ grp_count, int G, int n_pairs, int shard_start, int shard_n,
                                                           int4* __restrict__ work, int* __restrict__ n_work, int max_work) {
    __shared__ int warp_tot[32];
    __shared__ int running;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < G; base += 1024) {
        const int gi = base + tid;
        int nsub = 0, e = -1, s = 0, cnt = 0;
        if (gi < G) {
            e = grp_expert[gi] - shard_start;
            s = grp_start[gi];
            int en = grp_count ? s + grp_count[gi] : grp_start[gi + 1];
            if (en > n_pairs) en = n_pairs;
            cnt = en - s;
            if (e >= 0 && e < shard_n && cnt > 0 && s >= 0) nsub = (cnt + SK_TOK - 1) / SK_TOK;
        }
        int incl = nsub;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int woff = 0;
        for (int w = 0; w < warp; ++w) woff += warp_tot[w];
        int tot = 0;
        for (int w = 0; w < 32; ++w) tot += warp_tot[w];
        const int off = running + woff + incl - nsub;
        for (int i = 0; i < nsub; ++i) {
            const int rem = cnt - i * SK_TOK;
            if (off + i < max_work) work[off + i] = make_int4(e, s + i * SK_TOK, rem < SK_TOK ? rem : SK_TOK, gi);
        }
        __syncthreads();
        if (tid == 0) running += tot;
        __syncthreads();
    }
    if (tid == 0) *n_work = running < max_work ? running : max_work;
}

__global__ void skinny_zero_foreign_kernel(const int* __restrict__ grp_expert, const int* __restrict__ grp_start, const int* __restrict__ grp_count,
                                           int G, int n_pairs, int shard_start, int shard_n, float* __restrict__ out, long long out_ld, int N) {
    for (int gi = blockIdx.x; gi < G; gi += gridDim.x) {
        const int e = grp_expert[gi] - shard_start;
        if (e >= 0 && e < shard_n) continue;
        int s = grp_start[gi], en = grp_count ? s + grp_count[gi] : grp_start[gi + 1];
        if (en > n_pairs) en = n_pairs;
        if (s < 0) s = 0;
        for (int r = s; r < en; ++r)
            for (int n = threadIdx.x; n < N; n += blockDim.x) out[(long long)r * out_ld + n] = 0.f;
    }
}

// ------------------------------------------------------------------ host side
static int g_sm_count[64];
int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 132;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 132;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

template <int FMT, int EPI>
static int launch_one(const SkinnyArgs& a, int grid, size_t smem, cudaStream_t stream) {
    static bool attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_kernel<FMT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    skinny_kernel<FMT, EPI><<<grid, SK_THREADS, smem, stream>>>(a);
    B200_CHECK_LAUNCH();
    return 0;
}

template <int FMT>
static int launch_fmt(const SkinnyArgs& a, int epi, int grid, size_t smem, cudaStream_t stream) {
    switch (epi) {
        case SK_EPI_STORE_F32: return launch_one<FMT, SK_EPI_STORE_F32>(a, grid, smem, stream);
        case SK_EPI_ATOMIC_F32: return launch_one<FMT, SK_EPI_ATOMIC_F32>(a, grid, smem, stream);
        case SK_EPI_SWIGLU: return launch_one<FMT, SK_EPI_SWIGLU>(a, grid, smem, stream);
        case SK_EPI_STORE_BF16: return launch_one<FMT, SK_EPI_STORE_BF16>(a, grid, smem, stream);
    }
    return ERR_UNSUPPORTED;
}

int skinny_check(const SkinnyArgs& a, int fmt, int epi) {
    if (!a.w || !a.s || !a.x || !a.out) return ERR_BAD_ARG;
    if (!a.work && (a.n_work || a.dense_rows <= 0)) return ERR_BAD_ARG;
    const bool fp4 = fmt == SK_FMT_FP4_E8M0 || fmt == SK_FMT_FP4_BF16S;
    if (a.K <= 0 || a.N <= 0 || a.K % (fp4 ? 128 : 64) || a.N % 16) return ERR_BAD_SHAPE;
    if ((size_t)a.K * 16 + SK_RED_BYTES > 200 * 1024) return ERR_BAD_SHAPE;
    if (epi == SK_EPI_SWIGLU && (a.inter <= 0 || a.inter % 32 || a.N != 2 * a.inter)) return ERR_BAD_SHAPE;
    if (((uintptr_t)a.w & 15) || (a.w_estride & 15) || ((uintptr_t)a.x & 15) || (a.x_ld & 7)) return ERR_BAD_ALIGN;
    if (fmt == SK_FMT_FP4_E8M0 && (((uintptr_t)a.s & 3) || (a.s_rstride & 3) || (a.s_estride & 3))) return ERR_BAD_ALIGN;
    if (fmt == SK_FMT_FP8_F32B && (((uintptr_t)a.s & 3) || (a.s_rstride & 3))) return ERR_BAD_ALIGN;
    if (fmt == SK_FMT_FP4_BF16S && (((uintptr_t)a.s & 1) || (a.s_rstride & 1) || (a.s_estride & 1))) return ERR_BAD_ALIGN;
    return 0;
}

int skinny_launch(const SkinnyArgs& a, int fmt, int epi, cudaStream_t stream) {
    int rc = skinny_check(a, fmt, epi);
    if (rc) return rc;
    const size_t smem = (size_t)a.K * 16 + SK_RED_BYTES;
    const int grid = sm_count();
    switch (fmt) {
        case SK_FMT_FP4_E8M0: return launch_fmt<SK_FMT_FP4_E8M0>(a, epi, grid, smem, stream);
        case SK_FMT_FP4_BF16S: return launch_fmt<SK_FMT_FP4_BF16S>(a, epi, grid, smem, stream);
        case SK_FMT_FP8_E8M0: return launch_fmt<SK_FMT_FP8_E8M0>(a, epi, grid, smem, stream);
        case SK_FMT_FP8_F32B: return launch_fmt<SK_FMT_FP8_F32B>(a, epi, grid, smem, stream);
    }
    return ERR_UNSUPPORTED;
}

int skinny_plan(const int* grp_expert, const int* grp_start, const int* grp_count, int G, int n_pairs, int shard_start, int shard_n, int4* work,
                int* n_work, int max_work, cudaStream_t stream) {
    skinny_plan_kernel<<<1, 1024, 0, stream>>>(grp_expert, grp_start, grp_count, G, n_pairs, shard_start, shard_n, work, n_work, max_work);
    B200_CHECK_LAUNCH();
    return 0;
}

int skinny_zero_foreign(const int* grp_expert, const int* grp_start, const int* grp_count, int G, int n_pairs, int shard_start, int shard_n,
                        float* out, long long out_ld, int N, cudaStream_t stream) {
    int grid = G < 1024 ? (G > 0 ? G : 1) : 1024;
    skinny_zero_foreign_kernel<<<grid, 256, 0, stream>>>(grp_expert, grp_start, grp_count, G, n_pairs, shard_start, shard_n, out, out_ld, N);
    B200_CHECK_LAUNCH();
    return 0;
}

}  // namespace b200
