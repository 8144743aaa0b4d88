// Weight-streaming grouped "skinny" GEMM for decode: out[pair, n] = sum_k x[tok(pair), k] * W[expert][n, k] for groups
// of at most 8 tokens per expert (larger groups are cut into 8-token works that re-read the expert).
//
// Every weight byte is read once per work: one producer thread streams 32-row x 128-byte boxes of the weight matrix through a
// shared-memory ring with tensor-map bulk copies (128-byte swizzle) counted on mbarriers; the consumer warps fetch fragments with
// ldmatrix.x4, dequantise the 32-bit words in registers to packed bf16 with the block scale folded into the exponent, and contract
// them against the (<= 8) token columns with warp-level 16x8x16 tensor-core tiles that accumulate in fp32.  The K splits of a CTA
// are summed through shared memory.  Activations of the work's tokens sit in shared memory in the fragment order of the tile,
// pre-scaled by 2^ACT_SHIFT.  The dequantisation arithmetic, not HBM, bounds the FP4 form (about a quarter of the copy bandwidth);
// it is the engine for activations or scale formats the block-scaled tensor-core kernels (mxgemm.cu, wmgemm.cu) do not take.
//
// Replaces, for the sm_100a build, the reference's sm_80 kernels fp4_gemv_pairs (dsv41/cuda/fp4_gemv.cu:15),
// fp4_gemv_m1 (dsv41/cuda/fp4_gemv_m1.cu:57), fp4_gemm_tc8/16 (dsv41/cuda/fp4_tc.cu:52), fp8_gemv_m1
// (dsv41/cuda/fp8_gemv_m1.cu:55) and fp8_gemm_tc8/16 (dsv41/cuda/fp8_tc.cu:53) with one kernel template.
#include "common.cuh"
#include "skinny.cuh"
#include "tma.cuh"

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

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SK_CONSUMER_THREADS) : "memory"); }

// Device-visible error word: a wait that ran out of time records where it gave up instead of spinning forever.
__device__ int g_skinny_error = 0;

// ------------------------------------------------------------------ activation tile
// Shared-memory activation tile of one work (<= 8 token columns), in the register order of the tensor-core tile: 16-byte
// unit u = cu*32 + lane (lane = g*4 + t: token column g, quad lane t).  FP4: cu = k/32 (one 16-byte weight chunk of a row),
// the unit holds x[k0 + {0,4,1,5,2,6,3,7}], k0 = 32 cu + 8 t, matching the code pairs (j, j+4) of the lane's weight word.
// FP8: cu = k/32 covers the two 16-byte chunks 2 cu and 2 cu + 1; for each the unit holds x[kb + P(4t + {0,2,1,3})] with P
// the byte order of the weight container.  A warp reads 32 consecutive units: no bank conflicts.  Values are pre-scaled by
// 2^ACT_SHIFT.
template <int FMT>
__device__ void fill_act_tile(uint4* xs, const SkinnyArgs& a, int first, int ntok, int tid) {
    constexpr bool FP4 = FmtTraits<FMT>::FP4;
    const int K = a.K;
    const float up = u32_as_f32((uint32_t)(127 + ACT_SHIFT) << 23);
    for (int u = tid; u < K; u += SK_CONSUMER_THREADS) {
        const int t = u & 3, g = (u >> 2) & 7, cu = u >> 5;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < ntok) {
            const int pair = first + g;
            const long row = a.pair_tok ? a.pair_tok[pair] : pair;
            const __nv_bfloat16* xr = a.x + row * a.x_ld;
            float f[8];
            if (FP4) {
                const int k0 = cu * 32 + t * 8;
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
                f[0] = e[0]; f[1] = e[4]; f[2] = e[1]; f[3] = e[5]; f[4] = e[2]; f[5] = e[6]; f[6] = e[3]; f[7] = e[7];
            } else {
#pragma unroll
                for (int sl = 0; sl < 8; ++sl) {
                    const int kb = (2 * cu + (sl >> 2)) * 16;
                    const int q = ((sl & 1) << 1) | ((sl >> 1) & 1);  // slot order 0,2,1,3 within the lane's word
                    const int p = 4 * t + q;
                    f[sl] = __bfloat162float(xr[kb + (a.w_permk ? PERM_K16[p] : p)]);
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
// Work decomposition.  item = 64 weight rows of one work (SWIGLU epilogue: 32 gate rows + the 32 matching up rows).
// The rows of an item are streamed in stages of 64 rows x 512 bytes: a producer thread issues eight TMA box loads
// (32 rows x 128 bytes, 128-byte swizzle) per stage into a shared-memory ring and the bytes are counted on an mbarrier.
// 16 consumer warps = 2 row halves x 8 slices of 64 bytes; per 16-byte chunk column a warp fetches its 32 rows with one
// ldmatrix.x4 (conflict-free on the swizzled tile), dequantises the 32-bit words in registers and issues four
// tensor-core tiles against the activation columns.
struct ItemDesc {
    int wk, it;        // work index, item index within the work
    int expert, first, ntok;
    int row0a, row0b;  // first weight row of each 32-row half
};

template <int FMT, int EPI>
__global__ void __launch_bounds__(SK_THREADS, 1) skinny_kernel(const SkinnyArgs a, const __grid_constant__ CUtensorMap tmap) {
    using T = FmtTraits<FMT>;
    constexpr bool FP4 = T::FP4;
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    const int K = a.K, N = a.N;
    const int n_stages = a.n_stages;
    // the swizzled boxes need 1024-byte alignment: round the dynamic window up (the launch reserves the slack)
    uint8_t* ring = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);         // n_stages x 32 KB
    uint4* xs = reinterpret_cast<uint4*>(ring + (size_t)n_stages * SK_STAGE_BYTES);      // K units of 16 B
    float* red = reinterpret_cast<float*>(xs + K);                                       // [8 kq][64 rows][8 cols]
    __shared__ __align__(8) unsigned long long bars[2 * SK_MAX_STAGES];                  // full[s], empty[s]
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const long wrow_bytes = FP4 ? (K >> 1) : K;
    // Narrow items (a.rows32, never with the SwiGLU epilogue): 32 weight rows x 1024 bytes per stage instead of 64 x 512, the 16 warps
    // are 16 slices of one row half.  Twice as many items for the same matrix: a single GEMV of 4096 rows is 128 items, not 64, for
    // 148 SMs.
    const bool r32 = EPI != SK_EPI_SWIGLU && a.rows32 != 0;
    const int item_rows = r32 ? 32 : SK_ROWS, stage_row_bytes = r32 ? 2 * SK_STAGE_ROW_BYTES : SK_STAGE_ROW_BYTES, n_slices = r32 ? 16 : 8;
    const int nst = (int)((wrow_bytes + stage_row_bytes - 1) / stage_row_bytes);        // stages per item
    const int n_units = K >> 5;                                                         // activation units per token column
    const int ipw = (EPI == SK_EPI_SWIGLU) ? (a.inter >> 5) : ((N + item_rows - 1) / item_rows);
    // a launch may be tied to a device-side condition (see run_if in skinny.cuh): when it does not hold the kernel has nothing to do
    const bool skip = a.run_if && ((*a.run_if != 0) != (a.run_if_nonzero != 0));
    const int n_work = skip ? 0 : (a.n_work ? *a.n_work : a.n_work_host);
    const long total = (long)n_work * ipw;
    const long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[SK_MAX_STAGES + s]), SK_CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (lo >= hi) return;

    auto get_work = [&](int wk) -> int4 {
        if (a.work) return __ldg(a.work + wk);
        const int rem = a.dense_rows - wk * SK_TOK;  // dense mode: work wk = rows [8 wk, 8 wk + 8) of x against expert 0
        return make_int4(0, wk * SK_TOK, rem < SK_TOK ? rem : SK_TOK, 0);
    };
    auto make_desc = [&](int wk, int it) -> ItemDesc {
        ItemDesc d;
        d.wk = wk; d.it = it;
        const int4 w = get_work(wk);
        d.expert = w.x; d.first = w.y; d.ntok = w.z;
        if (EPI == SK_EPI_SWIGLU) { d.row0a = it * 32; d.row0b = a.inter + it * 32; }
        else { d.row0a = it * item_rows; d.row0b = it * item_rows + 32; }
        return d;
    };
    auto next_desc = [&](const ItemDesc& d) -> ItemDesc {
        int it = d.it + 1, wk = d.wk;
        if (it == ipw) { it = 0; ++wk; }
        return make_desc(wk, it);
    };
    const int wk_lo = (int)(lo / ipw), it_lo = (int)(lo - (long)wk_lo * ipw);

    if (warp == SK_CONSUMER_WARPS) {
        // ------------------------------------------------ producer: one thread, eight box loads per stage
        if (lane != 0) return;
        tma_prefetch_desc(&tmap);
        ItemDesc d = make_desc(wk_lo, it_lo);
        uint32_t n = 0;
        for (long item = lo; item < hi; ++item) {
            for (int st = 0; st < nst; ++st, ++n) {
                const uint32_t s = n % n_stages, ph = (n / n_stages) & 1;
                const uint32_t full = smem_u32(&bars[s]), empty = smem_u32(&bars[SK_MAX_STAGES + s]);
                if (!mbar_wait(empty, ph ^ 1, &abort_flag, &g_skinny_error, 1)) break;
                mbar_expect_tx(full, SK_STAGE_BYTES);
                const uint32_t dst = smem_u32(ring + (size_t)s * SK_STAGE_BYTES);
#pragma unroll
                for (int sl = 0; sl < 4; ++sl) {  // stage layout [row half][128-byte slab][32 rows][128 B]; narrow items: [slab 0..7][32 rows][128 B]
                    const int x = st * stage_row_bytes + sl * 128;
                    tma_load_3d(dst + sl * 4096, &tmap, x, d.row0a, d.expert, full);
                    if (r32) tma_load_3d(dst + 16384 + sl * 4096, &tmap, x + 512, d.row0a, d.expert, full);
                    else tma_load_3d(dst + 16384 + sl * 4096, &tmap, x, d.row0b, d.expert, full);
                }
            }
            if (abort_flag) break;
            if (item + 1 < hi) d = next_desc(d);
        }
        // leave only when every load this thread issued has landed (bounded wait on the last use of each ring slot)
        for (int k = 0; k < n_stages && k < (int)n; ++k) {
            const uint32_t m = n - 1 - k;
            const uint32_t s = m % n_stages, ph = (m / n_stages) & 1;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_test(smem_u32(&bars[s]), ph)) {
                if (global_timer_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(&g_skinny_error, 0, 3); break; }
            }
        }
        return;
    }

    // ---------------------------------------------------- consumer warps
    const int rh = r32 ? 0 : (warp & 1), kq = r32 ? warp : (warp >> 1);  // row half (32 rows), 64-byte slice of every stage row
    ItemDesc d = make_desc(wk_lo, it_lo);
    ItemDesc dn = d;
    auto scale_ptr = [&](const ItemDesc& q, int j) -> const uint8_t* {  // scale row of weight row g + 8 j of this warp's half
        const uint8_t* sb = a.s + (long long)q.expert * a.s_estride;
        const int r = min((rh ? q.row0b : q.row0a) + g + 8 * j, N - 1);
        if (FP4) return sb + (long)r * a.s_rstride;
        if (FMT == SK_FMT_FP8_E8M0) return sb + (long)(r >> 5) * a.s_rstride;
        return sb + (long)(r >> 7) * a.s_rstride;
    };
    // scale bits of this warp's slice of stage st.  FP4: k = 1024 st + 128 kq + [0, 128) = scale groups 4 c .. 4 c + 3 of the
    // row, c = 8 st + kq (one byte or bf16 each).  FP8: k = 512 st + 64 kq + [0, 64) = groups 2 c, 2 c + 1 (E8M0 per 32 k) or the
    // fp32 of block c >> 1 (per 128 k).
    auto load_scales = [&](const ItemDesc& q, int st, uint32_t (&sc)[4], uint32_t (&sc2)[4]) {
        const int c = st * n_slices + kq;
        if (c * (FP4 ? 128 : 64) >= K) { sc[0] = sc[1] = sc[2] = sc[3] = 0; sc2[0] = sc2[1] = sc2[2] = sc2[3] = 0; return; }
        if (FMT == SK_FMT_FP4_E8M0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[j] = ldg_stream4(scale_ptr(q, j) + 4 * c);
        } else if (FMT == SK_FMT_FP4_BF16S) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint2 v = *reinterpret_cast<const uint2*>(scale_ptr(q, j) + 8 * c);
                sc[j] = v.x;
                sc2[j] = v.y;
            }
        } else if (FMT == SK_FMT_FP8_E8M0) {
            const uint8_t* sp = scale_ptr(q, 0) + 2 * c;
            sc[0] = (uint32_t)sp[0] | ((uint32_t)sp[1] << 8);
        } else {
            sc[0] = ldg_stream4(scale_ptr(q, 0) + 4 * (c >> 1));
        }
    };

    uint32_t sc_cur[4], sc_nxt[4], sc2_cur[4] = {0, 0, 0, 0}, sc2_nxt[4] = {0, 0, 0, 0};
    load_scales(d, 0, sc_cur, sc2_cur);
    uint32_t n = 0;
    int cur_wk = -1;
    bool first_item = true;
    // ldmatrix row address of this lane inside a 32-row box: row l at l*128, 16-byte chunk cc stored at chunk cc ^ (l & 7)
    const uint32_t lm_row = (uint32_t)(rh * 16384 + (kq >> 1) * 4096 + lane * 128);
    const uint32_t lm_x = (uint32_t)(lane & 7);
    for (long item = lo; item < hi; ++item) {
        if (d.wk != cur_wk) {  // new work: the token columns change (every warp is past the previous item's compute)
            if (!first_item) consumer_sync();
            fill_act_tile<FMT>(xs, a, d.first, d.ntok, tid);
            consumer_sync();
            cur_wk = d.wk;
        }
        const bool has_next = item + 1 < hi;
        if (has_next) dn = next_desc(d);
        float acc[2][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[0][j] = acc[1][j] = 0.f;
        const bool bcol = g < d.ntok;
        for (int st = 0; st < nst; ++st, ++n) {
            const uint32_t s = n % n_stages, ph = (n / n_stages) & 1;
            // scales of the next stage (possibly of the next item) travel while this stage is computed
            if (st + 1 < nst) load_scales(d, st + 1, sc_nxt, sc2_nxt);
            else if (has_next) load_scales(dn, 0, sc_nxt, sc2_nxt);
            const bool ready = mbar_wait(smem_u32(&bars[s]), ph, &abort_flag, &g_skinny_error, 2);
            const int c = st * n_slices + kq;
            if (ready) {
                const uint32_t box = smem_u32(ring + (size_t)s * SK_STAGE_BYTES) + lm_row;
                if (FP4) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {  // chunk column i of the slice = scale group 4 c + i
                        const int cu = 4 * c + i;
                        uint32_t w[4];
                        ldmatrix_x4(box + ((((kq & 1) * 4 + i) ^ lm_x) << 4), w);
                        uint4 bv = make_uint4(0, 0, 0, 0);
                        if (bcol && cu < n_units) bv = lds128(xs + (cu * 32 + lane));
                        uint32_t mult[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (FMT == SK_FMT_FP4_E8M0) {
                                // both halves = 2^(s - 127) * 2^126 * 2^-ACT_SHIFT: exponent field s + 94.  Scale byte 0 needs no
                                // special case: the product with a code (<= 6 * 2^-126) underflows to zero in bf16.
                                mult[j] = __byte_perm(sc_cur[j], 0, 0x4440 | i) * 0x00800080u + bf16x2_pow2(126 - ACT_SHIFT);
                            } else {
                                const uint32_t raw = ((i & 2) ? sc2_cur[j] : sc_cur[j]) >> ((i & 1) * 16) & 0xFFFFu;
                                const float up = u32_as_f32((uint32_t)(127 + 126 - ACT_SHIFT) << 23);
                                const uint32_t h0 = f32_to_bf16_bits(bf16_bits_to_f32(raw) * up);
                                mult[j] = h0 | (h0 << 16);
                            }
                        }
                        uint32_t p0[4], p1[4], p2[4], p3[4];
                        dequant_fp4_word(w[0], mult[0], p0);
                        dequant_fp4_word(w[1], mult[1], p1);
                        dequant_fp4_word(w[2], mult[2], p2);
                        dequant_fp4_word(w[3], mult[3], p3);
                        mma_bf16_16816(acc[0], p0[0], p1[0], p0[1], p1[1], bv.x, bv.y);
                        mma_bf16_16816(acc[0], p0[2], p1[2], p0[3], p1[3], bv.z, bv.w);
                        mma_bf16_16816(acc[1], p2[0], p3[0], p2[1], p3[1], bv.x, bv.y);
                        mma_bf16_16816(acc[1], p2[2], p3[2], p2[3], p3[3], bv.z, bv.w);
                    }
                } else {
                    float blk[2][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) blk[0][j] = blk[1][j] = 0.f;
                    float (&d0)[4] = (FMT == SK_FMT_FP8_F32B) ? blk[0] : acc[0];
                    float (&d1)[4] = (FMT == SK_FMT_FP8_F32B) ? blk[1] : acc[1];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {  // 32-k scale group h of the slice = activation unit 2 c + h
                        const int cu = 2 * c + h;
                        uint32_t m;
                        if (FMT == SK_FMT_FP8_E8M0) {
                            // 2^(s - 127) * 2^120 * 2^-ACT_SHIFT: exponent field s + 88 (byte 0 underflows to zero like above)
                            m = __byte_perm(sc_cur[0], 0, 0x4440 | h) * 0x00800080u + bf16x2_pow2(120 - ACT_SHIFT);
                        } else {
                            m = bf16x2_pow2(127 + 120 - ACT_SHIFT);
                        }
                        uint4 bv = make_uint4(0, 0, 0, 0);
                        if (bcol && cu < n_units) bv = lds128(xs + (cu * 32 + lane));
#pragma unroll
                        for (int e = 0; e < 2; ++e) {  // 16-byte chunk column 2 h + e of the slice
                            uint32_t w[4];
                            ldmatrix_x4(box + ((((kq & 1) * 4 + 2 * h + e) ^ lm_x) << 4), w);
                            uint32_t p0[2], p1[2], p2[2], p3[2];
                            dequant_fp8_word(w[0], m, p0);
                            dequant_fp8_word(w[1], m, p1);
                            dequant_fp8_word(w[2], m, p2);
                            dequant_fp8_word(w[3], m, p3);
                            const uint32_t b0 = e ? bv.z : bv.x, b1 = e ? bv.w : bv.y;
                            mma_bf16_16816(d0, p0[0], p1[0], p0[1], p1[1], b0, b1);
                            mma_bf16_16816(d1, p2[0], p3[0], p2[1], p3[1], b0, b1);
                        }
                    }
                    if (FMT == SK_FMT_FP8_F32B) {
                        const float scl = u32_as_f32(sc_cur[0]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) { acc[0][j] = fmaf(scl, blk[0][j], acc[0][j]); acc[1][j] = fmaf(scl, blk[1][j], acc[1][j]); }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[SK_MAX_STAGES + s]));
#pragma unroll
            for (int j = 0; j < 4; ++j) { sc_cur[j] = sc_nxt[j]; sc2_cur[j] = sc2_nxt[j]; }
        }
        // partial sums of the 8 slices -> shared memory (after every warp has finished reading the previous item's sums)
        if (!first_item) consumer_sync();
        first_item = false;
        float* rp = red + (kq * item_rows + rh * 32) * 8;  // [slice][row of the item][token column]
        *reinterpret_cast<float2*>(rp + g * 8 + 2 * t) = make_float2(acc[0][0], acc[0][1]);
        *reinterpret_cast<float2*>(rp + (g + 8) * 8 + 2 * t) = make_float2(acc[0][2], acc[0][3]);
        *reinterpret_cast<float2*>(rp + (g + 16) * 8 + 2 * t) = make_float2(acc[1][0], acc[1][1]);
        *reinterpret_cast<float2*>(rp + (g + 24) * 8 + 2 * t) = make_float2(acc[1][2], acc[1][3]);
        consumer_sync();
        const int ntok = d.ntok, first = d.first, it = d.it;
        if (EPI == SK_EPI_SWIGLU) {
            // warp = token column, lane = column of the 32-wide quantisation group (dsv41/fused.py:285-306):
            // half 0 of the item holds the gate rows, half 1 the up rows
            if (warp < ntok) {
                float gt = 0.f, upv = 0.f;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    gt += red[(q * 64 + lane) * 8 + warp];
                    upv += red[(q * 64 + 32 + lane) * 8 + warp];
                }
                if (a.round_gu_bf16) { gt = round_bf16(gt); upv = round_bf16(upv); }
                const int pair = first + warp;
                const float h = swiglu_bf16(gt, upv, a.pair_w ? a.pair_w[pair] : 1.f, a.limit);
                const float s = fp8_group_scale(warp_max(fabsf(h)));
                const long orow = a.pair_out ? a.pair_out[pair] : pair;
                reinterpret_cast<__nv_bfloat16*>(a.out)[orow * a.out_ld + it * 32 + lane] = __float2bfloat16_rn(fp8_fake_quant_value(h, s));
            }
        } else {
            const int col = r32 ? (tid >> 5) : (tid >> 6), rr = r32 ? (tid & 31) : (tid & 63);
            const int nrow = it * item_rows + rr;
            if (col < SK_TOK && col < ntok && nrow < N) {
                float v = 0.f;
                if (r32) {
#pragma unroll
                    for (int q = 0; q < 16; ++q) v += red[(q * 32 + rr) * 8 + col];
                } else {
#pragma unroll
                    for (int q = 0; q < 8; ++q) v += red[(q * 64 + rr) * 8 + col];
                }
                const int pair = first + col;
                if (a.pair_w) v *= a.pair_w[pair];
                const long orow = a.pair_out ? a.pair_out[pair] : pair;
                if (EPI == SK_EPI_STORE_F32) reinterpret_cast<float*>(a.out)[orow * a.out_ld + nrow] = v;
                else if (EPI == SK_EPI_ATOMIC_F32) atomicAdd(reinterpret_cast<float*>(a.out) + orow * a.out_ld + nrow, v);
                else reinterpret_cast<__nv_bfloat16*>(a.out)[orow * a.out_ld + nrow] = __float2bfloat16_rn(v);
            }
        }
        if (has_next) d = dn;
    }
}

// ------------------------------------------------------------------ work list
// One block.  Groups g (expert grp_expert[g], pairs grp_start[g] .. grp_start[g+1]-1) that belong to this shard are cut
// into works of at most 8 pairs: work = {local expert, first pair, n pairs, group}.  Groups of other shards (and padded
// groups, expert -1) get their output rows zeroed when zero_out is set, as dsv41/cuda/fp4_tc.cu:66-72 does.
__global__ void __launch_bounds__(1024) skinny_plan_kernel(const int* __restrict__ grp_expert, const int* __restrict__ grp_start,
                                                           const int* __restrict__ grp_count, int G, int n_pairs, int shard_start, int shard_n,
                                                           int4* __restrict__ work, int* __restrict__ n_work, int max_work, int tpw) {
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
            if (e >= 0 && e < shard_n && cnt > 0 && s >= 0) nsub = (cnt + tpw - 1) / tpw;
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
            const int rem = cnt - i * tpw;
            if (off + i < max_work) work[off + i] = make_int4(e, s + i * tpw, rem < tpw ? rem : tpw, gi);
        }
        __syncthreads();
        if (tid == 0) running += tot;
        __syncthreads();
    }
    if (tid == 0) {
        *n_work = running < max_work ? running : max_work;
        if (running > max_work) atomicCAS(&g_skinny_error, 0, 91);  // the groups need more works than the list holds: results are incomplete
    }
}

// Zeroes the output rows of the pairs of foreign groups.  Pair p writes row pair_out[p] (p itself without pair_out), so that is the
// row cleared here too.
__global__ void skinny_zero_foreign_kernel(const int* __restrict__ grp_expert, const int* __restrict__ grp_start, const int* __restrict__ grp_count,
                                           int G, int n_pairs, int shard_start, int shard_n, const int* __restrict__ pair_out, float* __restrict__ out,
                                           long long out_ld, int N) {
    for (int gi = blockIdx.x; gi < G; gi += gridDim.x) {
        const int e = grp_expert[gi] - shard_start;
        if (e >= 0 && e < shard_n) continue;
        int s = grp_start[gi], en = grp_count ? s + grp_count[gi] : grp_start[gi + 1];
        if (en > n_pairs) en = n_pairs;
        if (s < 0) s = 0;
        for (int r = s; r < en; ++r) {
            const long long row = pair_out ? pair_out[r] : r;
            for (int n = threadIdx.x; n < N; n += blockDim.x) out[row * out_ld + n] = 0.f;
        }
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
static int launch_one(const SkinnyArgs& a, const CUtensorMap& tm, int grid, size_t smem, cudaStream_t stream) {
    static bool attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_kernel<FMT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_LIMIT);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    skinny_kernel<FMT, EPI><<<grid, SK_THREADS, smem, stream>>>(a, tm);
    B200_CHECK_LAUNCH();
    return 0;
}

template <int FMT>
static int launch_fmt(const SkinnyArgs& a, const CUtensorMap& tm, int epi, int grid, size_t smem, cudaStream_t stream) {
    switch (epi) {
        case SK_EPI_STORE_F32: return launch_one<FMT, SK_EPI_STORE_F32>(a, tm, grid, smem, stream);
        case SK_EPI_ATOMIC_F32: return launch_one<FMT, SK_EPI_ATOMIC_F32>(a, tm, grid, smem, stream);
        case SK_EPI_SWIGLU: return launch_one<FMT, SK_EPI_SWIGLU>(a, tm, grid, smem, stream);
        case SK_EPI_STORE_BF16: return launch_one<FMT, SK_EPI_STORE_BF16>(a, tm, grid, smem, stream);
    }
    return ERR_UNSUPPORTED;
}

int skinny_check(const SkinnyArgs& a, int fmt, int epi) {
    if (!a.w || !a.s || !a.x || !a.out) return ERR_BAD_ARG;
    if (!a.work && (a.n_work || a.dense_rows <= 0)) return ERR_BAD_ARG;
    const bool fp4 = fmt == SK_FMT_FP4_E8M0 || fmt == SK_FMT_FP4_BF16S;
    if (a.K <= 0 || a.N <= 0 || a.K % (fp4 ? 128 : 64) || a.N % 16) return ERR_BAD_SHAPE;
    if ((size_t)a.K * 16 + SK_RED_BYTES + 1024 + 2 * SK_STAGE_BYTES > (size_t)SK_SMEM_LIMIT) return ERR_BAD_SHAPE;  // K <= 9088
    if (epi == SK_EPI_SWIGLU && (a.inter <= 0 || a.inter % 32 || a.N != 2 * a.inter)) return ERR_BAD_SHAPE;
    if (((uintptr_t)a.w & 15) || (a.w_estride & 15) || ((uintptr_t)a.x & 15) || (a.x_ld & 7)) return ERR_BAD_ALIGN;
    if (fmt == SK_FMT_FP4_E8M0 && (((uintptr_t)a.s & 3) || (a.s_rstride & 3) || (a.s_estride & 3))) return ERR_BAD_ALIGN;
    if (fmt == SK_FMT_FP8_F32B && (((uintptr_t)a.s & 3) || (a.s_rstride & 3))) return ERR_BAD_ALIGN;
    if (fmt == SK_FMT_FP4_BF16S && (((uintptr_t)a.s & 7) || (a.s_rstride & 7) || (a.s_estride & 7))) return ERR_BAD_ALIGN;
    return 0;
}

int skinny_launch(const SkinnyArgs& a_in, int fmt, int epi, cudaStream_t stream) {
    int rc = skinny_check(a_in, fmt, epi);
    if (rc) return rc;
    SkinnyArgs a = a_in;
    const size_t fixed = (size_t)a.K * 16 + SK_RED_BYTES + 1024;
    int stages = (int)(((size_t)SK_SMEM_LIMIT - fixed) / SK_STAGE_BYTES);
    if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
    a.n_stages = stages;
    const size_t smem = fixed + (size_t)stages * SK_STAGE_BYTES;
    const int grid = sm_count();
    // 32-row items when they lower the largest share of weight rows a CTA gets (known on the host only when the work count is): a
    // GEMV of 4096 rows is 64 items of 64 rows for 148 SMs, one of 12288 rows is 192 (two for some CTAs, one for the others)
    a.rows32 = 0;
    if (epi != SK_EPI_SWIGLU && !a.n_work) {
        const long works = a.work ? a.n_work_host : (a.dense_rows + SK_TOK - 1) / SK_TOK;
        const long i64 = works * ((a.N + 63) / 64), i32 = works * ((a.N + 31) / 32);
        if ((i32 + grid - 1) / grid < 2 * ((i64 + grid - 1) / grid)) a.rows32 = 1;
    }
    const bool fp4 = fmt == SK_FMT_FP4_E8M0 || fmt == SK_FMT_FP4_BF16S;
    const uint64_t row_bytes = fp4 ? (uint64_t)a.K / 2 : (uint64_t)a.K;
    alignas(64) CUtensorMap tm;
    rc = make_weight_tmap(&tm, a.w, row_bytes, (uint64_t)a.N, (uint64_t)(a.n_experts > 0 ? a.n_experts : 1), (uint64_t)a.w_estride, 32);
    if (rc) return rc;
    switch (fmt) {
        case SK_FMT_FP4_E8M0: return launch_fmt<SK_FMT_FP4_E8M0>(a, tm, epi, grid, smem, stream);
        case SK_FMT_FP4_BF16S: return launch_fmt<SK_FMT_FP4_BF16S>(a, tm, epi, grid, smem, stream);
        case SK_FMT_FP8_E8M0: return launch_fmt<SK_FMT_FP8_E8M0>(a, tm, epi, grid, smem, stream);
        case SK_FMT_FP8_F32B: return launch_fmt<SK_FMT_FP8_F32B>(a, tm, epi, grid, smem, stream);
    }
    return ERR_UNSUPPORTED;
}

// copies and clears the device error word of the streaming kernels (the caller has synchronised the stream)
int skinny_device_error(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_skinny_error, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v) {
        int z = 0;
        cudaMemcpyToSymbol(g_skinny_error, &z, sizeof(int));
    }
    *out = v;
    return 0;
}

int skinny_plan(const int* grp_expert, const int* grp_start, const int* grp_count, int G, int n_pairs, int shard_start, int shard_n, int4* work,
                int* n_work, int max_work, cudaStream_t stream, int tpw) {
    skinny_plan_kernel<<<1, 1024, 0, stream>>>(grp_expert, grp_start, grp_count, G, n_pairs, shard_start, shard_n, work, n_work, max_work, tpw);
    B200_CHECK_LAUNCH();
    return 0;
}

int skinny_zero_foreign(const int* grp_expert, const int* grp_start, const int* grp_count, int G, int n_pairs, int shard_start, int shard_n,
                        const int* pair_out, float* out, long long out_ld, int N, cudaStream_t stream) {
    int grid = G < 1024 ? (G > 0 ? G : 1) : 1024;
    skinny_zero_foreign_kernel<<<grid, 256, 0, stream>>>(grp_expert, grp_start, grp_count, G, n_pairs, shard_start, shard_n, pair_out, out, out_ld, N);
    B200_CHECK_LAUNCH();
    return 0;
}

}  // namespace b200
