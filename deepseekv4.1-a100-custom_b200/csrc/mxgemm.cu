// Grouped expert GEMM on the 5th-generation tensor cores with hardware block scaling:
//     D[weight row, token] = sum_k  W[row, k] * 2^(sw[row, k/32] - 127)  *  q[token, k] * 2^(sx[token, k/32] - 127)
// W = packed E2M1 (FP4) or e4m3, q = e4m3 activations (the FP8 fake-quantised values of dsv41/quant.py:46-54 kept in
// quantised form), both with one E8M0 scale byte per 32 k -- exactly the operand formats of
// tcgen05.mma.kind::mxf8f6f4.block_scale, so the weights go HBM -> TMA -> shared memory -> tensor core with no
// arithmetic on the way, and the accumulators live in tensor memory (TMEM) in fp32.
//
// The tokens of a work (<= 128) are the M side of the tile (accumulator lanes), up to 256 weight rows are the N side: a
// 128 x 256 x 32 MMA runs in about 137 clocks, less than the fixed cost of issuing it and of handing a pipeline stage over, so
// every instruction and every stage carries as many weight bytes as it can.  Warp roles of the persistent CTA:
//   warp 0      TMA producer: boxes of the weight tile(s) and of the activation rows into a shared-memory ring
//   warp 1      allocates TMEM; one thread copies the scale atoms into TMEM (tcgen05.cp) and issues the MMAs
//   warps 4-7, 12-15  epilogue: a thread owns one token (TMEM lane) and reads its accumulator row with tcgen05.ld; SwiGLU + FP8
//               quantisation or store; the two groups split the columns
//   warps 8-11  scale loaders: one thread per tile row builds the 32x4x4 scale atoms in shared memory
// Every wait is bounded; a wait that runs out of time records a code in a device error word and the CTA runs to its end.
//
// Replaces, on B200, the reference's grouped FP4 kernels (dsv41/moe_kernels.py:341-378 for prefill; dsv41/cuda/fp4_tc.cu,
// fp4_tcw.cu, expert_chain.cu for decode) when the activation is FP8-quantised, which it always is inside the MoE layer
// (dsv41/model.py:2040, dsv41/fused.py:297-306).
#include <cuda_fp8.h>

#include "common.cuh"
#include "mxgemm.cuh"
#include "tma.cuh"
#include "tc5.cuh"

namespace b200 {

__device__ int g_mx_error = 0;

// ------------------------------------------------------------------ the kernel
// Tile orientation: the tokens of a work are the M side of the tensor-core tile (128 accumulator lanes, of which the first
// `ntok` carry data), the weight rows are the N side (up to 256 per MMA: the fixed cost per instruction and per pipeline stage is
// what bounds the kernel, so every instruction carries as many weight bytes as possible).  D[token, weight row] lives in TMEM
// columns [0, N_w).
//   dual (SwiGLU epilogue): N_w = 2 * rows_w, columns [0, rows_w) = gate rows row0.., columns [rows_w, 2 rows_w) = up rows
//   single:                 N_w = rows_w consecutive rows
// One launch runs up to two problems that share K, the tile shape and the token count per work (the routed experts and the
// shared expert of one layer step): the (work, tile) items of problem 0 are followed by those of problem 1 in one flat list that
// is cut evenly over the CTAs, so the small second problem fills the tail of the first.
__global__ void __launch_bounds__(MX_THREADS, 1) mx_gemm_kernel(const MxArgs a, const __grid_constant__ CUtensorMap tm_w0,
                                                                 const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_w1,
                                                                 const __grid_constant__ CUtensorMap tm_x1) {
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long bars[3 * MX_MAX_STAGES + 4];  // full_ab[s], full_sf[s], empty[s], acc_full[2], acc_empty[2]
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = a.n_stages, KB = a.kb, nd = a.nd, rows_w = a.rows_a;
    const int NW = a.dual ? 2 * rows_w : rows_w;   // N of the MMA
    const int n_sfb = (NW + 127) >> 7;             // scale atoms of the weight side
    const int n_atoms = 1 + n_sfb;
    uint8_t* base = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    // stage layout: [kb] token boxes (nd x 128 B), then [kb] weight tiles (NW x 128 B; dual: gate rows then up rows)
    const uint32_t x_box = (uint32_t)nd * 128u, w_tile = (uint32_t)NW * 128u;
    const uint32_t stage_bytes = (uint32_t)KB * (x_box + w_tile);
    uint8_t* ring = base;
    uint8_t* sf_ring = base + (size_t)NS * stage_bytes;   // per stage: [kb][n_atoms] atoms of 512 B
    const uint32_t sf_stage_bytes = (uint32_t)(KB * n_atoms) * 512u;
    float* stg = reinterpret_cast<float*>(sf_ring + (size_t)NS * sf_stage_bytes);  // staging of small accumulator tiles: [32 tokens][MX_STG_LD]
    auto bar_full_ab = [&](int s) { return smem_u32(&bars[s]); };
    auto bar_full_sf = [&](int s) { return smem_u32(&bars[MX_MAX_STAGES + s]); };
    auto bar_empty = [&](int s) { return smem_u32(&bars[2 * MX_MAX_STAGES + s]); };
    auto bar_acc_full = [&](int b) { return smem_u32(&bars[3 * MX_MAX_STAGES + b]); };
    auto bar_acc_empty = [&](int b) { return smem_u32(&bars[3 * MX_MAX_STAGES + 2 + b]); };

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full_ab(s), 1);
            mbar_init(bar_full_sf(s), 4);     // one arrival per scale-loader warp
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full(b), 1);
            mbar_init(bar_acc_empty(b), 8);   // one arrival per epilogue warp
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_sh), MX_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    // everything above touched no global memory: from here on the kernel before this one in the stream must have completed
    pdl_wait();
    pdl_launch_dependents();
    const int kblocks = a.K >> 7;                       // 128-wide k blocks
    const int spi = (kblocks + KB - 1) / KB;            // stages per item
    // items per work and items in all of each problem
    const int ipw0 = ((a.dual ? a.inter : a.p[0].N) + rows_w - 1) / rows_w;
    const int ipw1 = a.n_prob > 1 ? ((a.dual ? a.inter : a.p[1].N) + rows_w - 1) / rows_w : 1;
    const long items0 = (long)(a.p[0].n_work ? *a.p[0].n_work : a.p[0].n_work_host) * ipw0;
    const long items1 = a.n_prob > 1 ? (long)(a.p[1].n_work ? *a.p[1].n_work : a.p[1].n_work_host) * ipw1 : 0;
    // a launch may be tied to a device-side condition (run_if in mxgemm.cuh): when it does not hold there are no items
    const bool skip = a.run_if && ((*a.run_if != 0) != (a.run_if_nonzero != 0));
    const long total = skip ? 0 : items0 + items1;
    const long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    const int n_acc = (2 * NW <= MX_ACC_COLS_MAX) ? 2 : 1;  // two accumulator buffers (epilogue overlaps the next item) when they fit
    const uint32_t sf_col0 = (uint32_t)(n_acc * NW);        // the scale columns follow the accumulators


    // position in the flat item list: problem, work, tile of the work; `w` = {local expert, first token row, tokens, -}
    struct ItemCur { long item; int pr, wk, it; int4 w; };
    auto get_work = [&](int pr, int wk) -> int4 {
        const MxProb& P = a.p[pr];
        if (P.work) return __ldg(P.work + wk);
        const int rem = P.dense_rows - wk * nd;
        return make_int4(0, wk * nd, rem < nd ? rem : nd, 0);
    };
    auto locate = [&](long item, bool fetch) -> ItemCur {
        ItemCur c;
        c.item = item;
        c.pr = item >= items0 ? 1 : 0;
        const long rel = c.pr ? item - items0 : item;
        const int ipw = c.pr ? ipw1 : ipw0;
        c.wk = (int)(rel / ipw);
        c.it = (int)(rel - (long)c.wk * ipw);
        c.w = (fetch && item < total) ? get_work(c.pr, c.wk) : make_int4(0, 0, 0, 0);
        return c;
    };
    auto next_item = [&](ItemCur& c, bool fetch) {
        ++c.item;
        if (c.item >= hi) return;
        if (c.pr == 0 && c.item == items0) {
            c.pr = 1; c.wk = 0; c.it = 0;
            if (fetch) c.w = get_work(1, 0);
            return;
        }
        if (++c.it == (c.pr ? ipw1 : ipw0)) {
            c.it = 0;
            ++c.wk;
            if (fetch) c.w = get_work(c.pr, c.wk);
        }
    };

    if (lo < hi) {
        if (warp == 0) {
            // ------------------------------------------------ TMA producer (one thread)
            if (lane == 0) {
                tma_prefetch_desc(&tm_w0);
                tma_prefetch_desc(&tm_x0);
                if (a.n_prob > 1) { tma_prefetch_desc(&tm_w1); tma_prefetch_desc(&tm_x1); }
                ItemCur c = locate(lo, true);
                uint32_t n = 0;
                for (; c.item < hi && !abort_flag; next_item(c, true)) {
                    const CUtensorMap* tw = c.pr ? &tm_w1 : &tm_w0;
                    const CUtensorMap* tx = c.pr ? &tm_x1 : &tm_x0;
                    // packed FP4 boxes count the bytes actually written
                    const uint32_t w_tx = a.p[c.pr].a_fmt == MX_A_E2M1 ? w_tile / 2 : w_tile;
                    const int row0 = c.it * rows_w;
                    for (int st = 0; st < spi; ++st, ++n) {
                        const uint32_t s = n % NS, ph = (n / NS) & 1;
                        if (!mbar_wait(bar_empty(s), ph ^ 1, &abort_flag, &g_mx_error, 11)) break;
                        const int kb0 = st * KB, nkb = min(KB, kblocks - kb0);
                        mbar_expect_tx(bar_full_ab(s), (uint32_t)nkb * (x_box + w_tx));
                        const uint32_t dst = smem_u32(ring + (size_t)s * stage_bytes);
                        for (int b = 0; b < nkb; ++b) {
                            const int kx = (kb0 + b) * 128;  // element coordinate along K (bytes for e4m3, 4-bit elements for E2M1)
                            const uint32_t wdst = dst + (uint32_t)KB * x_box + (uint32_t)b * w_tile;
                            // dual: the weight map is 4-D {k, row within a half, half, expert}: one box fetches the gate rows and,
                            // right behind them in shared memory, the up rows
                            if (a.dual) tma_load_4d(wdst, tw, kx, row0, 0, c.w.x, bar_full_ab(s));
                            else tma_load_3d(wdst, tw, kx, row0, c.w.x, bar_full_ab(s));
                            tma_load_2d(dst + (uint32_t)b * x_box, tx, kx, c.w.y, bar_full_ab(s));
                        }
                    }
                }
                // every load issued above must have landed before the CTA may exit
                for (int k = 0; k < NS && k < (int)n; ++k) {
                    const uint32_t m = n - 1 - k, s = m % NS, ph = (m / NS) & 1;
                    const unsigned long long t0 = global_timer_ns();
                    while (!mbar_test(bar_full_ab(s), ph)) {
                        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(&g_mx_error, 0, 13); break; }
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer (one thread): scale atoms -> TMEM (tcgen05.cp), then the MMAs
            if (lane == 0) {
                uint32_t n = 0, acc_it = 0;
                for (long item = lo; item < hi && !abort_flag; ++item, ++acc_it) {
                    const int b_fmt = a.p[item >= items0 ? 1 : 0].a_fmt;  // weight format (the B operand); the tokens (A operand) are e4m3
                    const uint32_t buf = acc_it % n_acc, aph = (acc_it / n_acc) & 1;
                    if (!mbar_wait(bar_acc_empty(buf), aph ^ 1, &abort_flag, &g_mx_error, 21)) break;
                    tc_fence_after();
                    const uint32_t d0 = tmem_base + buf * NW;
                    uint32_t accumulate = 0;
                    for (int st = 0; st < spi; ++st, ++n) {
                        const uint32_t s = n % NS, ph = (n / NS) & 1;
                        if (!mbar_wait(bar_full_sf(s), ph, &abort_flag, &g_mx_error, 22)) break;
                        if (!mbar_wait(bar_full_ab(s), ph, &abort_flag, &g_mx_error, 23)) break;
                        tc_fence_after();
                        const int kb0 = st * KB, nkb = min(KB, kblocks - kb0);
                        const uint32_t sbase = smem_u32(ring + (size_t)s * stage_bytes);
                        const uint32_t sfs = smem_u32(sf_ring + (size_t)s * sf_stage_bytes);
                        for (int b = 0; b < nkb; ++b) {
                            // scale atoms of this k block -> TMEM: [tokens][weights 0][weights 1], 4 columns each
                            const uint32_t sfcol = tmem_base + sf_col0 + (s * KB + b) * n_atoms * 4;
                            for (int q = 0; q < n_atoms; ++q) tc_cp_sf(sfcol + q * 4, desc_sf_atom(sfs + (uint32_t)(b * n_atoms + q) * 512u));
                            const uint64_t dx = desc_sw128(sbase + (uint32_t)b * x_box);
                            const uint64_t dw = desc_sw128(sbase + (uint32_t)KB * x_box + (uint32_t)b * w_tile);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {  // 4 MMAs of K = 32: operand descriptors advance by 32 bytes inside the swizzled row
                                tc_mma_mx(d0, dx + 2 * j, dw + 2 * j, mx_idesc(b_fmt, NW, j), sfcol, sfcol + 4, accumulate);
                                accumulate = 1;
                            }
                        }
                        tc_commit(bar_empty(s));  // the stage (and its scale atoms) may be refilled once these MMAs have read it
                    }
                    tc_commit(bar_acc_full(buf));
                }
            }
        } else if (warp >= 8 && warp < 12) {
            // ------------------------------------------------ scale loaders: thread r feeds token r and weight rows r, r + 128 of the tile.
            // The loads of stage n + PD are in flight while stage n is stored (software pipeline over the flat stage sequence).
            const int r = tid - 256;
            const uint32_t atom_off = (uint32_t)(r & 31) * 16u + (uint32_t)(r >> 5) * 4u;
            struct Cur {
                ItemCur c; int st;
                const uint8_t *s_0, *s_1, *s_x; bool brow, w0, w1;
            };
            auto wrow = [&](int row0, int col) -> int {  // weight row of tile column col
                if (a.dual) return col < rows_w ? row0 + col : a.inter + row0 + (col - rows_w);
                return row0 + col;
            };
            auto setup = [&](Cur& u) {
                const MxProb& P = a.p[u.c.pr];
                const int row0 = u.c.it * rows_w;
                const uint8_t* sbase = P.s + (long long)u.c.w.x * P.s_estride;
                u.w0 = r < NW;
                u.w1 = r + 128 < NW;
                const int ra = min(wrow(row0, u.w0 ? r : 0), P.N - 1), rb = min(wrow(row0, u.w1 ? r + 128 : 0), P.N - 1);
                u.s_0 = sbase + (long)(ra >> P.s_row_shift) * P.s_rstride;
                u.s_1 = sbase + (long)(rb >> P.s_row_shift) * P.s_rstride;
                u.brow = r < u.c.w.z;
                u.s_x = P.xsf + (long)(u.c.w.y + (u.brow ? r : 0)) * P.xsf_ld;
            };
            auto advance = [&](Cur& u) {
                if (++u.st < spi) return;
                u.st = 0;
                next_item(u.c, true);
                if (u.c.item < hi) setup(u);
            };
            constexpr int PD = 3;
            uint32_t q[PD][3][4];
            auto load = [&](const Cur& u, uint32_t (&v)[3][4]) {
                if (u.c.item >= hi) return;
                const int kb0 = u.st * KB, nkb = min(KB, kblocks - kb0);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (b >= nkb) break;
                    const int g0 = (kb0 + b) * 4;  // first 32-k group of the k block
                    v[0][b] = u.brow ? ldg_stream4(u.s_x + g0) : 0x7F7F7F7Fu;
                    v[1][b] = u.w0 ? ldg_stream4(u.s_0 + g0) : 0x7F7F7F7Fu;
                    v[2][b] = u.w1 ? ldg_stream4(u.s_1 + g0) : 0x7F7F7F7Fu;
                }
            };
            Cur use;
            use.c = locate(lo, true);
            use.st = 0;
            setup(use);
            Cur ld = use;
#pragma unroll
            for (int i = 0; i < PD; ++i) { load(ld, q[i]); advance(ld); }
            uint32_t n = 0;
            while (use.c.item < hi && !abort_flag) {
#pragma unroll
                for (int i = 0; i < PD; ++i) {
                    if (use.c.item >= hi) break;
                    const uint32_t s = n % NS, ph = (n / NS) & 1;
                    const int kb0 = use.st * KB, nkb = min(KB, kblocks - kb0);
                    if (!mbar_wait(bar_empty(s), ph ^ 1, &abort_flag, &g_mx_error, 31)) break;
                    uint8_t* sf = sf_ring + (size_t)s * sf_stage_bytes + atom_off;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        if (b >= nkb) break;
                        *reinterpret_cast<uint32_t*>(sf + (size_t)(b * n_atoms) * 512) = q[i][0][b];
                        *reinterpret_cast<uint32_t*>(sf + (size_t)(b * n_atoms + 1) * 512) = q[i][1][b];
                        if (n_sfb == 2) *reinterpret_cast<uint32_t*>(sf + (size_t)(b * n_atoms + 2) * 512) = q[i][2][b];
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full_sf(s));  // arrivals on one barrier serialise: one per warp, not one per thread
                    advance(use);
                    ++n;
                    load(ld, q[i]);
                    advance(ld);
                }
            }
        } else if (warp >= 4) {
            // ------------------------------------------------ epilogue: warps 4-7 and 12-15.  Warp q (mod 4) reads TMEM lanes
            // 32 q .. 32 q + 31 = tokens; the two groups split the weight-row columns.  A thread owns one token.
            const int q = warp & 3, egrp = warp >= 12 ? 1 : 0;
            const int t = q * 32 + lane;
            ItemCur c = locate(lo, true);
            uint32_t acc_it = 0;
            // No early exit from this loop: the eight warps meet at named barriers, so all of them walk the same item sequence;
            // once a wait has run out of time every later wait returns at once and the loop drains quickly.
            for (; c.item < hi; next_item(c, true), ++acc_it) {
                const MxProb& P = a.p[c.pr];
                const int4 w = c.w;
                const uint32_t buf = acc_it % n_acc, aph = (acc_it / n_acc) & 1;
                // the row's routing weight and output row are fetched before the wait for the accumulator, not after it
                const bool tok_on = t < w.z;
                const int prow = w.y + (tok_on ? t : 0);
                const float pw = (P.pair_w && tok_on) ? __ldg(P.pair_w + prow) : 1.f;
                const long orow = (P.pair_out && tok_on) ? (long)__ldg(P.pair_out + prow) : (long)prow;
                const bool ready = mbar_wait(bar_acc_full(buf), aph, &abort_flag, &g_mx_error, 41);
                tc_fence_after();
                const int row0 = c.it * rows_w;
                const bool warp_on = ready && q * 32 < w.z;  // warp-uniform: some token of this warp exists
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * NW;
                if (w.z <= a.stg_rows) {
                    // ---- few tokens: a thread per token would leave most lanes idle for the whole epilogue.  The two warps that can
                    // read TMEM lanes 0-31 copy the tile to shared memory, the accumulator is handed back to the MMA issuer at once,
                    // and all eight warps then work on (token, group of 32 columns) tasks with one column per lane.
                    epi_bar();  // the tasks of the previous small tile are done: the staging buffer may be overwritten
                    if (ready && q == 0) {
                        const int cbase = egrp * (NW / 2);
                        for (int c0 = 0; c0 < NW / 2; c0 += 16) {
                            uint32_t g[16];
                            tc_ld16(t0 + cbase + c0, g);
                            tc_wait_ld();
                            if (lane < a.stg_rows)  // the buffer holds stg_rows token rows
#pragma unroll
                                for (int cc = 0; cc < 16; ++cc) stg[lane * MX_STG_LD + cbase + c0 + cc] = __uint_as_float(g[cc]);
                        }
                    }
                    tc_fence_before();
                    epi_bar();  // the copy is visible to all epilogue warps
                    if (lane == 0) mbar_arrive(bar_acc_empty(buf));
                    const int ew = q + 4 * egrp;
                    if (ready && P.epi == MX_EPI_SWIGLU_Q8) {
                        const int ngrp = rows_w >> 5;
                        for (int task = ew; task < w.z * ngrp; task += 8) {
                            const int tk = task / ngrp, gi = task - tk * ngrp;
                            if (row0 + gi * 32 >= a.inter) continue;
                            const int col = gi * 32 + lane;
                            float gt = stg[tk * MX_STG_LD + col], up = stg[tk * MX_STG_LD + rows_w + col];
                            if (P.round_gu_bf16) { gt = round_bf16(gt); up = round_bf16(up); }
                            const int pr_row = w.y + tk;
                            const float pwt = P.pair_w ? __ldg(P.pair_w + pr_row) : 1.f;
                            const long orw = P.pair_out ? (long)__ldg(P.pair_out + pr_row) : (long)pr_row;
                            const float h = swiglu_bf16(gt, up, pwt, a.limit);
                            const float sc = fp8_group_scale_bf16(warp_max(fabsf(h)));
                            const uint32_t sb = (f32_as_u32(sc) >> 23) & 0xFFu;
                            const float qv = fminf(fmaxf(h * u32_as_f32((254u - sb) << 23), -448.f), 448.f);
                            reinterpret_cast<uint8_t*>(P.out)[orw * P.out_ld + row0 + col] = (uint8_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3);
                            if (lane == 0) P.out_sf[orw * P.out_sf_ld + ((row0 + gi * 32) >> 5)] = (uint8_t)sb;
                        }
                    } else if (ready) {
                        const int nch = NW >> 5;  // 32-column chunks: a warp stores 128 contiguous bytes (fp32) per task
                        for (int task = ew; task < w.z * nch; task += 8) {
                            const int tk = task / nch, col = (task - tk * nch) * 32 + lane;
                            if (row0 + col >= P.N) continue;
                            const int pr_row = w.y + tk;
                            const float pwt = P.pair_w ? __ldg(P.pair_w + pr_row) : 1.f;
                            const long orw = P.pair_out ? (long)__ldg(P.pair_out + pr_row) : (long)pr_row;
                            const float v = stg[tk * MX_STG_LD + col] * pwt;
                            if (P.epi == MX_EPI_STORE_F32) reinterpret_cast<float*>(P.out)[orw * P.out_ld + row0 + col] = v;
                            else if (P.epi == MX_EPI_ATOMIC_F32) atomicAdd(reinterpret_cast<float*>(P.out) + orw * P.out_ld + row0 + col, v);
                            else reinterpret_cast<__nv_bfloat16*>(P.out)[orw * P.out_ld + row0 + col] = __float2bfloat16_rn(v);
                        }
                    }
                    continue;
                }
                if (warp_on) {
                    if (P.epi == MX_EPI_SWIGLU_Q8) {
                        // columns c = SwiGLU column row0 + c; 32 consecutive columns are one quantisation group (dsv41/fused.py:285-306)
                        for (int c0 = egrp * 32; c0 < rows_w; c0 += 64) {
                            uint32_t g[32], u[32];
                            tc_ld16(t0 + c0, *reinterpret_cast<uint32_t(*)[16]>(&g[0]));
                            tc_ld16(t0 + c0 + 16, *reinterpret_cast<uint32_t(*)[16]>(&g[16]));
                            tc_ld16(t0 + rows_w + c0, *reinterpret_cast<uint32_t(*)[16]>(&u[0]));
                            tc_ld16(t0 + rows_w + c0 + 16, *reinterpret_cast<uint32_t(*)[16]>(&u[16]));
                            tc_wait_ld();
                            if (!tok_on || row0 + c0 >= a.inter) continue;
                            float h[32], amax = 0.f;
#pragma unroll
                            for (int cc = 0; cc < 32; ++cc) {
                                float gt = __uint_as_float(g[cc]), up = __uint_as_float(u[cc]);
                                if (P.round_gu_bf16) { gt = round_bf16(gt); up = round_bf16(up); }
                                h[cc] = swiglu_bf16_fast(gt, up, pw, a.limit);
                                amax = fmaxf(amax, fabsf(h[cc]));
                            }
                            const float sc = fp8_group_scale_bf16(amax);  // amax is a bf16 value
                            const uint32_t sb = (f32_as_u32(sc) >> 23) & 0xFFu;
                            const float inv = u32_as_f32((254u - sb) << 23);  // 1 / sc, exact (sc is a power of two)
                            uint32_t o[8];
#pragma unroll
                            for (int cc = 0; cc < 8; ++cc) {  // |h / sc| <= 448 by the choice of sc; the conversion saturates anyway
                                const uint32_t lo2 = __nv_cvt_float2_to_fp8x2(make_float2(h[4 * cc] * inv, h[4 * cc + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                                const uint32_t hi2 = __nv_cvt_float2_to_fp8x2(make_float2(h[4 * cc + 2] * inv, h[4 * cc + 3] * inv), __NV_SATFINITE, __NV_E4M3);
                                o[cc] = lo2 | (hi2 << 16);
                            }
                            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(P.out) + orow * P.out_ld + row0 + c0);
                            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                            P.out_sf[orow * P.out_sf_ld + ((row0 + c0) >> 5)] = (uint8_t)sb;
                        }
                    } else {
                        for (int c0 = egrp * 16; c0 < NW; c0 += 32) {
                            uint32_t g[16];
                            tc_ld16(t0 + c0, g);
                            tc_wait_ld();
                            if (!tok_on) continue;
                            const int nrow = row0 + c0;
                            if (nrow + 16 <= P.N) {
                                if (P.epi == MX_EPI_STORE_F32) {
                                    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(P.out) + orow * P.out_ld + nrow);
#pragma unroll
                                    for (int cc = 0; cc < 4; ++cc)
                                        dst[cc] = make_float4(__uint_as_float(g[4 * cc]) * pw, __uint_as_float(g[4 * cc + 1]) * pw,
                                                              __uint_as_float(g[4 * cc + 2]) * pw, __uint_as_float(g[4 * cc + 3]) * pw);
                                } else if (P.epi == MX_EPI_ATOMIC_F32) {
                                    float* dst = reinterpret_cast<float*>(P.out) + orow * P.out_ld + nrow;
#pragma unroll
                                    for (int cc = 0; cc < 4; ++cc)  // one 16-byte reduction instead of four scalar ones
                                        red_add_v4(dst + 4 * cc, __uint_as_float(g[4 * cc]) * pw, __uint_as_float(g[4 * cc + 1]) * pw,
                                                   __uint_as_float(g[4 * cc + 2]) * pw, __uint_as_float(g[4 * cc + 3]) * pw);
                                } else {
                                    uint32_t o[8];
#pragma unroll
                                    for (int cc = 0; cc < 8; ++cc)
                                        o[cc] = f32_to_bf16_bits(__uint_as_float(g[2 * cc]) * pw) | (f32_to_bf16_bits(__uint_as_float(g[2 * cc + 1]) * pw) << 16);
                                    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(P.out) + orow * P.out_ld + nrow);
                                    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                                    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                                }
                            } else {  // ragged last tile
                                for (int cc = 0; cc < 16 && nrow + cc < P.N; ++cc) {
                                    const float v = __uint_as_float(g[cc]) * pw;
                                    if (P.epi == MX_EPI_STORE_F32) reinterpret_cast<float*>(P.out)[orow * P.out_ld + nrow + cc] = v;
                                    else if (P.epi == MX_EPI_ATOMIC_F32) atomicAdd(reinterpret_cast<float*>(P.out) + orow * P.out_ld + nrow + cc, v);
                                    else reinterpret_cast<__nv_bfloat16*>(P.out)[orow * P.out_ld + nrow + cc] = __float2bfloat16_rn(v);
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty(buf));  // the accumulator buffer may be overwritten once all 8 warps have read it
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, MX_TMEM_COLS);
    }
}

// ------------------------------------------------------------------ activation quantisation (+ row gather)
// one warp per (output row, group of 32): q = e4m3(x / s), s = 2^ceil(log2(amax / 448)) (dsv41/quant.py:46-54, quant_fp8)
__global__ void mx_quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, const int* __restrict__ src_row, int rows, int K,
                                        uint8_t* __restrict__ q8, uint8_t* __restrict__ sf) {
    const long gid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31, gpr = K >> 5;
    if (gid >= (long)rows * gpr) return;
    const int row = (int)(gid / gpr), grp = (int)(gid % gpr);
    const long src = src_row ? src_row[row] : row;
    const float v = __bfloat162float(x[src * x_ld + grp * 32 + lane]);
    const float s = fp8_group_scale(warp_max(fabsf(v)));
    const float q = fminf(fmaxf(__fdiv_rn(v, s), -448.f), 448.f);
    q8[(long)row * K + grp * 32 + lane] = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
    if (lane == 0) sf[(long)row * gpr + grp] = (uint8_t)((f32_as_u32(s) >> 23) & 0xFFu);
}

// 16-byte-aligned rows: a thread quantises 8 values (one 16-byte load) of MXQ_ROWS consecutive output rows, 4 threads share a group of
// 32.  The row indices and then the loads of all its rows are in flight together: with one row per thread the kernel is a chain of two
// dependent loads per thread and as many waves of threads as it takes (92 us for 28,672 rows of 4096 values; with 4 rows per thread 65 us).
// Two row sets in one launch: rows [0, rows) gather input rows through src_row (or take row r when src_row is null) into q8 / sf, rows
// [rows, rows + rows2) take input row r - rows into q8b / sfb (the layer quantises its pair-sorted copy and its token-order copy in one go).
constexpr int MXQ_ROWS = 4;
__global__ void __launch_bounds__(256) mx_quantize_rows_vec_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, const int* __restrict__ src_row,
                                                                   int rows, int K, uint8_t* __restrict__ q8, uint8_t* __restrict__ sf, int rows2,
                                                                   uint8_t* __restrict__ q8b, uint8_t* __restrict__ sfb) {
    pdl_wait();
    pdl_launch_dependents();
    const int tpr = K >> 3;  // threads per row
    const long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long rb = gid / tpr;
    const int c8 = (int)(gid - rb * tpr);
    const long total = (long)rows + rows2;
    bool on[MXQ_ROWS], second[MXQ_ROWS];
    long orow[MXQ_ROWS], src[MXQ_ROWS];
#pragma unroll
    for (int i = 0; i < MXQ_ROWS; ++i) {
        const long r = rb * MXQ_ROWS + i;
        on[i] = r < total;  // K % 32 == 0: the 4 threads of a group are on or off together
        second[i] = r >= rows;
        orow[i] = second[i] ? r - rows : r;
        src[i] = (on[i] && !second[i] && src_row) ? (long)__ldg(src_row + orow[i]) : orow[i];
    }
    uint4 raw[MXQ_ROWS];
#pragma unroll
    for (int i = 0; i < MXQ_ROWS; ++i) raw[i] = on[i] ? __ldg(reinterpret_cast<const uint4*>(x + src[i] * x_ld) + c8) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < MXQ_ROWS; ++i) {
        const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
        float v[8], amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[2 * j] = bf16_bits_to_f32(u[j] & 0xFFFFu);
            v[2 * j + 1] = bf16_bits_to_f32(u[j] >> 16);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        if (!on[i]) continue;
        const float sc = fp8_group_scale_bf16(amax);  // the inputs are bf16 values
        const uint32_t sb = (f32_as_u32(sc) >> 23) & 0xFFu;
        const float inv = u32_as_f32((254u - sb) << 23);  // 1 / sc, exact
        uint32_t o[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // |v / sc| <= 448 by the choice of sc; the conversion saturates anyway
            const uint32_t lo2 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h] * inv, v[4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi2 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h + 2] * inv, v[4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
            o[h] = lo2 | (hi2 << 16);
        }
        uint8_t* const qo = second[i] ? q8b : q8;
        uint8_t* const so = second[i] ? sfb : sf;
        *reinterpret_cast<uint2*>(qo + orow[i] * K + c8 * 8) = make_uint2(o[0], o[1]);
        if ((c8 & 3) == 0) so[orow[i] * (K >> 5) + (c8 >> 2)] = (uint8_t)sb;
    }
}

// The same quantisation with a check: `exact` (a device word the caller sets non-zero) is cleared when some value of x is NOT
// reproduced by its quantised form, i.e. when x was not already an FP8 fake-quantised tensor.  Inside the MoE layer the activations
// always are (dsv41/model.py:2040, dsv41/fused.py:297-306), which is what lets a caller that only has the bf16 tensor use the
// block-scaled tensor cores without changing a single output bit; launches that follow can be tied to the word (run_if).
// x_perm8: x is stored in the reference's 8-k permuted order (slot j of every 8 holds k = bit reversal of j, dsv41/cukern.py:267-273); a
// thread's 8 values are one such group, put back in natural order here.
__global__ void __launch_bounds__(256) mx_quantize_rows_check_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, const int* __restrict__ src_row, int rows,
                                                                     int K, uint8_t* __restrict__ q8, uint8_t* __restrict__ sf, int* __restrict__ exact, int x_perm8) {
    const int tpr = K >> 3;
    const long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool on = gid < (long)rows * tpr;
    const int row = on ? (int)(gid / tpr) : 0, c8 = on ? (int)(gid % tpr) : 0;
    const long src = src_row ? __ldg(src_row + row) : row;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (on) raw = __ldg(reinterpret_cast<const uint4*>(x + src * x_ld) + c8);
    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8], amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = bf16_bits_to_f32(u[i] & 0xFFFFu);
        v[2 * i + 1] = bf16_bits_to_f32(u[i] >> 16);
        amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    }
    if (x_perm8) {
        float t = v[1]; v[1] = v[4]; v[4] = t;
        t = v[3]; v[3] = v[6]; v[6] = t;
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!on) return;
    const float sc = fp8_group_scale_bf16(amax);
    const uint32_t sb = (f32_as_u32(sc) >> 23) & 0xFFu;
    const float inv = u32_as_f32((254u - sb) << 23);
    uint32_t o[2];
    bool same = true;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float qv = fminf(fmaxf(v[4 * h + e] * inv, -448.f), 448.f);
            const __nv_fp8_storage_t code = __nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3);
            w |= (uint32_t)code << (8 * e);
            same = same && (__half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3))) * sc == v[4 * h + e]);
        }
        o[h] = w;
    }
    *reinterpret_cast<uint2*>(q8 + (long)row * K + c8 * 8) = make_uint2(o[0], o[1]);
    if ((c8 & 3) == 0) sf[(long)row * (K >> 5) + (c8 >> 2)] = (uint8_t)sb;
    if (!same) *exact = 0;
}

// ------------------------------------------------------------------ host side
int sm_count();

static int make_tmap(CUtensorMap* tm, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                     const cuuint32_t* box) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, dt, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static int check_prob(const MxArgs& a, const MxProb& p) {
    if (!p.w || !p.s || !p.x8 || !p.xsf || !p.out) return ERR_BAD_ARG;
    if (p.a_fmt != MX_A_E2M1 && p.a_fmt != MX_A_E4M3) return ERR_UNSUPPORTED;
    if (p.N <= 0) return ERR_BAD_SHAPE;
    if (a.dual && (p.epi != MX_EPI_SWIGLU_Q8 || p.N != 2 * a.inter || !p.out_sf)) return ERR_BAD_SHAPE;
    if (!a.dual && p.epi == MX_EPI_SWIGLU_Q8) return ERR_BAD_SHAPE;
    if (((uintptr_t)p.w & 31) || (p.w_estride & 31) || ((uintptr_t)p.x8 & 15) || ((uintptr_t)p.s & 3) || (p.s_rstride & 3) || (p.s_estride & 3) ||
        ((uintptr_t)p.xsf & 3) || (p.xsf_ld & 3))
        return ERR_BAD_ALIGN;
    if (p.epi == MX_EPI_SWIGLU_Q8 && (((uintptr_t)p.out & 15) || (p.out_ld & 15))) return ERR_BAD_ALIGN;
    if (p.epi != MX_EPI_SWIGLU_Q8 && (((uintptr_t)p.out & 15) || (p.out_ld & 7))) return ERR_BAD_ALIGN;
    if (!p.work && (p.n_work || p.dense_rows <= 0)) return ERR_BAD_ARG;
    return 0;
}

static int make_prob_tmaps(const MxArgs& a, const MxProb& p, CUtensorMap* tm_w, CUtensorMap* tm_x) {
    const bool fp4 = p.a_fmt == MX_A_E2M1;
    const uint64_t row_bytes = fp4 ? (uint64_t)a.K / 2 : (uint64_t)a.K;
    const uint64_t experts = p.n_experts > 0 ? p.n_experts : 1;
    const cuuint64_t estride = (experts == 1 || p.w_estride == 0) ? row_bytes * (uint64_t)p.N : (cuuint64_t)p.w_estride;
    const CUtensorMapDataType dt = fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    int rc;
    if (a.dual) {  // {k, row within a half, half (gate | up), expert}: a box of two halves is one instruction; rows past `inter` read as zero
        cuuint64_t dims[4] = {(cuuint64_t)a.K, (cuuint64_t)a.inter, 2, experts};
        cuuint64_t strides[3] = {row_bytes, row_bytes * (uint64_t)a.inter, estride};
        cuuint32_t box[4] = {128, (cuuint32_t)a.rows_a, 2, 1};
        rc = make_tmap(tm_w, dt, 4, p.w, dims, strides, box);
    } else {
        cuuint64_t dims[3] = {(cuuint64_t)a.K, (cuuint64_t)p.N, experts};
        cuuint64_t strides[2] = {row_bytes, estride};
        cuuint32_t box[3] = {128, (cuuint32_t)a.rows_a, 1};
        rc = make_tmap(tm_w, dt, 3, p.w, dims, strides, box);
    }
    if (rc) return rc;
    cuuint64_t xdims[2] = {(cuuint64_t)a.K, (cuuint64_t)(p.x8_rows > 0 ? p.x8_rows : 1)};
    cuuint64_t xstrides[1] = {(cuuint64_t)a.K};
    cuuint32_t xbox[2] = {128, (cuuint32_t)a.nd};
    return make_tmap(tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p.x8, xdims, xstrides, xbox);
}

int mx_launch(const MxArgs& a_in, cudaStream_t stream) {
    MxArgs a = a_in;
    if (a.n_prob < 1 || a.n_prob > 2) return ERR_BAD_ARG;
    if (a.K <= 0 || a.K % 128) return ERR_BAD_SHAPE;
    if (a.nd < 16 || a.nd > 128 || a.nd % 16) return ERR_BAD_SHAPE;
    if (a.rows_a < 32 || a.rows_a % 32 || a.rows_a * (a.dual ? 2 : 1) > 256) return ERR_BAD_SHAPE;
    if (a.dual && (a.inter <= 0 || a.inter % 32)) return ERR_BAD_SHAPE;
    for (int i = 0; i < a.n_prob; ++i) {
        const int rc = check_prob(a, a.p[i]);
        if (rc) return rc;
    }
    const int NW = a.dual ? 2 * a.rows_a : a.rows_a;
    const int n_atoms = 1 + (NW + 127) / 128;
    // pipeline geometry.  Every stage costs a fixed round of barrier hand-offs, so stages are fat (two or more k blocks) when a ring
    // of three of them fits, which also keeps enough bytes in flight to cover the DRAM latency; otherwise two fat stages, which
    // measured faster than four or five thin ones.
    auto ring_for = [&](int kb, size_t& stage, size_t& sf_stage, size_t& slack) -> int {
        stage = (size_t)kb * ((size_t)a.nd * 128 + (size_t)NW * 128);
        sf_stage = (size_t)kb * n_atoms * 512;
        // 1 KB to align the ring; the token descriptors always span 128 rows (16 KB) from the start of a token box, which stays
        // inside the stage unless the stage is very small
        const size_t span = (size_t)a.nd * 128 + (size_t)kb * NW * 128;
        slack = 1024 + (span < 16384 ? 16384 - span : 0);  // + the staging buffer of the small-tile epilogue
        slack += (size_t)a.stg_rows * MX_STG_LD * 4;
        int st = (int)(((size_t)MX_SMEM_LIMIT - slack) / (stage + sf_stage));
        if (st > MX_MAX_STAGES) st = MX_MAX_STAGES;
        // scale columns in TMEM behind the accumulator buffers
        while (st > 1 && st * kb * n_atoms * 4 > MX_TMEM_COLS - (2 * NW <= MX_ACC_COLS_MAX ? 2 : 1) * NW) --st;
        return st;
    };
    // small-tile staging: 32 token rows when works are that small anyway, else 16 (the ring needs the shared memory more)
    a.stg_rows = a.nd <= 32 ? 32 : 16;
    int stages = 0;
    size_t stage = 0, sf_stage = 0, slack = 0;
    a.kb = 0;
    for (int kb = 4; kb >= 2 && !a.kb; --kb)
        if ((stages = ring_for(kb, stage, sf_stage, slack)) >= 3) a.kb = kb;
    if (!a.kb && (stages = ring_for(2, stage, sf_stage, slack)) >= 2) a.kb = 2;
    if (!a.kb) { stages = ring_for(1, stage, sf_stage, slack); a.kb = 1; }
    if (stages < 2) return ERR_BAD_SHAPE;
    a.n_stages = stages;
    size_t smem = (size_t)stages * (stage + sf_stage) + slack;
    if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: each CTA allocates all 512 TMEM columns

    alignas(64) CUtensorMap tm[4];
    for (int i = 0; i < 2; ++i) {
        const int rc = make_prob_tmaps(a, a.p[i < a.n_prob ? i : 0], &tm[2 * i], &tm[2 * i + 1]);
        if (rc) return rc;
    }
    static bool attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(mx_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM_LIMIT);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    const cudaError_t le = launch_pdl(mx_gemm_kernel, dim3(sm_count()), dim3(MX_THREADS), smem, stream, a, tm[0], tm[1], tm[2], tm[3]);
    return le == cudaSuccess ? 0 : (int)le;
}

int mx_device_error(int* out, cudaStream_t stream) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return (int)e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, g_mx_error, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v) {
        int z = 0;
        cudaMemcpyToSymbol(g_mx_error, &z, sizeof(int));
    }
    *out = v;
    return 0;
}

int mx_quantize_rows_check(const __nv_bfloat16* x, long long x_ld, const int* src_row, int rows, int K, uint8_t* q8, uint8_t* sf, int* exact, cudaStream_t stream,
                           int x_perm8) {
    if (!x || !q8 || !sf || !exact || rows < 0 || K <= 0 || K % 32) return ERR_BAD_ARG;
    if (((uintptr_t)x & 15) || x_ld % 8 || ((uintptr_t)q8 & 7)) return ERR_BAD_ALIGN;
    cudaError_t e = cudaMemsetAsync(exact, 1, sizeof(int), stream);  // non-zero: "exact so far"
    if (e != cudaSuccess) return (int)e;
    if (rows == 0) return 0;
    const long threads = (long)rows * (K / 8);
    mx_quantize_rows_check_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(x, x_ld, src_row, rows, K, q8, sf, exact, x_perm8);
    B200_CHECK_LAUNCH();
    return 0;
}

int mx_quantize_rows(const __nv_bfloat16* x, long long x_ld, const int* src_row, int rows, int K, uint8_t* q8, uint8_t* sf, cudaStream_t stream, int rows2,
                     uint8_t* q8b, uint8_t* sfb) {
    if (!x || !q8 || !sf || rows < 0 || rows2 < 0 || K <= 0 || K % 32 || (rows2 > 0 && (!q8b || !sfb))) return ERR_BAD_ARG;
    if (rows + rows2 == 0) return 0;
    if (!((uintptr_t)x & 15) && x_ld % 8 == 0 && !((uintptr_t)q8 & 7) && !((uintptr_t)q8b & 7)) {
        const long threads = (((long)rows + rows2 + MXQ_ROWS - 1) / MXQ_ROWS) * (K / 8);
        const cudaError_t le = launch_pdl(mx_quantize_rows_vec_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream, x, x_ld, src_row, rows, K, q8, sf,
                                          rows2, q8b, sfb);
        return le == cudaSuccess ? 0 : (int)le;
    }
    if (rows > 0) {
        const long warps = (long)rows * (K / 32);
        mx_quantize_rows_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(x, x_ld, src_row, rows, K, q8, sf);
        B200_CHECK_LAUNCH();
    }
    if (rows2 > 0) {
        const long warps = (long)rows2 * (K / 32);
        mx_quantize_rows_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(x, x_ld, nullptr, rows2, K, q8b, sfb);
        B200_CHECK_LAUNCH();
    }
    return 0;
}

}  // namespace b200
