// Decode-sized expert GEMM on the block-scaled tensor cores (tcgen05.mma kind::mxf8f6f4), laid out for a weight stream:
//     D[token, weight row] = sum_k  q[token, k] * 2^(sx[token, k/32] - 127)  *  W[row, k] * 2^(sw[row, k/32] - 127)
// A decode batch has at most 64 tokens but every expert it touches must be read from HBM once, so the kernel is built around the
// weight bytes:
//   * 256 weight rows (128 gate rows and their 128 up rows, or 256 consecutive rows of the down matrix) are the N side of ONE
//     instruction per 32 k, the tokens of the whole batch are its M side (128 lanes of which the first 16 .. 64 carry tokens).  An MMA
//     costs the tensor pipe about the same whether it is 128 x 16 or 128 x 256 wide (operand fetch, measured), so the widest N per
//     instruction gives the fewest tensor-pipe cycles per weight byte: 4 instructions per 128-wide k block of a tile;
//   * every expert is multiplied with ALL tokens of the batch and the epilogue keeps the (token, expert) pairs the router chose: no
//     gather of activation rows, no sorting of pairs, one work per distinct expert however many tokens share it;
//   * the scale bytes come as ready-made 512-byte atoms (scale_atoms() below rewrites the expert scales once, when a layer is built;
//     the producers of the activations write theirs in that form), so one thread moves everything with bulk copies: per 128-wide
//     k block a tensor-map box of the weights (FP4 is unpacked by the copy engine), a box of the tokens, 1 KB of weight scales and
//     512 B of token scales, all counted on one mbarrier;
//   * the k blocks of all tiles of the launch are cut EVENLY over the CTAs (one per SM): a CTA that ends inside a tile leaves its
//     partial accumulator in global memory, the CTA that finishes the tile adds the partial tiles in CTA order (deterministic) before
//     its epilogue.  A single token touches 6 experts = 112 tiles for 148 SMs; cut by tile a quarter of the machine would idle;
//   * the accumulator (128 lanes x 256 columns of TMEM) is copied to shared memory by the warps that can read the token lanes and
//     handed back to the tensor-core issuer at once; all eight epilogue warps then work on (token, 128 columns) tasks of the chosen
//     pairs with 16-byte accesses while the next tile's MMAs run.
// Warp roles: warp 0 copy producer, warp 1 TMEM allocation + scale copies (tcgen05.cp) + MMAs, warps 4-11 epilogue.  Every wait is
// bounded: a wait that runs out of time stores a code in a device error word and the CTA runs on.
//
// Replaces, for decode-sized batches on B200, dsv41/cuda/fp4_tc.cu, fp4_tcw.cu, fp4_gemv_m1.cu and the GEMM stages of
// dsv41/cuda/expert_chain.cu (routed experts), and fp8_gemv_m1.cu / fp8_tc.cu for the shared expert inside the layer.
#include <cuda_fp8.h>

#include "common.cuh"
#include "mxgemm.cuh"
#include "tc5.cuh"
#include "wmgemm.cuh"

namespace b200 {

__device__ int g_wm_error = 0;

// instruction descriptor: A = the tokens (e4m3), B = the weights (format code b_fmt), both K-major, M = 128, N = 256, E8M0 scales,
// byte j of the 4 scale bytes in a TMEM column for both operands
__device__ __forceinline__ uint32_t wm_idesc(int b_fmt, int j) {
    return ((uint32_t)j << 4) | (0u << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(WM_TILE_ROWS >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24) | ((uint32_t)j << 29);
}
__device__ __forceinline__ void wm_epi_bar() { asm volatile("bar.sync 2, 256;" ::: "memory"); }  // the eight epilogue warps
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

__global__ void __launch_bounds__(WM_THREADS, 1) wm_gemm_kernel(const WmArgs a, const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_x0,
                                                                 const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_x1) {
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long bars[2 * WM_MAX_STAGES + 2];  // full[s], empty[s], acc_full, acc_empty
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;
    __shared__ uint8_t s_slot[WM_NT_MAX];    // the current work's table over the tokens
    __shared__ int s_live[WM_NT_MAX + 1];    // tokens that take part, then their count at [WM_NT_MAX]
    __shared__ int s_pos[WM_NT_MAX];         // index of a token among the taking-part ones (-1: it does not)
    __shared__ uint8_t s_pred[WM_MAX_PRED];  // CTAs that hold earlier k blocks of the tile being finished (as distances back from this CTA), and their number
    __shared__ int s_npred;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = a.n_stages, NT = a.NT, KBLK = a.K >> 7;
    const int SR = NT < WM_STG_ROWS ? NT : WM_STG_ROWS;  // token rows the staging buffer holds
    uint8_t* base = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    // stage: [NT token rows x 128 B][256 weight rows x 128 B][weight scale atoms 2 x 512 B][token scale atom 512 B] (+ 512 B pad).
    // The token operand of an MMA spans 128 rows from the start of the token box: the rows behind the NT loaded ones are the weight
    // tile of the same stage; their accumulator lanes are never read.
    constexpr uint32_t W_TILE = (uint32_t)WM_TILE_ROWS * 128u;
    const uint32_t x_tile = (uint32_t)NT * 128u;
    const uint32_t stage_bytes = W_TILE + x_tile + 2048u;
    float* stg = reinterpret_cast<float*>(base + (size_t)NS * stage_bytes);  // staging of accumulator rows: [SR][WM_STG_LD]
    auto bar_full = [&](int s) { return smem_u32(&bars[s]); };
    auto bar_empty = [&](int s) { return smem_u32(&bars[WM_MAX_STAGES + s]); };
    const uint32_t bar_acc_full = smem_u32(&bars[2 * WM_MAX_STAGES]), bar_acc_empty = smem_u32(&bars[2 * WM_MAX_STAGES + 1]);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, 1);
        mbar_fence_init();
    }
    if (tid == 0) {  // the descriptors of the copies: fetched while the kernel before this one is still running
        tma_prefetch_desc(&tm_w0);
        tma_prefetch_desc(&tm_x0);
        if (a.n_prob > 1) { tma_prefetch_desc(&tm_w1); tma_prefetch_desc(&tm_x1); }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_sh), MX_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    // nothing above touched global memory: from here on the kernel before this one in the stream must have completed
    pdl_wait();
    pdl_launch_dependents();

    // (all unit arithmetic in 32 bits: 64-bit divisions on the lone threads that walk the sequence cost microseconds per launch)
    // ---- the flat sequence of k blocks: tiles of problem 0 (work-major) with those of problem 1 spread evenly among them; this CTA
    // owns units [lo, hi)
    const int tpw0 = a.dual ? (a.inter + 127) >> 7 : (a.p[0].N + WM_TILE_ROWS - 1) / WM_TILE_ROWS;
    const int tpw1 = a.n_prob > 1 ? (a.dual ? (a.inter + 127) >> 7 : (a.p[1].N + WM_TILE_ROWS - 1) / WM_TILE_ROWS) : 1;
    const int tiles0 = (a.p[0].n_work ? *a.p[0].n_work : a.p[0].n_work_host) * tpw0;
    const int tiles1 = a.n_prob > 1 ? (a.p[1].n_work ? *a.p[1].n_work : a.p[1].n_work_host) * tpw1 : 0;
    const int tiles = tiles0 + tiles1;
    const int U = tiles * KBLK;
    const int G = gridDim.x;
    const int gap = tiles1 > 0 ? tiles / tiles1 : 1;
    // The cut is even in TIME, not in k blocks: a k block of an FP8 matrix (the shared expert) is twice the bytes of a packed FP4 one.
    // cost_at(u) = weight of the k blocks before u; CTA c starts at the first u whose cost reaches c / G of the total.
    // (measured: a k block of an FP8 matrix takes about 1.5 times as long as a packed FP4 one, not twice: weights 3 and 2)
    const int wc0 = a.p[0].a_fmt == MX_A_E2M1 ? 2 : 3, wc1 = (a.n_prob > 1 && a.p[1].a_fmt != MX_A_E2M1) ? 3 : 2;
    const int gap_i = (int)gap, t1_i = (int)tiles1, tile_c0 = wc0 * KBLK, tile_c1 = wc1 * KBLK;
    const int period_c = (gap_i - 1) * tile_c0 + tile_c1;      // cost of `gap` consecutive tiles while problem 1 has tiles left
    const int cost_all = (int)(tiles0 * tile_c0 + tiles1 * tile_c1);
    auto cost_at = [&](int u) -> int {
        const int tile = u / KBLK, within = u - tile * KBLK;
        const int nb = t1_i > 0 ? (tile / gap_i < t1_i ? tile / gap_i : t1_i) : 0;
        const bool is1 = t1_i > 0 && tile % gap_i == gap_i - 1 && tile / gap_i < t1_i;
        return (tile - nb) * tile_c0 + nb * tile_c1 + within * (is1 ? wc1 : wc0);
    };
    auto unit_lo = [&](int c) -> int {  // the first unit whose preceding cost reaches c / G of the total (closed form of the inverse of cost_at)
        if (!a.split_k) return (tiles * c / G) * KBLK;
        if (c <= 0) return 0;
        if (c >= G) return U;
        const int x = (int)((long long)cost_all * c / G);  // the one 64-bit division
        int tile, rem, w;
        if (t1_i > 0 && x < t1_i * period_c) {
            const int j = x / period_c, r = x - j * period_c;
            if (r < (gap_i - 1) * tile_c0) { const int q = r / tile_c0; tile = j * gap_i + q; rem = r - q * tile_c0; w = wc0; }
            else { tile = j * gap_i + gap_i - 1; rem = r - (gap_i - 1) * tile_c0; w = wc1; }
        } else {
            const int y = x - t1_i * period_c, q = y / tile_c0;
            tile = t1_i * gap_i + q; rem = y - q * tile_c0; w = wc0;
        }
        return tile * KBLK + (rem + w - 1) / w;
    };
    const int lo = unit_lo(blockIdx.x), hi = unit_lo(blockIdx.x + 1);
    const int nwork0 = (int)(tiles0 / tpw0) > 0 ? (int)(tiles0 / tpw0) : 1, nwork1 = (int)(tiles1 / tpw1) > 0 ? (int)(tiles1 / tpw1) : 1;
    // a prime that does not divide the length of the list is coprime to it (three candidates: their product exceeds any list)
    const int wstride0 = nwork0 % 29 ? 29 : (nwork0 % 31 ? 31 : 37);

    struct Seg { int tile; int kb0, kb1, pr, wk, it, e; };
    auto seg_at = [&](int u) -> Seg {
        Seg s;
        s.tile = u / KBLK;
        s.kb0 = (int)(u - s.tile * KBLK);
        const int end = (s.tile + 1) * KBLK;
        s.kb1 = (int)((end < hi ? end : hi) - s.tile * KBLK);
        // the tiles of problem 1 (the shared expert) are spread evenly through the sequence, one after
        // every `gap - 1` tiles of problem 0, so that no CTA gets more than its share of them
        const int nb = s.tile / gap < tiles1 ? s.tile / gap : tiles1;   // tiles of problem 1 before this position
        s.pr = (tiles1 > 0 && s.tile % gap == gap - 1 && s.tile / gap < tiles1) ? 1 : 0;
        // Order of a problem's tiles: tile index major, works minor, the works taken with a stride coprime to their number.  Tiles of
        // an expert that many tokens chose cost more (more accumulator rows to move out); consecutive positions of the sequence then
        // belong to experts far apart in the work list, so every CTA's share is a mix.
        const int rel = (int)(s.pr ? nb : s.tile - nb);
        const int nw = s.pr ? nwork1 : nwork0;
        s.it = rel / nw;
        const int j = rel - s.it * nw;
        s.wk = s.pr ? j : (j * wstride0) % nw;
        s.e = a.p[s.pr].work ? __ldg(a.p[s.pr].work + s.wk) : 0;
        return s;
    };
    // Order of this CTA's segments: a CTA that ends inside a tile computes that trailing share FIRST and publishes it at once, then
    // walks the rest of its range in order.  The CTA that finishes the tile needs the share for its first epilogue, about as many
    // k blocks later; published at the end of the range instead, every CTA would wait for the whole range of the one before it.
    // ... and a CTA that begins inside a tile and finishes it (it then adds the shares of the CTAs before it) computes that leading
    // part LAST: one of those CTAs may lie inside the tile with its whole range and publish only at its end, and a leading part done
    // first would wait for it with the accumulator in hand.  Order: trailing share, whole tiles, leading part.
    const bool has_head = a.split_k && (lo % KBLK != 0) && ((lo / KBLK + 1) * KBLK <= hi);
    const int head_end = has_head ? (lo / KBLK + 1) * KBLK : lo;  // leading part = [lo, head_end)
    const int tail_floor = (hi / KBLK) * KBLK;
    const int tail_start = (a.split_k && hi % KBLK != 0) ? (tail_floor > head_end ? tail_floor : head_end) : hi;  // trailing share = [tail_start, hi)
    struct It { int u; int ph; bool done; };
    auto it_enter = [&](It& it, int ph) {  // the first non-empty part from `ph` on
        for (; ph < 3; ++ph) {
            if (ph == 0 && tail_start < hi) { it = It{tail_start, 0, false}; return; }
            if (ph == 1 && head_end < tail_start) { it = It{head_end, 1, false}; return; }
            if (ph == 2 && lo < head_end) { it = It{lo, 2, false}; return; }
        }
        it = It{hi, 3, true};
    };
    auto it_begin = [&]() -> It {
        It it;
        it_enter(it, 0);
        return it;
    };
    auto it_next = [&](It& it, const Seg& sg) {
        if (it.ph == 1) {
            const int u = sg.tile * KBLK + sg.kb1;
            if (u < tail_start) { it.u = u; return; }
        }
        it_enter(it, it.ph + 1);
    };

    if (lo < hi) {
        if (warp == 0) {
            // ------------------------------------------------ copy producer (one thread)
            if (lane == 0) {
                uint32_t n = 0, s = 0, ph = 0;  // k blocks issued, their stage and the stage's phase
                for (It it = it_begin(); !it.done && !abort_flag;) {
                    const Seg sg = seg_at(it.u);
                    const WmProb& P = a.p[sg.pr];
                    const CUtensorMap* tw = sg.pr ? &tm_w1 : &tm_w0;
                    const CUtensorMap* tx = sg.pr ? &tm_x1 : &tm_x0;
                    const uint32_t w_tx = P.a_fmt == MX_A_E2M1 ? W_TILE / 2 : W_TILE;  // packed FP4 boxes count the bytes read
                    const int row0 = sg.it * (a.dual ? 128 : WM_TILE_ROWS);
                    const int xrow = P.x_per_work ? sg.wk * NT : 0;
                    const uint8_t* wat = P.w_atoms + (long long)sg.e * P.atoms_estride + ((long long)sg.it * KBLK) * 1024;
                    const uint8_t* xat = P.x_atoms + ((long long)(P.x_per_work ? sg.wk : 0) * KBLK) * 512;
                    for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++n) {
                        if (!mbar_wait(bar_empty(s), ph ^ 1, &abort_flag, &g_wm_error, 11)) break;
                        mbar_expect_tx(bar_full(s), w_tx + x_tile + 1536u);
                        const uint32_t dst = smem_u32(base + (size_t)s * stage_bytes);
                        const int kx = kb * 128;  // element coordinate along K
                        if (a.dual) tma_load_4d(dst + x_tile, tw, kx, row0, 0, sg.e, bar_full(s));
                        else tma_load_3d(dst + x_tile, tw, kx, row0, sg.e, bar_full(s));
                        tma_load_2d(dst, tx, kx, xrow, bar_full(s));
                        bulk_load(dst + x_tile + W_TILE, wat + (long long)kb * 1024, 1024u, bar_full(s));
                        bulk_load(dst + x_tile + W_TILE + 1024u, xat + (long long)kb * 512, 512u, bar_full(s));
                        if (++s == (uint32_t)NS) { s = 0; ph ^= 1; }
                    }
                    it_next(it, sg);
                }
                // every copy issued above must have landed before the CTA may exit
                for (int k = 0; k < NS && k < (int)n; ++k) {
                    const uint32_t m = n - 1 - k, sl = m % NS, pl = (m / NS) & 1;
                    const unsigned long long t0 = global_timer_ns();
                    while (!mbar_test(bar_full(sl), pl)) {
                        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(&g_wm_error, 0, 13); break; }
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ tensor-core issuer (one thread)
            if (lane == 0) {
                uint32_t acc_it = 0, s = 0, ph = 0;
                for (It it = it_begin(); !it.done && !abort_flag; ++acc_it) {
                    const Seg sg = seg_at(it.u);
                    const int b_fmt = a.p[sg.pr].a_fmt;
                    // the accumulator is free again once the epilogue warps have read the previous tile out of it
                    if (!mbar_wait(bar_acc_empty, (acc_it & 1) ^ 1, &abort_flag, &g_wm_error, 21)) break;
                    tc_fence_after();
                    uint32_t accumulate = 0;
                    for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                        if (!mbar_wait(bar_full(s), ph, &abort_flag, &g_wm_error, 22)) break;
                        tc_fence_after();
                        const uint32_t sbase = smem_u32(base + (size_t)s * stage_bytes);
                        const uint32_t sfs = sbase + x_tile + W_TILE;
                        const uint32_t sfcol = tmem_base + WM_SF_COL0 + s * 12;  // [weight rows 0-127][weight rows 128-255][tokens], 4 columns each
#pragma unroll
                        for (int q = 0; q < 3; ++q) tc_cp_sf(sfcol + q * 4, desc_sf_atom(sfs + (uint32_t)q * 512u));
                        const uint64_t dx = desc_sw128(sbase), dw = desc_sw128(sbase + x_tile);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {  // 4 MMAs of K = 32: the operand descriptors advance by 32 bytes inside the swizzled row
                            tc_mma_mx(tmem_base, dx + 2 * j, dw + 2 * j, wm_idesc(b_fmt, j), sfcol + 8, sfcol, accumulate);
                            accumulate = 1;
                        }
                        tc_commit(bar_empty(s));  // the stage may be refilled once these MMAs (and scale copies) have read it
                        if (++s == (uint32_t)NS) { s = 0; ph ^= 1; }
                    }
                    tc_commit(bar_acc_full);
                    it_next(it, sg);
                }
            }
        } else if (warp >= 4) {
            // ------------------------------------------------ epilogue, warps 4-11.  The accumulator rows of the tokens that take part
            // are copied to a staging buffer in shared memory by the warps that can read their TMEM lanes (warp = lane quadrant x column
            // half), the accumulator goes back to the tensor-core issuer at once, and all eight warps then move the rows to global memory
            // with 16-byte accesses (adding the shares of the CTAs that held earlier k blocks of the tile on the way).
            const int ew = warp - 4, et = tid - 128, quad = warp & 3, chalf = ew >> 2;
            uint32_t acc_it = 0;
            // no early exit: the eight warps meet at named barriers, so all of them walk the same segment sequence; once a wait has run
            // out of time every later wait returns at once
            for (It it = it_begin(); !it.done; ++acc_it) {
                const Seg sg = seg_at(it.u);
                it_next(it, sg);
                const WmProb& P = a.p[sg.pr];
                const bool owner = sg.kb1 == KBLK;
                wm_epi_bar();  // the tasks of the previous segment are done: its tables and the staging buffer may be overwritten
                if (et < NT)   // which tokens take part: the work's table, for a share of a tile as for a finished tile (same rows in both)
                    s_slot[et] = P.slot ? __ldg(P.slot + (size_t)sg.wk * NT + et) : (uint8_t)(et < P.tokens ? 1 : 0);
                wm_epi_bar();
                // the taking-part tokens, compacted: s_live[i] = i-th such token, s_pos[t] = its index (-1: token t does not take part)
                if (ew == 0) {
                    const bool l0 = lane < NT && s_slot[lane] != 0, l1 = lane + 32 < NT && s_slot[lane + 32] != 0;
                    const uint32_t m0 = __ballot_sync(0xffffffffu, l0), m1 = __ballot_sync(0xffffffffu, l1);
                    const int p0i = __popc(m0 & ((1u << lane) - 1)), p1i = __popc(m0) + __popc(m1 & ((1u << lane) - 1));
                    if (l0) s_live[p0i] = lane;
                    if (l1) s_live[p1i] = lane + 32;
                    s_pos[lane] = l0 ? p0i : -1;
                    s_pos[lane + 32] = l1 ? p1i : -1;
                    if (lane == 0) s_live[WM_NT_MAX] = __popc(m0) + __popc(m1);
                }
                // the CTAs that hold the k blocks [0, kb0) of this tile, in CTA order (one thread finds them, all wait for their shares)
                if (et == 0) {
                    int np = 0;
                    if (owner && sg.kb0 > 0) {
                        const int u0 = sg.tile * KBLK;
                        int c_first = (int)((long long)cost_at(u0) * G / cost_all);
                        if (c_first >= (int)blockIdx.x) c_first = (int)blockIdx.x - 1;
                        if (c_first < 0) c_first = 0;
                        while (c_first + 1 < (int)blockIdx.x && unit_lo(c_first + 1) <= u0) ++c_first;
                        while (c_first > 0 && unit_lo(c_first) > u0) --c_first;
                        int ulo = unit_lo(c_first);
                        for (int c = c_first; c < (int)blockIdx.x && np < WM_MAX_PRED; ++c) {
                            const int unext = unit_lo(c + 1);
                            if (unext != ulo) s_pred[np++] = (uint8_t)((int)blockIdx.x - c);  // a CTA without work leaves nothing
                            ulo = unext;
                        }
                    }
                    s_npred = np;
                }
                wm_epi_bar();
                const int n_pred = s_npred;
                {
                    for (int pi = 0; pi < n_pred; ++pi) {
                        const int c = (int)blockIdx.x - s_pred[pi];
                        unsigned long long ts = 0;
                        for (uint32_t i = 0; !abort_flag && ld_acquire(a.flags + c) != a.flag_value; ++i) {
                            __nanosleep(64);
                            if ((i & 63u) == 63u) {
                                const unsigned long long tn = global_timer_ns();
                                if (ts == 0) ts = tn;
                                else if (tn - ts > WAIT_LIMIT_NS) { abort_flag = 1; atomicCAS(&g_wm_error, 0, 42); break; }
                            }
                        }
                    }
                }
                wm_epi_bar();
                const int n_live = s_live[WM_NT_MAX];
                const bool ready = mbar_wait(bar_acc_full, acc_it & 1, &abort_flag, &g_wm_error, 41);
                tc_fence_after();
                // where the rows go: the partial-tile buffer of this CTA, or the output rows of the tokens
                const int row0 = sg.it * (a.dual ? 128 : WM_TILE_ROWS);
                const int epi = P.epi, topk = P.topk;
                const bool has_slot = P.slot != nullptr;
                const long long out_ld = P.out_ld;
                char* const outp = reinterpret_cast<char*>(P.out);
                const int esz = epi == WM_EPI_STORE_BF16 ? 2 : 4;
                // columns of half h: gate | up matrices put the gate values at [row0, ..) and the up values at [inter + row0, ..)
                const long col_h[2] = {(long)row0, a.dual ? (long)a.inter + row0 : (long)row0 + 128};
                const int lim0 = a.dual ? a.inter - row0 : P.N - row0, lim1 = a.dual ? a.inter - row0 : P.N - row0 - 128;
                const int ok_h[2] = {lim0 < 128 ? (lim0 > 0 ? lim0 : 0) : 128, lim1 < 128 ? (lim1 > 0 ? lim1 : 0) : 128};
                for (int p0 = 0; p0 < (n_live > 0 ? n_live : 1); p0 += SR) {
                    if (p0) wm_epi_bar();  // the tasks of the previous pass are done
                    if (quad * 32 < NT && n_live > 0) {
                        const int t = quad * 32 + lane;
                        const int pos = t < NT ? s_pos[t] : -1;
                        const bool mine = pos >= p0 && pos < p0 + SR;
                        if (__any_sync(0xffffffffu, mine)) {
                            const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + chalf * 128;
                            float4* row = reinterpret_cast<float4*>(stg + (size_t)(mine ? pos - p0 : 0) * WM_STG_LD + chalf * 128);
#pragma unroll
                            for (int c0 = 0; c0 < 128; c0 += 32) {
                                uint32_t g[32];
                                tc_ld16(t0 + c0, *reinterpret_cast<uint32_t(*)[16]>(&g[0]));
                                tc_ld16(t0 + c0 + 16, *reinterpret_cast<uint32_t(*)[16]>(&g[16]));
                                tc_wait_ld();
                                if (mine)
#pragma unroll
                                    for (int k = 0; k < 8; ++k)
                                        row[(c0 >> 2) + k] = make_float4(__uint_as_float(g[4 * k]), __uint_as_float(g[4 * k + 1]), __uint_as_float(g[4 * k + 2]), __uint_as_float(g[4 * k + 3]));
                            }
                        }
                    }
                    tc_fence_before();
                    wm_epi_bar();  // the copy is complete and visible to all epilogue warps
                    if (et == 0 && p0 + SR >= n_live) mbar_arrive(bar_acc_empty);
                    const int n_pass = n_live - p0 < SR ? n_live - p0 : SR;
                    if (!ready) continue;
                    if (owner && epi == WM_EPI_SWIGLU_Q8) {
                        // task = (row, 32 SwiGLU columns = one quantisation group): gate column c and up column 128 + c of the row
                        // (dsv41/fused.py:285-306).  Used for the smallest batches, where the few rows of a tile cost less here than a
                        // kernel of their own between the two GEMMs.  The shares of earlier CTAs are added on the way.
                        uint8_t* const o8 = reinterpret_cast<uint8_t*>(P.out);
                        for (int task = ew; task < n_pass * 4; task += WM_EPI_WARPS) {
                            const int r = task >> 2, g = task & 3, t = s_live[p0 + r], col = row0 + g * 32 + lane;
                            if (row0 + g * 32 >= a.inter) continue;
                            float gt = stg[(size_t)r * WM_STG_LD + g * 32 + lane], up = stg[(size_t)r * WM_STG_LD + 128 + g * 32 + lane];
                            for (int pi = 0; pi < n_pred; pi += 4) {  // four shares in flight, added in CTA order
                                float pg[4], pu[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const int pq = pi + q < n_pred ? pi + q : n_pred - 1;
                                    const float* src = a.partial + ((size_t)(blockIdx.x - s_pred[pq]) * WM_NT_MAX + t) * WM_TILE_ROWS + g * 32 + lane;
                                    pg[q] = __ldcg(src);
                                    pu[q] = __ldcg(src + 128);
                                }
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    if (pi + q < n_pred) { gt += pg[q]; up += pu[q]; }
                            }
                            if (P.round_gu_bf16) { gt = round_bf16(gt); up = round_bf16(up); }
                            const float pw = P.pair_w ? __ldg(P.pair_w + (size_t)t * topk + s_slot[t] - 1) : 1.f;
                            const float h = swiglu_bf16(gt, up, pw, a.limit);
                            const float sc = fp8_group_scale_bf16(warp_max(fabsf(h)));
                            const uint32_t sb = (f32_as_u32(sc) >> 23) & 0xFFu;
                            const float qv = fminf(fmaxf(h * u32_as_f32((254u - sb) << 23), -448.f), 448.f);
                            o8[((size_t)sg.wk * NT + t) * out_ld + col] = (uint8_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3);
                            if (lane == 0) P.out_atoms[((size_t)sg.wk * (a.inter >> 7) + sg.it) * 512 + (t & 31) * 16 + (t >> 5) * 4 + g] = (uint8_t)sb;
                        }
                        continue;
                    }
                    // task = (row of the staging buffer, column half): a lane moves 4 consecutive values; two tasks per warp and turn
                    for (int base_task = ew * 2; base_task < n_pass * 2; base_task += 2 * WM_EPI_WARPS) {
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int task = base_task + u;
                            if (task >= n_pass * 2) continue;
                            const int r = task >> 1, h = task & 1, t = s_live[p0 + r], c = 4 * lane;
                            float4 v = *reinterpret_cast<const float4*>(stg + (size_t)r * WM_STG_LD + h * 128 + c);
                            if (!owner) {
                                *reinterpret_cast<float4*>(a.partial + ((size_t)blockIdx.x * WM_NT_MAX + t) * WM_TILE_ROWS + h * 128 + c) = v;
                                continue;
                            }
                            for (int pi = 0; pi < n_pred; pi += 4) {  // the shares of the CTAs before this one: four in flight, added in CTA order
                                float4 p4[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const int pq = pi + q < n_pred ? pi + q : n_pred - 1;
                                    p4[q] = __ldcg(reinterpret_cast<const float4*>(a.partial + ((size_t)(blockIdx.x - s_pred[pq]) * WM_NT_MAX + t) * WM_TILE_ROWS + h * 128 + c));
                                }
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    if (pi + q < n_pred) { v.x += p4[q].x; v.y += p4[q].y; v.z += p4[q].z; v.w += p4[q].w; }
                            }
                            if (c >= ok_h[h]) continue;
                            const long orow = has_slot ? (long)t * topk + s_slot[t] - 1 : (long)t;
                            char* dst = outp + (orow * out_ld + col_h[h] + c) * esz;
                            if (c + 4 <= ok_h[h]) {
                                if (esz == 4) *reinterpret_cast<float4*>(dst) = v;
                                else *reinterpret_cast<uint2*>(dst) = make_uint2(f32_to_bf16_bits(v.x) | (f32_to_bf16_bits(v.y) << 16), f32_to_bf16_bits(v.z) | (f32_to_bf16_bits(v.w) << 16));
                            } else {
                                const float vv[4] = {v.x, v.y, v.z, v.w};
                                for (int k = 0; k < 4 && c + k < ok_h[h]; ++k) {
                                    if (esz == 4) reinterpret_cast<float*>(dst)[k] = vv[k];
                                    else reinterpret_cast<__nv_bfloat16*>(dst)[k] = __float2bfloat16_rn(vv[k]);
                                }
                            }
                        }
                    }
                }
                if (!owner) {  // publish this CTA's share
                    __threadfence();
                    wm_epi_bar();
                    if (et == 0 && ready) st_release(a.flags + blockIdx.x, a.flag_value);
                }
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

// ------------------------------------------------------------------ scale atoms
// The tensor cores take the E8M0 scales of 128 operand rows x 4 groups of 32 k from 4 TMEM columns, filled by a copy of a 512-byte
// "atom" whose byte (r % 32) * 16 + (r / 32) * 4 + g is the scale of row r, group g.  This kernel rewrites a scale tensor in the
// checkpoint's order ([expert][row >> row_shift][K / 32] bytes; one row of scales per weight row for the experts, per 32 rows for
// the dense FP8 format) into the atoms a tile of wm_gemm_kernel needs, in the order it reads them:
//     dst[expert][tile][k block][row block 0 | row block 1][512]
// dual (gate | up matrix): tile t = gate rows 128 t .. 128 t + 127 and up rows inter + 128 t ..; else rows 256 t .. 256 t + 255.
// Rows past the matrix get the byte 127 (scale 1; their weights read as zero).  One thread per (atom, row).
__global__ void scale_atoms_kernel(const uint8_t* __restrict__ s, int row_shift, int s_cols, long long s_estride, int n_experts, int N, int kblk, int dual, int inter,
                                   int tiles, uint8_t* __restrict__ dst) {
    const long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long total = (long)n_experts * tiles * kblk * 256;
    if (gid >= total) return;
    const int r = (int)(gid & 127), rb = (int)(gid >> 7) & 1;
    long rest = gid >> 8;
    const int kb = (int)(rest % kblk);
    rest /= kblk;
    const int t = (int)(rest % tiles), e = (int)(rest / tiles);
    int row;
    bool ok;
    if (dual) {
        row = (rb ? inter : 0) + t * 128 + r;
        ok = t * 128 + r < inter;
    } else {
        row = t * 256 + rb * 128 + r;
        ok = row < N;
    }
    uint32_t v = 0x7F7F7F7Fu;
    if (ok) v = *reinterpret_cast<const uint32_t*>(s + (long long)e * s_estride + (long long)(row >> row_shift) * s_cols + kb * 4);
    *reinterpret_cast<uint32_t*>(dst + (gid >> 7) * 512 + (r & 31) * 16 + (r >> 5) * 4) = v;
}

// ------------------------------------------------------------------ host side
int sm_count();

static int wm_tiles(int N, int dual) { return dual ? (N / 2 + 127) / 128 : (N + WM_TILE_ROWS - 1) / WM_TILE_ROWS; }

size_t scale_atoms_bytes(int n_experts, int N, int K, int dual) {
    if (n_experts <= 0 || N <= 0 || K <= 0) return 0;
    return (size_t)n_experts * wm_tiles(N, dual) * (K / 128) * 1024;
}

int scale_atoms(const uint8_t* s, int row_shift, int s_cols, int n_experts, int N, int K, int dual, uint8_t* dst, cudaStream_t stream) {
    if (!s || !dst || n_experts < 1 || N < 1) return ERR_BAD_ARG;
    if (K <= 0 || K % 128 || (dual && (N % 2 || (N / 2) % 32)) || s_cols < K / 32) return ERR_BAD_SHAPE;
    if (((uintptr_t)s & 3) || (s_cols & 3) || ((uintptr_t)dst & 15)) return ERR_BAD_ALIGN;
    const int tiles = wm_tiles(N, dual), kblk = K / 128;
    const long long estride = (long long)((N + (1 << row_shift) - 1) >> row_shift) * s_cols;
    const long total = (long)n_experts * tiles * kblk * 256;
    scale_atoms_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(s, row_shift, s_cols, estride, n_experts, N, kblk, dual, N / 2, tiles, dst);
    B200_CHECK_LAUNCH();
    return 0;
}

static int make_tmap(CUtensorMap* tm, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, dt, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static int wm_prob_tmaps(const WmArgs& a, const WmProb& p, CUtensorMap* tm_w, CUtensorMap* tm_x) {
    const bool fp4 = p.a_fmt == MX_A_E2M1;
    const uint64_t row_bytes = fp4 ? (uint64_t)a.K / 2 : (uint64_t)a.K;
    const uint64_t experts = p.n_experts > 0 ? p.n_experts : 1;
    const cuuint64_t estride = (experts == 1 || p.w_estride == 0) ? row_bytes * (uint64_t)p.N : (cuuint64_t)p.w_estride;
    const CUtensorMapDataType dt = fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    int rc;
    if (a.dual) {  // {k, row within a half, half (gate | up), expert}: one box = 128 gate rows and, behind them in shared memory, their up rows
        cuuint64_t dims[4] = {(cuuint64_t)a.K, (cuuint64_t)a.inter, 2, experts};
        cuuint64_t strides[3] = {row_bytes, row_bytes * (uint64_t)a.inter, estride};
        cuuint32_t box[4] = {128, 128, 2, 1};
        rc = make_tmap(tm_w, dt, 4, p.w, dims, strides, box);
    } else {
        cuuint64_t dims[3] = {(cuuint64_t)a.K, (cuuint64_t)p.N, experts};
        cuuint64_t strides[2] = {row_bytes, estride};
        cuuint32_t box[3] = {128, WM_TILE_ROWS, 1};
        rc = make_tmap(tm_w, dt, 3, p.w, dims, strides, box);
    }
    if (rc) return rc;
    cuuint64_t xdims[2] = {(cuuint64_t)a.K, (cuuint64_t)(p.x8_rows > 0 ? p.x8_rows : 1)};
    cuuint64_t xstrides[1] = {(cuuint64_t)a.K};
    cuuint32_t xbox[2] = {128, (cuuint32_t)a.NT};
    return make_tmap(tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p.x8, xdims, xstrides, xbox);
}

int wm_launch(const WmArgs& a_in, cudaStream_t stream) {
    WmArgs a = a_in;
    if (a.n_prob < 1 || a.n_prob > 2) return ERR_BAD_ARG;
    if (a.K <= 0 || a.K % 128 || a.K / 128 > WM_MAX_PRED) return ERR_BAD_SHAPE;
    if (a.NT != 16 && a.NT != 32 && a.NT != 64) return ERR_BAD_SHAPE;
    if (a.dual && (a.inter <= 0 || a.inter % 32)) return ERR_BAD_SHAPE;
    if (a.split_k && (!a.partial || !a.flags)) return ERR_BAD_ARG;
    for (int i = 0; i < a.n_prob; ++i) {
        const WmProb& p = a.p[i];
        if (!p.w || !p.w_atoms || !p.x8 || !p.x_atoms || !p.out) return ERR_BAD_ARG;
        if (p.a_fmt != MX_A_E2M1 && p.a_fmt != MX_A_E4M3) return ERR_UNSUPPORTED;
        if (p.N <= 0 || (a.dual && p.N != 2 * a.inter)) return ERR_BAD_SHAPE;
        if (p.epi != WM_EPI_STORE_F32 && p.epi != WM_EPI_STORE_BF16 && p.epi != WM_EPI_SWIGLU_Q8) return ERR_UNSUPPORTED;
        if (p.epi == WM_EPI_SWIGLU_Q8 && (!a.dual || !p.out_atoms)) return ERR_BAD_ARG;
        if (p.epi != WM_EPI_SWIGLU_Q8 && ((p.out_ld & (p.epi == WM_EPI_STORE_BF16 ? 7 : 3)) || ((uintptr_t)p.out & 15))) return ERR_BAD_ALIGN;
        if (((uintptr_t)p.w & 31) || (p.w_estride & 31) || ((uintptr_t)p.x8 & 15) || ((uintptr_t)p.w_atoms & 15) || (p.atoms_estride & 15) || ((uintptr_t)p.x_atoms & 15))
            return ERR_BAD_ALIGN;
        if (!p.work && p.n_work) return ERR_BAD_ARG;
    }
    const size_t stage = (size_t)WM_TILE_ROWS * 128 + (size_t)a.NT * 128 + 2048;
    const size_t stg = (size_t)(a.NT < WM_STG_ROWS ? a.NT : WM_STG_ROWS) * WM_STG_LD * sizeof(float);
    int stages = (int)(((size_t)MX_SMEM_LIMIT - 1024 - stg) / stage);
    if (stages > WM_MAX_STAGES) stages = WM_MAX_STAGES;
    if (stages * 12 > MX_TMEM_COLS - WM_SF_COL0) stages = (MX_TMEM_COLS - WM_SF_COL0) / 12;
    if (stages < 2) return ERR_BAD_SHAPE;
    a.n_stages = stages;
    const size_t smem = (size_t)stages * stage + stg + 1024;

    alignas(64) CUtensorMap tm[4];
    for (int i = 0; i < 2; ++i) {
        const int rc = wm_prob_tmaps(a, a.p[i < a.n_prob ? i : 0], &tm[2 * i], &tm[2 * i + 1]);
        if (rc) return rc;
    }
    static bool attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(wm_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM_LIMIT);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    int grid = sm_count();
    if (a.split_k && a.max_ctas > 0 && grid > a.max_ctas) grid = a.max_ctas;
    const cudaError_t le = launch_pdl(wm_gemm_kernel, dim3(grid), dim3(WM_THREADS), smem, stream, a, tm[0], tm[1], tm[2], tm[3]);
    return le == cudaSuccess ? 0 : (int)le;
}

int wm_device_error(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_wm_error, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v) {
        int z = 0;
        cudaMemcpyToSymbol(g_wm_error, &z, sizeof(int));
    }
    *out = v;
    return 0;
}

}  // namespace b200
