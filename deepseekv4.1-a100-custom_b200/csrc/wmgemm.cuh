// Internal interface of the decode-sized block-scaled tensor-core GEMM (wmgemm.cu): the tokens of the batch (at most 64) on the
// M side of the tile, 256 weight rows on the N side, the k range of the whole launch cut evenly over the CTAs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int WM_THREADS = 384;      // warp 0: copy producer, warp 1: tensor-core issuer, warps 4-11: epilogue (warps 2-3 idle)
constexpr int WM_MAX_STAGES = 8;
constexpr int WM_NT_MAX = 64;        // token columns of a tile
constexpr int WM_TILE_ROWS = 256;    // weight rows of a tile = N of the MMA: two blocks of 128 (gate | up, or consecutive)
constexpr int WM_SF_COL0 = 256;      // TMEM: the scale columns follow the accumulator (128 lanes x 256 columns)
constexpr int WM_EPI_WARPS = 8;
constexpr int WM_MAX_PRED = 80;      // CTAs whose shares of one tile a finishing CTA adds: each holds at least one of the tile's k blocks (K <= 10240)
constexpr int WM_STG_ROWS = 32;      // token rows of the staging buffer (tiles with more taking-part tokens take two passes)
constexpr int WM_STG_LD = 260;       // its row stride in floats: 16-byte aligned rows, conflict-free for 16-byte row writes and reads
constexpr size_t WM_PARTIAL_BYTES = (size_t)WM_NT_MAX * WM_TILE_ROWS * sizeof(float);  // one CTA's partial tile: [token][column]

enum { WM_EPI_STORE_F32 = 0, WM_EPI_SWIGLU_Q8 = 1, WM_EPI_STORE_BF16 = 2 };

// One problem of a launch: a set of expert matrices (or one dense matrix) against the token columns.
struct WmProb {
    const void* w;            // weights [experts][N rows][K]: packed E2M1 (two per byte) or e4m3 bytes
    long long w_estride;      // bytes between experts
    int n_experts;
    int a_fmt;                // operand format code of the weights (MX_A_E2M1 / MX_A_E4M3)
    const uint8_t* w_atoms;   // scale atoms of the weights, see scale_atoms(): [expert][tile][k block][2][512]
    long long atoms_estride;  // bytes between experts
    int N;                    // weight rows (gate | up: 2 * inter)
    const uint8_t* x8;        // token activations, e4m3 bytes [rows][K]
    long long x8_rows;        // rows the buffer holds (bound of the tensor map)
    const uint8_t* x_atoms;   // scale atoms of the tokens: [group][k block][512]
    int x_per_work;           // 1: work w reads rows [w * NT, w * NT + NT) and atom group w; 0: rows [0, NT), group 0 for every work
    const int* work;          // local expert of each work; nullptr = one work over expert 0
    const int* n_work;        // device count of works (nullptr: n_work_host)
    int n_work_host;
    const uint8_t* slot;      // [work][NT]: 0 = token not routed to the work's expert, else 1 + its top-k slot; nullptr = tokens 0..tokens-1 all take part
    int tokens;
    int topk;
    int epi;
    void* out;                // STORE: fp32 or bf16 [token * topk + slot - 1][N] (no slot table: [token][N]); gate | up matrices: the gate
    long long out_ld;         // values of a row in columns [0, inter), the up values in [inter, 2 inter).  SWIGLU_Q8: e4m3 [work * NT + token][inter]
    uint8_t* out_atoms;       // SWIGLU_Q8: scale atoms of the output rows, [work][inter / 128][512]
    const float* pair_w;      // SWIGLU_Q8: routing weights [token * topk + slot - 1] (nullptr: 1)
    int round_gu_bf16;        // SWIGLU_Q8: round gate / up to bf16 first (shared expert)
};

struct WmArgs {
    WmProb p[2];
    int n_prob;
    int K;
    int NT;            // token columns: multiple of 16, <= WM_NT_MAX
    int dual;          // 1: row block 0 = gate rows, row block 1 = the up rows `inter` further down
    int inter;
    float limit;
    int n_stages;      // set by wm_launch
    int split_k;       // 1: the k blocks of all tiles are cut evenly over the CTAs; partial tiles meet through `partial` / `flags`
    float* partial;    // [grid][WM_NT_MAX][WM_TILE_ROWS] fp32
    int* flags;        // [grid], all different from flag_value when the kernel starts
    int flag_value;
    int max_ctas;      // CTAs `partial` and `flags` are sized for (0: no limit)
};

int wm_launch(const WmArgs& a, cudaStream_t stream);
int wm_device_error(int* out);
// bytes of the scale atoms of `n_experts` matrices of N rows (dual: N = 2 * inter) and K columns
size_t scale_atoms_bytes(int n_experts, int N, int K, int dual);
// s: E8M0 bytes [expert][N >> row_shift][s_cols]; dst: [expert][tile][K / 128][2][512]
int scale_atoms(const uint8_t* s, int row_shift, int s_cols, int n_experts, int N, int K, int dual, uint8_t* dst, cudaStream_t stream);

}  // namespace b200
