// Internal interface of the weight-streaming skinny GEMM (skinny.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int SK_CONSUMER_WARPS = 16;    // 2 row halves x 8 slices of 64 bytes
constexpr int SK_CONSUMER_THREADS = SK_CONSUMER_WARPS * 32;
constexpr int SK_THREADS = SK_CONSUMER_THREADS + 32;  // + 1 producer warp (bulk copies)
constexpr int SK_ROWS = 64;              // weight rows per item
constexpr int SK_TOK = 8;                // token columns per work (one 8-wide tensor-core tile)
constexpr int SK_STAGE_ROW_BYTES = 512;  // bytes of each row per stage
constexpr int SK_STAGE_BYTES = SK_ROWS * SK_STAGE_ROW_BYTES;  // eight boxes of 32 rows x 128 bytes
constexpr int SK_MAX_STAGES = 8;
constexpr int SK_RED_BYTES = 8 * 64 * 8 * 4;  // partial sums of the 8 slices
constexpr int SK_SMEM_LIMIT = 227 * 1024 - 2048;

// weight formats (also the `fmt` values of the C-ABI)
enum { SK_FMT_FP4_E8M0 = 0, SK_FMT_FP4_BF16S = 1, SK_FMT_FP8_E8M0 = 2, SK_FMT_FP8_F32B = 3 };
// epilogues
enum { SK_EPI_STORE_F32 = 0, SK_EPI_ATOMIC_F32 = 1, SK_EPI_SWIGLU = 2, SK_EPI_STORE_BF16 = 3 };

struct SkinnyArgs {
    const uint8_t* w;       // weights: [experts][N][K/2] packed E2M1 or [experts][N][K] e4m3
    long long w_estride;    // bytes between experts
    int n_experts;          // experts held by w (bounds of the tensor map); 0 = 1
    const uint8_t* s;       // scales (format dependent)
    long long s_estride;    // bytes between experts
    int s_rstride;          // bytes between scale rows (FP4: per weight row; FP8: per 32- or 128-row block)
    int N, K;
    const __nv_bfloat16* x; // activations, row-major
    long long x_ld;         // elements between rows
    int x_perm8;            // x is in the 8-k permuted layout of dsv41/cukern.py:267-273
    int w_permk;            // FP8 weight bytes are in the 16-k order of dsv41/w8.py:21-23
    const int4* work;       // {local expert, first pair, n pairs (1..8), group}; nullptr = dense mode over dense_rows
    int dense_rows;
    const int* n_work;      // device count of works, or nullptr to use n_work_host
    int n_work_host;
    const int* pair_tok;    // x row of each pair (nullptr: the pair index)
    const int* pair_out;    // output row of each pair (nullptr: the pair index)
    const float* pair_w;    // optional weight per pair
    void* out;
    long long out_ld;       // elements between output rows
    float limit;            // SwiGLU clamp (epilogue SK_EPI_SWIGLU)
    int inter;              // N == 2*inter for SK_EPI_SWIGLU
    int round_gu_bf16;      // round gate/up to bf16 before SwiGLU (shared expert)
    int n_stages;           // ring depth, set by skinny_launch from the shared-memory budget
    int rows32;             // items of 32 weight rows instead of 64 (set by skinny_launch when 64-row items would leave SMs without work)
    const int* run_if;      // optional device word: the launch does its work only if (*run_if != 0) == (run_if_nonzero != 0)
    int run_if_nonzero;
};

int sm_count();
int skinny_device_error(int* out);  // device error word of the streaming kernels (1-3: a wait ran out of time, 91: work list overflow)
int skinny_check(const SkinnyArgs& a, int fmt, int epi);
int skinny_launch(const SkinnyArgs& a, int fmt, int epi, cudaStream_t stream);
int skinny_plan(const int* grp_expert, const int* grp_start, const int* grp_count, int G, int n_pairs, int shard_start, int shard_n, int4* work,
                int* n_work, int max_work, cudaStream_t stream, int tpw = SK_TOK);
int skinny_zero_foreign(const int* grp_expert, const int* grp_start, const int* grp_count, int G, int n_pairs, int shard_start, int shard_n,
                        const int* pair_out, float* out, long long out_ld, int N, cudaStream_t stream);

}  // namespace b200
