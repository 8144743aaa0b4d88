// Internal interface of the block-scaled tensor-core grouped GEMM (mxgemm.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int MX_THREADS = 512;   // 16 warps: TMA producer, MMA issuer, 2 spare, 4 epilogue, 4 scale loaders, 4 more epilogue
constexpr int MX_TMEM_COLS = 512;
constexpr int MX_ACC_COLS_MAX = 384;  // TMEM columns the accumulator buffers may take; the rest holds the scale factors
constexpr int MX_MAX_STAGES = 8;
constexpr int MX_STG_LD = 257;                      // row stride (floats) of the small-tile staging buffer: odd, so that both the
                                                    // per-token writes and the per-column reads are free of bank conflicts
constexpr int MX_SMEM_LIMIT = 227 * 1024 - 1024;  // dynamic shared memory: the 227 KB a block may use minus the kernel's static 1 KB

enum { MX_EPI_STORE_F32 = 0, MX_EPI_SWIGLU_Q8 = 1, MX_EPI_STORE_BF16 = 2, MX_EPI_ATOMIC_F32 = 3 };
enum { MX_A_E4M3 = 0, MX_A_E2M1 = 5 };  // operand format codes of the tensor-core instruction descriptor

// One GEMM problem of a launch: a weight set against activation rows.
struct MxProb {
    // weights [experts][N rows][K], packed E2M1 (two per byte) or e4m3 bytes
    const void* w;
    long long w_estride;    // bytes between experts
    int n_experts;
    int a_fmt;              // MX_A_E2M1 / MX_A_E4M3 (operand format code of the weights)
    const uint8_t* s;       // E8M0 scale bytes, one per (scale row, 32 k)
    long long s_estride;    // bytes between experts
    int s_rstride;          // bytes between scale rows
    int s_row_shift;        // scale row of weight row r = r >> s_row_shift (0: per row, 5: per 32 rows)
    int N;
    // activations as e4m3 bytes [rows][K] with E8M0 scale bytes [rows][K/32]
    const uint8_t* x8;
    long long x8_rows;      // rows the buffer holds (bound of the tensor map)
    const uint8_t* xsf;
    int xsf_ld;
    // works: {local expert, first activation row, rows (1..nd), -}; nullptr = dense mode over dense_rows rows, expert 0
    const int4* work;
    const int* n_work;
    int n_work_host;
    int dense_rows;
    int epi;
    const int* pair_out;    // output row of activation row p (nullptr: p)
    const float* pair_w;    // optional weight per activation row
    void* out;              // f32 / bf16 [rows][N] or, for SWIGLU, e4m3 bytes [rows][inter]
    long long out_ld;
    uint8_t* out_sf;        // SWIGLU: E8M0 scale bytes [rows][inter/32]
    int out_sf_ld;
    int round_gu_bf16;
};

// A launch: one or two problems with the same K, tile shape and epilogue family (both SWIGLU, or both stores).
struct MxArgs {
    MxProb p[2];
    int n_prob;
    int K;
    int nd;                 // tokens per work = token rows fetched per tile (multiple of 16, <= 128; the tile spans 128 accumulator lanes)
    int rows_a;             // weight rows per tile half: the MMA covers rows_a (single) or 2 * rows_a (dual) weight rows
    int dual;               // 1: gate rows r and up rows inter + r side by side in one tile, epilogue SWIGLU
    int kb;                 // 128-wide k blocks per pipeline stage
    int n_stages;
    int stg_rows;           // token rows of the small-tile staging buffer (set by mx_launch): works up to this size take the staged epilogue
    float limit;
    int inter;
    const int* run_if;      // optional device word: the launch does its work only if (*run_if != 0) == (run_if_nonzero != 0)
    int run_if_nonzero;
};

int mx_launch(const MxArgs& a, cudaStream_t stream);
// quantise as mx_quantize_rows and clear *exact (set non-zero first, on the stream) if x is not reproduced exactly by its quantised form
int mx_quantize_rows_check(const __nv_bfloat16* x, long long x_ld, const int* src_row, int rows, int K, uint8_t* q8, uint8_t* sf, int* exact, cudaStream_t stream,
                           int x_perm8 = 0);
int mx_device_error(int* out, cudaStream_t stream);  // copies and clears the device error word (synchronises the stream)

// bf16 [rows][K] -> e4m3 bytes + E8M0 scale byte per 32 (the FP8 fake quantisation of dsv41/quant.py:46-54 kept in
// quantised form); optional row gather: output row p reads input row src_row[p]
// a second row set (rows2 > 0): input rows 0 .. rows2-1, ungathered, into q8b / sfb in the same launch
int mx_quantize_rows(const __nv_bfloat16* x, long long x_ld, const int* src_row, int rows, int K, uint8_t* q8, uint8_t* sf, cudaStream_t stream, int rows2 = 0,
                     uint8_t* q8b = nullptr, uint8_t* sfb = nullptr);

}  // namespace b200
