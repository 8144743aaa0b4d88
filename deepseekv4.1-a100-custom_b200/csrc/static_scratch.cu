// Grouped FP4 expert GEMM whose scratch is a fixed array in the library's own device image, so that the call itself obtains no
// memory from anybody: no workspace argument, no cudaMalloc / cudaFree, no pool.  Same kernels and same results as
// b200_fp4_grouped_gemm (chain.cu); only the home of the work list differs.  There is no counterpart in the reference.
//
// What lives in the array: the list of works the planning kernel cuts the groups into (one int4 per work, at most one work
// per pair) followed by the work count.  The planning kernel rewrites the count and every entry the GEMM kernel will read on
// every call, so NOTHING in the array has to start at zero and nothing has to be cleared between calls.
//
// Sharing: each device has ONE such array and every call on that device uses it.  Calls issued to the same stream run one
// after the other and are safe.  Calls that may overlap on the device (different streams, different host threads with
// different streams) race on the array and produce garbage: serialise them with events or use the workspace form.
//
// First call on a device: the address of the array is looked up with cudaGetSymbolAddress and cached.  That look-up may make
// the runtime load the device image, so make the first call per device during set-up, before any stream capture begins.
#include <mutex>

#include "b200_moe.h"
#include "common.cuh"
#include "skinny.cuh"

namespace b200 {

constexpr int STATIC_MAX_PAIRS = B200_STATIC_MAX_PAIRS;                       // 4096 pairs
constexpr size_t STATIC_WORK_BYTES = (((size_t)STATIC_MAX_PAIRS + 1) * 16 + 255) & ~(size_t)255;  // int4 work list, rounded up to 256 bytes
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_WORK_BYTES + 256;              // + the work count on the 256-byte line behind it: 66,048 bytes

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static std::mutex g_scratch_mutex;
static void* g_scratch_ptr[MAX_DEVICES];  // per device, filled on the first call there

// Address of the array on the current device; 0 and *rc set when the runtime refuses.
static unsigned char* scratch_of_current_device(int* rc) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
    if (dev < 0 || dev >= MAX_DEVICES) { *rc = ERR_UNSUPPORTED; return nullptr; }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
        if (!p || ((uintptr_t)p & 255)) { *rc = ERR_BAD_ALIGN; return nullptr; }
        g_scratch_ptr[dev] = p;
    }
    return static_cast<unsigned char*>(g_scratch_ptr[dev]);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_fp4_grouped_gemm_static(const void* x, long long x_ld, int x_perm8, const void* w, long long w_estride, const void* s,
                                            long long s_estride, int fmt, int n_local_experts, int N, int K, const int* grp_expert,
                                            const int* grp_start, const int* grp_count, int n_groups, const int* pair_tok, const int* pair_out,
                                            const float* pair_w, int n_pairs, int shard_start, int shard_n, int zero_out, int accumulate, float* out,
                                            long long out_ld, cudaStream_t stream) {
    if (!x || !w || !s || !grp_expert || !grp_start || !out || n_groups < 0 || n_pairs < 0 || n_local_experts < 1) return ERR_BAD_ARG;
    if (fmt != SK_FMT_FP4_E8M0 && fmt != SK_FMT_FP4_BF16S) return ERR_UNSUPPORTED;
    if (n_pairs > STATIC_MAX_PAIRS) return ERR_TOO_LARGE;  // the array holds one work per pair at most
    if (n_pairs == 0 || n_groups == 0) return 0;
    int rc = 0;
    unsigned char* scratch = scratch_of_current_device(&rc);
    if (!scratch) return rc;
    int4* work = reinterpret_cast<int4*>(scratch);
    int* n_work = reinterpret_cast<int*>(scratch + STATIC_WORK_BYTES);

    SkinnyArgs a{};
    a.w = (const uint8_t*)w; a.w_estride = w_estride; a.n_experts = n_local_experts;
    a.s = (const uint8_t*)s; a.s_estride = s_estride;
    a.s_rstride = (K / 32) * (fmt == SK_FMT_FP4_BF16S ? 2 : 1);
    a.N = N; a.K = K;
    a.x = (const __nv_bfloat16*)x; a.x_ld = x_ld; a.x_perm8 = x_perm8;
    a.work = work; a.n_work = n_work;
    a.pair_tok = pair_tok; a.pair_out = pair_out; a.pair_w = pair_w;
    a.out = out; a.out_ld = out_ld;
    const int epi = accumulate ? SK_EPI_ATOMIC_F32 : SK_EPI_STORE_F32;
    rc = skinny_check(a, fmt, epi);
    if (rc) return rc;
    if (shard_n > n_local_experts) shard_n = n_local_experts;
    rc = skinny_plan(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, work, n_work, n_pairs, stream);
    if (rc) return rc;
    if (zero_out && !accumulate) {
        rc = skinny_zero_foreign(grp_expert, grp_start, grp_count, n_groups, n_pairs, shard_start, shard_n, pair_out, out, out_ld, N, stream);
        if (rc) return rc;
    }
    return skinny_launch(a, fmt, epi, stream);
}
