// Device-side bucketing of (row, expert) pairs for the grouped expert GEMMs: the replacement of the reference's GroupedPairs
// (dsv41/moe_kernels.py:76-158), which builds the same tables from a stable argsort, bincount, cumsum and repeat_interleave.
// Here it is a counting sort in three launches with no host synchronisation and no dynamic sizes:
//   1. histogram of the expert ids;
//   2. one block scans the histogram: first sorted position of every expert, and the tile table (tiles of at most block_m pairs of one
//      expert, in expert order); the table has a fixed capacity of n_experts + n_pairs / block_m entries, unused entries carry expert -1
//      and count 0, which the GEMM launchers skip;
//   3. one block per expert walks the pairs in their original order and writes those of its expert, in that order, behind the
//      expert's first position (so the sort is stable, like the reference's), together with their rows and weights.
#include "b200_moe.h"
#include "common.cuh"

namespace b200 {

constexpr int GP_MAX_EXPERTS = 1024;

__global__ void gp_hist_kernel(const int* __restrict__ expert, int P, int E, int* __restrict__ cnt) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int e = expert[p];
    if (e >= 0 && e < E) atomicAdd(cnt + e, 1);
}

__global__ void __launch_bounds__(GP_MAX_EXPERTS) gp_scan_kernel(const int* __restrict__ cnt, int E, int block_m, int max_tiles, int* __restrict__ first,
                                                                int* __restrict__ tile_expert, int* __restrict__ tile_start, int* __restrict__ tile_count,
                                                                int* __restrict__ n_tiles) {
    __shared__ int wp[32], wt[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = tid < E ? cnt[tid] : 0;
    const int nt = (c + block_m - 1) / block_m;
    int ip = c, it = nt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int vp = __shfl_up_sync(0xffffffffu, ip, o), vt = __shfl_up_sync(0xffffffffu, it, o);
        if (lane >= o) { ip += vp; it += vt; }
    }
    if (lane == 31) { wp[warp] = ip; wt[warp] = it; }
    __syncthreads();
    int bp = ip - c, bt = it - nt, total = 0;
    for (int w = 0; w < 32; ++w) {
        if (w < warp) { bp += wp[w]; bt += wt[w]; }
        total += wt[w];
    }
    if (tid < E) {
        first[tid] = bp;
        for (int i = 0; i < nt; ++i) {
            const int rem = c - i * block_m;
            tile_expert[bt + i] = tid;
            tile_start[bt + i] = bp + i * block_m;
            tile_count[bt + i] = rem < block_m ? rem : block_m;
        }
    }
    for (int i = total + tid; i < max_tiles; i += blockDim.x) {  // unused capacity: skipped by the GEMM launchers
        tile_expert[i] = -1;
        tile_start[i] = 0;
        tile_count[i] = 0;
    }
    if (tid == 0) *n_tiles = total;
}

__global__ void __launch_bounds__(256) gp_place_kernel(const int* __restrict__ expert, int P, const int* __restrict__ first, const int* __restrict__ row_in,
                                                       const int* __restrict__ row_out, const float* __restrict__ weight, int* __restrict__ order,
                                                       int* __restrict__ s_expert, int* __restrict__ s_row_in, int* __restrict__ s_row_out,
                                                       float* __restrict__ s_weight) {
    __shared__ int wsum[8];
    __shared__ int running;
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) running = first[e];
    __syncthreads();
    for (int base = 0; base < P; base += 256) {
        const int p = base + tid;
        const bool mine = p < P && expert[p] == e;
        const uint32_t m = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) wsum[warp] = __popc(m);
        __syncthreads();
        int off = running + __popc(m & ((1u << lane) - 1)), tot = 0;
        for (int w = 0; w < 8; ++w) {
            if (w < warp) off += wsum[w];
            tot += wsum[w];
        }
        if (mine) {
            order[off] = p;
            s_expert[off] = e;
            s_row_in[off] = row_in ? row_in[p] : p;
            s_row_out[off] = row_out ? row_out[p] : p;
            s_weight[off] = weight ? weight[p] : 1.f;
        }
        __syncthreads();
        if (tid == 0) running += tot;
        __syncthreads();
    }
}

// out[i] = src[order[i]] for the rows and weights of a second GEMM over the same buckets (dsv41/moe_kernels.py:134-158)
__global__ void gp_gather_kernel(const int* __restrict__ order, int P, const int* __restrict__ row_in, const int* __restrict__ row_out,
                                 const float* __restrict__ weight, int* __restrict__ s_row_in, int* __restrict__ s_row_out, float* __restrict__ s_weight) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P) return;
    const int p = order[i];
    if (row_in) s_row_in[i] = row_in[p];
    if (row_out) s_row_out[i] = row_out[p];
    if (weight) s_weight[i] = weight[p];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_group_pairs_max_tiles(int n_pairs, int n_experts, int block_m) {
    if (n_pairs < 0 || n_experts < 1 || block_m < 1) return 0;
    return n_experts + n_pairs / block_m;
}

extern "C" size_t b200_group_pairs_workspace_bytes(int n_experts) { return (size_t)(2 * (n_experts > 0 ? n_experts : 0) + 64) * sizeof(int); }

extern "C" int b200_group_pairs(const int* expert, const int* row_in, const int* row_out, const float* weight, int n_pairs, int n_experts, int block_m,
                                int* order, int* s_expert, int* s_row_in, int* s_row_out, float* s_weight, int* tile_expert, int* tile_start,
                                int* tile_count, int* n_tiles, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!expert || !order || !s_expert || !s_row_in || !s_row_out || !s_weight || !tile_expert || !tile_start || !tile_count || !n_tiles || !workspace)
        return ERR_BAD_ARG;
    if (n_pairs < 0 || block_m < 1) return ERR_BAD_ARG;
    if (n_experts < 1 || n_experts > GP_MAX_EXPERTS) return ERR_BAD_SHAPE;
    if (workspace_bytes < b200_group_pairs_workspace_bytes(n_experts) || ((uintptr_t)workspace & 3)) return ERR_WORKSPACE;
    int* cnt = (int*)workspace;
    int* first = cnt + n_experts;
    cudaError_t ce;
    if ((ce = cudaMemsetAsync(cnt, 0, sizeof(int) * n_experts, stream)) != cudaSuccess) return (int)ce;
    if (n_pairs > 0) {
        // pairs with an id outside the expert range are dropped: the slots they leave unused at the end of the sorted arrays hold row 0 /
        // weight 0, so that a kernel that walks all n_pairs slots (a row gather) stays inside its tensors
        int* const i32[4] = {order, s_expert, s_row_in, s_row_out};
        for (int* p : i32)
            if ((ce = cudaMemsetAsync(p, 0, sizeof(int) * (size_t)n_pairs, stream)) != cudaSuccess) return (int)ce;
        if ((ce = cudaMemsetAsync(s_weight, 0, sizeof(float) * (size_t)n_pairs, stream)) != cudaSuccess) return (int)ce;
        gp_hist_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(expert, n_pairs, n_experts, cnt);
        B200_CHECK_LAUNCH();
    }
    gp_scan_kernel<<<1, GP_MAX_EXPERTS, 0, stream>>>(cnt, n_experts, block_m, b200_group_pairs_max_tiles(n_pairs, n_experts, block_m), first, tile_expert, tile_start,
                                                   tile_count, n_tiles);
    B200_CHECK_LAUNCH();
    if (n_pairs > 0) {
        gp_place_kernel<<<n_experts, 256, 0, stream>>>(expert, n_pairs, first, row_in, row_out, weight, order, s_expert, s_row_in, s_row_out, s_weight);
        B200_CHECK_LAUNCH();
    }
    return 0;
}

extern "C" int b200_regroup_pairs(const int* order, int n_pairs, const int* row_in, const int* row_out, const float* weight, int* s_row_in, int* s_row_out,
                                  float* s_weight, cudaStream_t stream) {
    if (!order || n_pairs < 0 || (row_in && !s_row_in) || (row_out && !s_row_out) || (weight && !s_weight)) return ERR_BAD_ARG;
    if (n_pairs == 0) return 0;
    gp_gather_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(order, n_pairs, row_in, row_out, weight, s_row_in, s_row_out, s_weight);
    B200_CHECK_LAUNCH();
    return 0;
}
