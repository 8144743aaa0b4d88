// Expert-parallel decode step over peer memory: the exchange of one MoE layer step between the GPUs of a node done by three small
// kernels with ordinary peer stores and flag words, no collective library call and no host round trip.
//
// Every rank owns a slab of device memory that all ranks can address (CUDA IPC mapping, one cudaMalloc per rank):
//     inbox_x   [max tokens][x_row_bytes]        token rows of ALL ranks, in global token order
//     inbox_l   [max tokens][l_row_bytes]        their router logits
//     partials  [max tokens][world][dim] fp32    routed partial sums of this rank's own tokens, one row per contributing rank
//     flags_in  [world], flags_out [world]       int32, count upwards
// One step on rank r, all stream-ordered (`seq` is a device word holding the step number):
//     dispatch   the rank's token rows and logits go to every rank's inbox (its own included) at the rows of its global token
//                range; the last block to finish publishes seq to flags_in[r] of every rank           (ep_dispatch_kernel)
//     wait       until flags_in[0 .. world) >= seq: every rank's rows have arrived                      (ep_wait_kernel)
//     compute    the rank's experts over all tokens -> fp32 partial row per token                      (the layer's own launches)
//     return     row t of the partial sums goes to partials[t - first[h]][r] on the home rank h of token t; the last block
//                publishes seq to flags_out[r] of every rank                                            (ep_return_kernel)
//     wait       until flags_out[0 .. world) >= seq, then seq += 1                                      (ep_wait_kernel)
//     combine    out[t] = bf16(sum over ranks in rank order of partials[t][.] + shared expert row)      (moe_combine_kernel)
// Buffers can be reused by the next step without further handshakes: a rank passes the second wait of step s only after every
// peer has finished reading its inbox of step s (a peer signals flags_out after its compute), and a peer writes partial rows of
// step s + 1 only after this rank's dispatch of step s + 1, which follows its combine of step s in stream order.
//
// Follows the protocol of the reference's expert-parallel decode runtime (packet push + flag per peer, partial rows returned per
// sender and summed in rank order: dsv41/ep.py:69-80, 356-525, dsv41/cuda/p2p.cu:6-82) with three differences: activations travel
// with the router logits and every rank routes all tokens itself (the compute path is the single-GPU one), one kernel does copy +
// fan-out + signal, and every wait is bounded: after the limit it stores 3003 (arrival) or 3004 (return) in the device error word
// and the step runs on, so a missing peer costs a wrong result that the host learns of, never a hung GPU.
#include "b200_moe.h"
#include "common.cuh"
#include "tma.cuh"
#include <string.h>

namespace b200 {

// device addresses of the messaging error word and of the wait limit (p2p.cu)
int p2p_words(int** error_word, const unsigned long long** limit_ns);

namespace {

__device__ __forceinline__ int ep_ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ep_st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// the last block of the grid to get here publishes the step number to one flag per rank
__device__ __forceinline__ void publish_when_last(int* const* flags, int world, const int* seq, unsigned int* counter) {
    __shared__ int last;
    __threadfence_system();
    __syncthreads();
    const unsigned int n_blocks = gridDim.x * gridDim.y;
    if (threadIdx.x == 0) last = atomicInc(counter, n_blocks - 1) == n_blocks - 1;
    __syncthreads();
    if (last) {
        __threadfence_system();
        const int v = *seq;
        for (int d = threadIdx.x; d < world; d += blockDim.x) ep_st_release_sys(flags[d], v);
    }
}

// grid (local tokens, world): block (t, d) copies token t's activation row and logits row into rank d's inbox
__global__ void ep_dispatch_kernel(b200_ep_peers P, const uint4* __restrict__ x, const uint4* __restrict__ logits, int n_rows) {
    const int t = blockIdx.x, d = blockIdx.y;
    if (t < n_rows) {
        const int x16 = P.x_row_bytes >> 4, l16 = P.l_row_bytes >> 4;
        const long long row = P.first[P.rank] + t;
        uint4* dx = (uint4*)P.inbox_x[d] + row * x16;
        uint4* dl = (uint4*)P.inbox_l[d] + row * l16;
        const uint4* sx = x + (long long)t * x16;
        const uint4* sl = logits + (long long)t * l16;
        for (int i = threadIdx.x; i < x16; i += blockDim.x) dx[i] = sx[i];
        for (int i = threadIdx.x; i < l16; i += blockDim.x) dl[i] = sl[i];
    }
    publish_when_last(P.flags_in, P.world, P.seq, P.counter);
}

// grid (tokens, column chunks): block (t, c) sends its chunk of partial row t to the home rank of token t
__global__ void ep_return_kernel(b200_ep_peers P, const uint4* __restrict__ part) {
    const int t = blockIdx.x;
    int h = 0;
    while (h + 1 < P.world && t >= P.first[h + 1]) ++h;
    const int d16 = P.dim >> 2;  // fp32 row in 16-byte words
    const int per = (d16 + gridDim.y - 1) / gridDim.y;
    const int lo = blockIdx.y * per, hi = min(d16, lo + per);
    uint4* dst = (uint4*)P.partials[h] + ((long long)(t - P.first[h]) * P.world + P.rank) * d16;
    const uint4* src = part + (long long)t * d16;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = src[i];
    publish_when_last(P.flags_out, P.world, P.seq, P.counter + 1);
}

// one block: wait until the first n flags have reached the step number, or the limit runs out; then optionally advance the step
__global__ void ep_wait_kernel(const int* __restrict__ flags, int n, int* seq, int bump, int code, int* error_word,
                               const unsigned long long* __restrict__ limit_ns) {
    const int v = *seq;
    const unsigned long long limit = *limit_ns;
    unsigned long long t0 = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        for (unsigned it = 0; ep_ld_acquire_sys(flags + i) < v; ++it) {
            __nanosleep(64);
            if ((it & 15u) == 15u) {
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > limit) {
                    atomicCAS(error_word, 0, code);
                    break;
                }
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (bump && threadIdx.x == 0) *seq = v + 1;
}

int check_peers(const b200_ep_peers* P) {
    if (!P || !P->first || !P->inbox_x || !P->inbox_l || !P->flags_in || !P->partials || !P->flags_out || !P->seq || !P->counter) return ERR_BAD_ARG;
    if (P->world < 1 || P->world > B200_EP_MAX_RANKS || P->rank < 0 || P->rank >= P->world || P->dim <= 0) return ERR_BAD_SHAPE;
    if ((P->x_row_bytes & 15) || (P->l_row_bytes & 15) || (P->dim & 3) || P->x_row_bytes <= 0 || P->l_row_bytes <= 0) return ERR_BAD_ALIGN;
    return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_ep_dispatch(const b200_ep_peers* peers, const void* x_local, const void* logits_local, int local_tokens, cudaStream_t stream) {
    if (int rc = check_peers(peers)) return rc;
    if (local_tokens < 0 || (local_tokens > 0 && (!x_local || !logits_local))) return ERR_BAD_ARG;
    if (((uintptr_t)x_local & 15) || ((uintptr_t)logits_local & 15)) return ERR_BAD_ALIGN;
    // a rank without tokens still signals: one row of blocks that copies nothing
    ep_dispatch_kernel<<<dim3(local_tokens > 0 ? local_tokens : 1, peers->world), 256, 0, stream>>>(*peers, (const uint4*)x_local, (const uint4*)logits_local,
                                                                                                  local_tokens);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_ep_return(const b200_ep_peers* peers, const float* partial, int tokens, cudaStream_t stream) {
    if (int rc = check_peers(peers)) return rc;
    if (!partial || tokens <= 0) return ERR_BAD_ARG;
    if ((uintptr_t)partial & 15) return ERR_BAD_ALIGN;
    const int d16 = peers->dim >> 2;
    const int chunks = d16 >= 1024 ? 4 : d16 >= 512 ? 2 : 1;
    ep_return_kernel<<<dim3(tokens, chunks), 256, 0, stream>>>(*peers, (const uint4*)partial);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_ep_wait(const int* flags, int n, int* seq, int advance, int which, cudaStream_t stream) {
    if (!flags || !seq || n < 1 || n > B200_EP_MAX_RANKS) return ERR_BAD_ARG;
    int* err = nullptr;
    const unsigned long long* limit = nullptr;
    if (int rc = p2p_words(&err, &limit)) return rc;
    ep_wait_kernel<<<1, 32, 0, stream>>>(flags, n, seq, advance, which ? 4 : 3, err, limit);
    B200_CHECK_LAUNCH();
    return 0;
}

/* ---- set-up calls (not stream-ordered; they may synchronise and allocate) */
extern "C" int b200_ep_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return ERR_BAD_ARG;
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(*ptr, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200_ep_free(void* ptr) {
    const cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200_ep_export(const void* ptr, void* handle) {
    if (!ptr || !handle) return ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == B200_EP_HANDLE_BYTES, "handle size");
    const cudaError_t e = cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle, const_cast<void*>(ptr));
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200_ep_open(const void* handle, void** ptr) {
    if (!ptr || !handle) return ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200_ep_close(void* ptr) {
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? 0 : (int)e;
}
