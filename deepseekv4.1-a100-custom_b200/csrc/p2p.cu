// Device-side messaging between GPUs for the expert-parallel decode protocol: copies by kernel stores into memory another GPU can
// see (a peer mapping, an IPC mapping or symmetric memory; local memory works the same), flag signal / wait kernels and a sequence
// counter, all stream-ordered so that a whole decode step runs without host round trips.  Replaces dsv41/cuda/p2p.cu
// (dsv41/cukern.py:348-434) with one difference that matters on shared machines: EVERY WAIT IS BOUNDED.  A wait that does not see its
// flag within the limit stores a code in the device error word (b200_device_error: 3001 plain wait, 3002 masked wait) and returns, so
// the stream, the context and the GPU stay usable; the caller learns of the failure at its next b200_device_error.
// No multicast or switch-side reduction is used: the fan-out to several destinations is a loop of ordinary stores.
#include "b200_moe.h"
#include "common.cuh"
#include "tma.cuh"

namespace b200 {

__device__ int g_p2p_error = 0;
__device__ unsigned long long g_p2p_wait_limit_ns = WAIT_LIMIT_NS;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// 16-byte copy, grid-stride
__global__ void p2p_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n16) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// row b of src -> dst_base[seq[b]][row_idx[b]]: the layout of the reference's per-sequence inboxes (dsv41/cukern.py:357-366)
__global__ void p2p_copy_row_kernel(uint4* __restrict__ dst_base, const long long* __restrict__ row_idx, const uint4* __restrict__ src, int row16, int nb,
                                    long long bstride16, const long long* __restrict__ seq) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)row16 * nb) return;
    const int b = (int)(i / row16), j = (int)(i - (long long)b * row16);
    dst_base[seq[b] * bstride16 + row_idx[b] * row16 + j] = src[i];
}

// publish the value at seq_ptr to n flag words (addresses in `flags`), after everything earlier in the stream
__global__ void p2p_signal_kernel(int* const* __restrict__ flags, int n, const int* __restrict__ seq_ptr) {
    __threadfence_system();
    const int v = *seq_ptr;
    for (int i = threadIdx.x; i < n; i += blockDim.x) st_release_sys(flags[i], v);
}

// wait until every (unmasked) flag has reached the value at seq_ptr, or the limit runs out
__global__ void p2p_wait_kernel(const int* __restrict__ flags, int n, const int* __restrict__ seq_ptr, const int* __restrict__ mask) {
    const int v = *seq_ptr;
    const unsigned long long limit = g_p2p_wait_limit_ns;
    unsigned long long t0 = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (mask && !mask[i]) continue;
        for (unsigned it = 0; ld_acquire_sys(flags + i) < v; ++it) {
            __nanosleep(100);
            if ((it & 15u) == 15u) {
                const unsigned long long t = global_timer_ns();
                if (t0 == 0) t0 = t;
                else if (t - t0 > limit) {
                    atomicCAS(&g_p2p_error, 0, mask ? 2 : 1);
                    return;
                }
            }
        }
    }
    __threadfence_system();
}

__global__ void p2p_seq_bump_kernel(int* seq) { *seq += 1; }

// src -> every destination in dsts (ordinary stores, one destination after the other), then the last block to finish publishes the
// value at seq_ptr to the flags (one per destination); `counter` starts at zero and resets itself
__global__ void p2p_fanout_kernel(uint4* const* __restrict__ dsts, int ndst, const uint4* __restrict__ src, long long n16, int* const* __restrict__ flags,
                                  const int* __restrict__ seq_ptr, unsigned int* __restrict__ counter) {
    __shared__ int last;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        for (int d = 0; d < ndst; ++d) dsts[d][i] = v;
    }
    if (!flags) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicInc(counter, gridDim.x - 1) == gridDim.x - 1;
    __syncthreads();
    if (last) {
        __threadfence_system();
        const int v = *seq_ptr;
        for (int d = threadIdx.x; d < ndst; d += blockDim.x) st_release_sys(flags[d], v);
    }
}

__global__ void p2p_stamp_kernel(long long* dst) { *dst = (long long)global_timer_ns(); }

int p2p_device_error(int* out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_p2p_error, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v) {
        int z = 0;
        cudaMemcpyToSymbol(g_p2p_error, &z, sizeof(int));
    }
    *out = v;
    return 0;
}

int sm_count();

// device addresses of the error word and the wait limit, for kernels of other translation units (per device; looked up every call:
// cudaGetSymbolAddress is a table look-up once the module is loaded)
int p2p_words(int** error_word, const unsigned long long** limit_ns) {
    cudaError_t e = cudaGetSymbolAddress((void**)error_word, g_p2p_error);
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)limit_ns, g_p2p_wait_limit_ns);
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_p2p_copy(void* dst, const void* src, long long nbytes, cudaStream_t stream) {
    if (!dst || !src || nbytes < 0) return ERR_BAD_ARG;
    if ((nbytes & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)src & 15)) return ERR_BAD_ALIGN;
    if (nbytes == 0) return 0;
    const long long n16 = nbytes / 16;
    long long blocks = (n16 + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    p2p_copy_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, stream>>>((uint4*)dst, (const uint4*)src, n16);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_p2p_copy_row(void* dst_base, const long long* row_idx, const void* src, long long row_bytes, int n_rows, long long batch_stride_bytes,
                                 const long long* seq, cudaStream_t stream) {
    if (!dst_base || !row_idx || !src || !seq || n_rows < 0 || row_bytes <= 0) return ERR_BAD_ARG;
    if ((row_bytes & 15) || (batch_stride_bytes & 15) || ((uintptr_t)dst_base & 15) || ((uintptr_t)src & 15)) return ERR_BAD_ALIGN;
    if (n_rows == 0) return 0;
    const long long total = row_bytes / 16 * n_rows;
    p2p_copy_row_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((uint4*)dst_base, row_idx, (const uint4*)src, (int)(row_bytes / 16), n_rows,
                                                                             batch_stride_bytes / 16, seq);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_p2p_signal(int* const* flag_ptrs, int n, const int* seq, cudaStream_t stream) {
    if (!flag_ptrs || !seq || n < 0) return ERR_BAD_ARG;
    if (n == 0) return 0;
    p2p_signal_kernel<<<1, 32, 0, stream>>>(flag_ptrs, n, seq);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_p2p_wait(const int* flags, int n, const int* seq, const int* mask, cudaStream_t stream) {
    if (!flags || !seq || n < 0) return ERR_BAD_ARG;
    if (n == 0) return 0;
    p2p_wait_kernel<<<1, 32, 0, stream>>>(flags, n, seq, mask);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_p2p_seq_bump(int* seq, cudaStream_t stream) {
    if (!seq) return ERR_BAD_ARG;
    p2p_seq_bump_kernel<<<1, 1, 0, stream>>>(seq);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_p2p_multicast(void* const* dst_ptrs, int n_dst, const void* src, long long nbytes, int* const* flag_ptrs, const int* seq,
                                  unsigned int* counter, cudaStream_t stream) {
    if (!dst_ptrs || !src || n_dst < 0 || nbytes < 0 || (flag_ptrs && (!seq || !counter))) return ERR_BAD_ARG;
    if ((nbytes & 15) || ((uintptr_t)src & 15)) return ERR_BAD_ALIGN;
    if (n_dst == 0) return 0;
    const long long n16 = nbytes / 16;
    long long blocks = (n16 + 1023) / 1024;
    if (blocks < 1) blocks = 1;
    const long long cap = (long long)sm_count() * 2;
    p2p_fanout_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 1024, 0, stream>>>((uint4* const*)dst_ptrs, n_dst, (const uint4*)src, n16, flag_ptrs, seq, counter);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_p2p_stamp(long long* dst, cudaStream_t stream) {
    if (!dst) return ERR_BAD_ARG;
    p2p_stamp_kernel<<<1, 1, 0, stream>>>(dst);
    B200_CHECK_LAUNCH();
    return 0;
}

extern "C" int b200_memcpy_async(void* dst, const void* src, long long nbytes, cudaStream_t stream) {
    if (!dst || !src || nbytes < 0) return ERR_BAD_ARG;
    if (nbytes == 0) return 0;
    const cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDefault, stream);
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200_set_wait_limit_ns(unsigned long long ns) {
    if (ns == 0) ns = WAIT_LIMIT_NS;
    const cudaError_t e = cudaMemcpyToSymbol(g_p2p_wait_limit_ns, &ns, sizeof(ns));
    return e == cudaSuccess ? 0 : (int)e;
}
