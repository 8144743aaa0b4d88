// Tensor-map (TMA) plumbing: host-side descriptor encoding through the driver entry point (no link against libcuda),
// device-side mbarrier / bulk-tensor PTX wrappers with bounded waits.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 3-D byte tensor [experts][rows][row_bytes] (row pitch = row_bytes, expert pitch = expert_stride bytes) read in boxes of
// box_rows x 128 bytes with the 128-byte swizzle; out-of-range parts of a box are filled with zeros.
inline int make_weight_tmap(CUtensorMap* tm, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t experts, uint64_t expert_stride,
                            uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    if (experts == 0) experts = 1;
    if (experts == 1 || expert_stride == 0) expert_stride = rows * row_bytes;
    cuuint64_t dims[3] = {row_bytes, rows, experts};
    cuuint64_t strides[2] = {row_bytes, expert_stride};
    cuuint32_t box[3] = {128, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

#ifdef __CUDACC__
// ------------------------------------------------------------------ device
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// One box of a 3-D tensor map -> shared memory; completion counted in bytes on an mbarrier.  x (bytes) must be a
// multiple of 16.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst), "l"(tm),
                 "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) { asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory"); }

// four 8x8 b16 matrices: lane l supplies the address of row (l & 7) of matrix (l >> 3); lane (g, t) receives the 32-bit
// word t of row g of each matrix
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// Bounded wait on an mbarrier phase.  `abort_flag` (shared memory) short-circuits every later wait of the CTA once one
// wait has run out of time, so the CTA still runs to its end (barriers stay matched) and returns; `where` is recorded in
// the device error word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err_word, int where, unsigned backoff_ns = 0) {
    if (*abort_flag) return false;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (backoff_ns) __nanosleep(backoff_ns);  // roles off the critical path leave the issue slots to the others
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            unsigned long long t = global_timer_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(err_word, 0, where);
                return false;
            }
        }
    }
}
#endif

}  // namespace b200
