// Shared device helpers for the sm_100a MoE kernels: number-format arithmetic (exact restatements of the
// reference definitions, dsv41/quant.py and dsv41/fused.py:11-34), small PTX wrappers and error codes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ------------------------------------------------------------------ return codes of the C-ABI
// 0 = ok, >0 = cudaError_t of the failed runtime call, <0 = argument error detected before any launch.
enum : int {
    ERR_BAD_ARG = -1,       // null pointer / non-positive size
    ERR_BAD_SHAPE = -2,     // divisibility or range rule violated (see the entry point's comment)
    ERR_BAD_ALIGN = -3,     // pointer or stride not aligned as required
    ERR_WORKSPACE = -4,     // caller-provided workspace too small
    ERR_UNSUPPORTED = -5,   // format / mode not implemented
    ERR_TOO_LARGE = -6,     // size beyond a fixed maximum (static-scratch entry point)
};

#define B200_CHECK_LAUNCH()                          \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)

// ------------------------------------------------------------------ programmatic dependent launch
// The kernels of a layer step are launched with the programmatic-serialisation attribute: a kernel may be placed on SMs that the
// kernel before it in the stream has already left and run its prologue there (barrier set-up, TMEM allocation, descriptor fetch)
// instead of waiting for the whole grid to drain.  pdl_wait() blocks until the preceding kernel has completed and its writes
// are visible; every kernel launched this way calls it before it touches global memory, so the usual stream order holds for data.
// Launched without the attribute both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------ bit casts / bf16
__device__ __forceinline__ float u32_as_f32(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t f32_as_u32(float f) { return __float_as_uint(f); }
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
// round-to-nearest-even fp32 -> bf16 bits (NaN preserved)
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

// ------------------------------------------------------------------ power-of-two activation scale
// 2^ceil(log2 a) for a > 0 (normal fp32), from the IEEE bits: exponent + 1 when the mantissa is non-zero
// (dsv41/fused.py:11-16, dsv41/quant.py:34-42).
__device__ __forceinline__ float pow2_ceil(float a) {
    uint32_t b = f32_as_u32(a);
    uint32_t e = (b >> 23) & 0xFF;
    if (b & 0x7FFFFF) e += 1;
    return u32_as_f32(e << 23);
}

// nearest float8_e4m3fn value of v (|v| <= 448), ties to even, as fp32 (dsv41/fused.py:25-34).
__device__ __forceinline__ float round_e4m3(float v) {
    float a = fabsf(v);
    int e = (int)((f32_as_u32(a) >> 23) & 0xFF) - 127;  // floor(log2 a) for normal a; very small a clamps below
    e = e < -6 ? -6 : e;
    float ulp = u32_as_f32((uint32_t)(e - 3 + 127) << 23);
    float inv = u32_as_f32((uint32_t)(3 - e + 127) << 23);  // 1/ulp, exact power of two
    float r = rintf(a * inv) * ulp;
    r = fminf(r, 448.f);
    return copysignf(r, v);
}

// per-group FP8 fake quantisation scale from the group's amax (dsv41/quant.py:46-54): amax >= 1e-4,
// s = 2^ceil(log2(amax / 448)) with an IEEE division.
__device__ __forceinline__ float fp8_group_scale(float amax) {
    amax = fmaxf(amax, 1e-4f);
    return pow2_ceil(__fdiv_rn(amax, 448.f));
}

// Same scale without the division, valid when amax carries at most 8 significant bits (a bf16 value, or the 1e-4 floor):
// amax = M * 2^E, 448 = 1.75 * 2^8, so ceil(log2(amax / 448)) = E - 8 + (M > 1.75); amax / 448 can only be a power of two
// when M == 1.75 exactly.
__device__ __forceinline__ float fp8_group_scale_bf16(float amax) {
    amax = fmaxf(amax, 1e-4f);
    const uint32_t b = f32_as_u32(amax);
    const uint32_t e = ((b >> 23) & 0xFF) - 8 + ((b & 0x7FFFFF) > 0x600000 ? 1 : 0);
    return u32_as_f32(e << 23);
}

// quantise-dequantise one value with a power-of-two scale s (division by s is exact)
__device__ __forceinline__ float fp8_fake_quant_value(float v, float s) {
    float q = __fdiv_rn(v, s);
    q = fminf(fmaxf(q, -448.f), 448.f);
    return round_e4m3(q) * s;
}

// SwiGLU of the reference with its clamps (dsv41/fused.py:291-296, dsv41/cpu/moe_cpu.cpp:364-366):
// wt * silu(min(g, L)) * clamp(u, -L, L), then the bf16 cast that precedes the FP8 fake quantisation.
__device__ __forceinline__ float swiglu_bf16(float g, float u, float wt, float limit) {
    if (limit > 0.f) {
        u = fminf(fmaxf(u, -limit), limit);
        g = fminf(g, limit);
    }
    // g / (1 + e^-g) with an IEEE division, as the reference computes it.  Below g = -80 the denominator leaves the range the
    // hardware divides without its (very slow) denormal path; there silu(g) = g * e^g to within one ulp of a value < 1e-32.
    float sl = __fdiv_rn(g, 1.f + expf(-fmaxf(g, -80.f)));
    if (g < -80.f) sl = g * expf(g);
    float v = wt * sl * u;
    return round_bf16(v);
}

// The same function on the special-function unit: e^-g as ex2.approx, the quotient as an approximate division.  The result differs
// from swiglu_bf16 by a few fp32 ulp before the bf16 cast, i.e. in about one bf16 result in ten thousand; used where the epilogue of a
// tensor-core tile has to keep up with the tile's MMAs (128 x 128 results per tile).  e^-g overflows to +inf below g = -88: the quotient
// is then -0, which is what the exact value (|silu| < 1e-36) rounds to in bf16.
__device__ __forceinline__ float swiglu_bf16_fast(float g, float u, float wt, float limit) {
    if (limit > 0.f) {
        u = fminf(fmaxf(u, -limit), limit);
        g = fminf(g, limit);
    }
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    const float sl = __fdividef(g, 1.f + e);
    return round_bf16(wt * sl * u);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------ streaming loads
// 16-byte weight load that bypasses L1 allocation (weights are read exactly once per launch).
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// ------------------------------------------------------------------ warp-level tensor-core tile (16 x 8 x 16, bf16 -> fp32)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// packed bf16x2 multiply a*b (+0); subnormal inputs are honoured, which the exact FP4/FP8 -> bf16 bit placement
// below relies on.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(0u));
    return d;
}

// Activations are pre-multiplied by 2^ACT_SHIFT and weights by 2^-ACT_SHIFT so that the bf16 scale multiplier
// 2^(scale_byte - 1 - ACT_SHIFT) stays inside the bf16 exponent range for every E8M0 byte in [40, 160].
constexpr int ACT_SHIFT = 32;

}  // namespace b200
