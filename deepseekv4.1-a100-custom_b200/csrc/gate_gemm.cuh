// Router projection (gate_gemm.cu): fp32 logits from the hidden state and the gate matrix, k range split over blocks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace b200 {

constexpr int GATE_MAX_SPLITS = 32;

// number of k splits the launcher would use for this shape (the caller sizes the output: splits x T x E floats)
int gate_gemm_splits(int T, int E, int D);
// out[s][t][e] = partial logits of split s; their sum over s, in order, is x @ w^T.  x: fp32 rows (xf) or bf16 rows (xb).
int gate_gemm(const float* xf, long long xf_ld, const __nv_bfloat16* xb, long long xb_ld, const float* w, int T, int E, int D, int splits, float* out,
              cudaStream_t stream);

}  // namespace b200
