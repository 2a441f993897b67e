// Host interface of the FP8 block quantisers and the blockwise-scaled FP8 GEMM (fp8_sm100.cu).
#pragma once
#include <cuda_runtime.h>

namespace lf {

// x bf16 [M, K] (K % 128 == 0) -> q e4m3 [M, K], scales fp32 [M, K/128]; x ~= q * scale. pow2: power-of-two scales.
int quant_1x128(const void* x, void* q, float* scales, long long M, int K, int pow2, cudaStream_t st);
// w bf16 [N, K] (both % 128 == 0) -> q e4m3 [N, K], scales fp32 [N/128, K/128].
int quant_128x128(const void* w, void* q, float* scales, int N, int K, int pow2, cudaStream_t st);
// D bf16 [M, N] = (A_q, sa) x (B_q, sb)^T with A_q [M, K], B_q [N, K] e4m3, K % 128 == 0, N % 128 == 0.
int gemm_fp8_blockwise(const void* Aq, const float* sa, const void* Bq, const float* sb, void* D, long long ldd, int M,
                       int N, int K, int* status, cudaStream_t stream);

}  // namespace lf
