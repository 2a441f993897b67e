// Host interface of the grouped (per-expert) tcgen05 GEMM (grouped_gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.h"

namespace lf {

// One expert's problem; lives in DEVICE memory when the kernel runs (filled on the host, copied over).
struct alignas(64) GroupDesc {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  void* D;          // [M, N] row-major, leading dim ldd; bf16 (out_mode 0) or fp32 (1 store, 2 accumulate)
  long long ldd;
  int M, N, K;
  int out_mode;
};

// Fills `d` (host memory) for D[M,N] = op(A) op(B). Operand layouts as in GemmArgs. Returns 0 or a negative code.
int grouped_gemm_fill_desc(GroupDesc* d, const void* A, long long lda, const void* B, long long ldb, void* D,
                           long long ldd, int M, int N, int K, bool a_mn, bool b_mn, int out_mode);

// Number of output tiles of one group (entries it contributes to the tile table).
int grouped_gemm_tiles_for(int M, int N);

// `groups_dev`: device array of GroupDesc; `tiles_dev`: device array of int2 {group, tile index in group}.
int grouped_gemm_launch(const GroupDesc* groups_dev, const void* tiles_dev, int num_tiles, bool a_mn, bool b_mn,
                        int* status, cudaStream_t stream);

}  // namespace lf
