// Host interface of the tcgen05 bf16 GEMM (gemm_sm100.cu). Plain C++ types only,
// so that both the torch binding and raw-pointer callers can use it.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace lf {

struct GemmArgs {
  const void* A = nullptr;  // bf16; [M,K] (K-major) or [K,M] (MN-major), row-major with leading dim lda
  const void* B = nullptr;  // bf16; [N,K] (K-major) or [K,N] (MN-major), row-major with leading dim ldb
  void* D = nullptr;        // [M,N] row-major, leading dim ldd; bf16 (out_mode 0) or fp32 (1, 2)
  long long lda = 0, ldb = 0, ldd = 0;
  int M = 0, N = 0, K = 0;
  bool a_mn_major = false;
  bool b_mn_major = false;
  int out_mode = 0;                 // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (D += result)
  const void* bias = nullptr;       // bf16 [N], optional
  const void* residual = nullptr;   // bf16 [M, ldr], optional, out_mode 0 only
  long long ldr = 0;
  float alpha = 1.0f;
  int* status = nullptr;            // device int; receives an error code if a bounded wait gives up
  int max_ctas = 0;                 // 0 = one CTA per SM; >0 leaves SMs free for a concurrent kernel
};

// Returns 0 on success, a negative code when arguments violate the alignment
// rules (all leading dimensions multiples of 8 elements, 16-byte aligned bases).
int gemm_bf16(const GemmArgs& args, cudaStream_t stream);

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld,
                      int box_rows, int box_cols);
// Same for 1-byte elements (fp8): `cols`, `ld` and `box_cols` in bytes; box_cols = 128 (one swizzle row).
int make_tmap_u8_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                    int box_cols);

}  // namespace lf
