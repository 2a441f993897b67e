// Grouped bf16 GEMM for MoE experts on sm_100a: ONE persistent launch covers every local expert.
//
// Each group g (one expert) has its own problem D_g[M_g, N_g] = op(A_g) * op(B_g) with its own TMA
// descriptors, held in a device array of `GroupDesc`. A flat tile table lists (group, tile) pairs;
// CTAs walk it with the same TMA -> tcgen05.mma -> TMEM -> epilogue pipeline as the dense GEMM
// (gemm_sm100.cu). Per-expert descriptors make ragged row counts exact: TMA zero-fills rows past
// the expert's last token, so forward / dgrad tiles never read a neighbour's tokens and the wgrad
// contraction over an expert's tokens stops at its last row.
//
//   forward : Y_e[n_e, N]   = X_e[n_e, K]  * W_e[N, K]^T     (A K-major,  B K-major)
//   dgrad   : dX_e[n_e, K]  = dY_e[n_e, N] * W_e[N, K]       (A K-major,  B MN-major)
//   wgrad   : dW_e[N, K]   += dY_e^T       * X_e             (A MN-major, B MN-major, fp32 accumulate)
//
// Replaces TE GroupedLinear / grouped cuBLAS in the reference
// (loongforge/models/foundation/qwen3/qwen_layer_spec.py:46-55).
#include "sm100_ptx.cuh"
#include "grouped_gemm_sm100.h"

namespace lf {

static constexpr int GG_BM = 128, GG_BN = 256, GG_BK = 64, GG_UMMA_K = 16, GG_STAGES = 4, GG_THREADS = 192;
static constexpr int GG_A_BYTES = GG_BM * GG_BK * 2, GG_B_BYTES = GG_BN * GG_BK * 2;
static constexpr int GG_STAGE_BYTES = GG_A_BYTES + GG_B_BYTES;
static constexpr int GG_SMEM_BYTES = GG_STAGES * GG_STAGE_BYTES + 1024 + 256;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GG_THREADS, 1)
grouped_gemm_kernel(const GroupDesc* __restrict__ groups, const int2* __restrict__ tiles, int num_tiles, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tbuf = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GG_STAGES * GG_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + GG_STAGES;
  uint64_t* tmem_full = bars + 2 * GG_STAGES;
  uint64_t* tmem_empty = bars + 2 * GG_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GG_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GG_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * GG_BN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int2 tl = tiles[t];
        const GroupDesc* g = groups + tl.x;
        const int tiles_n = (g->N + GG_BN - 1) / GG_BN;
        const int tm = tl.y / tiles_n, tn = tl.y - tm * tiles_n;
        const int k_blocks = (g->K + GG_BK - 1) / GG_BK;
        tmap_acquire(&g->tmap_a);
        tmap_acquire(&g->tmap_b);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % GG_STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / GG_STAGES) & 1) ^ 1, abort_flag)) {
            atomicCAS(status, 0, LF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = tbuf + s * GG_STAGE_BYTES;
          uint8_t* sb = sa + GG_A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], GG_STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < GG_BM / 64; ++j)
              tma_load_2d(sa + j * (GG_BK * 128), &g->tmap_a, &full_bar[s], tm * GG_BM + j * 64, kb * GG_BK);
          } else {
            tma_load_2d(sa, &g->tmap_a, &full_bar[s], kb * GG_BK, tm * GG_BM);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < GG_BN / 64; ++j)
              tma_load_2d(sb + j * (GG_BK * 128), &g->tmap_b, &full_bar[s], tn * GG_BN + j * 64, kb * GG_BK);
          } else {
            tma_load_2d(sb, &g->tmap_b, &full_bar[s], kb * GG_BK, tn * GG_BN);
          }
        }
      }
      if (*abort_flag) {
        const uint32_t first = it > GG_STAGES ? it - GG_STAGES : 0;
        for (uint32_t j = first; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[j % GG_STAGES], (j / GG_STAGES) & 1))
            if (clock64() - t0 > (LF_WAIT_BUDGET_CYCLES >> 4)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, GG_BM, GG_BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++acc_it) {
        const GroupDesc* g = groups + tiles[t].x;
        const int k_blocks = (g->K + GG_BK - 1) / GG_BK;
        const uint32_t acc = acc_it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((acc_it >> 1) & 1) ^ 1, abort_flag)) {
          atomicCAS(status, 0, LF_ERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * GG_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % GG_STAGES;
          if (!mbar_wait(&full_bar[s], (it / GG_STAGES) & 1, abort_flag)) {
            atomicCAS(status, 0, LF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tbuf + s * GG_STAGE_BYTES);
          const uint32_t sb = sa + GG_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GG_BK / GG_UMMA_K; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * (GG_UMMA_K * 128), GG_BK * 128, 1024)
                                     : make_smem_desc_sw128(sa + kk * (GG_UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * (GG_UMMA_K * 128), GG_BK * 128, 1024)
                                     : make_smem_desc_sw128(sb + kk * (GG_UMMA_K * 2), 16, 1024);
            tc_mma_f16_ss(tmem_d, da, db, idesc, (kb | kk) != 0);
          }
          tc_commit(&empty_bar[s]);
        }
        // a group with K == 0 (expert without tokens in wgrad) contributes nothing: the epilogue skips it
        if (ok) tc_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t acc_it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++acc_it) {
      const int2 tl = tiles[t];
      const GroupDesc* g = groups + tl.x;
      const int tiles_n = (g->N + GG_BN - 1) / GG_BN;
      const int tm = tl.y / tiles_n, tn = tl.y - tm * tiles_n;
      const uint32_t acc = acc_it & 1;
      if (!mbar_wait_warp(&tmem_full[acc], (acc_it >> 1) & 1, abort_flag)) {
        if (lane == 0) atomicCAS(status, 0, LF_ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * GG_BM + quarter * 32 + lane;
      const bool row_ok = row < g->M && g->K > 0;
      const uint32_t taddr = tmem_base + acc * GG_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int N = g->N;
#pragma unroll 1
      for (int c0 = 0; c0 < GG_BN; c0 += 32) {
        const int col = tn * GG_BN + c0;
        if (col >= N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c0, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (g->out_mode == 0) {
          __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(g->D) + static_cast<long long>(row) * g->ldd + col;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col + j + 8 <= N) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
              *reinterpret_cast<uint4*>(d + j) = o;
            }
          }
        } else {
          float* d = reinterpret_cast<float*>(g->D) + static_cast<long long>(row) * g->ldd + col;
          const bool accumulate = g->out_mode == 2;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (col + j + 4 <= N) {
              float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                     __uint_as_float(r[j + 3]));
              if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(d + j);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(d + j) = o;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * GG_BN);
  }
}

int grouped_gemm_fill_desc(GroupDesc* d, const void* A, long long lda, const void* B, long long ldb, void* D,
                           long long ldd, int M, int N, int K, bool a_mn, bool b_mn, int out_mode) {
  int rc;
  // a group without rows still needs valid descriptors: describe one (never stored) row
  const int Mm = M > 0 ? M : 1, Kk = K > 0 ? K : 1;
  if (a_mn)
    rc = make_tmap_bf16_2d(&d->tmap_a, A, Kk, Mm, lda, GG_BK, 64);
  else
    rc = make_tmap_bf16_2d(&d->tmap_a, A, Mm, Kk, lda, GG_BM, GG_BK);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_bf16_2d(&d->tmap_b, B, Kk, N, ldb, GG_BK, 64);
  else
    rc = make_tmap_bf16_2d(&d->tmap_b, B, N, Kk, ldb, GG_BN, GG_BK);
  if (rc) return rc;
  d->D = D;
  d->ldd = ldd;
  d->M = M;
  d->N = N;
  d->K = K;
  d->out_mode = out_mode;
  return 0;
}

int grouped_gemm_tiles_for(int M, int N) { return ((M + GG_BM - 1) / GG_BM) * ((N + GG_BN - 1) / GG_BN); }

template <bool A_MN, bool B_MN>
static int gg_launch(const GroupDesc* groups, const int2* tiles, int num_tiles, int* status, cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<A_MN, B_MN>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GG_SMEM_BYTES) != cudaSuccess) return -4;
    attr = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int grid = num_tiles < sms ? num_tiles : sms;
  if (grid <= 0) return 0;
  kern<<<grid, GG_THREADS, GG_SMEM_BYTES, stream>>>(groups, tiles, num_tiles, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int grouped_gemm_launch(const GroupDesc* groups_dev, const void* tiles_dev, int num_tiles, bool a_mn, bool b_mn,
                        int* status, cudaStream_t stream) {
  const int2* tiles = static_cast<const int2*>(tiles_dev);
  if (a_mn && b_mn) return gg_launch<true, true>(groups_dev, tiles, num_tiles, status, stream);
  if (!a_mn && b_mn) return gg_launch<false, true>(groups_dev, tiles, num_tiles, status, stream);
  if (!a_mn && !b_mn) return gg_launch<false, false>(groups_dev, tiles, num_tiles, status, stream);
  return gg_launch<true, false>(groups_dev, tiles, num_tiles, status, stream);
}

}  // namespace lf
