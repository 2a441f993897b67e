// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   TMA (cp.async.bulk.tensor) -> 128B-swizzled shared memory -> tcgen05.mma with
//   fp32 accumulators in TMEM (double buffered) -> tcgen05.ld epilogue.
//
// D[M,N] = op(A) * op(B) (+ bias) (+ residual), fp32 accumulate.
//   A operand "K-major"  : global A [M,K] row-major          (forward / dgrad activations)
//   A operand "MN-major" : global At[K,M] row-major          (wgrad: dY^T)
//   B operand "K-major"  : global B [N,K] row-major          (forward: weight [out,in])
//   B operand "MN-major" : global Bt[K,N] row-major          (dgrad: weight, wgrad: X)
// so that forward (X*W^T), dgrad (dY*W) and wgrad (dY^T*X) all run without a
// transposed copy of any operand.
//
// Roles inside one CTA (192 threads, 1 CTA per SM, grid = min(tiles, #SM)):
//   warp 0   : TMA producer (one elected lane)
//   warp 1   : TMEM allocation + tcgen05.mma issue (one elected lane)
//   warps 2-5: epilogue; warp w drains TMEM lanes 32*(w%4) .. 32*(w%4)+31
//
// Replaces the cuBLASLt GEMMs behind TE's Column/RowParallelLinear in the
// reference (loongforge/models/dispatch.py:45-54).
#include "sm100_ptx.cuh"
#include "gemm_sm100.h"

namespace lf {

static constexpr int BM = 128;
static constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
static constexpr int UMMA_K = 16;
static constexpr int NUM_THREADS = 192;
static constexpr int NUM_EPI_WARPS = 4;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  // epilogue transpose patches: one [32 rows x 32 fp32 columns] patch per epilogue warp, rows padded by 16 bytes so
  // that the 16-byte stores of a warp spread over all banks
  static constexpr int STG_ROW = 144;
  static constexpr int STG_BYTES = NUM_EPI_WARPS * 32 * STG_ROW;
  // +1024 for manual 1024-byte alignment of the swizzled tiles, +256 for barriers
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_BYTES + 1024 + 256;
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n;
  int out_mode;          // 0: bf16 store, 1: fp32 store, 2: fp32 accumulate (D += acc)
  void* D;               // [M, ldd]
  long long ldd;         // leading dimension of D in elements
  const __nv_bfloat16* bias;      // [N] or nullptr   (out_mode 0/1)
  const __nv_bfloat16* residual;  // [M, ldr] or nullptr (out_mode 0)
  long long ldr;
  float alpha;           // scales the accumulator before bias/residual
  int* status;           // device int, set to an LF_ERR_* code when a wait gives up
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Group GROUP_M row-tiles so that one wave of CTAs reuses the same B tiles from L2.
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % rows);
  tn = r / rows;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* stage_base = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_base + Cfg::STG_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;   // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = tiles + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmap_a, &full_bar[s], tm * BM + j * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[s], kb * BK, tm * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmap_b, &full_bar[s], tn * BN + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[s], kb * BK, tn * BN);
          }
        }
      }
      // Copies issued by this thread complete on full_bar[]; when the MMA warp
      // stopped consuming (abort) wait, bounded, until they have landed so that no
      // bulk copy is in flight when the CTA exits.
      if (*abort_flag) {
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[j % STAGES], (j / STAGES) & 1)) {
            if (clock64() - t0 > (LF_WAIT_BUDGET_CYCLES >> 4)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, BM, BN);
      uint32_t it = 0;
      uint32_t acc_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
        const uint32_t acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            tc_mma_f16_ss(tmem_d, da, db, idesc, (kb | kk) != 0);
          }
          tc_commit(&empty_bar[s]);  // stage is free once these MMAs retire
        }
        if (ok) tc_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lane quarter this warp may touch
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // Drain: every thread reads 32 accumulator columns of ITS row from TMEM and parks them in a shared-memory patch;
      // the warp then walks the patch transposed, four rows per instruction with eight lanes per row, so that bias,
      // residual, the fp32 read-modify-write of accumulate mode and the stores all touch full contiguous row segments.
      const int row0 = tm * BM + quarter * 32;  // first row of this warp's patch
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      uint8_t* stg = stage_base + quarter * (32 * Cfg::STG_ROW);
      const int piece = lane & 7;   // four consecutive columns of a row
      const int rsub = lane >> 3;   // row inside a group of four
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col = tn * BN + c0;
        if (col >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c0, r);
        tmem_ld_wait();
        __syncwarp();  // the previous chunk's readers are done with the patch
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(stg + lane * Cfg::STG_ROW + j * 4) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        __syncwarp();
        const int c = col + piece * 4;  // first of this lane's four columns
        const bool full4 = c + 4 <= p.N;
        float bias4[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.bias != nullptr) {
#pragma unroll
          for (int t = 0; t < 4; ++t)
            if (c + t < p.N) bias4[t] = __bfloat162float(p.bias[c + t]);
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + rsub;
          const int row = row0 + rr;
          if (row >= p.M || c >= p.N) continue;
          const float4 a4 = *reinterpret_cast<const float4*>(stg + rr * Cfg::STG_ROW + piece * 16);
          float v[4] = {a4.x * p.alpha + bias4[0], a4.y * p.alpha + bias4[1], a4.z * p.alpha + bias4[2],
                        a4.w * p.alpha + bias4[3]};
          if (p.out_mode == 0) {
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + c;
            const __nv_bfloat16* rs = p.residual ? p.residual + static_cast<long long>(row) * p.ldr + c : nullptr;
            if (full4) {
              if (rs) {
                const uint2 q = *reinterpret_cast<const uint2*>(rs);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
                const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
                v[0] += f0.x; v[1] += f0.y; v[2] += f1.x; v[3] += f1.y;
              }
              uint2 o;
              o.x = pack_bf16x2(v[0], v[1]);
              o.y = pack_bf16x2(v[2], v[3]);
              *reinterpret_cast<uint2*>(d) = o;
            } else {
              for (int t = 0; t < 4; ++t)
                if (c + t < p.N) {
                  float x = v[t];
                  if (rs) x += __bfloat162float(rs[t]);
                  d[t] = __float2bfloat16(x);
                }
            }
          } else {
            float* d = reinterpret_cast<float*>(p.D) + static_cast<long long>(row) * p.ldd + c;
            const bool accumulate = p.out_mode == 2;
            if (full4) {
              float4 o = make_float4(v[0], v[1], v[2], v[3]);
              if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(d);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(d) = o;
            } else {
              for (int t = 0; t < 4; ++t)
                if (c + t < p.N) d[t] = accumulate ? d[t] + v[t] : v[t];
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
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  // cuTensorMapEncodeTiled is a driver call: it needs a CUDA context bound to THIS thread, which
  // autograd worker threads do not have until a runtime call binds the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix (leading dimension `ld`
// elements), box = [box_rows, 64 columns], 128-byte swizzle, zero fill out of bounds.
int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld,
                      int box_rows, int box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ((ld * 2) & 15) != 0) return -2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

int make_tmap_u8_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                    int box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld & 15) != 0) return -2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}


template <int BN, bool A_MN, bool B_MN>
static int launch_cfg(const GemmArgs& a, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap ta, tb;
  int rc;
  if (A_MN)
    rc = make_tmap_bf16_2d(&ta, a.A, a.K, a.M, a.lda, BK, 64);
  else
    rc = make_tmap_bf16_2d(&ta, a.A, a.M, a.K, a.lda, BM, BK);
  if (rc) return rc;
  if (B_MN)
    rc = make_tmap_bf16_2d(&tb, a.B, a.K, a.N, a.ldb, BK, 64);
  else
    rc = make_tmap_bf16_2d(&tb, a.B, a.N, a.K, a.ldb, BN, BK);
  if (rc) return rc;
  GemmParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.out_mode = a.out_mode;
  p.D = a.D; p.ldd = a.ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ldr = a.ldr;
  p.alpha = a.alpha;
  p.status = a.status;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN>;
  // per device: the shared-memory opt-in of this instantiation and the SM count (a process may drive several GPUs)
  constexpr int kMaxDev = 64;
  static bool attr_set[kMaxDev] = {};
  static int num_sms[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -4;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -4;
    cudaDeviceGetAttribute(&num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    attr_set[dev] = true;
  }
  const int dev_sms = num_sms[dev];
  int sms = a.max_ctas > 0 ? (a.max_ctas < dev_sms ? a.max_ctas : dev_sms) : dev_sms;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sms ? tiles : sms;
  if (grid <= 0) return 0;
  kern<<<grid, NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return 0;
  // Alignment rules of the vectorised epilogue and of TMA (16-byte rows).
  if ((a.ldd % 8) != 0 || (a.lda % 8) != 0 || (a.ldb % 8) != 0) return -2;
  if (a.residual != nullptr && (a.ldr % 8) != 0) return -2;
  const bool small_n = a.N <= 128;
  const int key = (small_n ? 4 : 0) | (a.a_mn_major ? 2 : 0) | (a.b_mn_major ? 1 : 0);
  switch (key) {
    case 0: return launch_cfg<256, false, false>(a, stream);
    case 1: return launch_cfg<256, false, true>(a, stream);
    case 2: return launch_cfg<256, true, false>(a, stream);
    case 3: return launch_cfg<256, true, true>(a, stream);
    case 4: return launch_cfg<128, false, false>(a, stream);
    case 5: return launch_cfg<128, false, true>(a, stream);
    case 6: return launch_cfg<128, true, false>(a, stream);
    default: return launch_cfg<128, true, true>(a, stream);
  }
}

}  // namespace lf
