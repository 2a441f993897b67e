// FP8 (e4m3) block quantisers and the blockwise-scaled FP8 GEMM for sm_100a.
//
//   quant_1x128   : bf16 [M, K] -> e4m3 [M, K] + fp32 scales [M, K/128]   (activations; one warp per 128-wide group)
//   quant_128x128 : bf16 [N, K] -> e4m3 [N, K] + fp32 scales [N/128, K/128] (weights; one CTA per block)
//   gemm_fp8_blockwise : D[M, N] (bf16) = sum_kb (sa[m, kb] * sb[n/128, kb]) * (A_q[m, kb-block] . B_q[n, kb-block])
//
// The GEMM runs tcgen05.mma.kind::f8f6f4 (128 x 128 x 32 per instruction) on 128B-swizzled K-major tiles
// (one 128-byte swizzle row = 128 fp8 values = one scale block). Every 128-wide K block is accumulated into a FRESH
// TMEM accumulator (double buffered); the epilogue warps read it, multiply by the two block scales and add it to fp32
// register accumulators — the two-level accumulation that blockwise FP8 recipes use to keep precision.
// Roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 scale-and-accumulate epilogue.
//
// Replaces TE's Float8BlockQuantizer and blockwise FP8 GEMM that the reference uses for DeepSeek-V3.2 FP8 training
// (loongforge/models/common/experimental_attention_variant/dsa_fused_kernels.py:2308-2346 quantiser call sites).
#include <cuda_fp8.h>

#include "fp8_sm100.h"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace lf {

static constexpr float kE4M3Max = 448.0f;

__device__ __forceinline__ float warp_absmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float block_scale(float amax, int pow2) {
  // exact arithmetic (the file is built with fast-math): IEEE division, and the next power of two from the bits
  float s = __fdiv_rn(fmaxf(amax, 1e-12f), kE4M3Max);
  if (pow2) {
    const uint32_t bits = __float_as_uint(s);  // positive, normal
    const uint32_t e = (bits >> 23) + ((bits & 0x7fffffu) ? 1u : 0u);
    s = __uint_as_float(e << 23);
  }
  return s;
}

// One warp per (row, 128-column group): lane handles 4 consecutive values.
__global__ void __launch_bounds__(256) quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                          float* __restrict__ scales, long long M, int K, int pow2) {
  const int lane = threadIdx.x & 31;
  const int groups = K >> 7;
  const long long total = M * groups;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += stride) {
    const long long row = w / groups;
    const int g = static_cast<int>(w - row * groups);
    const long long base = row * K + g * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(x + base);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
    amax = warp_absmax(amax);
    const float s = block_scale(amax, pow2);
    const float inv = 1.0f / s;
    __nv_fp8x4_e4m3 packed(make_float4(a.x * inv, a.y * inv, b.x * inv, b.y * inv));
    *reinterpret_cast<uint32_t*>(q + base) = *reinterpret_cast<uint32_t*>(&packed);
    if (lane == 0) scales[w] = s;
  }
}

// One CTA (256 threads) per 128 x 128 block: thread t handles row t/2, half-row (64 values) t%2.
__global__ void __launch_bounds__(256) quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                                            float* __restrict__ scales, int N, int K, int pow2) {
  __shared__ float red[8];
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int r = threadIdx.x >> 1, half = threadIdx.x & 1;
  const long long base = static_cast<long long>(nb * 128 + r) * K + kb * 128 + half * 64;
  float v[64];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 raw = *reinterpret_cast<const uint4*>(w + base + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      v[i * 8 + 2 * j] = f.x;
      v[i * 8 + 2 * j + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = warp_absmax(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = block_scale(amax, pow2);
  const float inv = 1.0f / s;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    __nv_fp8x4_e4m3 packed(make_float4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv));
    *reinterpret_cast<uint32_t*>(q + base + 4 * i) = *reinterpret_cast<uint32_t*>(&packed);
  }
  if (threadIdx.x == 0) scales[static_cast<long long>(nb) * gridDim.x + kb] = s;
}

int quant_1x128(const void* x, void* q, float* scales, long long M, int K, int pow2, cudaStream_t st) {
  if (K % 128 != 0) return -1;
  if (M == 0) return 0;
  const long long warps = M * (K / 128);
  long long grid = (warps + 7) / 8;
  if (grid > 148 * 16) grid = 148 * 16;
  quant_1x128_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                                  static_cast<uint8_t*>(q), scales, M, K, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int quant_128x128(const void* w, void* q, float* scales, int N, int K, int pow2, cudaStream_t st) {
  if (K % 128 != 0 || N % 128 != 0) return -1;
  if (N == 0) return 0;
  quant_128x128_kernel<<<dim3(K / 128, N / 128), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w),
                                                               static_cast<uint8_t*>(q), scales, N, K, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// ------------------------------------------------------------------------------------------------ FP8 GEMM
static constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128, F8_UMMA_K = 32, F8_STAGES = 6, F8_THREADS = 192;
static constexpr int F8_A_BYTES = F8_BM * F8_BK, F8_B_BYTES = F8_BN * F8_BK, F8_STAGE_BYTES = F8_A_BYTES + F8_B_BYTES;
static constexpr int F8_SMEM_BYTES = F8_STAGES * F8_STAGE_BYTES + 1024 + 256;

struct Fp8GemmParams {
  int M, N, K, tiles_m, tiles_n;
  const float* sa;   // [M, K/128]
  const float* sb;   // [N/128, K/128]
  __nv_bfloat16* D;  // [M, ldd]
  long long ldd;
  int* status;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_blockwise_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const Fp8GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F8_STAGES * F8_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + F8_STAGES;
  uint64_t* tmem_full = bars + 2 * F8_STAGES;       // [2] one per partial-accumulator buffer
  uint64_t* tmem_empty = bars + 2 * F8_STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F8_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = p.K / F8_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * F8_BN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % F8_STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / F8_STAGES) & 1) ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * F8_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], F8_STAGE_BYTES);
          // x coordinate in ELEMENTS of the uint8 map: kb * 128 bytes, a multiple of 16
          tma_load_2d(sa, &tmap_a, &full_bar[s], kb * F8_BK, tm * F8_BM);
          tma_load_2d(sa + F8_A_BYTES, &tmap_b, &full_bar[s], kb * F8_BK, tn * F8_BN);
        }
      }
      if (*abort_flag) {  // let copies already in flight land before the CTA exits
        const uint32_t first = it > F8_STAGES ? it - F8_STAGES : 0;
        for (uint32_t j = first; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[j % F8_STAGES], (j / F8_STAGES) & 1))
            if (clock64() - t0 > (LF_WAIT_BUDGET_CYCLES >> 4)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(0, 0, false, false, F8_BM, F8_BN);  // e4m3 x e4m3 -> fp32
      uint32_t it = 0;  // counts k-blocks globally: stage = it % STAGES, partial buffer = it & 1
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % F8_STAGES;
          const uint32_t buf = it & 1;
          if (!mbar_wait(&tmem_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_EMPTY);
            ok = false;
            break;
          }
          if (!mbar_wait(&full_bar[s], (it / F8_STAGES) & 1, abort_flag)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a0 = smem_u32(smem + s * F8_STAGE_BYTES);
          const uint32_t b0 = a0 + F8_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < F8_BK / F8_UMMA_K; ++kk) {
            const uint64_t da = make_smem_desc_sw128(a0 + kk * F8_UMMA_K, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(b0 + kk * F8_UMMA_K, 16, 1024);
            tc_mma_f8_ss(tmem_base + buf * F8_BN, da, db, idesc, kk != 0);
          }
          tc_commit(&empty_bar[s]);
          tc_commit(&tmem_full[buf]);
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int row = tm * F8_BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      float acc[F8_BN];
#pragma unroll
      for (int c = 0; c < F8_BN; ++c) acc[c] = 0.f;
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1;
        if (!mbar_wait_warp(&tmem_full[buf], (it >> 1) & 1, abort_flag)) {
          if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const float sc = (row_ok ? p.sa[static_cast<long long>(row) * k_blocks + kb] : 0.f) *
                         p.sb[static_cast<long long>(tn) * k_blocks + kb];
        const uint32_t taddr = tmem_base + buf * F8_BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < F8_BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c0 + j] = fmaf(__uint_as_float(r[j]), sc, acc[c0 + j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }
      if (!ok) break;
      if (row_ok) {
        __nv_bfloat16* d = p.D + static_cast<long long>(row) * p.ldd + tn * F8_BN;
#pragma unroll
        for (int c = 0; c < F8_BN; c += 8) {
          if (tn * F8_BN + c + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16x2(acc[c], acc[c + 1]);
            o.y = pack_bf16x2(acc[c + 2], acc[c + 3]);
            o.z = pack_bf16x2(acc[c + 4], acc[c + 5]);
            o.w = pack_bf16x2(acc[c + 6], acc[c + 7]);
            *reinterpret_cast<uint4*>(d + c) = o;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * F8_BN);
  }
}

int gemm_fp8_blockwise(const void* Aq, const float* sa, const void* Bq, const float* sb, void* D, long long ldd, int M,
                       int N, int K, int* status, cudaStream_t stream) {
  if (K % 128 != 0 || N % 128 != 0 || ldd % 8 != 0) return -2;
  if (M == 0) return 0;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_u8_2d(&ta, Aq, M, K, K, F8_BM, F8_BK))) return rc;
  if ((rc = make_tmap_u8_2d(&tb, Bq, N, K, K, F8_BN, F8_BK))) return rc;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gemm_fp8_blockwise_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES) !=
        cudaSuccess)
      return -4;
    attr = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  Fp8GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + F8_BM - 1) / F8_BM;
  p.tiles_n = N / F8_BN;
  p.sa = sa; p.sb = sb;
  p.D = static_cast<__nv_bfloat16*>(D);
  p.ldd = ldd;
  p.status = status;
  const int tiles = p.tiles_m * p.tiles_n;
  gemm_fp8_blockwise_kernel<<<tiles < sms ? tiles : sms, F8_THREADS, F8_SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
