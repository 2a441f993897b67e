// Expert-parallel token exchange over NVLink peer memory: the MoE all-to-all pair as two kernels that
// also do the permutation and the top-k reduction, so no send/receive staging buffers, no index_add.
//
//   moe_push : row x[token(j)] of every (token, expert) pair j is STORED straight into its final,
//              expert-sorted row of the destination rank's receive buffer (all-to-all dispatch +
//              permute + sort-by-local-expert in one pass); optionally one fp32 scalar per pair
//              (the router probability) travels with it. The kernel ends by releasing an arrival
//              flag on every peer.
//   moe_pull : out[t] = sum over the k pairs of token t of the pair's row LOADED from the rank that
//              owns the expert (all-to-all combine + un-permute + top-k sum in one pass, fixed
//              summation order); optionally gathers one fp32 scalar per pair.
//   moe_signal / moe_wait : cross-rank epoch flags (release / bounded acquire spin).
//
// Backward of push is pull and vice versa. Replaces the NCCL all_to_all(v) + permute / unpermute of
// Megatron's alltoall token dispatcher that the reference's MoE layers use
// (loongforge/models/foundation/qwen3/qwen_layer_spec.py:46-55 -> megatron MoELayer).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "moe_peer.h"
#include "wait_budget.h"
#include "sm100_ptx.cuh"

namespace lf {

__device__ __forceinline__ int mp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mp_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct MoePeerPtrs {
  __nv_bfloat16* buf[kMoeMaxPeers];
  float* scal[kMoeMaxPeers];
  int* flags[kMoeMaxPeers];
};

// grid: one CTA per pair (grid-stride), 128 threads, 16-byte vectors
__global__ void __launch_bounds__(128) moe_push_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int H,
                                                       const int* __restrict__ pair_token,
                                                       const int* __restrict__ pair_row, const int* __restrict__ pair_dst,
                                                       const float* __restrict__ pair_scal, MoePeerPtrs pp, int P,
                                                       int cap_rows, int* done_counter, int rank, int world, int kind,
                                                       int epoch, int* status) {
  const int vecs = H >> 3;
  for (int j = blockIdx.x; j < P; j += gridDim.x) {
    const int row = pair_row[j], d = pair_dst[j];
    if (row < 0 || row >= cap_rows || d < 0 || d >= world) {
      if (threadIdx.x == 0) atomicCAS(status, 0, LF_ERR_BAD_INDEX);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(pair_token[j]) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(pp.buf[d] + static_cast<long long>(row) * H);
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = src[i];
    if (pair_scal != nullptr && threadIdx.x == 0) pp.scal[d][row] = pair_scal[j];
  }
  // last CTA out releases the arrival flag on every peer
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(done_counter, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      __threadfence_system();
      *done_counter = 0;
      for (int r = 0; r < world; ++r) mp_st_release_sys(pp.flags[r] + kind * kMoeMaxPeers + rank, epoch);
    }
  }
}

// grid: one CTA per token (grid-stride), 128 threads
__global__ void __launch_bounds__(128) moe_pull_kernel(__nv_bfloat16* __restrict__ out, long long ldo, int H, int T, int k,
                                                       const int* __restrict__ slot_pair,  // [T*k] -> pair index
                                                       const int* __restrict__ pair_row, const int* __restrict__ pair_dst,
                                                       float* __restrict__ slot_scal, MoePeerPtrs pp, int cap_rows,
                                                       int world, int* status) {
  const int vecs = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = 0.f;
      for (int kk = 0; kk < k; ++kk) {
        const int j = slot_pair[t * k + kk];
        const int row = pair_row[j], d = pair_dst[j];
        if (row < 0 || row >= cap_rows || d < 0 || d >= world) continue;
        const uint4 v = reinterpret_cast<const uint4*>(pp.buf[d] + static_cast<long long>(row) * H)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float2 f = __bfloat1622float2(h[c]);
          acc[2 * c] += f.x;
          acc[2 * c + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ldo)[i] = o;
    }
    if (slot_scal != nullptr && threadIdx.x < k) {
      const int j = slot_pair[t * k + threadIdx.x];
      const int row = pair_row[j], d = pair_dst[j];
      const bool ok = row >= 0 && row < cap_rows && d >= 0 && d < world;
      if (!ok) atomicCAS(status, 0, LF_ERR_BAD_INDEX);
      slot_scal[t * k + threadIdx.x] = ok ? pp.scal[d][row] : 0.f;
    }
  }
}

__global__ void moe_signal_kernel(MoePeerPtrs pp, int rank, int world, int kind, int epoch) {
  __threadfence_system();
  if (threadIdx.x < world) mp_st_release_sys(pp.flags[threadIdx.x] + kind * kMoeMaxPeers + rank, epoch);
}

// One warp; lane r waits (bounded) for rank r's flag. On timeout the status word is set and the kernel returns.
__global__ void moe_wait_kernel(const int* flags_local, int world, int kind, int epoch, int* status,
                                long long budget) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const int* p = flags_local + kind * kMoeMaxPeers + r;
  if (mp_ld_acquire_sys(p) >= epoch) return;
  const long long t0 = clock64();
  while (mp_ld_acquire_sys(p) < epoch) {
    __nanosleep(100);
    if (clock64() - t0 > budget) {
      atomicCAS(status, 0, LF_ERR_WAIT_PEER);
      return;
    }
  }
}

static MoePeerPtrs to_ptrs(const MoePeerBufs& b) {
  MoePeerPtrs p;
  for (int r = 0; r < kMoeMaxPeers; ++r) {
    p.buf[r] = static_cast<__nv_bfloat16*>(b.buf[r]);
    p.scal[r] = b.scal[r];
    p.flags[r] = b.flags[r];
  }
  return p;
}

static int mp_grid(int n) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int cap = sms * 16;
  return n < cap ? (n > 0 ? n : 1) : cap;
}

int moe_push(const MoePeerBufs& b, const void* x, long long ldx, int H, const int* pair_token, const int* pair_row,
             const int* pair_dst, const float* pair_scal, int P, int* done_counter, int kind, int epoch, int* status,
             cudaStream_t st) {
  if (H % 8 != 0 || ldx % 8 != 0 || b.world < 1 || b.world > kMoeMaxPeers) return -1;
  moe_push_kernel<<<mp_grid(P), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, H, pair_token, pair_row, pair_dst,
                                              pair_scal, to_ptrs(b), P, b.cap_rows, done_counter, b.rank, b.world, kind,
                                              epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_pull(const MoePeerBufs& b, void* out, long long ldo, int H, int T, int k, const int* slot_pair,
             const int* pair_row, const int* pair_dst, float* slot_scal, int* status, cudaStream_t st) {
  if (H % 8 != 0 || ldo % 8 != 0 || k > 128 || b.world < 1 || b.world > kMoeMaxPeers) return -1;
  if (T <= 0) return 0;
  moe_pull_kernel<<<mp_grid(T), 128, 0, st>>>(static_cast<__nv_bfloat16*>(out), ldo, H, T, k, slot_pair, pair_row,
                                              pair_dst, slot_scal, to_ptrs(b), b.cap_rows, b.world, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_signal(const MoePeerBufs& b, int kind, int epoch, cudaStream_t st) {
  moe_signal_kernel<<<1, 32, 0, st>>>(to_ptrs(b), b.rank, b.world, kind, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_wait(const MoePeerBufs& b, int kind, int epoch, int* status, cudaStream_t st) {
  moe_wait_kernel<<<1, 32, 0, st>>>(b.flags[b.rank], b.world, kind, epoch, status, g_peer_wait_cycles);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
