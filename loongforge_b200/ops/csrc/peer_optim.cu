// Data-parallel optimizer step over NVLink peer memory: the gradient reduce-scatter and the parameter all-gather are
// folded into the two elementwise kernels that touch the same bytes anyway.
//
//   grad_pull_reduce : every rank LOADS its shard of the gradient bucket from all data-parallel peers, sums, scales,
//                      stores the reduced shard locally and accumulates its squared norm (for clipping) — one pass
//                      instead of NCCL reduce-scatter + scale + sum-of-squares.
//   adam_push        : AdamW on the shard, then the refreshed bf16 weights are STORED into every peer's parameter
//                      buffer — one pass instead of Adam + NCCL all-gather.
//
// Between the two only the scalar grad-norm all-reduce remains. Ordering across ranks uses release / acquire epoch
// flags with bounded waits (status word on timeout). Counterpart of the distributed optimizer's reduce-scatter ->
// FusedAdam -> all-gather sequence the reference configures (loongforge/train/training_utils.py:943-991).
#include <cuda_bf16.h>

#include "peer_optim.h"
#include "wait_budget.h"
#include "sm100_ptx.cuh"

namespace lf {

struct PeerPtrs {
  void* p[kOptMaxPeers];
};

static PeerPtrs to_ptrs(const PeerTable& t) {
  PeerPtrs o;
  for (int i = 0; i < kOptMaxPeers; ++i) o.p[i] = t.ptr[i];
  return o;
}

__global__ void __launch_bounds__(256) grad_pull_reduce_kernel(PeerPtrs grads, int world, int rank, long long start,
                                                               long long n4, float scale, float* __restrict__ sumsq) {
  __shared__ float red[8];
  float ss = 0.f;
  float4* mine = reinterpret_cast<float4*>(static_cast<float*>(grads.p[rank]) + start);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // fixed summation order (rank 0, 1, ...) on every rank: replicas that reduce the same data agree bit for bit
    for (int r = 0; r < world; ++r) {
      const float4 g = reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + start)[i];
      acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    mine[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(sumsq, t);
  }
}

__device__ __forceinline__ float po_master_from_parts(__nv_bfloat16 w, short lo) {
  const unsigned hi = static_cast<unsigned>(__bfloat16_as_ushort(w)) << 16;
  return __uint_as_float(hi + static_cast<unsigned>(static_cast<int>(lo)));
}

__global__ void __launch_bounds__(256) adam_push_kernel(PeerPtrs params, int world, int rank, long long start,
                                                        long long n, short* __restrict__ lo,
                                                        const float* __restrict__ grad, float* __restrict__ m,
                                                        float* __restrict__ v, float lr, float beta1, float beta2,
                                                        float eps, float wd, float bc1, float bc2, float grad_scale) {
  const __nv_bfloat16* w_local = static_cast<const __nv_bfloat16*>(params.p[rank]) + start;
  // two elements per thread so that the peer stores are 4-byte
  const long long n2 = n >> 1;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    __nv_bfloat16 wn[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long long e = 2 * i + j;
      const float g = grad[e] * grad_scale;
      const float mi = beta1 * m[e] + (1.f - beta1) * g;
      const float vi = beta2 * v[e] + (1.f - beta2) * g * g;
      float p = po_master_from_parts(w_local[e], lo[e]);
      p -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * p);
      wn[j] = __float2bfloat16_rn(p);
      const unsigned hi = static_cast<unsigned>(__bfloat16_as_ushort(wn[j])) << 16;
      lo[e] = static_cast<short>(static_cast<int>(__float_as_uint(p) - hi));
      m[e] = mi;
      v[e] = vi;
    }
    const unsigned packed = static_cast<unsigned>(__bfloat16_as_ushort(wn[0])) |
                            (static_cast<unsigned>(__bfloat16_as_ushort(wn[1])) << 16);
    for (int r = 0; r < world; ++r)
      reinterpret_cast<unsigned*>(static_cast<__nv_bfloat16*>(params.p[r]) + start)[i] = packed;
  }
}

__global__ void peer_signal_kernel(PeerPtrs flags, int world, int rank, int epoch) {
  __threadfence_system();
  if (threadIdx.x < world)
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(static_cast<int*>(flags.p[threadIdx.x]) + rank), "r"(epoch)
                 : "memory");
}

__global__ void peer_wait_kernel(const int* flags_local, int world, int epoch, int* status, long long budget) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const int* p = flags_local + r;
  const long long t0 = clock64();
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (v >= epoch) return;
    __nanosleep(100);
    if (clock64() - t0 > budget) {
      atomicCAS(status, 0, LF_ERR_WAIT_PEER);
      return;
    }
  }
}

static int grid_for_n(long long work) {
  long long g = (work + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : static_cast<int>(g);
}

int grad_pull_reduce(const PeerTable& grads, long long start, long long n, float scale, float* sumsq, cudaStream_t st) {
  if ((start & 3) || (n & 3) || grads.world < 1 || grads.world > kOptMaxPeers) return -1;
  if (n == 0) return 0;
  grad_pull_reduce_kernel<<<grid_for_n(n >> 2), 256, 0, st>>>(to_ptrs(grads), grads.world, grads.rank, start, n >> 2,
                                                              scale, sumsq);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int adam_push(const PeerTable& params, long long start, long long n, short* lo, const float* grad, float* m, float* v,
              float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
              cudaStream_t st) {
  if ((start & 1) || (n & 1) || params.world < 1 || params.world > kOptMaxPeers) return -1;
  if (n == 0) return 0;
  adam_push_kernel<<<grid_for_n(n >> 1), 256, 0, st>>>(to_ptrs(params), params.world, params.rank, start, n, lo, grad, m,
                                                       v, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int peer_signal(const PeerTable& flags, int epoch, cudaStream_t st) {
  peer_signal_kernel<<<1, 32, 0, st>>>(to_ptrs(flags), flags.world, flags.rank, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int peer_wait(const PeerTable& flags, int epoch, int* status, cudaStream_t st) {
  peer_wait_kernel<<<1, 32, 0, st>>>(static_cast<const int*>(flags.ptr[flags.rank]), flags.world, epoch, status,
                                    g_peer_wait_cycles);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
