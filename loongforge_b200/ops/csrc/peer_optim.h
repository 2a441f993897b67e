// Host interface of the data-parallel optimizer kernels over NVLink peer memory (peer_optim.cu).
#pragma once
#include <cuda_runtime.h>

namespace lf {

constexpr int kOptMaxPeers = 8;

struct PeerTable {
  void* ptr[kOptMaxPeers] = {};  // same symmetric buffer on every rank of the data-parallel group; index = DP rank
  int world = 1, rank = 0;
};

// Gradient reduce-scatter by PULL, fused with scaling and the squared-norm partial:
//   my_shard[i] = scale * sum_r grads[r][start + i]   (fp32),  *sumsq += sum_i my_shard[i]^2
// `start`, `n` in elements; n % 4 == 0 and start % 4 == 0. The result overwrites this rank's own shard in place.
int grad_pull_reduce(const PeerTable& grads, long long start, long long n, float scale, float* sumsq, cudaStream_t st);

// AdamW on this rank's shard (fp32 master kept as bf16 weight + int16 remainder) fused with the parameter
// all-gather by PUSH: the refreshed bf16 weights are stored to params[r][start + i] on every rank r.
// grad / m / v / lo point at the LOCAL shard (n elements); params are the full symmetric bf16 buffers.
int adam_push(const PeerTable& params, long long start, long long n, short* lo, const float* grad, float* m, float* v,
              float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
              cudaStream_t st);

// Epoch flags for ordering across ranks: flags[r] points at rank r's int[kOptMaxPeers] array (symmetric).
int peer_signal(const PeerTable& flags, int epoch, cudaStream_t st);
int peer_wait(const PeerTable& flags, int epoch, int* status, cudaStream_t st);

}  // namespace lf
