// Fused tensor-parallel GEMMs over NVLink peer memory (peer_gemm.cu).
//
//   ag_gemm : Y[T, N] = all_gather(X)[T, K] * op(B)      (sequence-parallel all-gather -> GEMM)
//   gemm_rs : Y[T/W, N] = reduce_scatter(X[T, K] * op(B)) (+ residual)   (GEMM -> reduce-scatter)
//
// Both are ONE kernel launch per rank: the collective's bytes move with SM-issued bulk copies /
// stores to and from peer pointers while the tcgen05 tiles run, gated by per-tile flags.
// All peer buffers come from one symmetric allocation per rank (same layout on every rank).
#pragma once
#include <cuda_runtime.h>

namespace lf {

constexpr int kMaxPeers = 8;

struct AgGemmArgs {
  // X shards: peer_x[r] points at rank r's [rows_per_rank, K] bf16 shard (own shard included)
  const void* peer_x[kMaxPeers] = {};
  int* peer_sync[kMaxPeers] = {};   // per rank: int[kMaxPeers] arrival counters (symmetric)
  void* x_full = nullptr;           // local [T, K] bf16 gather buffer (own rows are copied too)
  int* chunk_flags = nullptr;       // local int[T / 128]: row block r of x_full is complete when == epoch
  const void* B = nullptr;          // weight: [N, K] (K-major) or [K, N] (MN-major), leading dim ldb
  long long ldb = 0;
  bool b_mn_major = false;
  void* out = nullptr;              // [T, N] bf16, leading dim ldo
  long long ldo = 0;
  const void* bias = nullptr;
  int rank = 0, world = 1, rows_per_rank = 0, K = 0, N = 0;
  int epoch = 1;                    // strictly increasing per call on this (buffer, group)
  int copy_ctas = 8;
  int* status = nullptr;
};

struct GemmRsArgs {
  const void* A = nullptr;          // [T, K] bf16 local activations (leading dim lda)
  long long lda = 0;
  const void* B = nullptr;          // [N, K] or [K, N]
  long long ldb = 0;
  bool b_mn_major = false;
  // receive buffers: peer_recv[r] = rank r's bf16 [2 parities][world sources][rows_per_rank][N]
  void* peer_recv[kMaxPeers] = {};
  // tile counters: peer_tile_flags[r] = rank r's int [2][world][tiles_per_rank]
  int* peer_tile_flags[kMaxPeers] = {};
  void* out = nullptr;              // [T / world, N] bf16
  long long ldo = 0;
  const void* residual = nullptr;   // [T / world, N] bf16 or nullptr
  long long ldr = 0;
  int rank = 0, world = 1, T = 0, K = 0, N = 0;
  int call_index = 0;               // 0, 1, 2, ... per (buffer, group); parity selects the receive buffer
  int* status = nullptr;
};

int ag_gemm(const AgGemmArgs& a, cudaStream_t stream);
int gemm_rs(const GemmRsArgs& a, cudaStream_t stream);

}  // namespace lf
