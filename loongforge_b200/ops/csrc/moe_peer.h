// Host interface of the expert-parallel token exchange over peer memory (moe_peer.cu).
#pragma once
#include <cuda_runtime.h>

namespace lf {

constexpr int kMoeMaxPeers = 8;

// Symmetric buffers of one expert-parallel group; index r = rank r of the group (own rank included).
struct MoePeerBufs {
  void* buf[kMoeMaxPeers] = {};    // bf16 [cap_rows, H] rows, written by push / read by pull
  float* scal[kMoeMaxPeers] = {};  // fp32 [cap_rows] one scalar per row
  int* flags[kMoeMaxPeers] = {};   // int [2 kinds][kMoeMaxPeers] arrival epochs
  int rank = 0, world = 1, cap_rows = 0;
};

// Pair j = one (token, expert) assignment: x[pair_token[j]] goes to row pair_row[j] of rank pair_dst[j].
// Ends by releasing flag (kind, rank) = epoch on every peer. `done_counter`: zero-initialised device int.
int moe_push(const MoePeerBufs& b, const void* x, long long ldx, int H, const int* pair_token, const int* pair_row,
             const int* pair_dst, const float* pair_scal, int P, int* done_counter, int kind, int epoch, int* status,
             cudaStream_t st);
// out[t] = sum_{kk<k} row of pair slot_pair[t*k+kk]; slot_scal[t*k+kk] = that row's scalar (optional).
int moe_pull(const MoePeerBufs& b, void* out, long long ldo, int H, int T, int k, const int* slot_pair,
             const int* pair_row, const int* pair_dst, float* slot_scal, int* status, cudaStream_t st);
int moe_signal(const MoePeerBufs& b, int kind, int epoch, cudaStream_t st);
// Waits (bounded by the run-time peer budget of wait_budget.h) until every rank's flag of `kind` reached `epoch`; sets *status on timeout.
int moe_wait(const MoePeerBufs& b, int kind, int epoch, int* status, cudaStream_t st);

}  // namespace lf
