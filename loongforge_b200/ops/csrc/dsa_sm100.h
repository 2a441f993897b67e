// Host interface of the DeepSeek sparse attention kernels (dsa_sm100.cu).
#pragma once
#include <cuda_runtime.h>

namespace lf {

// Top-k sparse attention on the absorbed multi-latent form (key dims 576 = 512 latent + 64 rope, value = the first
// 512 key dims). q [m, H <= 128, 576] bf16 with element strides (q_ts, q_hs); kv [n_kv, 576] bf16 with row stride
// kv_ts; idx [m, topk] int32, -1 = empty slot; o [m, H, 512] bf16 with strides (o_ts, o_hs); lse [m, H] fp32 (natural
// log-sum-exp of the scaled scores over the selected keys, -inf when a token selected nothing).
struct SparseMlaArgs {
  const void* q = nullptr;
  long long q_ts = 0, q_hs = 0;
  const void* kv = nullptr;
  long long kv_ts = 0;
  const int* idx = nullptr;
  int topk = 0, m = 0, H = 0, n_kv = 0;
  float scale = 1.f;
  void* o = nullptr;
  long long o_ts = 0, o_hs = 0;
  float* lse = nullptr;
  float* pmean = nullptr;  // sparse_mla_probs only: [m, topk] fp32
  int* status = nullptr;
};

// 0 on success, negative on invalid arguments (alignment: strides multiples of 8 elements, bases 16-byte aligned).
int sparse_mla_fwd(const SparseMlaArgs& a, cudaStream_t stream);

// Second pass for the indexer loss: with `lse` of the forward as INPUT, writes pmean[m, s] = mean over heads of the
// attention probability of selected slot s (0 for empty slots). `o` is not used.
int sparse_mla_probs(const SparseMlaArgs& a, cudaStream_t stream);

// Lightning-indexer logits logits[t, j] = sum_h w[t, h] * relu(q[t, h, :] . k[j, :]) for the keys j in
// [k_start[t], k_end[t]) of every query t (entries outside that range are left unwritten). q [m, Hi, 128] bf16
// contiguous, Hi in {32, 64, 128, 256}; k [n, 128] bf16 with row stride k_ld; w [m, Hi] fp32; logits [m, ld] fp32.
struct IndexerArgs {
  const void* q = nullptr;
  const void* k = nullptr;
  long long k_ld = 128;
  const float* w = nullptr;
  const int* k_start = nullptr;
  const int* k_end = nullptr;
  float* logits = nullptr;
  long long ld = 0;
  int m = 0, n = 0, Hi = 64;
  int* status = nullptr;
};
int indexer_logits(const IndexerArgs& a, cudaStream_t stream);

// Indices of the `topk` largest logits of every row inside [k_start, k_end) (unordered; -1 pads short rows) -> out
// [m, topk] int32. `max_len` bounds k_end - k_start over all rows and must not exceed 49152.
int topk_range(const float* logits, long long ld, const int* k_start, const int* k_end, int* out, int m, int topk,
               int max_len, cudaStream_t stream);

}  // namespace lf
