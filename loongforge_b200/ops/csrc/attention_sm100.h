// Host interface of the tcgen05 flash-attention kernels (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>

namespace lf {

// Packed-token ("thd") attention, head dim D <= 128 (a multiple of 8), bf16 in/out, fp32 softmax statistics.
// Queries ([Tq] tokens) and keys / values ([Tk] tokens) may differ in length (context-parallel chunks, prefixes):
// a causal mask is aligned to the bottom right, query row i of a sequence sees keys j <= i + (k_len - q_len).
// Q head h belongs to KV group g = h / R (R = Hq / Hkv) and is element offset
// t*q_ts + g*q_gs + (h % R)*q_hs from `q`; K/V head g of token t is at t*k_ts + g*k_hs.
// This lets q, k and v be views into ONE packed [T, Hkv, R + 2, 128] QKV buffer (and dq, dk,
// dv views into one packed gradient buffer), so no split/concat copies are needed.
// o and dout are [Tq, Hq, D] with strides (o_ts, o_hs) / (do_ts, do_hs).
struct AttnArgs {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  void* o = nullptr;
  float* lse = nullptr;        // [Hq, Tq] natural-log sum-exp of the scaled scores (-inf: the row saw no key)
  const void* dout = nullptr;  // backward only
  void* dq = nullptr;
  void* dk = nullptr;
  void* dv = nullptr;
  float* delta = nullptr;      // [Hq, Tq] scratch: rowsum(dO * O)
  int Tq = 0, Tk = 0, Hq = 0, Hkv = 0, D = 128;
  long long q_ts = 0, q_gs = 0, q_hs = 0;
  long long k_ts = 0, k_hs = 0, v_ts = 0, v_hs = 0;
  long long o_ts = 0, o_hs = 0, do_ts = 0, do_hs = 0;
  long long dq_ts = 0, dq_gs = 0, dq_hs = 0, dk_ts = 0, dk_hs = 0, dv_ts = 0, dv_hs = 0;
  float scale = 1.0f;
  bool causal = true;
  // device int32 [num_seqs + 1] sequence boundaries on the query and on the key side; nullptr = one sequence.
  // cu_seqlens_k == nullptr means "same as the query side".
  const int* cu_seqlens_q = nullptr;
  const int* cu_seqlens_k = nullptr;
  int num_seqs = 1;
  int* status = nullptr;
};

// Return 0 on success, negative on invalid arguments (alignment: every stride a multiple of 8).
int attn_fwd(const AttnArgs& a, cudaStream_t stream);
int attn_bwd(const AttnArgs& a, cudaStream_t stream);

}  // namespace lf
