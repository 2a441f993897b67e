// MoE router: score function + (group-limited) top-k + dense probs / routing map / per-expert counts in ONE
// launch, one warp per token with the whole expert row in registers; and its backward.
//
// Semantics follow Megatron's topk_softmax_with_capacity as the reference carries it
// (loongforge/models/foundation/ernie4_5_vl/ernie_router.py:32-140):
//   score 0  softmax over the selected k logits (post-softmax);   aux scores = softmax over all experts
//   score 1  softmax over all experts, top-k of it (pre-softmax); aux scores = the same softmax
//   score 2  sigmoid, selected values normalised by their sum when k > 1; aux scores = s / sum(s)
// `bias` (optional, fp32 [E]) shifts the SELECTION scores only. Group-limited selection keeps the
// `group_topk` groups with the largest sum of their top-(k / group_topk) selection scores.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "elementwise.h"

namespace lf {

static constexpr int RT_MAX_SLOTS = 16;  // experts per lane: E <= 512
static constexpr int RT_MAX_K = 32;

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, a.v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, a.i, o);
    if (ov > a.v || (ov == a.v && oi < a.i)) {
      a.v = ov;
      a.i = oi;
    }
  }
  return a;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename TIn>
__device__ __forceinline__ float load_logit(const TIn* p);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename TIn, int SLOTS>
__global__ void __launch_bounds__(128) router_fwd_kernel(const TIn* __restrict__ logits, const float* __restrict__ bias,
                                                         float* __restrict__ probs, uint8_t* __restrict__ map,
                                                         float* __restrict__ aux, int* __restrict__ topk_idx,
                                                         int* __restrict__ counts, int T, int E, int k, int score,
                                                         int num_groups, int group_topk, float scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const TIn* row = logits + static_cast<long long>(t) * E;
  float l[SLOTS], s[SLOTS], sel[SLOTS];
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int e = lane + 32 * j;
    l[j] = e < E ? load_logit<TIn>(row + e) : -FLT_MAX;
    mx = fmaxf(mx, l[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  if (score == 2) {
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      s[j] = lane + 32 * j < E ? 1.f / (1.f + __expf(-l[j])) : 0.f;
      sum += s[j];
    }
  } else {
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      s[j] = lane + 32 * j < E ? __expf(l[j] - mx) : 0.f;
      sum += s[j];
    }
  }
  sum = warp_sum(sum);
  const float inv = score == 2 ? 1.f / (sum + 1e-20f) : 1.f / sum;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int e = lane + 32 * j;
    if (score != 2) s[j] *= inv;  // full softmax
    if (e < E) {
      aux[static_cast<long long>(t) * E + e] = score == 2 ? s[j] * inv : s[j];
      const float base = score == 0 ? l[j] : s[j];
      sel[j] = base + (bias != nullptr ? bias[e] : 0.f);
    } else {
      sel[j] = -FLT_MAX;
    }
  }
  // ---- group-limited selection: mask out experts of groups that are not kept
  if (num_groups > 1 && group_topk > 0 && group_topk < num_groups) {
    const int per = E / num_groups;
    const int m = max(k / group_topk, 1);
    float gscore = -FLT_MAX;  // lane g holds the score of group g (num_groups <= 32)
    for (int g = 0; g < num_groups; ++g) {
      uint32_t taken = 0;
      float acc = 0.f;
      for (int r = 0; r < m; ++r) {
        ArgMax best{-FLT_MAX, 0x7fffffff};
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
          const int e = lane + 32 * j;
          if (e < E && e / per == g && !((taken >> j) & 1u) && (sel[j] > best.v || (sel[j] == best.v && e < best.i))) {
            best.v = sel[j];
            best.i = e;
          }
        }
        best = warp_argmax(best);
        if (best.i != 0x7fffffff) {
          acc += best.v;
          if ((best.i & 31) == lane) taken |= 1u << (best.i >> 5);
        }
      }
      if (lane == g) gscore = acc;
    }
    uint32_t keep = 0;
    for (int r = 0; r < group_topk; ++r) {
      ArgMax best{(keep >> lane) & 1u ? -FLT_MAX : gscore, lane < num_groups && !((keep >> lane) & 1u) ? lane : 0x7fffffff};
      if (best.i == 0x7fffffff) best.v = -FLT_MAX;
      best = warp_argmax(best);
      if (best.i != 0x7fffffff) keep |= 1u << best.i;
    }
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      const int e = lane + 32 * j;
      if (e < E && !((keep >> (e / per)) & 1u)) sel[j] = -FLT_MAX;
    }
  }
  // ---- top-k by k rounds of warp arg-max
  uint32_t chosen = 0;  // bit j: this lane's slot j is selected
  float csum = 0.f, cmax = -FLT_MAX;
  for (int r = 0; r < k; ++r) {
    ArgMax best{-FLT_MAX, 0x7fffffff};
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      const int e = lane + 32 * j;
      if (e < E && !((chosen >> j) & 1u) && (sel[j] > best.v || (sel[j] == best.v && e < best.i))) {
        best.v = sel[j];
        best.i = e;
      }
    }
    best = warp_argmax(best);
    if (best.i == 0x7fffffff) break;
    if ((best.i & 31) == lane) chosen |= 1u << (best.i >> 5);
    if (lane == 0) topk_idx[static_cast<long long>(t) * k + r] = best.i;
  }
  // ---- values of the selected experts
  if (score == 0) {
#pragma unroll
    for (int j = 0; j < SLOTS; ++j)
      if ((chosen >> j) & 1u) cmax = fmaxf(cmax, l[j]);
    cmax = warp_max(cmax);
  }
  float v[SLOTS];
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    v[j] = 0.f;
    if ((chosen >> j) & 1u) {
      v[j] = score == 0 ? __expf(l[j] - cmax) : s[j];
      csum += v[j];
    }
  }
  csum = warp_sum(csum);
  float norm = 1.f;
  if (score == 0) norm = 1.f / csum;
  if (score == 2 && k > 1) norm = 1.f / (csum + 1e-20f);
  norm *= scale;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int e = lane + 32 * j;
    if (e < E) {
      const bool on = (chosen >> j) & 1u;
      probs[static_cast<long long>(t) * E + e] = on ? v[j] * norm : 0.f;
      map[static_cast<long long>(t) * E + e] = on ? 1 : 0;
      if (on && counts != nullptr) atomicAdd(&counts[e], 1);
    }
  }
}

// Backward: dlogits [T, E] fp32 from dprobs (read only at selected experts) and daux (optional).
// Scores are recomputed from the logits; only the routing map is saved by the forward.
template <typename TIn, int SLOTS>
__global__ void __launch_bounds__(128) router_bwd_kernel(const TIn* __restrict__ logits, const uint8_t* __restrict__ map,
                                                         const float* __restrict__ dprobs, const float* __restrict__ daux,
                                                         float* __restrict__ dlogits, int T, int E, int k, int score,
                                                         float scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const long long base = static_cast<long long>(t) * E;
  float l[SLOTS], s[SLOTS], dp[SLOTS], da[SLOTS], out[SLOTS];
  bool on[SLOTS];
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int e = lane + 32 * j;
    const bool ok = e < E;
    l[j] = ok ? load_logit<TIn>(logits + base + e) : -FLT_MAX;
    mx = fmaxf(mx, l[j]);
    on[j] = ok && map[base + e] != 0;
    dp[j] = on[j] ? dprobs[base + e] : 0.f;
    da[j] = ok && daux != nullptr ? daux[base + e] : 0.f;
  }
  mx = warp_max(mx);
  float S = 0.f;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const bool ok = lane + 32 * j < E;
    s[j] = !ok ? 0.f : (score == 2 ? 1.f / (1.f + __expf(-l[j])) : __expf(l[j] - mx));
    S += s[j];
  }
  S = warp_sum(S);
  if (score != 2) {
    const float inv = 1.f / S;
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) s[j] *= inv;  // full softmax
  }
  if (score == 0) {
    // probs = scale * softmax over the selected logits; aux = full softmax
    float cmax = -FLT_MAX, csum = 0.f, p[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j)
      if (on[j]) cmax = fmaxf(cmax, l[j]);
    cmax = warp_max(cmax);
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      p[j] = on[j] ? __expf(l[j] - cmax) : 0.f;
      csum += p[j];
    }
    csum = warp_sum(csum);
    float d1 = 0.f, d2 = 0.f;
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      p[j] /= csum;
      d1 += dp[j] * p[j];
      d2 += da[j] * s[j];
    }
    d1 = warp_sum(d1);
    d2 = warp_sum(d2);
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) out[j] = scale * p[j] * (dp[j] - d1) + s[j] * (da[j] - d2);
  } else if (score == 1) {
    float d = 0.f;
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      da[j] += dp[j] * scale;
      d += da[j] * s[j];
    }
    d = warp_sum(d);
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) out[j] = s[j] * (da[j] - d);
  } else {
    const float Se = S + 1e-20f;
    float C = 0.f, d1 = 0.f, d2 = 0.f;
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      if (on[j]) C += s[j];
      d1 += dp[j] * s[j];
      d2 += da[j] * s[j];
    }
    C = warp_sum(C) + 1e-20f;
    d1 = warp_sum(d1);
    d2 = warp_sum(d2);
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      float ds = da[j] / Se - d2 / (Se * Se);
      if (on[j]) ds += k > 1 ? scale * (dp[j] / C - d1 / (C * C)) : scale * dp[j];
      out[j] = ds * s[j] * (1.f - s[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int e = lane + 32 * j;
    if (e < E) dlogits[base + e] = out[j];
  }
}

template <typename TIn>
static int router_fwd_t(const RouterArgs& a, cudaStream_t st) {
  const int warps = 4;
  const dim3 grid((a.T + warps - 1) / warps), block(warps * 32);
  const TIn* lg = static_cast<const TIn*>(a.logits);
#define LF_RT_FWD(S)                                                                                             \
  router_fwd_kernel<TIn, S><<<grid, block, 0, st>>>(lg, a.bias, a.probs, a.map, a.aux, a.topk_idx, a.counts, a.T, \
                                                    a.E, a.k, a.score, a.num_groups, a.group_topk, a.scale)
  if (a.E <= 64) LF_RT_FWD(2);
  else if (a.E <= 128) LF_RT_FWD(4);
  else if (a.E <= 256) LF_RT_FWD(8);
  else LF_RT_FWD(16);
#undef LF_RT_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <typename TIn>
static int router_bwd_t(const RouterArgs& a, cudaStream_t st) {
  const int warps = 4;
  const dim3 grid((a.T + warps - 1) / warps), block(warps * 32);
  const TIn* lg = static_cast<const TIn*>(a.logits);
#define LF_RT_BWD(S)                                                                                         \
  router_bwd_kernel<TIn, S><<<grid, block, 0, st>>>(lg, a.map, a.dprobs, a.daux, a.dlogits, a.T, a.E, a.k, \
                                                    a.score, a.scale)
  if (a.E <= 64) LF_RT_BWD(2);
  else if (a.E <= 128) LF_RT_BWD(4);
  else if (a.E <= 256) LF_RT_BWD(8);
  else LF_RT_BWD(16);
#undef LF_RT_BWD
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

static int router_check(const RouterArgs& a) {
  if (a.T <= 0) return 1;
  if (a.E <= 0 || a.E > 32 * RT_MAX_SLOTS || a.k <= 0 || a.k > RT_MAX_K || a.k > a.E) return -1;
  if (a.num_groups > 1 && (a.num_groups > 32 || a.E % a.num_groups != 0)) return -2;
  return 0;
}

int router_fwd(const RouterArgs& a, cudaStream_t st) {
  const int rc = router_check(a);
  if (rc != 0) return rc < 0 ? rc : 0;
  return a.logits_bf16 ? router_fwd_t<__nv_bfloat16>(a, st) : router_fwd_t<float>(a, st);
}

int router_bwd(const RouterArgs& a, cudaStream_t st) {
  const int rc = router_check(a);
  if (rc != 0) return rc < 0 ? rc : 0;
  return a.logits_bf16 ? router_bwd_t<__nv_bfloat16>(a, st) : router_bwd_t<float>(a, st);
}

}  // namespace lf
