// Bandwidth-bound kernels of the transformer layer, written for HBM3e: 16-byte
// vector accesses, one pass over the activations wherever the row fits in registers.
//   RMSNorm fwd/bwd      (TE LayerNormLinear norm part / apex FusedRMSNorm in the reference,
//                         loongforge/models/common/local_layers/local_norm.py:14-26)
//   RoPE fwd/bwd         (TE fused_rope with the mscale patch,
//                         patches/TransformerEngine_v2.9/.../fused_rope.cu.patch:1-179, and the Triton
//                         rotary kernels in .../experimental_attention_variant/dsa_fused_kernels.py:69-603)
//   SwiGLU fwd/bwd       (fused_bias_swiglu, loongforge/models/dispatch.py:56)
//   cross-entropy stats + in-place dlogits for the chunked linear+CE path
//                        (docs/source/features/fused_linear_cross_entropy.md:7-44)
//   fused AdamW on flat shards with fp32 or bf16 moments
//                        (patches/.../optimizers/fused_adam.py.patch:18-350)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "elementwise.h"

namespace lf {

using bf16 = __nv_bfloat16;

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
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? sh[l] : 0.f;
  t = warp_sum(t);
  return t;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? sh[l] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

// ============================================================== RMSNorm forward
// One CTA per row; the row lives in registers between the two passes (H <= 8*256*VPT).
constexpr int NORM_THREADS = 256;
constexpr int NORM_VPT = 4;  // uint4 chunks per thread held in registers -> H <= 8192

__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                   float* __restrict__ rstd, int H, long long x_stride, long long y_stride, float eps,
                   float w_offset) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  uint4* yr = reinterpret_cast<uint4*>(y + row * y_stride);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const int nvec = H >> 3;
  uint4 cache[NORM_VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_VPT; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      cache[i] = xr[v];
      float f[8];
      unpack8(cache[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  for (int v = threadIdx.x + NORM_VPT * NORM_THREADS; v < nvec; v += NORM_THREADS) {
    float f[8];
    unpack8(xr[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum<NORM_THREADS>(ss, sh);
  const float r = rsqrtf(ss / static_cast<float>(H) + eps);
  if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < NORM_VPT; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float f[8], g[8];
      unpack8(cache[i], f);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * r * (g[j] + w_offset);
      yr[v] = pack8(f);
    }
  }
  for (int v = threadIdx.x + NORM_VPT * NORM_THREADS; v < nvec; v += NORM_THREADS) {
    float f[8], g[8];
    unpack8(xr[v], f);
    unpack8(wr[v], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * (g[j] + w_offset);
    yr[v] = pack8(f);
  }
}

// ============================================================== RMSNorm backward
// Persistent grid: CTA b handles rows b, b+grid, ...; keeps its partial dw in
// registers and writes one fp32 row of `dw_partial[grid, H]` (scratch); a second
// kernel sums the partials. dx = rstd*(w*dy) - x*rstd^3*mean(w*dy*x) (+ dx_residual).
// VPT = uint4 chunks per thread (H <= VPT * 8 * NORM_THREADS). The loads of the NEXT row are issued before the block
// reduction of the current one, so the reduction's two barriers do not leave the memory system idle.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS, VPT <= 2 ? 3 : 1)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                   const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H, float w_offset) {
  __shared__ float sh[32];
  const int nvec = H >> 3;
  float dwacc[VPT][8];
  uint4 cw[VPT], nx[VPT], ng[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    const int v = threadIdx.x + i * NORM_THREADS;
    cw[i] = v < nvec ? reinterpret_cast<const uint4*>(w)[v] : make_uint4(0u, 0u, 0u, 0u);
    nx[i] = ng[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  auto load_row = [&](long long row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        nx[i] = xr[v];
        ng[i] = gr[v];
      }
    }
  };
  if (blockIdx.x < T) load_row(blockIdx.x);
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
    uint4* or_ = reinterpret_cast<uint4*>(dx + row * H);
    const float r = rstd[row];
    uint4 cx[VPT], cg[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      cx[i] = nx[i];
      cg[i] = ng[i];
    }
    if (row + gridDim.x < T) load_row(row + gridDim.x);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float fx[8], fg[8], fw[8];
        unpack8(cx[i], fx);
        unpack8(cg[i], fg);
        unpack8(cw[i], fw);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += fg[j] * (fw[j] + w_offset) * fx[j];
          dwacc[i][j] += fg[j] * fx[j] * r;
        }
      }
    }
    dot = block_sum<NORM_THREADS>(dot, sh);
    const float c = dot * r * r * r / static_cast<float>(H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float fx[8], fg[8], fw[8], o[8];
        unpack8(cx[i], fx);
        unpack8(cg[i], fg);
        unpack8(cw[i], fw);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * fg[j] * (fw[j] + w_offset) - c * fx[j];
        if (rr) {
          float fr[8];
          unpack8(rr[v], fr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += fr[j];
        }
        or_[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float4* d = reinterpret_cast<float4*>(dw_partial + static_cast<long long>(blockIdx.x) * H + v * 8);
      d[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      d[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// dw[h] (+)= sum_p partial[p, h]; output fp32 (accumulate) or bf16 (store).
__global__ void colsum_partials_kernel(const float* __restrict__ partial, int P, int H, float* __restrict__ out_f32,
                                       bf16* __restrict__ out_bf16, int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[static_cast<long long>(p) * H + h];
  if (out_f32) out_f32[h] = accumulate ? out_f32[h] + s : s;
  if (out_bf16) out_bf16[h] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[h]) + s : s);
}

// ============================================================== RoPE
// x viewed as [T, heads, D] with token stride `t_stride` and head stride `h_stride`
// (elements). Heads are organised in groups of `group` consecutive heads; only the
// first `rope_in_group` heads of each group rotate (packed QKV: q heads and the k
// head rotate, the v head does not). freqs[T, rot_dim/2] fp32 angles; cos/sin are
// scaled by `mscale` (YaRN). interleaved=0: pairs (i, i+rot/2); 1: pairs (2i, 2i+1).
// `sign` = +1 forward, -1 backward (inverse rotation). In place.
// One CTA per token: the rot_dim / 2 (cos, sin) pairs of the token are computed once into shared memory and reused by
// all heads; rotating heads are processed eight bf16 at a time when the layout allows 16-byte accesses.
constexpr int ROPE_MAX_HALF = 256;
__global__ void rope_kernel(bf16* __restrict__ x, const float* __restrict__ freqs, int T, int heads, int D,
                            int rot_dim, int rot_offset, long long t_stride, long long h_stride, int group,
                            int rope_in_group, int interleaved, float mscale, float sign,
                            const int* __restrict__ pos_ids, int vec_ok) {
  __shared__ float cs[ROPE_MAX_HALF], sn[ROPE_MAX_HALF];
  const int t = blockIdx.x;
  const int half = rot_dim >> 1;
  const long long frow = pos_ids ? pos_ids[t] : t;
  const float* fr = freqs + frow * half;
  bf16* xt = x + static_cast<long long>(t) * t_stride;
  const bool cached = half <= ROPE_MAX_HALF;
  if (cached) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float s, c;
      sincosf(fr[i], &s, &c);
      sn[i] = s * mscale * sign;
      cs[i] = c * mscale;
    }
    __syncthreads();
  }
  if (cached && vec_ok) {
    if (!interleaved) {
      const int hv = half >> 3;  // 16-byte chunks per half
      for (int idx = threadIdx.x; idx < heads * hv; idx += blockDim.x) {
        const int h = idx / hv, v = idx - h * hv;
        if ((h % group) >= rope_in_group) continue;
        uint4* p0 = reinterpret_cast<uint4*>(xt + h * h_stride + rot_offset) + v;
        uint4* p1 = reinterpret_cast<uint4*>(xt + h * h_stride + rot_offset + half) + v;
        float a[8], b[8], o0[8], o1[8];
        unpack8(*p0, a);
        unpack8(*p1, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float c = cs[v * 8 + j], s = sn[v * 8 + j];
          o0[j] = a[j] * c - b[j] * s;
          o1[j] = b[j] * c + a[j] * s;
        }
        *p0 = pack8(o0);
        *p1 = pack8(o1);
      }
    } else {
      const int rv = rot_dim >> 3;  // 16-byte chunks of the rotated span: four (even, odd) pairs each
      for (int idx = threadIdx.x; idx < heads * rv; idx += blockDim.x) {
        const int h = idx / rv, v = idx - h * rv;
        if ((h % group) >= rope_in_group) continue;
        uint4* p = reinterpret_cast<uint4*>(xt + h * h_stride + rot_offset) + v;
        float e[8], o[8];
        unpack8(*p, e);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float c = cs[v * 4 + j], s = sn[v * 4 + j];
          o[2 * j] = e[2 * j] * c - e[2 * j + 1] * s;
          o[2 * j + 1] = e[2 * j + 1] * c + e[2 * j] * s;
        }
        *p = pack8(o);
      }
    }
    return;
  }
  const int total = heads * half;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int h = idx / half;
    const int i = idx - h * half;
    if ((h % group) >= rope_in_group) continue;
    float s, c;
    if (cached) {
      s = sn[i];
      c = cs[i];
    } else {
      sincosf(fr[i], &s, &c);
      s *= mscale * sign;
      c *= mscale;
    }
    bf16* xh = xt + h * h_stride + rot_offset;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(xh[i0]);
    const float b = __bfloat162float(xh[i1]);
    xh[i0] = __float2bfloat16(a * c - b * s);
    xh[i1] = __float2bfloat16(b * c + a * s);
  }
}

// ============================================================== Hadamard (n = 128)
// y = x H_128 / sqrt(128) on rows of 128 bf16 (the rotation of the lightning indexer's q / k). One warp per row, four
// consecutive elements per lane: two butterfly stages inside the lane, five across lanes by shuffles. H is symmetric
// and orthogonal, so the same kernel is its own backward.
__global__ void hadamard128_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint2 raw = reinterpret_cast<const uint2*>(x + row * 128)[lane];
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float v0 = __bfloat162float(p0.x), v1 = __bfloat162float(p0.y), v2 = __bfloat162float(p1.x), v3 = __bfloat162float(p1.y);
  // strides 1 and 2: inside the lane
  float a = v0 + v1, b = v0 - v1, c = v2 + v3, d = v2 - v3;
  v0 = a + c; v1 = b + d; v2 = a - c; v3 = b - d;
  // strides 4 .. 64: lane distance 1 .. 16
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool up = (lane & m) != 0;
    const float o0 = __shfl_xor_sync(0xffffffffu, v0, m), o1 = __shfl_xor_sync(0xffffffffu, v1, m);
    const float o2 = __shfl_xor_sync(0xffffffffu, v2, m), o3 = __shfl_xor_sync(0xffffffffu, v3, m);
    v0 = up ? o0 - v0 : v0 + o0;
    v1 = up ? o1 - v1 : v1 + o1;
    v2 = up ? o2 - v2 : v2 + o2;
    v3 = up ? o3 - v3 : v3 + o3;
  }
  const float sc = 0.08838834764831845f;  // 1 / sqrt(128)
  uint2 out;
  *reinterpret_cast<__nv_bfloat162*>(&out.x) = __floats2bfloat162_rn(v0 * sc, v1 * sc);
  *reinterpret_cast<__nv_bfloat162*>(&out.y) = __floats2bfloat162_rn(v2 * sc, v3 * sc);
  reinterpret_cast<uint2*>(y + row * 128)[lane] = out;
}

// ============================================================== SwiGLU
// in [T, 2F] = [gate | up]; out[T, F] = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, long long T, int F) {
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / fv;
    const int v = static_cast<int>(i - t * fv);
    const uint4* row = reinterpret_cast<const uint4*>(in + t * 2 * F);
    float g[8], u[8], o[8];
    unpack8(row[v], g);
    unpack8(row[fv + v], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<uint4*>(out + t * F)[v] = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ in, bf16* __restrict__ din,
                                  long long T, int F) {
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / fv;
    const int v = static_cast<int>(i - t * fv);
    const uint4* row = reinterpret_cast<const uint4*>(in + t * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[v], g);
    unpack8(row[fv + v], u);
    unpack8(reinterpret_cast<const uint4*>(dout + t * F)[v], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
    }
    uint4* orow = reinterpret_cast<uint4*>(din + t * 2 * F);
    orow[v] = pack8(dg);
    orow[fv + v] = pack8(du);
  }
}

// ============================================================== cross entropy
// Pass 1: per-row max and sum(exp(x - max)) over this rank's vocab slice, and the
// target logit when the label falls inside [vocab_start, vocab_start + V).
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const bf16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_max,
                float* __restrict__ row_sum, float* __restrict__ tgt_logit, int V, long long ld, int vocab_start,
                int valid_v) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const bf16* lr = logits + row * ld;
  const int nvec = V >> 3;
  float m = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v * 8 + j < valid_v) m = fmaxf(m, f[j]);
  }
  m = block_max<CE_THREADS>(m, sh);
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v * 8 + j < valid_v) s += __expf(f[j] - m);
  }
  s = block_sum<CE_THREADS>(s, sh);
  if (threadIdx.x == 0) {
    row_max[row] = m;
    row_sum[row] = s;
    const long long lab = labels[row] - vocab_start;
    tgt_logit[row] = (lab >= 0 && lab < valid_v) ? __bfloat162float(lr[lab]) : 0.f;
  }
}
// Pass 2 (after the TP reduction of max / sum): logits <- (softmax - onehot) * row_scale, in place.
// gmax/gsum are the GLOBAL max and sum(exp(x - gmax)).
__global__ void __launch_bounds__(CE_THREADS)
ce_dlogits_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ gmax,
                  const float* __restrict__ gsum, const float* __restrict__ row_scale, int V, long long ld,
                  int vocab_start, int valid_v) {
  const long long row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const int nvec = V >> 3;
  const float m = gmax[row];
  const float inv = 1.f / gsum[row];
  const float sc = row_scale[row];
  const long long lab = labels[row] - vocab_start;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = v * 8 + j;
      float p = (col < valid_v) ? __expf(f[j] - m) * inv : 0.f;
      if (col == lab) p -= 1.f;
      f[j] = p * sc;
    }
    reinterpret_cast<uint4*>(lr)[v] = pack8(f);
  }
}

// ============================================================== fused AdamW
// Flat shard update. master fp32; grad fp32 or bf16; moments fp32 or bf16;
// optionally writes the bf16 model copy. grad is multiplied by grad_scale first
// (1/loss-scale x clip coefficient).
template <typename GT, typename MT>
__global__ void adam_kernel(float* __restrict__ master, const GT* __restrict__ grad, MT* __restrict__ m,
                            MT* __restrict__ v, bf16* __restrict__ model_out, long long n, float lr, float beta1,
                            float beta2, float eps, float wd, float bc1, float bc2, float grad_scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = static_cast<float>(grad[i]) * grad_scale;
    float mi = static_cast<float>(m[i]);
    float vi = static_cast<float>(v[i]);
    mi = beta1 * mi + (1.f - beta1) * g;
    vi = beta2 * vi + (1.f - beta2) * g * g;
    float p = master[i];
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * p;
    p -= lr * upd;
    master[i] = p;
    m[i] = static_cast<MT>(mi);
    v[i] = static_cast<MT>(vi);
    if (model_out) model_out[i] = __float2bfloat16(p);
  }
}

// AdamW with the fp32 master weight stored as (bf16 model weight, int16 remainder):
//   master_bits = (bf16_bits << 16) + remainder,  bf16 = round-to-nearest-even(master)
// The pair is an exact fp32 value, so the update is bit-identical to the fp32-master kernel while
// the optimizer keeps 2 instead of 4 extra bytes per parameter.
__device__ __forceinline__ float master_from_parts(bf16 w, short lo) {
  const unsigned hi = static_cast<unsigned>(__bfloat16_as_ushort(w)) << 16;
  return __uint_as_float(hi + static_cast<unsigned>(static_cast<int>(lo)));
}
__device__ __forceinline__ void master_to_parts(float p, bf16& w, short& lo) {
  w = __float2bfloat16_rn(p);
  const unsigned hi = static_cast<unsigned>(__bfloat16_as_ushort(w)) << 16;
  lo = static_cast<short>(static_cast<int>(__float_as_uint(p) - hi));
}
template <typename GT, typename MT>
__global__ void adam_remainder_kernel(bf16* __restrict__ w, short* __restrict__ lo, const GT* __restrict__ grad,
                                      MT* __restrict__ m, MT* __restrict__ v, long long n, float lr, float beta1,
                                      float beta2, float eps, float wd, float bc1, float bc2, float grad_scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = static_cast<float>(grad[i]) * grad_scale;
    float mi = static_cast<float>(m[i]);
    float vi = static_cast<float>(v[i]);
    mi = beta1 * mi + (1.f - beta1) * g;
    vi = beta2 * vi + (1.f - beta2) * g * g;
    float p = master_from_parts(w[i], lo[i]);
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * p;
    p -= lr * upd;
    bf16 wn;
    short ln;
    master_to_parts(p, wn, ln);
    w[i] = wn;
    lo[i] = ln;
    m[i] = static_cast<MT>(mi);
    v[i] = static_cast<MT>(vi);
  }
}
// remainder <-> fp32 master conversion (checkpointing, initialisation)
__global__ void master_split_kernel(const float* __restrict__ master, bf16* __restrict__ w, short* __restrict__ lo,
                                    long long n, int write_w) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    bf16 wn;
    short ln;
    master_to_parts(master[i], wn, ln);
    if (write_w) w[i] = wn;
    lo[i] = ln;
  }
}
__global__ void master_join_kernel(const bf16* __restrict__ w, const short* __restrict__ lo, float* __restrict__ master,
                                   long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    master[i] = master_from_parts(w[i], lo[i]);
}

// sum of squares of a flat buffer into a single fp32 (atomic add of block partials)
// ---- small rows (H = 64 / 128 / 256, e.g. per-head QK norm): one WARP per row, VPL elements per lane.
template <int VPL>
struct alignas(2 * VPL) BfVec {
  bf16 v[VPL];
};
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                        float* __restrict__ rstd, long long T, long long x_stride, long long y_stride, float eps,
                        float w_offset) {
  using V = BfVec<VPL>;
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const V wv = reinterpret_cast<const V*>(w)[lane];
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < T;
       row += warps) {
    const V xv = reinterpret_cast<const V*>(x + row * x_stride)[lane];
    float f[VPL], ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      f[j] = __bfloat162float(xv.v[j]);
      ss += f[j] * f[j];
    }
    ss = warp_sum_f(ss);
    const float r = rsqrtf(ss / static_cast<float>(32 * VPL) + eps);
    if (lane == 0 && rstd != nullptr) rstd[row] = r;
    V o;
#pragma unroll
    for (int j = 0; j < VPL; ++j) o.v[j] = __float2bfloat16_rn(f[j] * r * (__bfloat162float(wv.v[j]) + w_offset));
    reinterpret_cast<V*>(y + row * y_stride)[lane] = o;
  }
}

template <int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_warp_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                        const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                        float* __restrict__ dw_partial, long long T, float w_offset) {
  using V = BfVec<VPL>;
  constexpr int H = 32 * VPL;
  __shared__ float sh[8][H];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const long long warps = static_cast<long long>(gridDim.x) * 8;
  const V wv = reinterpret_cast<const V*>(w)[lane];
  float fw[VPL], dwacc[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    fw[j] = __bfloat162float(wv.v[j]) + w_offset;
    dwacc[j] = 0.f;
  }
  for (long long row = static_cast<long long>(blockIdx.x) * 8 + wid; row < T; row += warps) {
    const V xv = reinterpret_cast<const V*>(x + row * H)[lane];
    const V gv = reinterpret_cast<const V*>(dy + row * H)[lane];
    const float r = rstd[row];
    float fx[VPL], fg[VPL], dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      fx[j] = __bfloat162float(xv.v[j]);
      fg[j] = __bfloat162float(gv.v[j]);
      dot += fg[j] * fw[j] * fx[j];
      dwacc[j] += fg[j] * fx[j] * r;
    }
    dot = warp_sum_f(dot);
    const float c = dot * r * r * r / static_cast<float>(H);
    V o;
    if (dres != nullptr) {
      const V rv = reinterpret_cast<const V*>(dres + row * H)[lane];
#pragma unroll
      for (int j = 0; j < VPL; ++j)
        o.v[j] = __float2bfloat16_rn(r * fg[j] * fw[j] - c * fx[j] + __bfloat162float(rv.v[j]));
    } else {
#pragma unroll
      for (int j = 0; j < VPL; ++j) o.v[j] = __float2bfloat16_rn(r * fg[j] * fw[j] - c * fx[j]);
    }
    reinterpret_cast<V*>(dx + row * H)[lane] = o;
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) sh[wid][lane * VPL + j] = dwacc[j];
  __syncthreads();
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) s += sh[q][h];
    dw_partial[static_cast<long long>(blockIdx.x) * H + h] = s;
  }
}

template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float sh[32];
  float s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = static_cast<float>(x[i]);
    s += f * f;
  }
  s = block_sum<256>(s, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] += sum of the per-CTA partials, added up in a fixed order: the result does not depend on which CTA finished
// first, so the gradient norm (and with it the clipping factor) is the same bit pattern on every run.
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int count, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < count; i += 256) s += partial[i];
  s = block_sum<256>(s, sh);
  if (threadIdx.x == 0) out[0] += s;
}

// ---------------------------------------------------------------------------- launchers
static inline int grid_for(long long work, int threads, int cap = 148 * 8) {
  long long g = (work + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long T, int H, long long x_stride,
                 long long y_stride, float eps, float w_offset, cudaStream_t s) {
  if (T == 0) return;
  if ((H == 64 || H == 128 || H == 256) && x_stride % 8 == 0 && y_stride % 8 == 0) {
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w);
    bf16* yp = static_cast<bf16*>(y);
    const int grid = grid_for(T, 8, 148 * 8);
    if (H == 64)
      rmsnorm_fwd_warp_kernel<2><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, T, x_stride, y_stride, eps, w_offset);
    else if (H == 128)
      rmsnorm_fwd_warp_kernel<4><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, T, x_stride, y_stride, eps, w_offset);
    else
      rmsnorm_fwd_warp_kernel<8><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, T, x_stride, y_stride, eps, w_offset);
    return;
  }
  rmsnorm_fwd_kernel<<<static_cast<unsigned>(T), NORM_THREADS, 0, s>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<bf16*>(y), rstd, H, x_stride, y_stride,
      eps, w_offset);
}

int rmsnorm_bwd_grid(long long T) { return static_cast<int>(T < 148 * 4 ? (T > 0 ? T : 1) : 148 * 4); }

void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                 float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, long long T, int H, float w_offset,
                 cudaStream_t s) {
  if (T == 0) return;
  const int grid = rmsnorm_bwd_grid(T);
  if (H == 64 || H == 128 || H == 256) {
    const bf16 *gp = static_cast<const bf16*>(dy), *xp = static_cast<const bf16*>(x), *wp = static_cast<const bf16*>(w);
    const bf16* rp = static_cast<const bf16*>(dres);
    bf16* op = static_cast<bf16*>(dx);
    if (H == 64)
      rmsnorm_bwd_warp_kernel<2><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_partial, T, w_offset);
    else if (H == 128)
      rmsnorm_bwd_warp_kernel<4><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_partial, T, w_offset);
    else
      rmsnorm_bwd_warp_kernel<8><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_partial, T, w_offset);
    colsum_partials_kernel<<<(H + 255) / 256, 256, 0, s>>>(dw_partial, grid, H, dw_f32, static_cast<bf16*>(dw_bf16),
                                                           accumulate);
    return;
  }
  const bf16 *gp = static_cast<const bf16*>(dy), *xp = static_cast<const bf16*>(x), *wp = static_cast<const bf16*>(w);
  const bf16* rp = static_cast<const bf16*>(dres);
  bf16* op = static_cast<bf16*>(dx);
  const int nvec = H >> 3, Ti = static_cast<int>(T);
  if (nvec <= NORM_THREADS)
    rmsnorm_bwd_kernel<1><<<grid, NORM_THREADS, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_partial, Ti, H, w_offset);
  else if (nvec <= 2 * NORM_THREADS)
    rmsnorm_bwd_kernel<2><<<grid, NORM_THREADS, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_partial, Ti, H, w_offset);
  else
    rmsnorm_bwd_kernel<NORM_VPT><<<grid, NORM_THREADS, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_partial, Ti, H, w_offset);
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, s>>>(dw_partial, grid, H, dw_f32, static_cast<bf16*>(dw_bf16),
                                                         accumulate);
}

void rope_inplace(void* x, const float* freqs, const int* pos_ids, int T, int heads, int D, int rot_dim,
                  int rot_offset, long long t_stride, long long h_stride, int group, int rope_in_group,
                  int interleaved, float mscale, float sign, cudaStream_t s) {
  if (T == 0) return;
  // 16-byte accesses need aligned rows, heads, rotated span and halves
  const int vec_ok = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (t_stride % 8 == 0) && (h_stride % 8 == 0) &&
                     (rot_offset % 8 == 0) && (rot_dim % 16 == 0);
  const int work = vec_ok ? heads * (rot_dim / 16) : heads * (rot_dim / 2);
  const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
  rope_kernel<<<T, threads, 0, s>>>(static_cast<bf16*>(x), freqs, T, heads, D, rot_dim, rot_offset, t_stride,
                                    h_stride, group, rope_in_group, interleaved, mscale, sign, pos_ids, vec_ok);
}

void hadamard128(const void* x, void* y, long long rows, cudaStream_t s) {
  if (rows == 0) return;
  hadamard128_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>(static_cast<const bf16*>(x),
                                                                          static_cast<bf16*>(y), rows);
}

void swiglu_fwd(const void* in, void* out, long long T, int F, cudaStream_t s) {
  if (T == 0) return;
  swiglu_fwd_kernel<<<grid_for(T * (F >> 3), 256), 256, 0, s>>>(static_cast<const bf16*>(in),
                                                                 static_cast<bf16*>(out), T, F);
}
void swiglu_bwd(const void* dout, const void* in, void* din, long long T, int F, cudaStream_t s) {
  if (T == 0) return;
  swiglu_bwd_kernel<<<grid_for(T * (F >> 3), 256), 256, 0, s>>>(static_cast<const bf16*>(dout),
                                                                 static_cast<const bf16*>(in),
                                                                 static_cast<bf16*>(din), T, F);
}

void ce_stats(const void* logits, const long long* labels, float* row_max, float* row_sum, float* tgt, long long T,
              int V, long long ld, int vocab_start, int valid_v, cudaStream_t s) {
  if (T == 0) return;
  ce_stats_kernel<<<static_cast<unsigned>(T), CE_THREADS, 0, s>>>(static_cast<const bf16*>(logits), labels, row_max,
                                                                  row_sum, tgt, V, ld, vocab_start, valid_v);
}
void ce_dlogits(void* logits, const long long* labels, const float* gmax, const float* gsum, const float* row_scale,
                long long T, int V, long long ld, int vocab_start, int valid_v, cudaStream_t s) {
  if (T == 0) return;
  ce_dlogits_kernel<<<static_cast<unsigned>(T), CE_THREADS, 0, s>>>(static_cast<bf16*>(logits), labels, gmax, gsum,
                                                                    row_scale, V, ld, vocab_start, valid_v);
}

void adam_step(float* master, const void* grad, int grad_is_bf16, void* m, void* v, int moments_bf16,
               void* model_out, long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
               float bc2, float grad_scale, cudaStream_t s) {
  if (n == 0) return;
  const int grid = grid_for(n, 256, 148 * 16);
  bf16* mo = static_cast<bf16*>(model_out);
  if (grad_is_bf16) {
    if (moments_bf16)
      adam_kernel<bf16, bf16><<<grid, 256, 0, s>>>(master, static_cast<const bf16*>(grad), static_cast<bf16*>(m),
                                                   static_cast<bf16*>(v), mo, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                                   grad_scale);
    else
      adam_kernel<bf16, float><<<grid, 256, 0, s>>>(master, static_cast<const bf16*>(grad), static_cast<float*>(m),
                                                    static_cast<float*>(v), mo, n, lr, beta1, beta2, eps, wd, bc1,
                                                    bc2, grad_scale);
  } else {
    if (moments_bf16)
      adam_kernel<float, bf16><<<grid, 256, 0, s>>>(master, static_cast<const float*>(grad), static_cast<bf16*>(m),
                                                    static_cast<bf16*>(v), mo, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                                    grad_scale);
    else
      adam_kernel<float, float><<<grid, 256, 0, s>>>(master, static_cast<const float*>(grad), static_cast<float*>(m),
                                                     static_cast<float*>(v), mo, n, lr, beta1, beta2, eps, wd, bc1,
                                                     bc2, grad_scale);
  }
}

void adam_step_remainder(void* w, void* lo, const void* grad, int grad_is_bf16, void* m, void* v, int moments_bf16,
                         long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                         float grad_scale, cudaStream_t s) {
  if (n == 0) return;
  const int grid = grid_for(n, 256, 148 * 16);
  bf16* wp = static_cast<bf16*>(w);
  short* lp = static_cast<short*>(lo);
  if (grad_is_bf16) {
    if (moments_bf16)
      adam_remainder_kernel<bf16, bf16><<<grid, 256, 0, s>>>(wp, lp, static_cast<const bf16*>(grad), static_cast<bf16*>(m),
                                                             static_cast<bf16*>(v), n, lr, beta1, beta2, eps, wd, bc1,
                                                             bc2, grad_scale);
    else
      adam_remainder_kernel<bf16, float><<<grid, 256, 0, s>>>(wp, lp, static_cast<const bf16*>(grad),
                                                              static_cast<float*>(m), static_cast<float*>(v), n, lr,
                                                              beta1, beta2, eps, wd, bc1, bc2, grad_scale);
  } else {
    if (moments_bf16)
      adam_remainder_kernel<float, bf16><<<grid, 256, 0, s>>>(wp, lp, static_cast<const float*>(grad),
                                                              static_cast<bf16*>(m), static_cast<bf16*>(v), n, lr,
                                                              beta1, beta2, eps, wd, bc1, bc2, grad_scale);
    else
      adam_remainder_kernel<float, float><<<grid, 256, 0, s>>>(wp, lp, static_cast<const float*>(grad),
                                                               static_cast<float*>(m), static_cast<float*>(v), n, lr,
                                                               beta1, beta2, eps, wd, bc1, bc2, grad_scale);
  }
}
void master_split(const float* master, void* w, void* lo, long long n, int write_w, cudaStream_t s) {
  if (n == 0) return;
  master_split_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, s>>>(master, static_cast<bf16*>(w), static_cast<short*>(lo),
                                                                 n, write_w);
}
void master_join(const void* w, const void* lo, float* master, long long n, cudaStream_t s) {
  if (n == 0) return;
  master_join_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, s>>>(static_cast<const bf16*>(w),
                                                                static_cast<const short*>(lo), master, n);
}

int sumsq_partials(long long n) { return grid_for(n, 256, 148 * 8); }

void sumsq(const void* x, int is_bf16, long long n, float* out, float* partial, cudaStream_t s) {
  if (n == 0) return;
  const int grid = sumsq_partials(n);
  if (is_bf16)
    sumsq_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<const bf16*>(x), n, partial);
  else
    sumsq_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), n, partial);
  sumsq_final_kernel<<<1, 256, 0, s>>>(partial, grid, out);
}

}  // namespace lf

// ============================================================================ allocation-free RMSNorm backward
// See rmsnorm_bwd_noalloc.h. The per-CTA partial weight gradients go to a scratch array that is
// part of the library image instead of a per-call allocation.
#include "rmsnorm_bwd_noalloc.h"

static __device__ __align__(256) float g_rmsnorm_noalloc_scratch[LF_RMSNORM_NOALLOC_MAX_CTAS * LF_RMSNORM_NOALLOC_MAX_H];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_dev_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal
}  // namespace

extern "C" int lf_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                      float* dw, long long T, int H, float w_offset, cudaStream_t stream) {
  if (H <= 0 || H > LF_RMSNORM_NOALLOC_MAX_H || (H % 8) != 0 || T < 0) return LF_NOALLOC_ERR_TOO_LARGE;
  // the kernels count rows with a 32-bit int: a larger T would wrap, so it is refused, not narrowed
  if (T > LF_RMSNORM_NOALLOC_MAX_T) return LF_NOALLOC_ERR_TOO_LARGE;
  if (T == 0) return LF_NOALLOC_OK;
  const void* ptrs[6] = {dy, x, w, rstd, dx, dw};
  for (const void* p : ptrs)
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) != 0) return LF_NOALLOC_ERR_BAD_POINTER;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return LF_NOALLOC_ERR_CUDA;
  float* scratch = g_scratch_dev_ptr[dev];
  if (scratch == nullptr) {
    // One-time set-up for this device (it is current): in host code the array's name is only a
    // stand-in for the symbol, so ask the runtime for its address in device memory.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_rmsnorm_noalloc_scratch) != cudaSuccess || p == nullptr) return LF_NOALLOC_ERR_CUDA;
    scratch = static_cast<float*>(p);
    g_scratch_dev_ptr[dev] = scratch;
  }
  // An error left behind by earlier, unrelated work on this device must not be reported as this call's.
  if (cudaPeekAtLastError() != cudaSuccess) return LF_NOALLOC_ERR_CUDA;
  const int grid = static_cast<int>(T < LF_RMSNORM_NOALLOC_MAX_CTAS ? T : LF_RMSNORM_NOALLOC_MAX_CTAS);
  // Every CTA writes its full row [0, H) of the scratch and the column sum reads exactly rows
  // [0, grid) x [0, H): stale contents of earlier calls are never read, so no clearing is needed.
  lf::rmsnorm_bwd_kernel<lf::NORM_VPT><<<grid, lf::NORM_THREADS, 0, stream>>>(
      static_cast<const lf::bf16*>(dy), static_cast<const lf::bf16*>(x), static_cast<const lf::bf16*>(w), rstd,
      nullptr, static_cast<lf::bf16*>(dx), scratch, static_cast<int>(T), H, w_offset);
  lf::colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(scratch, grid, H, dw, nullptr, 0);
  return cudaGetLastError() == cudaSuccess ? LF_NOALLOC_OK : LF_NOALLOC_ERR_CUDA;
}
