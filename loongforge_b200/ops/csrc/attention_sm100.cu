// Flash attention for sm_100a (head dim 128, bf16, packed tokens, causal / bidirectional, GQA,
// variable-length sequences through cu_seqlens).
//
// All matrix products run on tcgen05.mma with fp32 accumulators in TMEM; operands are staged by
// TMA into 128-byte-swizzled shared memory. Every tile is 128 x 128 bf16 in a "two-box" format:
// two [128 rows x 64 columns] swizzled boxes of 16 KB. Such a tile can be read by the tensor
// core either K-major (rows = M/N index, columns = contraction) or MN-major (rows = contraction,
// columns = M/N index), so Q, K, V, dO and the probability tiles are never transposed:
//
//   forward : S = Q K^T          (A = Q  K-major,  B = K  K-major)
//             O += P V           (A = P  K-major,  B = V  MN-major)
//   dK/dV   : S = Q K^T, dP = dO V^T
//             dV += P^T dO       (A = P  MN-major, B = dO MN-major)
//             dK += dS^T Q       (A = dS MN-major, B = Q  MN-major)
//   dQ      : S, dP as above;  dQ += dS K   (A = dS K-major, B = K MN-major)
//
// Warp roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2-5 = softmax / gradient math, one thread per tile row (TMEM lane). Every mbarrier wait
// is bounded; a wait that gives up sets the status word and all roles unwind.
//
// Replaces TE DotProductAttention / flash-attn in the reference
// (loongforge/models/common/local_layers/local_attention.py:23,147-158).
#include "sm100_ptx.cuh"
#include "attention_sm100.h"
#include <cstdio>
#include <cstdlib>

namespace lf {

static constexpr int AT_THREADS = 192;
static constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KB
static constexpr int BOX_BYTES = 128 * 64 * 2;    // 16 KB
static constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  int T, Hq, Hkv, R;
  float scale_log2;  // scale * log2(e)
  float scale;
  int causal;
  const int* cu_seqlens;
  int num_seqs;
  int* status;
  __nv_bfloat16* o;
  long long o_ts, o_hs;
  float* lse;
  float* delta;
  __nv_bfloat16 *dq, *dk, *dv;
  long long dq_ts, dq_gs, dq_hs, dk_ts, dk_hs, dv_ts, dv_hs;
};

// ------------------------------------------------------------------------- tile helpers
// TMA load of a [128 tokens x 128 dims] tile of head (c1[, c2]) starting at token `tok`.
__device__ __forceinline__ void load_tile_q(uint8_t* smem, const CUtensorMap* m, uint64_t* bar, int j, int g, int tok) {
  // 4-D map: (d, head-in-group, group, token)
  for (int b = 0; b < 2; ++b) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];" ::"r"(smem_u32(smem + b * BOX_BYTES)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(b * 64), "r"(j), "r"(g), "r"(tok)
        : "memory");
  }
}
__device__ __forceinline__ void load_tile_kv(uint8_t* smem, const CUtensorMap* m, uint64_t* bar, int g, int tok) {
  for (int b = 0; b < 2; ++b) tma_load_3d(smem + b * BOX_BYTES, m, bar, b * 64, g, tok);
}

// One 128x128x128 product on tiles in the two-box format. *_mn selects the MN-major view.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_tile(uint32_t tmem_d, uint32_t a_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, 128, 128);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + kk * 2048, BOX_BYTES, 1024)
                             : make_smem_desc_sw128(a_base + (kk >> 2) * BOX_BYTES + (kk & 3) * 32, 16, 1024);
    const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + kk * 2048, BOX_BYTES, 1024)
                             : make_smem_desc_sw128(b_base + (kk >> 2) * BOX_BYTES + (kk & 3) * 32, 16, 1024);
    tc_mma_f16_ss(tmem_d, da, db, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// Store 32 consecutive columns [c0, c0+32) of row `row` into a two-box swizzled tile.
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row, int c0, const float (&v)[32]) {
  uint8_t* base = tile + (c0 >> 6) * BOX_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
  const int chunk0 = (c0 & 63) >> 3;  // 16-byte chunk index within the 128-byte row
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = pack_bf16x2(v[c * 8 + 0], v[c * 8 + 1]);
    q.y = pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
    q.z = pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
    q.w = pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
    *reinterpret_cast<uint4*>(base + (((chunk0 + c) ^ (row & 7)) << 4)) = q;
  }
}

// Locate q-block `blk` among the sequences: returns false when blk is past the end.
__device__ __forceinline__ bool locate_block(int blk, const int* cu, int num_seqs, int T, int& seq_start,
                                             int& seq_len, int& blk_in_seq) {
  if (cu == nullptr) {
    seq_start = 0;
    seq_len = T;
    blk_in_seq = blk;
    return blk * 128 < T;
  }
  int acc = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int a = cu[s], b = cu[s + 1];
    const int nb = (b - a + 127) >> 7;
    if (blk < acc + nb) {
      seq_start = a;
      seq_len = b - a;
      blk_in_seq = blk - acc;
      return true;
    }
    acc += nb;
  }
  return false;
}

struct SharedCtl {
  uint64_t bars[16];
  uint32_t tmem_slot;
  int abort_flag;
};

// =========================================================================== forward
// smem: Q tile | K[2] | V[2] | P tile | control
struct FwdSmem {
  static constexpr int Q = 0;
  static constexpr int K = TILE_BYTES;
  static constexpr int V = 3 * TILE_BYTES;
  static constexpr int P = 5 * TILE_BYTES;
  static constexpr int CTL = 6 * TILE_BYTES;
  static constexpr int BYTES = 6 * TILE_BYTES + 256 + 1024;
};
enum { F_Q = 0, F_KV_FULL = 1, F_KV_EMPTY = 3, F_S_FULL = 5, F_P_FULL = 7, F_O_DONE = 8 };

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + FwdSmem::CTL);
  uint64_t* bars = ctl->bars;
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int g = head / p.R, jh = head % p.R;

  int seq_start, seq_len, qb;
  // launch the long (late) query blocks first: with a causal mask they do the most work
  const bool live = locate_block(gridDim.x - 1 - blockIdx.x, p.cu_seqlens, p.num_seqs, p.T, seq_start, seq_len, qb);
  if (!live) return;  // uniform for the whole CTA
  const int q0 = qb * 128;
  const int n_kv = p.causal ? min((seq_len + 127) >> 7, qb + 1) : ((seq_len + 127) >> 7);

  if (threadIdx.x == 0) {
    mbar_init(&bars[F_Q], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[F_KV_FULL + s], 1);
      mbar_init(&bars[F_KV_EMPTY + s], 1);
      mbar_init(&bars[F_S_FULL + s], 1);
    }
    mbar_init(&bars[F_P_FULL], 4);
    mbar_init(&bars[F_O_DONE], 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t tmem_s0 = tmem, tmem_o = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars[F_Q], TILE_BYTES);
      load_tile_q(smem + FwdSmem::Q, &tq, &bars[F_Q], jh, g, seq_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&bars[F_KV_EMPTY + s], ((j >> 1) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[F_KV_FULL + s], 2 * TILE_BYTES);
        load_tile_kv(smem + FwdSmem::K + s * TILE_BYTES, &tk, &bars[F_KV_FULL + s], g, seq_start + j * 128);
        load_tile_kv(smem + FwdSmem::V + s * TILE_BYTES, &tv, &bars[F_KV_FULL + s], g, seq_start + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sq = smem_u32(smem + FwdSmem::Q), sp = smem_u32(smem + FwdSmem::P);
      bool ok = mbar_wait(&bars[F_Q], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[F_KV_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        mma_tile<false, false>(tmem_s0, sq, smem_u32(smem + FwdSmem::K), false);
        tc_commit(&bars[F_S_FULL + 0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv) {
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(&bars[F_KV_FULL + s1], ((j + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          mma_tile<false, false>(tmem_s0 + s1 * 128, sq, smem_u32(smem + FwdSmem::K + s1 * TILE_BYTES), false);
          tc_commit(&bars[F_S_FULL + s1]);
        }
        ok = mbar_wait(&bars[F_P_FULL], j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile<false, true>(tmem_o, sp, smem_u32(smem + FwdSmem::V + s * TILE_BYTES), j > 0);
        tc_commit(&bars[F_KV_EMPTY + s]);
        tc_commit(&bars[F_O_DONE]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // tile row == TMEM lane
    const int qi = q0 + row;              // position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m_ref = -INFINITY;  // running reference maximum in the log2 domain (scaled scores)
    float l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      ok = mbar_wait(&bars[F_S_FULL + s], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t ts = tmem_s0 + s * 128 + lane_off;
      const int kv0 = j * 128;
      const bool need_mask = (kv0 + 128 > seq_len) || (p.causal && kv0 + 127 > q0);
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(ts + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(r[i]);
          if (need_mask) {
            const int kj = kv0 + c0 + i;
            if (kj >= seq_len || (p.causal && kj > qi)) x = -INFINITY;
          }
          mx = fmaxf(mx, x);
        }
      }
      mx *= p.scale_log2;
      // Lazy rescale: keep the old reference unless the maximum grew by more than 2^8; then all
      // exponentials stay below 256 and the accumulated O / l remain consistent with m_ref.
      float m_new = m_ref;
      if (mx > m_ref + 8.f || m_ref == -INFINITY) m_new = fmaxf(mx, m_ref);
      const bool rescale = (m_new != m_ref) && (j > 0);
      const unsigned any = __ballot_sync(0xffffffffu, rescale);
      // P of the previous block must have been consumed, and O complete, before touching either
      if (j > 0) {
        ok = mbar_wait(&bars[F_O_DONE], (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
      }
      const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
      if (any) {
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_o + lane_off + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x16(tmem_o + lane_off + c0, r);
        }
        tmem_st_wait();
      }
      l_sum *= alpha;
      m_ref = m_new;
      // pass 2: probabilities -> shared memory (bf16), row sum
      const float mref_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(ts + c0, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(r[i]) * p.scale_log2 - mref_safe;
          if (need_mask) {
            const int kj = kv0 + c0 + i;
            if (kj >= seq_len || (p.causal && kj > qi)) x = -INFINITY;
          }
          const float e = exp2f(x);
          pv[i] = e;
          l_sum += e;
        }
        store_row_chunk(smem + FwdSmem::P, row, c0, pv);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[F_P_FULL]);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && n_kv > 0) ok = mbar_wait(&bars[F_O_DONE], (n_kv - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      const bool valid = qi < seq_len;
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      const long long tok = seq_start + qi;
      __nv_bfloat16* orow = p.o + tok * p.o_ts + static_cast<long long>(head) * p.o_hs;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_o + lane_off + c0, r);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            q.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            q.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            q.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + i) = q;
          }
        }
      }
      if (valid) p.lse[static_cast<long long>(head) * p.T + tok] = (m_ref + log2f(l_sum)) * (1.f / LOG2E);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// =========================================================================== backward: delta
// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (token, head).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ o,
                                  float* __restrict__ delta, int T, int Hq, long long do_ts, long long do_hs,
                                  long long o_ts, long long o_hs) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(T) * Hq) return;
  const int t = static_cast<int>(w / Hq), h = static_cast<int>(w % Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(dout + t * do_ts + h * do_hs + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(o + t * o_ts + h * o_hs + lane * 4);
  const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(bh[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// =========================================================================== backward: dK, dV
// One CTA per (kv block, kv head); loops over the R query heads of the group and over the
// query blocks that attend to this kv block. smem: K | V | Q | dO | P | dS | control.
struct BkvSmem {
  static constexpr int K = 0, V = TILE_BYTES, Q = 2 * TILE_BYTES, DO = 3 * TILE_BYTES, P = 4 * TILE_BYTES,
                       DS = 5 * TILE_BYTES, CTL = 6 * TILE_BYTES, BYTES = 6 * TILE_BYTES + 256 + 1024;
};
enum { B_KV = 0, B_QDO_FULL = 1, B_QDO_EMPTY = 2, B_S_FULL = 3, B_PDS_FULL = 4, B_ACC_DONE = 5 };

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + BkvSmem::CTL);
  uint64_t* bars = ctl->bars;
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y;

  int seq_start, seq_len, kb;
  if (!locate_block(blockIdx.x, p.cu_seqlens, p.num_seqs, p.T, seq_start, seq_len, kb)) return;
  const int kv0 = kb * 128;
  const int n_qb_total = (seq_len + 127) >> 7;
  const int qb_first = p.causal ? kb : 0;
  const int n_iter = (n_qb_total - qb_first) * p.R;  // iteration it -> head it % R, q block qb_first + it / R

  if (threadIdx.x == 0) {
    mbar_init(&bars[B_KV], 1);
    mbar_init(&bars[B_QDO_FULL], 1);
    mbar_init(&bars[B_QDO_EMPTY], 1);
    mbar_init(&bars[B_S_FULL], 1);
    mbar_init(&bars[B_PDS_FULL], 4);
    mbar_init(&bars[B_ACC_DONE], 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars[B_KV], 2 * TILE_BYTES);
      load_tile_kv(smem + BkvSmem::K, &tk, &bars[B_KV], g, seq_start + kv0);
      load_tile_kv(smem + BkvSmem::V, &tv, &bars[B_KV], g, seq_start + kv0);
      for (int it = 0; it < n_iter; ++it) {
        if (!mbar_wait(&bars[B_QDO_EMPTY], (it & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        const int jh = it % p.R, qb = qb_first + it / p.R;
        mbar_arrive_expect_tx(&bars[B_QDO_FULL], 2 * TILE_BYTES);
        load_tile_q(smem + BkvSmem::Q, &tq, &bars[B_QDO_FULL], jh, g, seq_start + qb * 128);
        load_tile_q(smem + BkvSmem::DO, &tdo, &bars[B_QDO_FULL], jh, g, seq_start + qb * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sk = smem_u32(smem + BkvSmem::K), sv = smem_u32(smem + BkvSmem::V);
      const uint32_t sq = smem_u32(smem + BkvSmem::Q), sdo = smem_u32(smem + BkvSmem::DO);
      const uint32_t sp = smem_u32(smem + BkvSmem::P), sds = smem_u32(smem + BkvSmem::DS);
      bool ok = mbar_wait(&bars[B_KV], 0, abort_flag);
      for (int it = 0; it < n_iter && ok; ++it) {
        ok = mbar_wait(&bars[B_QDO_FULL], it & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile<false, false>(t_s, sq, sk, false);    // S  = Q K^T
        mma_tile<false, false>(t_dp, sdo, sv, false);  // dP = dO V^T
        tc_commit(&bars[B_S_FULL]);
        ok = mbar_wait(&bars[B_PDS_FULL], it & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile<true, true>(t_dv, sp, sdo, it > 0);   // dV += P^T dO
        mma_tile<true, true>(t_dk, sds, sq, it > 0);   // dK += dS^T Q
        tc_commit(&bars[B_QDO_EMPTY]);
        tc_commit(&bars[B_ACC_DONE]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int jh = it % p.R, qb = qb_first + it / p.R;
      const int head = g * p.R + jh;
      const int qi = qb * 128 + row;  // this thread's query row
      const bool q_valid = qi < seq_len;
      const long long tok = seq_start + qi;
      const float lse2 = q_valid ? p.lse[static_cast<long long>(head) * p.T + tok] * LOG2E : 0.f;
      const float dlt = q_valid ? p.delta[static_cast<long long>(head) * p.T + tok] : 0.f;
      ok = mbar_wait(&bars[B_S_FULL], it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      // P and dS tiles of the previous iteration must have been consumed by the MMAs
      if (it > 0) {
        ok = mbar_wait(&bars[B_ACC_DONE], (it - 1) & 1, abort_flag);
        if (!ok) break;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(t_s + lane_off + c0, rs);
        tmem_ld_32x32b_x32(t_dp + lane_off + c0, rd);
        tmem_ld_wait();
        float pv[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kj = kv0 + c0 + i;
          const bool keep = q_valid && kj < seq_len && (!p.causal || kj <= qi);
          const float pr = keep ? exp2f(__uint_as_float(rs[i]) * p.scale_log2 - lse2) : 0.f;
          pv[i] = pr;
          ds[i] = pr * (__uint_as_float(rd[i]) - dlt) * p.scale;
        }
        store_row_chunk(smem + BkvSmem::P, row, c0, pv);
        store_row_chunk(smem + BkvSmem::DS, row, c0, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_PDS_FULL]);
    }
    if (ok && n_iter > 0) ok = mbar_wait(&bars[B_ACC_DONE], (n_iter - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      const int kj = kv0 + row;
      const bool valid = kj < seq_len;
      const long long tok = seq_start + kj;
      __nv_bfloat16* dvrow = p.dv + tok * p.dv_ts + static_cast<long long>(g) * p.dv_hs;
      __nv_bfloat16* dkrow = p.dk + tok * p.dk_ts + static_cast<long long>(g) * p.dk_hs;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t a[32], b[32];
        if (n_iter > 0) {
          tmem_ld_32x32b_x32(t_dv + lane_off + c0, a);
          tmem_ld_32x32b_x32(t_dk + lane_off + c0, b);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = b[i] = 0u;
        }
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
            q.y = pack_bf16x2(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
            q.z = pack_bf16x2(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
            q.w = pack_bf16x2(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
            *reinterpret_cast<uint4*>(dvrow + c0 + i) = q;
            q.x = pack_bf16x2(__uint_as_float(b[i]), __uint_as_float(b[i + 1]));
            q.y = pack_bf16x2(__uint_as_float(b[i + 2]), __uint_as_float(b[i + 3]));
            q.z = pack_bf16x2(__uint_as_float(b[i + 4]), __uint_as_float(b[i + 5]));
            q.w = pack_bf16x2(__uint_as_float(b[i + 6]), __uint_as_float(b[i + 7]));
            *reinterpret_cast<uint4*>(dkrow + c0 + i) = q;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// =========================================================================== backward: dQ
// One CTA per (q block, q head); loops over kv blocks. smem: Q | dO | K | V | dS | control.
struct BqSmem {
  static constexpr int Q = 0, DO = TILE_BYTES, K = 2 * TILE_BYTES, V = 3 * TILE_BYTES, DS = 4 * TILE_BYTES,
                       CTL = 5 * TILE_BYTES, BYTES = 5 * TILE_BYTES + 256 + 1024;
};
enum { Q_QDO = 0, Q_KV_FULL = 1, Q_KV_EMPTY = 2, Q_S_FULL = 3, Q_DS_FULL = 4, Q_ACC_DONE = 5 };

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                   const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + BqSmem::CTL);
  uint64_t* bars = ctl->bars;
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int g = head / p.R, jh = head % p.R;

  int seq_start, seq_len, qb;
  if (!locate_block(gridDim.x - 1 - blockIdx.x, p.cu_seqlens, p.num_seqs, p.T, seq_start, seq_len, qb)) return;
  const int q0 = qb * 128;
  const int n_kv = p.causal ? min((seq_len + 127) >> 7, qb + 1) : ((seq_len + 127) >> 7);

  if (threadIdx.x == 0) {
    mbar_init(&bars[Q_QDO], 1);
    mbar_init(&bars[Q_KV_FULL], 1);
    mbar_init(&bars[Q_KV_EMPTY], 1);
    mbar_init(&bars[Q_S_FULL], 1);
    mbar_init(&bars[Q_DS_FULL], 4);
    mbar_init(&bars[Q_ACC_DONE], 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dq = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars[Q_QDO], 2 * TILE_BYTES);
      load_tile_q(smem + BqSmem::Q, &tq, &bars[Q_QDO], jh, g, seq_start + q0);
      load_tile_q(smem + BqSmem::DO, &tdo, &bars[Q_QDO], jh, g, seq_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        if (!mbar_wait(&bars[Q_KV_EMPTY], (j & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[Q_KV_FULL], 2 * TILE_BYTES);
        load_tile_kv(smem + BqSmem::K, &tk, &bars[Q_KV_FULL], g, seq_start + j * 128);
        load_tile_kv(smem + BqSmem::V, &tv, &bars[Q_KV_FULL], g, seq_start + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sq = smem_u32(smem + BqSmem::Q), sdo = smem_u32(smem + BqSmem::DO);
      const uint32_t sk = smem_u32(smem + BqSmem::K), sv = smem_u32(smem + BqSmem::V);
      const uint32_t sds = smem_u32(smem + BqSmem::DS);
      bool ok = mbar_wait(&bars[Q_QDO], 0, abort_flag);
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = mbar_wait(&bars[Q_KV_FULL], j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile<false, false>(t_s, sq, sk, false);
        mma_tile<false, false>(t_dp, sdo, sv, false);
        tc_commit(&bars[Q_S_FULL]);
        ok = mbar_wait(&bars[Q_DS_FULL], j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile<false, true>(t_dq, sds, sk, j > 0);  // dQ += dS K
        tc_commit(&bars[Q_KV_EMPTY]);
        tc_commit(&bars[Q_ACC_DONE]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + row;
    const bool q_valid = qi < seq_len;
    const long long tok = seq_start + qi;
    const float lse2 = q_valid ? p.lse[static_cast<long long>(head) * p.T + tok] * LOG2E : 0.f;
    const float dlt = q_valid ? p.delta[static_cast<long long>(head) * p.T + tok] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int kv0 = j * 128;
      ok = mbar_wait(&bars[Q_S_FULL], j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      if (j > 0) {
        ok = mbar_wait(&bars[Q_ACC_DONE], (j - 1) & 1, abort_flag);
        if (!ok) break;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(t_s + lane_off + c0, rs);
        tmem_ld_32x32b_x32(t_dp + lane_off + c0, rd);
        tmem_ld_wait();
        float ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kj = kv0 + c0 + i;
          const bool keep = q_valid && kj < seq_len && (!p.causal || kj <= qi);
          const float pr = keep ? exp2f(__uint_as_float(rs[i]) * p.scale_log2 - lse2) : 0.f;
          ds[i] = pr * (__uint_as_float(rd[i]) - dlt) * p.scale;
        }
        store_row_chunk(smem + BqSmem::DS, row, c0, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[Q_DS_FULL]);
    }
    if (ok && n_kv > 0) ok = mbar_wait(&bars[Q_ACC_DONE], (n_kv - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      __nv_bfloat16* dqrow = p.dq + tok * p.dq_ts + static_cast<long long>(g) * p.dq_gs + jh * p.dq_hs;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t a[32];
        tmem_ld_32x32b_x32(t_dq + lane_off + c0, a);
        tmem_ld_wait();
        if (q_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
            q.y = pack_bf16x2(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
            q.z = pack_bf16x2(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
            q.w = pack_bf16x2(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
            *reinterpret_cast<uint4*>(dqrow + c0 + i) = q;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// =========================================================================== host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_encode_fn() {
  // cuTensorMapEncodeTiled is a driver call: it needs a CUDA context bound to THIS thread, which
  // autograd worker threads do not have until a runtime call binds the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 4-D map (d, head-in-group, group, token) with box (64, 1, 1, 128).
static int make_map_q(CUtensorMap* m, const void* ptr, int T, int groups, int R, long long ts, long long gs,
                      long long hs) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ts % 8) || (gs % 8) || (hs % 8)) return -2;
  cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(R), static_cast<cuuint64_t>(groups), static_cast<cuuint64_t>(T)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(hs) * 2, static_cast<cuuint64_t>(gs) * 2,
                           static_cast<cuuint64_t>(ts) * 2};
  // a degenerate dimension of extent 1 may carry any (16-byte aligned, non-zero) stride
  if (R == 1) strides[0] = 256;
  if (groups == 1) strides[1] = strides[0] * (R > 1 ? R : 1);
  cuuint32_t box[4] = {64, 1, 1, 128};
  cuuint32_t es[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}
// 3-D map (d, head, token) with box (64, 1, 128).
static int make_map_kv(CUtensorMap* m, const void* ptr, int T, int heads, long long ts, long long hs) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ts % 8) || (hs % 8)) return -2;
  cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(T)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(hs) * 2, static_cast<cuuint64_t>(ts) * 2};
  if (heads == 1) strides[0] = 256;
  cuuint32_t box[3] = {64, 1, 128};
  cuuint32_t es[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}

static AttnParams make_params(const AttnArgs& a) {
  AttnParams p;
  p.T = a.T; p.Hq = a.Hq; p.Hkv = a.Hkv; p.R = a.Hq / a.Hkv;
  p.scale = a.scale;
  p.scale_log2 = a.scale * LOG2E;
  p.causal = a.causal ? 1 : 0;
  p.cu_seqlens = a.cu_seqlens;
  p.num_seqs = a.num_seqs;
  p.status = a.status;
  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.o_ts = a.o_ts; p.o_hs = a.o_hs;
  p.lse = a.lse;
  p.delta = a.delta;
  p.dq = static_cast<__nv_bfloat16*>(a.dq);
  p.dk = static_cast<__nv_bfloat16*>(a.dk);
  p.dv = static_cast<__nv_bfloat16*>(a.dv);
  p.dq_ts = a.dq_ts; p.dq_gs = a.dq_gs; p.dq_hs = a.dq_hs;
  p.dk_ts = a.dk_ts; p.dk_hs = a.dk_hs; p.dv_ts = a.dv_ts; p.dv_hs = a.dv_hs;
  return p;
}

static int max_blocks(const AttnArgs& a) {
  // every sequence may add one partial block
  return (a.T + 127) / 128 + (a.cu_seqlens ? a.num_seqs : 0);
}

int attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.T == 0) return 0;
  if (a.Hq % a.Hkv) return -2;
  if ((a.o_ts % 8) || (a.o_hs % 8)) return -2;
  const int R = a.Hq / a.Hkv;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map_q(&tq, a.q, a.T, a.Hkv, R, a.q_ts, a.q_gs, a.q_hs))) return rc;
  if ((rc = make_map_kv(&tk, a.k, a.T, a.Hkv, a.k_ts, a.k_hs))) return rc;
  if ((rc = make_map_kv(&tv, a.v, a.T, a.Hkv, a.v_ts, a.v_hs))) return rc;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem::BYTES) !=
        cudaSuccess)
      return -4;
    attr = true;
  }
  const AttnParams p = make_params(a);
  dim3 grid(max_blocks(a), a.Hq);
  attn_fwd_kernel<<<grid, AT_THREADS, FwdSmem::BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#define LF_DBG(msg) do { if (getenv("LF_DEBUG")) { fprintf(stderr, "[lf::attn_bwd] %s\n", msg); fflush(stderr); } } while (0)

int attn_bwd(const AttnArgs& a, cudaStream_t stream) {
  LF_DBG("enter");
  if (a.T == 0) return 0;
  if (a.Hq % a.Hkv) return -2;
  const int R = a.Hq / a.Hkv;
  if ((a.do_ts % 8) || (a.do_hs % 8) || (a.dq_ts % 8) || (a.dq_gs % 8) || (a.dq_hs % 8) || (a.dk_ts % 8) ||
      (a.dk_hs % 8) || (a.dv_ts % 8) || (a.dv_hs % 8))
    return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_map_q(&tq, a.q, a.T, a.Hkv, R, a.q_ts, a.q_gs, a.q_hs))) return rc;
  if ((rc = make_map_kv(&tk, a.k, a.T, a.Hkv, a.k_ts, a.k_hs))) return rc;
  if ((rc = make_map_kv(&tv, a.v, a.T, a.Hkv, a.v_ts, a.v_hs))) return rc;
  // dO is [T, Hq, 128]: group stride R * head stride
  if ((rc = make_map_q(&tdo, a.dout, a.T, a.Hkv, R, a.do_ts, a.do_hs * R, a.do_hs))) return rc;
  LF_DBG("maps encoded");
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BkvSmem::BYTES) !=
            cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BqSmem::BYTES) !=
            cudaSuccess)
      return -4;
    attr = true;
  }
  LF_DBG("attributes set");
  const AttnParams p = make_params(a);
  const long long warps = static_cast<long long>(a.T) * a.Hq;
  attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a.dout), static_cast<const __nv_bfloat16*>(a.o), a.delta, a.T, a.Hq, a.do_ts,
      a.do_hs, a.o_ts, a.o_hs);
  LF_DBG("delta launched");
  dim3 grid_kv(max_blocks(a), a.Hkv);
  attn_bwd_dkdv_kernel<<<grid_kv, AT_THREADS, BkvSmem::BYTES, stream>>>(tq, tk, tv, tdo, p);
  LF_DBG("dkdv launched");
  dim3 grid_q(max_blocks(a), a.Hq);
  attn_bwd_dq_kernel<<<grid_q, AT_THREADS, BqSmem::BYTES, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
