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

static constexpr int AT_THREADS = 192;      // forward: 2 control warps + 4 softmax warps
static constexpr int AT_BWD_THREADS = 320;  // backward: 2 control warps + 8 math warps (2 per TMEM lane quarter)
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
// smem: Q tile | K[2] | V[2] | P[2] | control
struct FwdSmem {
  static constexpr int Q = 0;
  static constexpr int K = TILE_BYTES;
  static constexpr int V = 3 * TILE_BYTES;
  static constexpr int P = 5 * TILE_BYTES;
  static constexpr int CTL = 7 * TILE_BYTES;
  static constexpr int BYTES = 7 * TILE_BYTES + 256 + 1024;
};
enum { F_Q = 0, F_KV_FULL = 1, F_KV_EMPTY = 3, F_S_FULL = 5, F_P_FULL = 7, F_P_EMPTY = 9, F_O_DONE = 11 };

// Pipeline per kv block j (S and P are double buffered, index j & 1):
//   MMA warp : S[j+1] = Q K[j+1]^T is issued BEFORE waiting for P[j], so the tensor core computes
//              the next scores while the softmax warps work on block j; then O += P[j] V[j].
//   softmax  : reads S[j] once into registers, row max, (rare) lazy rescale of O, exponentials ->
//              P[j] in shared memory; it only waits for P[j-2]'s consumer, never for O += P[j-1] V[j-1],
//              unless a rescale is needed.
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
      mbar_init(&bars[F_P_FULL + s], 4);
      mbar_init(&bars[F_P_EMPTY + s], 1);
    }
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
        ok = mbar_wait(&bars[F_P_FULL + s], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile<false, true>(tmem_o, sp + s * TILE_BYTES, smem_u32(smem + FwdSmem::V + s * TILE_BYTES), j > 0);
        tc_commit(&bars[F_KV_EMPTY + s]);
        tc_commit(&bars[F_P_EMPTY + s]);
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
      ok = mbar_wait_warp(&bars[F_S_FULL + s], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t ts = tmem_s0 + s * 128 + lane_off;
      const int kv0 = j * 128;
      // the whole score row of this thread in registers: one TMEM pass
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld_32x32b_x32(ts, r0);
      tmem_ld_32x32b_x32(ts + 32, r1);
      tmem_ld_32x32b_x32(ts + 64, r2);
      tmem_ld_32x32b_x32(ts + 96, r3);
      tmem_ld_wait();
      const bool need_mask = (kv0 + 128 > seq_len) || (p.causal && kv0 + 127 > q0);
      if (need_mask) {
        const int lim = min(seq_len, p.causal ? qi + 1 : seq_len) - kv0;  // columns [0, lim) stay
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i >= lim) r0[i] = 0xff800000u;
          if (i + 32 >= lim) r1[i] = 0xff800000u;
          if (i + 64 >= lim) r2[i] = 0xff800000u;
          if (i + 96 >= lim) r3[i] = 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        mx0 = fmaxf(mx0, __uint_as_float(r0[i]));
        mx1 = fmaxf(mx1, __uint_as_float(r1[i]));
        mx2 = fmaxf(mx2, __uint_as_float(r2[i]));
        mx3 = fmaxf(mx3, __uint_as_float(r3[i]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      // Lazy rescale: keep the old reference unless the maximum grew by more than 2^8; then all
      // exponentials stay below 256 and the accumulated O / l remain consistent with m_ref.
      float m_new = m_ref;
      if (mx > m_ref + 8.f || m_ref == -INFINITY) m_new = fmaxf(mx, m_ref);
      const bool rescale = (m_new != m_ref) && (j > 0);
      const unsigned any = __ballot_sync(0xffffffffu, rescale);
      const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
      if (any) {
        // O must be complete (O += P[j-1] V[j-1] retired) before its rows are rescaled
        ok = mbar_wait_warp(&bars[F_O_DONE], (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
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
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      // P[s] was last read by O += P[j-2] V[j-2]
      ok = mbar_wait_warp(&bars[F_P_EMPTY + s], ((j >> 1) & 1) ^ 1, abort_flag);
      if (!ok) break;
      uint8_t* ptile = smem + FwdSmem::P + s * TILE_BYTES;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) { pv[i] = exp2f(fmaf(__uint_as_float(r0[i]), p.scale_log2, neg_m)); l0 += pv[i]; }
        store_row_chunk(ptile, row, 0, pv);
#pragma unroll
        for (int i = 0; i < 32; ++i) { pv[i] = exp2f(fmaf(__uint_as_float(r1[i]), p.scale_log2, neg_m)); l1 += pv[i]; }
        store_row_chunk(ptile, row, 32, pv);
#pragma unroll
        for (int i = 0; i < 32; ++i) { pv[i] = exp2f(fmaf(__uint_as_float(r2[i]), p.scale_log2, neg_m)); l2 += pv[i]; }
        store_row_chunk(ptile, row, 64, pv);
#pragma unroll
        for (int i = 0; i < 32; ++i) { pv[i] = exp2f(fmaf(__uint_as_float(r3[i]), p.scale_log2, neg_m)); l3 += pv[i]; }
        store_row_chunk(ptile, row, 96, pv);
      }
      l_sum += (l0 + l1) + (l2 + l3);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[F_P_FULL + s]);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && n_kv > 0) ok = mbar_wait_warp(&bars[F_O_DONE], (n_kv - 1) & 1, abort_flag);
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
// One CTA per (64-row kv block, kv head); loops over the R query heads of the group and over the
// 128-row query blocks that attend to this kv block. Per iteration (all on tcgen05, N = 64):
//   S  = Q K^T, dP = dO V^T                      [128 q x 64 kv] fp32 in TMEM (double buffered)
//   P  = exp2(S*scale*log2e - lse), dS = P (dP - delta) scale   -> bf16 tiles in shared memory (x2)
//   dV^T += dO^T P,  dK^T += Q^T dS              [128 d x 64 kv] fp32 in TMEM
// The transposed accumulators keep M = 128 for every MMA; Q, dO, P and dS tiles are read MN-major
// where the contraction runs over their rows, so nothing is transposed in memory. Q/dO, S/dP and
// P/dS are all double buffered: TMA, the score MMAs of iteration it+1 and the gradient MMAs of
// iteration it overlap the math warps' work on iteration it.
struct BkvSmem {
  static constexpr int KVB = 64 * 128 * 2;  // 16 KB: [64 kv rows x 128 d]
  static constexpr int PB = 128 * 64 * 2;   // 16 KB: [128 q rows x 64 kv]
  static constexpr int K = 0, V = KVB, Q = 2 * KVB, DO = Q + 2 * TILE_BYTES, P = DO + 2 * TILE_BYTES, DS = P + 2 * PB,
                       CTL = DS + 2 * PB, BYTES = CTL + 256 + 1024;
};
enum { B_KV = 0, B_QDO_FULL = 1, B_QDO_EMPTY = 3, B_S_FULL = 5, B_PDS_FULL = 7, B_PDS_EMPTY = 9, B_ACC_DONE = 11 };

// 128 x 64 x 128 product. A: two-box tile [128 x 128] (K-major: rows = M) or MN-major (rows = contraction).
// B (N = 64): K-major [64 rows x 128 contraction] as two 8 KB boxes, or MN-major [128 contraction rows x 64].
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_tile_n64(uint32_t tmem_d, uint32_t a_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, 128, 64);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + kk * 2048, BOX_BYTES, 1024)
                             : make_smem_desc_sw128(a_base + (kk >> 2) * BOX_BYTES + (kk & 3) * 32, 16, 1024);
    const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + kk * 2048, 16, 1024)
                             : make_smem_desc_sw128(b_base + (kk >> 2) * (64 * 128) + (kk & 3) * 32, 16, 1024);
    tc_mma_f16_ss(tmem_d, da, db, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

__global__ void __launch_bounds__(AT_BWD_THREADS, 1)
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

  // kv blocks are 64 rows: locate by 128-row block, then take the half
  int seq_start, seq_len, kb128;
  if (!locate_block(blockIdx.x >> 1, p.cu_seqlens, p.num_seqs, p.T, seq_start, seq_len, kb128)) return;
  const int kv0 = kb128 * 128 + (blockIdx.x & 1) * 64;
  if (kv0 >= seq_len) return;
  const int n_qb_total = (seq_len + 127) >> 7;
  const int qb_first = p.causal ? kb128 : 0;
  const int n_iter = (n_qb_total - qb_first) * p.R;  // iteration it -> head it % R, q block qb_first + it / R

  if (threadIdx.x == 0) {
    mbar_init(&bars[B_KV], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[B_QDO_FULL + s], 1);
      mbar_init(&bars[B_QDO_EMPTY + s], 1);
      mbar_init(&bars[B_S_FULL + s], 1);
      mbar_init(&bars[B_PDS_FULL + s], 8);
      mbar_init(&bars[B_PDS_EMPTY + s], 1);
    }
    mbar_init(&bars[B_ACC_DONE], 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 320;  // S[2], dP[2] 64 cols each

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars[B_KV], 2 * BkvSmem::KVB);
      for (int b = 0; b < 2; ++b) {
        tma_load_3d(smem + BkvSmem::K + b * (64 * 128), &tk, &bars[B_KV], b * 64, g, seq_start + kv0);
        tma_load_3d(smem + BkvSmem::V + b * (64 * 128), &tv, &bars[B_KV], b * 64, g, seq_start + kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it & 1;
        if (!mbar_wait(&bars[B_QDO_EMPTY + s], ((it >> 1) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        const int jh = it % p.R, qb = qb_first + it / p.R;
        mbar_arrive_expect_tx(&bars[B_QDO_FULL + s], 2 * TILE_BYTES);
        load_tile_q(smem + BkvSmem::Q + s * TILE_BYTES, &tq, &bars[B_QDO_FULL + s], jh, g, seq_start + qb * 128);
        load_tile_q(smem + BkvSmem::DO + s * TILE_BYTES, &tdo, &bars[B_QDO_FULL + s], jh, g, seq_start + qb * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sk = smem_u32(smem + BkvSmem::K), sv = smem_u32(smem + BkvSmem::V);
      const uint32_t sq = smem_u32(smem + BkvSmem::Q), sdo = smem_u32(smem + BkvSmem::DO);
      const uint32_t sp = smem_u32(smem + BkvSmem::P), sds = smem_u32(smem + BkvSmem::DS);
      bool ok = mbar_wait(&bars[B_KV], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[B_QDO_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        mma_tile_n64<false, false>(t_s, sq, sk, false);    // S[0]  = Q K^T
        mma_tile_n64<false, false>(t_dp, sdo, sv, false);  // dP[0] = dO V^T
        tc_commit(&bars[B_S_FULL + 0]);
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_iter) {
          const int s1 = (it + 1) & 1;
          ok = mbar_wait(&bars[B_QDO_FULL + s1], ((it + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          mma_tile_n64<false, false>(t_s + s1 * 64, sq + s1 * TILE_BYTES, sk, false);
          mma_tile_n64<false, false>(t_dp + s1 * 64, sdo + s1 * TILE_BYTES, sv, false);
          tc_commit(&bars[B_S_FULL + s1]);
        }
        ok = mbar_wait(&bars[B_PDS_FULL + s], (it >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_tile_n64<true, true>(t_dv, sdo + s * TILE_BYTES, sp + s * BkvSmem::PB, it > 0);  // dV^T += dO^T P
        mma_tile_n64<true, true>(t_dk, sq + s * TILE_BYTES, sds + s * BkvSmem::PB, it > 0);  // dK^T += Q^T dS
        tc_commit(&bars[B_QDO_EMPTY + s]);
        tc_commit(&bars[B_PDS_EMPTY + s]);
        if (it == n_iter - 1) tc_commit(&bars[B_ACC_DONE]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    // two warps share each TMEM lane quarter; each takes 32 of the 64 tile columns
    const int quarter = warp & 3;
    const int cbeg = ((warp - 2) >> 2) * 32;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const int jh = it % p.R, qb = qb_first + it / p.R;
      const int head = g * p.R + jh;
      const int qi = qb * 128 + row;  // this thread's query row
      const bool q_valid = qi < seq_len;
      const long long tok = seq_start + qi;
      const float neg_lse2 = q_valid ? -p.lse[static_cast<long long>(head) * p.T + tok] * LOG2E : 0.f;
      const float dlt = q_valid ? p.delta[static_cast<long long>(head) * p.T + tok] : 0.f;
      // columns [0, lim) of this row are kept (sequence end, causal diagonal, invalid query row)
      const int lim = q_valid ? (min(seq_len, p.causal ? qi + 1 : seq_len) - kv0) : 0;
      ok = mbar_wait_warp(&bars[B_S_FULL + s], (it >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t rs[32], rd[32];
      tmem_ld_32x32b_x32(t_s + s * 64 + lane_off + cbeg, rs);
      tmem_ld_32x32b_x32(t_dp + s * 64 + lane_off + cbeg, rd);
      tmem_ld_wait();
      float pv[32], ds[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float pr = exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, neg_lse2));
        if (cbeg + i >= lim) pr = 0.f;
        pv[i] = pr;
        ds[i] = pr * (__uint_as_float(rd[i]) - dlt) * p.scale;
      }
      // P[s] / dS[s] were last read by the gradient MMAs of iteration it - 2
      ok = mbar_wait_warp(&bars[B_PDS_EMPTY + s], ((it >> 1) & 1) ^ 1, abort_flag);
      if (!ok) break;
      store_row_chunk(smem + BkvSmem::P + s * BkvSmem::PB, row, cbeg, pv);
      store_row_chunk(smem + BkvSmem::DS + s * BkvSmem::PB, row, cbeg, ds);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_PDS_FULL + s]);
    }
    if (ok && n_iter > 0) ok = mbar_wait_warp(&bars[B_ACC_DONE], 0, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      // accumulators are transposed: TMEM lane = head-dim index d, column = kv row
      tc_fence_after_sync();
      uint32_t a[32], b[32];
      if (n_iter > 0) {
        tmem_ld_32x32b_x32(t_dv + lane_off + cbeg, a);
        tmem_ld_32x32b_x32(t_dk + lane_off + cbeg, b);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) a[i] = b[i] = 0u;
      }
      const int d = row;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int kj = kv0 + cbeg + i;
        if (kj < seq_len) {
          const long long tok = seq_start + kj;
          p.dv[tok * p.dv_ts + static_cast<long long>(g) * p.dv_hs + d] = __float2bfloat16(__uint_as_float(a[i]));
          p.dk[tok * p.dk_ts + static_cast<long long>(g) * p.dk_hs + d] = __float2bfloat16(__uint_as_float(b[i]));
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
// One CTA per (q block, q head); loops over kv blocks j.
// smem: Q | dO | K[2] | V[2] | dS | control.   TMEM: S[2] | dP | dQ.
// MMA issue order keeps the tensor core busy while the math warps work on block j:
//   S[j+1] (and S[j+2]) are computed ahead into the spare S buffer, dP[j+1] is issued as soon as
//   the math warps have drained dP[j], and dQ += dS[j] K[j] runs under the math of block j+1.
struct BqSmem {
  static constexpr int Q = 0, DO = TILE_BYTES, K = 2 * TILE_BYTES, V = 4 * TILE_BYTES, DS = 6 * TILE_BYTES,
                       CTL = 7 * TILE_BYTES, BYTES = 7 * TILE_BYTES + 256 + 1024;
};
enum { Q_QDO = 0, Q_KV_FULL = 1, Q_KV_EMPTY = 3, Q_S_FULL = 5, Q_DS_FULL = 6, Q_ACC_DONE = 7 };

__global__ void __launch_bounds__(AT_BWD_THREADS, 1)
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[Q_KV_FULL + s], 1);
      mbar_init(&bars[Q_KV_EMPTY + s], 1);
    }
    mbar_init(&bars[Q_S_FULL], 1);
    mbar_init(&bars[Q_DS_FULL], 8);
    mbar_init(&bars[Q_ACC_DONE], 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t t_s0 = tmem, t_dp = tmem + 256, t_dq = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars[Q_QDO], 2 * TILE_BYTES);
      load_tile_q(smem + BqSmem::Q, &tq, &bars[Q_QDO], jh, g, seq_start + q0);
      load_tile_q(smem + BqSmem::DO, &tdo, &bars[Q_QDO], jh, g, seq_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&bars[Q_KV_EMPTY + s], ((j >> 1) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[Q_KV_FULL + s], 2 * TILE_BYTES);
        load_tile_kv(smem + BqSmem::K + s * TILE_BYTES, &tk, &bars[Q_KV_FULL + s], g, seq_start + j * 128);
        load_tile_kv(smem + BqSmem::V + s * TILE_BYTES, &tv, &bars[Q_KV_FULL + s], g, seq_start + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sq = smem_u32(smem + BqSmem::Q), sdo = smem_u32(smem + BqSmem::DO);
      const uint32_t sk = smem_u32(smem + BqSmem::K), sv = smem_u32(smem + BqSmem::V);
      const uint32_t sds = smem_u32(smem + BqSmem::DS);
      bool ok = mbar_wait(&bars[Q_QDO], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[Q_KV_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        mma_tile<false, false>(t_s0, sq, sk, false);    // S[0]
        mma_tile<false, false>(t_dp, sdo, sv, false);   // dP[0]
        tc_commit(&bars[Q_S_FULL]);
        if (n_kv > 1) {
          ok = mbar_wait(&bars[Q_KV_FULL + 1], 0, abort_flag);
          if (ok) {
            tc_fence_after_sync();
            mma_tile<false, false>(t_s0 + 128, sq, sk + TILE_BYTES, false);  // S[1]
          }
        }
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait(&bars[Q_DS_FULL], j & 1, abort_flag);  // math of block j done: dS[j] ready, dP free
        if (!ok) break;
        tc_fence_after_sync();
        if (j + 1 < n_kv) {
          mma_tile<false, false>(t_dp, sdo, sv + ((j + 1) & 1) * TILE_BYTES, false);  // dP[j+1]
          tc_commit(&bars[Q_S_FULL]);                                                  // S[j+1], dP[j+1] ready
        }
        mma_tile<false, true>(t_dq, sds, sk + s * TILE_BYTES, j > 0);  // dQ += dS[j] K[j]
        tc_commit(&bars[Q_KV_EMPTY + s]);
        tc_commit(&bars[Q_ACC_DONE]);
        if (j + 2 < n_kv) {
          ok = mbar_wait(&bars[Q_KV_FULL + s], ((j + 2) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          mma_tile<false, false>(t_s0 + s * 128, sq, sk + s * TILE_BYTES, false);  // S[j+2]
        }
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    const int quarter = warp & 3;
    const int cbeg = ((warp - 2) >> 2) * 64;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + row;
    const bool q_valid = qi < seq_len;
    const long long tok = seq_start + qi;
    const float lse2 = q_valid ? p.lse[static_cast<long long>(head) * p.T + tok] * LOG2E : 0.f;
    const float dlt = q_valid ? p.delta[static_cast<long long>(head) * p.T + tok] : 0.f;
    const float neg_lse2 = -lse2;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int kv0 = j * 128;
      ok = mbar_wait_warp(&bars[Q_S_FULL], j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const int lim = q_valid ? (min(seq_len, p.causal ? qi + 1 : seq_len) - kv0) : 0;
      const uint32_t t_s = t_s0 + (j & 1) * 128;
      uint32_t rs0[32], rd0[32], rs1[32], rd1[32];
      tmem_ld_32x32b_x32(t_s + lane_off + cbeg, rs0);
      tmem_ld_32x32b_x32(t_dp + lane_off + cbeg, rd0);
      tmem_ld_32x32b_x32(t_s + lane_off + cbeg + 32, rs1);
      tmem_ld_32x32b_x32(t_dp + lane_off + cbeg + 32, rd1);
      tmem_ld_wait();
      float ds0[32], ds1[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float pr = exp2f(fmaf(__uint_as_float(rs0[i]), p.scale_log2, neg_lse2));
        if (cbeg + i >= lim) pr = 0.f;
        ds0[i] = pr * (__uint_as_float(rd0[i]) - dlt) * p.scale;
        float pr1 = exp2f(fmaf(__uint_as_float(rs1[i]), p.scale_log2, neg_lse2));
        if (cbeg + 32 + i >= lim) pr1 = 0.f;
        ds1[i] = pr1 * (__uint_as_float(rd1[i]) - dlt) * p.scale;
      }
      // the dS tile is single buffered: dQ += dS[j-1] K[j-1] must have retired
      if (j > 0) {
        ok = mbar_wait_warp(&bars[Q_ACC_DONE], (j - 1) & 1, abort_flag);
        if (!ok) break;
      }
      store_row_chunk(smem + BqSmem::DS, row, cbeg, ds0);
      store_row_chunk(smem + BqSmem::DS, row, cbeg + 32, ds1);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[Q_DS_FULL]);
    }
    if (ok && n_kv > 0) ok = mbar_wait_warp(&bars[Q_ACC_DONE], (n_kv - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      __nv_bfloat16* dqrow = p.dq + tok * p.dq_ts + static_cast<long long>(g) * p.dq_gs + jh * p.dq_hs;
#pragma unroll 1
      for (int c0 = cbeg; c0 < cbeg + 64; c0 += 32) {
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
static int make_map_kv(CUtensorMap* m, const void* ptr, int T, int heads, long long ts, long long hs,
                       int box_rows = 128) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ts % 8) || (hs % 8)) return -2;
  cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(T)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(hs) * 2, static_cast<cuuint64_t>(ts) * 2};
  if (heads == 1) strides[0] = 256;
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
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

int attn_bwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.T == 0) return 0;
  if (a.Hq % a.Hkv) return -2;
  const int R = a.Hq / a.Hkv;
  if ((a.do_ts % 8) || (a.do_hs % 8) || (a.dq_ts % 8) || (a.dq_gs % 8) || (a.dq_hs % 8) || (a.dk_ts % 8) ||
      (a.dk_hs % 8) || (a.dv_ts % 8) || (a.dv_hs % 8))
    return -2;
  CUtensorMap tq, tk, tv, tdo, tk64, tv64;
  int rc;
  if ((rc = make_map_q(&tq, a.q, a.T, a.Hkv, R, a.q_ts, a.q_gs, a.q_hs))) return rc;
  if ((rc = make_map_kv(&tk, a.k, a.T, a.Hkv, a.k_ts, a.k_hs))) return rc;
  if ((rc = make_map_kv(&tv, a.v, a.T, a.Hkv, a.v_ts, a.v_hs))) return rc;
  if ((rc = make_map_kv(&tk64, a.k, a.T, a.Hkv, a.k_ts, a.k_hs, 64))) return rc;
  if ((rc = make_map_kv(&tv64, a.v, a.T, a.Hkv, a.v_ts, a.v_hs, 64))) return rc;
  // dO is [T, Hq, 128]: group stride R * head stride
  if ((rc = make_map_q(&tdo, a.dout, a.T, a.Hkv, R, a.do_ts, a.do_hs * R, a.do_hs))) return rc;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BkvSmem::BYTES) !=
            cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BqSmem::BYTES) !=
            cudaSuccess)
      return -4;
    attr = true;
  }
  const AttnParams p = make_params(a);
  const long long warps = static_cast<long long>(a.T) * a.Hq;
  attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a.dout), static_cast<const __nv_bfloat16*>(a.o), a.delta, a.T, a.Hq, a.do_ts,
      a.do_hs, a.o_ts, a.o_hs);
  dim3 grid_kv(2 * max_blocks(a), a.Hkv);
  attn_bwd_dkdv_kernel<<<grid_kv, AT_BWD_THREADS, BkvSmem::BYTES, stream>>>(tq, tk64, tv64, tdo, p);
  dim3 grid_q(max_blocks(a), a.Hq);
  attn_bwd_dq_kernel<<<grid_q, AT_BWD_THREADS, BqSmem::BYTES, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
