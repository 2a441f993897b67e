// Flash attention for sm_100a: bf16, head dim <= 128, packed tokens, causal (bottom-right aligned) or
// bidirectional, GQA, variable-length sequences with separate query / key boundaries.
//
// All matrix products run on tcgen05.mma with fp32 accumulators in TMEM; operands are staged by TMA into
// 128-byte-swizzled shared memory as "two-box" tiles: a [rows x 128] bf16 tile is two [rows x 64] swizzled
// boxes. Such a tile can be read by the tensor core either K-major (rows = M/N index, columns =
// contraction) or MN-major (rows = contraction, columns = M/N index), so Q, K, V and dO are never
// transposed. Head dims below 128 are zero-filled by TMA inside the tile (the tensor map's inner extent is
// the true head dim), so a 80-wide vision head runs through the same 128-wide tiles.
//
// The softmax probabilities (and dS in the backward) never go through shared memory: the math warps
// write them as packed bf16 straight into the TMEM columns of the scores they were computed from, and the
// next tcgen05.mma takes its A operand from TMEM.
//
//   forward : CTA = 256 query rows (two 128-row tiles in ping-pong: the tensor core works on one tile
//             while the softmax warps work on the other), loop over 128-row kv blocks
//               S_t = Q_t K^T                  (A, B shared memory, K-major)
//               O_t += P_t V                   (A = P_t in TMEM, B = V MN-major)
//   dK/dV   : CTA = 128 kv rows, loop over 64-row query blocks of every query head of the group; scores
//             are computed TRANSPOSED so that the kv row is the TMEM lane
//               S^T = K Q^T, dP^T = V dO^T     (N = 64)
//               dV += P^T dO, dK += dS^T Q     (A = P^T / dS^T in TMEM, B = dO / Q MN-major)
//   dQ      : CTA = 128 query rows, loop over 128-row kv blocks
//               S = Q K^T, dP = dO V^T,  dQ += dS K   (A = dS in TMEM, B = K MN-major)
//
// Every mbarrier wait is bounded; a wait that gives up sets the status word and all roles unwind.
//
// Replaces TE DotProductAttention / flash-attn in the reference
// (loongforge/models/common/local_layers/local_attention.py:23,147-158) and the thd / windowed attention
// of its vision towers (loongforge/models/encoder/qwen2_vl_vision_models/vision_model.py:54-160).
#include "sm100_ptx.cuh"
#include "attention_sm100.h"
#include <cstdio>
#include <cstdlib>

namespace lf {

static constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KB: [128 rows x 128 d]
static constexpr int BOX_BYTES = 128 * 64 * 2;    // 16 KB
static constexpr int HTILE_BYTES = 64 * 128 * 2;  // 16 KB: [64 rows x 128 d]
static constexpr int HBOX_BYTES = 64 * 64 * 2;    // 8 KB
static constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  int Tq, Tk, Hq, Hkv, R, D;
  float scale_log2;  // scale * log2(e)
  float scale;
  int causal;
  const int* cu_q;
  const int* cu_k;
  int num_seqs;
  int* status;
  __nv_bfloat16* o;
  long long o_ts, o_hs;
  float* lse;
  float* delta;
  __nv_bfloat16 *dq, *dk, *dv;
  long long dq_ts, dq_gs, dq_hs, dk_ts, dk_hs, dv_ts, dv_hs;
};

// One sequence of the packed batch: token offsets and lengths on the query and on the key side.
struct Seq {
  int q0, qn, k0, kn;
};

// ------------------------------------------------------------------------- tile helpers
// TMA load of a [ROWS tokens x 128 dims] tile (two boxes) of query-type tensors: 4-D map (d, head-in-group,
// group, token). Dims past the head dim are zero-filled.
template <int ROWS>
__device__ __forceinline__ void load_tile_q(uint8_t* smem, const CUtensorMap* m, uint64_t* bar, int j, int g, int tok) {
  for (int b = 0; b < 2; ++b) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];" ::"r"(smem_u32(smem + b * (ROWS * 128))),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(b * 64), "r"(j), "r"(g), "r"(tok)
        : "memory");
  }
}
// Key-type tensors: 3-D map (d, head, token).
template <int ROWS>
__device__ __forceinline__ void load_tile_kv(uint8_t* smem, const CUtensorMap* m, uint64_t* bar, int g, int tok) {
  for (int b = 0; b < 2; ++b) tma_load_3d(smem + b * (ROWS * 128), m, bar, b * 64, g, tok);
}

// D[128 x N] (+)= A B^T over the 128 head dims; A = [128 rows x 128 d] tile, B = [N rows x 128 d] tile, both
// K-major in shared memory.
template <int N>
__device__ __forceinline__ void mma_ss_kmajor(uint32_t tmem_d, uint32_t a_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc(1, 1, false, false, 128, N);
  constexpr uint32_t b_box = N * 128;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t da = make_smem_desc_sw128(a_base + (kk >> 2) * BOX_BYTES + (kk & 3) * 32, 16, 1024);
    const uint64_t db = make_smem_desc_sw128(b_base + (kk >> 2) * b_box + (kk & 3) * 32, 16, 1024);
    tc_mma_f16_ss(tmem_d, da, db, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// D[128 x 128] (+)= A B with A [128 x 16*KSTEPS] packed bf16 in TMEM (row = lane, two values per 32-bit column) and
// B = [16*KSTEPS rows x 128 d] tile read MN-major from shared memory (rows = contraction). The packed A columns are
// written by one or two math warps per TMEM lane quarter, each only over columns it has itself finished reading:
//   A_LAYOUT 0: one writer, k-step kk at column 8 kk;
//   A_LAYOUT 1: two writers of 32 fp32 columns each (64-column score buffer): k-steps {0,1} at 0, {2,3} at 32;
//   A_LAYOUT 2: two writers of 64 fp32 columns each (128-column score buffer): k-steps {0..3} at 0, {4..7} at 64.
template <int KSTEPS, int A_LAYOUT>
__device__ __forceinline__ void mma_ts_bmn(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc(1, 1, false, true, 128, 128);
  constexpr uint32_t b_box = KSTEPS * 16 * 128;  // bytes of one [rows x 64] box
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    const uint64_t db = make_smem_desc_sw128(b_base + kk * 2048, b_box, 1024);
    const uint32_t a = A_LAYOUT == 1   ? tmem_a + (kk >> 1) * 32 + (kk & 1) * 8
                       : A_LAYOUT == 2 ? tmem_a + (kk >> 2) * 64 + (kk & 3) * 8
                                       : tmem_a + kk * 8;
    tc_mma_f16_ts(tmem_d, a, db, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// Sequence that holds block `blk` when every sequence is cut into blocks of `rows` tokens along the query side
// (BY_K = false) or the key side (BY_K = true); false when blk is past the end.
template <bool BY_K>
__device__ __forceinline__ bool locate_block(int blk, int rows, const AttnParams& p, Seq& s, int& blk_in_seq) {
  if (p.cu_q == nullptr) {
    s.q0 = 0; s.qn = p.Tq; s.k0 = 0; s.kn = p.Tk;
    blk_in_seq = blk;
    return blk * rows < (BY_K ? p.Tk : p.Tq);
  }
  int acc = 0;
  for (int i = 0; i < p.num_seqs; ++i) {
    const int qa = p.cu_q[i], qb = p.cu_q[i + 1], ka = p.cu_k[i], kb = p.cu_k[i + 1];
    const int n = BY_K ? kb - ka : qb - qa;
    const int nb = (n + rows - 1) / rows;
    if (blk < acc + nb) {
      s.q0 = qa; s.qn = qb - qa; s.k0 = ka; s.kn = kb - ka;
      blk_in_seq = blk - acc;
      return true;
    }
    acc += nb;
  }
  return false;
}

// Number of keys a 128-row query tile starting at row `q_first` of its sequence can see (0 for a tile past the end).
// Causal masks are aligned to the bottom right: query row i sees keys j <= i + (kn - qn).
__device__ __forceinline__ int visible_keys(const Seq& s, int q_first, int rows, int causal) {
  if (q_first >= s.qn) return 0;
  int lim = s.kn;
  if (causal) lim = min(lim, q_first + rows + (s.kn - s.qn));
  return max(lim, 0);
}

// Wait of a math warp. All lanes execute the blocking try_wait: its wake-up latency is far below that of a polled
// test_wait + nanosleep, and the softmax / gradient math sits on the critical path between two tensor-core products.
__device__ __forceinline__ bool math_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_wait(bar, parity, abort_flag);
}

struct SharedCtl {
  uint64_t bars[24];
  uint32_t tmem_slot;
  int abort_flag;
};

// =========================================================================== forward
// smem: Q[2 tiles] | K[2 stages] | V[2 stages] | control.   TMEM: S0 | S1 | O0 | O1 (128 columns each); the packed
// probabilities P_t overwrite columns [0, 64) of S_t.
struct FwdSmem {
  static constexpr int Q = 0;
  static constexpr int K = 2 * TILE_BYTES;
  static constexpr int V = 4 * TILE_BYTES;
  static constexpr int CTL = 6 * TILE_BYTES;
  static constexpr int BYTES = 6 * TILE_BYTES + 256 + 1024;
};
static constexpr int FWD_THREADS = 320;  // TMA warp, MMA warp, 4 softmax warps per query tile
enum { F_Q = 0, F_K_FULL = 1, F_K_EMPTY = 3, F_V_FULL = 5, F_V_EMPTY = 7, F_S_FULL = 9, F_P_FULL = 11, F_O_DONE = 13 };

// Issue order of the MMA warp for kv block j (both tiles t = 0, 1 active):
//   O_0 += P_0[j] V[j];  S_0[j+1] = Q_0 K[j+1]^T;  O_1 += P_1[j] V[j];  S_1[j+1] = Q_1 K[j+1]^T
// so while the softmax warps of tile 0 work on S_0[j+1] the tensor core runs tile 1's products and vice versa.
// tcgen05.mma instructions execute in issue order, which is what makes the aliasing safe: S_t[j+1] overwrites the
// columns of P_t[j] only after O_t += P_t[j] V[j] has read them.
__global__ void __launch_bounds__(FWD_THREADS, 1)
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

  Seq sq;
  int qb;
  // launch the long (late) query blocks first: with a causal mask they do the most work
  if (!locate_block<false>(gridDim.x - 1 - blockIdx.x, 256, p, sq, qb)) return;  // uniform for the whole CTA
  const int q0 = qb * 256;
  const int off = sq.kn - sq.qn;
  int n_kv[2];
  n_kv[0] = (visible_keys(sq, q0, 128, p.causal) + 127) >> 7;
  n_kv[1] = (visible_keys(sq, q0 + 128, 128, p.causal) + 127) >> 7;
  const int n_max = max(n_kv[0], n_kv[1]);

  if (threadIdx.x == 0) {
    mbar_init(&bars[F_Q], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[F_K_FULL + s], 1);
      mbar_init(&bars[F_K_EMPTY + s], 1);
      mbar_init(&bars[F_V_FULL + s], 1);
      mbar_init(&bars[F_V_EMPTY + s], 1);
      mbar_init(&bars[F_S_FULL + s], 1);
      mbar_init(&bars[F_P_FULL + s], 4);
      mbar_init(&bars[F_O_DONE + s], 1);
    }
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;

  if (warp == 0) {
    if (lane == 0 && n_max > 0) {
      mbar_arrive_expect_tx(&bars[F_Q], 2 * TILE_BYTES);
      load_tile_q<128>(smem + FwdSmem::Q, &tq, &bars[F_Q], jh, g, sq.q0 + q0);
      load_tile_q<128>(smem + FwdSmem::Q + TILE_BYTES, &tq, &bars[F_Q], jh, g, sq.q0 + q0 + 128);
      for (int j = 0; j < n_max; ++j) {
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&bars[F_K_EMPTY + s], par, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[F_K_FULL + s], TILE_BYTES);
        load_tile_kv<128>(smem + FwdSmem::K + s * TILE_BYTES, &tk, &bars[F_K_FULL + s], g, sq.k0 + j * 128);
        if (!mbar_wait(&bars[F_V_EMPTY + s], par, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[F_V_FULL + s], TILE_BYTES);
        load_tile_kv<128>(smem + FwdSmem::V + s * TILE_BYTES, &tv, &bars[F_V_FULL + s], g, sq.k0 + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_max > 0) {
      const uint32_t sq_addr = smem_u32(smem + FwdSmem::Q);
      const uint32_t sk = smem_u32(smem + FwdSmem::K), sv = smem_u32(smem + FwdSmem::V);
      bool ok = mbar_wait(&bars[F_Q], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[F_K_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < 2; ++t) {
          if (n_kv[t] > 0) {
            mma_ss_kmajor<128>(tmem + t * 128, sq_addr + t * TILE_BYTES, sk, false);
            tc_commit(&bars[F_S_FULL + t]);
          }
        }
        tc_commit(&bars[F_K_EMPTY + 0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j & 1, s1 = s ^ 1;
        bool k_ready = false, v_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < n_kv[t]) {
            if (!v_ready) {
              ok = mbar_wait(&bars[F_V_FULL + s], (j >> 1) & 1, abort_flag);
              if (!ok) break;
              v_ready = true;
            }
            ok = mbar_wait(&bars[F_P_FULL + t], j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            mma_ts_bmn<8, 0>(tmem + 256 + t * 128, tmem + t * 128, sv + s * TILE_BYTES, j > 0);  // O_t += P_t V
            tc_commit(&bars[F_O_DONE + t]);
          }
          if (j + 1 < n_kv[t]) {
            if (!k_ready) {
              ok = mbar_wait(&bars[F_K_FULL + s1], ((j + 1) >> 1) & 1, abort_flag);
              if (!ok) break;
              k_ready = true;
              tc_fence_after_sync();
            }
            mma_ss_kmajor<128>(tmem + t * 128, sq_addr + t * TILE_BYTES, sk + s1 * TILE_BYTES, false);  // S_t[j+1]
            tc_commit(&bars[F_S_FULL + t]);
          }
        }
        if (!ok) break;
        tc_commit(&bars[F_V_EMPTY + s]);
        if (j + 1 < n_max) tc_commit(&bars[F_K_EMPTY + s1]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int t = (warp - 2) >> 2;  // query tile of this warp
    const int quarter = warp & 3;   // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;
    const int qi = q0 + t * 128 + row;  // position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t ts = tmem + t * 128 + lane_off;
    const uint32_t to = tmem + 256 + t * 128 + lane_off;
    const int my_n = n_kv[t];
    const int q_first = q0 + t * 128;
    // keys [0, row_lim) are visible to this row
    const int row_lim = min(sq.kn, p.causal ? qi + off + 1 : sq.kn);
    float m_ref = -INFINITY;  // running reference maximum in the log2 domain (scaled scores)
    float l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < my_n && ok; ++j) {
      ok = math_wait(&bars[F_S_FULL + t], j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const int kv0 = j * 128;
      // the whole score row of this thread in registers: one TMEM pass
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld_32x32b_x32(ts, r0);
      tmem_ld_32x32b_x32(ts + 32, r1);
      tmem_ld_32x32b_x32(ts + 64, r2);
      tmem_ld_32x32b_x32(ts + 96, r3);
      tmem_ld_wait();
      // only tiles cut by the sequence end or by the causal diagonal need the mask (warp-uniform test)
      const bool need_mask = (kv0 + 128 > sq.kn) || (p.causal && kv0 + 128 > q_first + off + 1);
      if (need_mask) {
        const int lim = row_lim - kv0;  // columns [0, lim) stay
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
        ok = math_wait(&bars[F_O_DONE + t], (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(to + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x16(to + c0, r);
        }
      }
      l_sum *= alpha;
      m_ref = m_new;
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      // exponentials, packed two bf16 per 32-bit TMEM column over the first 64 columns of S_t
      float l0 = 0.f, l1 = 0.f;
      {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = exp2f(fmaf(__uint_as_float(r0[2 * i]), p.scale_log2, neg_m));
          const float b = exp2f(fmaf(__uint_as_float(r0[2 * i + 1]), p.scale_log2, neg_m));
          l0 += a; l1 += b;
          pk[i] = pack_bf16x2(a, b);
        }
        tmem_st_32x32b_x16(ts, pk);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = exp2f(fmaf(__uint_as_float(r1[2 * i]), p.scale_log2, neg_m));
          const float b = exp2f(fmaf(__uint_as_float(r1[2 * i + 1]), p.scale_log2, neg_m));
          l0 += a; l1 += b;
          pk[i] = pack_bf16x2(a, b);
        }
        tmem_st_32x32b_x16(ts + 16, pk);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = exp2f(fmaf(__uint_as_float(r2[2 * i]), p.scale_log2, neg_m));
          const float b = exp2f(fmaf(__uint_as_float(r2[2 * i + 1]), p.scale_log2, neg_m));
          l0 += a; l1 += b;
          pk[i] = pack_bf16x2(a, b);
        }
        tmem_st_32x32b_x16(ts + 32, pk);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = exp2f(fmaf(__uint_as_float(r3[2 * i]), p.scale_log2, neg_m));
          const float b = exp2f(fmaf(__uint_as_float(r3[2 * i + 1]), p.scale_log2, neg_m));
          l0 += a; l1 += b;
          pk[i] = pack_bf16x2(a, b);
        }
        tmem_st_32x32b_x16(ts + 48, pk);
      }
      l_sum += l0 + l1;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[F_P_FULL + t]);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && my_n > 0) ok = math_wait(&bars[F_O_DONE + t], (my_n - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      const bool valid = qi < sq.qn;
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      const long long tok = sq.q0 + qi;
      __nv_bfloat16* orow = p.o + tok * p.o_ts + static_cast<long long>(head) * p.o_hs;
#pragma unroll 1
      for (int c0 = 0; c0 < p.D; c0 += 32) {
        uint32_t r[32];
        if (my_n > 0) {
          tmem_ld_32x32b_x32(to + c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;  // a row block that sees no key at all
        }
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (c0 + i < p.D) {
              uint4 q;
              q.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              q.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              q.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              q.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c0 + i) = q;
            }
          }
        }
      }
      if (valid)
        p.lse[static_cast<long long>(head) * p.Tq + tok] =
            l_sum > 0.f ? (m_ref + log2f(l_sum)) * (1.f / LOG2E) : -INFINITY;
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
                                  float* __restrict__ delta, int T, int Hq, int D, long long do_ts, long long do_hs,
                                  long long o_ts, long long o_hs) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(T) * Hq) return;
  const int t = static_cast<int>(w / Hq), h = static_cast<int>(w % Hq);
  float s = 0.f;
  if (lane * 4 < D) {
    const uint2 a = *reinterpret_cast<const uint2*>(dout + t * do_ts + h * do_hs + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(o + t * o_ts + h * o_hs + lane * 4);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(bh[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// =========================================================================== backward: dK, dV
// One CTA per (128-row kv block, kv head); loops over the R query heads of the group and over the 64-row query
// blocks that see this kv block. The scores are computed transposed, so that the kv row is the TMEM lane and the
// probabilities can feed the gradient products as TMEM A operands:
//   S^T  = K Q^T, dP^T = V dO^T                       [128 kv x 64 q] fp32 in TMEM (double buffered)
//   P^T  = exp2(S^T*scale*log2e - lse_q), dS^T = P^T (dP^T - delta_q) scale   -> packed bf16 over S^T / dP^T
//   dV  += P^T dO,  dK += dS^T Q                      [128 kv x 128 d] fp32 in TMEM
// Per-query statistics (-lse*log2e, delta) of the 64 rows of a block are staged in shared memory by the TMA warp.
// Q / dO tiles run through a ring of four stages so that their loads are issued well ahead of their use.
// TMEM columns: S^T[0] 0..63 | S^T[1] 64..127 | dP^T[0] 128..191 | dP^T[1] 192..255 | dV 256..383 | dK 384..511.
// Inside a 64-column S^T / dP^T buffer the math warp that owns query columns [32h, 32h+32) writes its 32 packed
// values to columns [32h, 32h+16): it only ever overwrites columns it has itself finished reading.
struct BkvSmem {
  static constexpr int STAGES = 4;
  static constexpr int K = 0, V = TILE_BYTES, Q = 2 * TILE_BYTES, DO = Q + STAGES * HTILE_BYTES,
                       STAT = DO + STAGES * HTILE_BYTES,  // per stage: 64 x (-lse*log2e) then 64 x delta
                       CTL = STAT + STAGES * 512, BYTES = CTL + 256 + 1024;
};
static constexpr int BWD_THREADS = 320;  // TMA warp, MMA warp, 8 math warps (2 per TMEM lane quarter)
enum { B_KV = 0, B_QDO_FULL = 1, B_QDO_EMPTY = 5, B_S_FULL = 9, B_PDS_FULL = 11, B_ACC_DONE = 13 };

__global__ void __launch_bounds__(BWD_THREADS, 1)
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
  constexpr int ST = BkvSmem::STAGES;

  Seq sq;
  int kb;
  if (!locate_block<true>(blockIdx.x, 128, p, sq, kb)) return;
  const int kv0 = kb * 128;
  const int off = sq.kn - sq.qn;
  // query rows i >= kv0 - off see this block (causal); query blocks are 64 rows
  const int n_qb_total = (sq.qn + 63) >> 6;
  const int qb_first = p.causal ? (max(kv0 - off, 0) >> 6) : 0;
  const int n_iter = max(n_qb_total - qb_first, 0) * p.R;  // iteration it -> head it % R, q block qb_first + it / R

  if (threadIdx.x == 0) {
    mbar_init(&bars[B_KV], 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&bars[B_QDO_FULL + s], 2);  // TMA transaction + statistics written by the TMA warp
      mbar_init(&bars[B_QDO_EMPTY + s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[B_S_FULL + s], 1);
      mbar_init(&bars[B_PDS_FULL + s], 8);
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
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

  if (warp == 0) {
    if (n_iter > 0) {
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars[B_KV], 2 * TILE_BYTES);
        load_tile_kv<128>(smem + BkvSmem::K, &tk, &bars[B_KV], g, sq.k0 + kv0);
        load_tile_kv<128>(smem + BkvSmem::V, &tv, &bars[B_KV], g, sq.k0 + kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % ST;
        int ok = 1;
        if (lane == 0) {
          if (!mbar_wait(&bars[B_QDO_EMPTY + s], ((it / ST) & 1) ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
            ok = 0;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const int jh = it % p.R, qb = qb_first + it / p.R;
        const int head = g * p.R + jh;
        if (lane == 0) {
          mbar_arrive_expect_tx(&bars[B_QDO_FULL + s], 2 * HTILE_BYTES);
          load_tile_q<64>(smem + BkvSmem::Q + s * HTILE_BYTES, &tq, &bars[B_QDO_FULL + s], jh, g, sq.q0 + qb * 64);
          load_tile_q<64>(smem + BkvSmem::DO + s * HTILE_BYTES, &tdo, &bars[B_QDO_FULL + s], jh, g, sq.q0 + qb * 64);
        }
        // statistics of the block's 64 query rows; rows past the sequence end get -lse = -inf (probability 0)
        float* stat = reinterpret_cast<float*>(smem + BkvSmem::STAT + s * 512);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int qi = qb * 64 + h * 32 + lane;
          float nl = -INFINITY, dl = 0.f;
          if (qi < sq.qn) {
            const long long idx = static_cast<long long>(head) * p.Tq + sq.q0 + qi;
            const float l = p.lse[idx];
            nl = (l == -INFINITY) ? -INFINITY : -l * LOG2E;  // a row that saw no key keeps probability 0
            dl = p.delta[idx];
          }
          stat[h * 32 + lane] = nl;
          stat[64 + h * 32 + lane] = dl;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_QDO_FULL + s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      const uint32_t sk = smem_u32(smem + BkvSmem::K), sv = smem_u32(smem + BkvSmem::V);
      const uint32_t sqa = smem_u32(smem + BkvSmem::Q), sdo = smem_u32(smem + BkvSmem::DO);
      bool ok = mbar_wait(&bars[B_KV], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[B_QDO_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        mma_ss_kmajor<64>(t_s, sk, sqa, false);    // S^T[0]  = K Q^T
        mma_ss_kmajor<64>(t_dp, sv, sdo, false);   // dP^T[0] = V dO^T
        tc_commit(&bars[B_S_FULL + 0]);
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int b = it & 1, s = it % ST;
        if (it + 1 < n_iter) {
          const int b1 = b ^ 1, s1 = (it + 1) % ST;
          ok = mbar_wait(&bars[B_QDO_FULL + s1], ((it + 1) / ST) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          mma_ss_kmajor<64>(t_s + b1 * 64, sk, sqa + s1 * HTILE_BYTES, false);
          mma_ss_kmajor<64>(t_dp + b1 * 64, sv, sdo + s1 * HTILE_BYTES, false);
          tc_commit(&bars[B_S_FULL + b1]);
        }
        ok = mbar_wait(&bars[B_PDS_FULL + b], (it >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_ts_bmn<4, 1>(t_dv, t_s + b * 64, sdo + s * HTILE_BYTES, it > 0);   // dV += P^T dO
        mma_ts_bmn<4, 1>(t_dk, t_dp + b * 64, sqa + s * HTILE_BYTES, it > 0);  // dK += dS^T Q
        tc_commit(&bars[B_QDO_EMPTY + s]);
        if (it == n_iter - 1) tc_commit(&bars[B_ACC_DONE]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    // two warps share each TMEM lane quarter; each takes 32 of the 64 query columns
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;  // kv row of this thread inside the block
    const int kj = kv0 + row;             // position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int b = it & 1, s = it % ST;
      const int qb = qb_first + it / p.R;
      const int qc0 = qb * 64 + half * 32;  // first query row of this warp's columns
      ok = math_wait(&bars[B_QDO_FULL + s], (it / ST) & 1, abort_flag);  // statistics visible
      if (ok) ok = math_wait(&bars[B_S_FULL + b], (it >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t rs[32], rd[32];
      tmem_ld_32x32b_x32(t_s + b * 64 + lane_off + half * 32, rs);
      tmem_ld_32x32b_x32(t_dp + b * 64 + lane_off + half * 32, rd);
      tmem_ld_wait();
      const float4* nl4 = reinterpret_cast<const float4*>(smem + BkvSmem::STAT + s * 512) + half * 8;
      const float4* dl4 = nl4 + 16;
      // query column c (row qc0 + c of the sequence) sees this kv row iff kj <= qc0 + c + off, i.e. c >= first
      const bool need_mask = p.causal && (kv0 + 127 > qc0 + off);
      const int first = need_mask ? kj - off - qc0 : 0;
      uint32_t pp[16], pd[16];
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 nl = nl4[c4], dl = dl4[c4];
        const float nls[4] = {nl.x, nl.y, nl.z, nl.w}, dls[4] = {dl.x, dl.y, dl.z, dl.w};
        float pr[4], ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = c4 * 4 + e;
          float x = exp2f(fmaf(__uint_as_float(rs[c]), p.scale_log2, nls[e]));
          if (c < first) x = 0.f;
          pr[e] = x;
          ds[e] = x * (__uint_as_float(rd[c]) - dls[e]) * p.scale;
        }
        pp[c4 * 2] = pack_bf16x2(pr[0], pr[1]);
        pp[c4 * 2 + 1] = pack_bf16x2(pr[2], pr[3]);
        pd[c4 * 2] = pack_bf16x2(ds[0], ds[1]);
        pd[c4 * 2 + 1] = pack_bf16x2(ds[2], ds[3]);
      }
      tmem_st_32x32b_x16(t_s + b * 64 + lane_off + half * 32, pp);
      tmem_st_32x32b_x16(t_dp + b * 64 + lane_off + half * 32, pd);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_PDS_FULL + b]);
    }
    if (ok && n_iter > 0) ok = math_wait(&bars[B_ACC_DONE], 0, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      // TMEM lane = kv row, column = head dim; this warp stores head dims [64 half, 64 half + 64)
      tc_fence_after_sync();
      const bool valid = kj < sq.kn;
      const long long tok = sq.k0 + kj;
      __nv_bfloat16* dvrow = p.dv + tok * p.dv_ts + static_cast<long long>(g) * p.dv_hs;
      __nv_bfloat16* dkrow = p.dk + tok * p.dk_ts + static_cast<long long>(g) * p.dk_hs;
#pragma unroll 1
      for (int c0 = half * 64; c0 < half * 64 + 64 && c0 < p.D; c0 += 32) {
        uint32_t a[32], bq[32];
        if (n_iter > 0) {
          tmem_ld_32x32b_x32(t_dv + lane_off + c0, a);
          tmem_ld_32x32b_x32(t_dk + lane_off + c0, bq);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = bq[i] = 0u;  // a kv block no query sees
        }
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (c0 + i < p.D) {
              uint4 x, y;
              x.x = pack_bf16x2(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
              x.y = pack_bf16x2(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
              x.z = pack_bf16x2(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
              x.w = pack_bf16x2(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
              y.x = pack_bf16x2(__uint_as_float(bq[i]), __uint_as_float(bq[i + 1]));
              y.y = pack_bf16x2(__uint_as_float(bq[i + 2]), __uint_as_float(bq[i + 3]));
              y.z = pack_bf16x2(__uint_as_float(bq[i + 4]), __uint_as_float(bq[i + 5]));
              y.w = pack_bf16x2(__uint_as_float(bq[i + 6]), __uint_as_float(bq[i + 7]));
              *reinterpret_cast<uint4*>(dvrow + c0 + i) = x;
              *reinterpret_cast<uint4*>(dkrow + c0 + i) = y;
            }
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
// One CTA per (128-row q block, q head); loops over 128-row kv blocks j.
// smem: Q | dO | K[3 stages] | V[2 stages] | control.   TMEM: S[2] | dP | dQ (128 columns each); the packed dS[j]
// overwrites S[j & 1] (each math warp writes only columns it has finished reading: the warp that owns score columns
// [64h, 64h+64) writes its 32 packed columns at [64h, 64h+32)).
// MMA issue order keeps the tensor core busy while the math warps work on block j:
//   S[j+1] (and S[j+2]) are computed ahead into the spare S buffer, dP[j+1] is issued as soon as the math warps have
//   drained dP[j], and dQ += dS[j] K[j] runs under the math of block j+1. K needs three stages because K[j] is read
//   last (by dQ) while K[j+2] is already wanted for S[j+2]; V[j] is free as soon as dP[j] is done.
struct BqSmem {
  static constexpr int Q = 0, DO = TILE_BYTES, K = 2 * TILE_BYTES, V = 5 * TILE_BYTES, CTL = 7 * TILE_BYTES,
                       BYTES = 7 * TILE_BYTES + 256 + 1024;
};
enum { Q_QDO = 0, Q_K_FULL = 1, Q_K_EMPTY = 4, Q_V_FULL = 7, Q_V_EMPTY = 9, Q_S_FULL = 11, Q_DS_FULL = 12, Q_ACC_DONE = 13 };

__global__ void __launch_bounds__(BWD_THREADS, 1)
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

  Seq sq;
  int qb;
  if (!locate_block<false>(gridDim.x - 1 - blockIdx.x, 128, p, sq, qb)) return;
  const int q0 = qb * 128;
  const int off = sq.kn - sq.qn;
  const int n_kv = (visible_keys(sq, q0, 128, p.causal) + 127) >> 7;

  if (threadIdx.x == 0) {
    mbar_init(&bars[Q_QDO], 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&bars[Q_K_FULL + s], 1);
      mbar_init(&bars[Q_K_EMPTY + s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[Q_V_FULL + s], 1);
      mbar_init(&bars[Q_V_EMPTY + s], 1);
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
    if (lane == 0 && n_kv > 0) {
      mbar_arrive_expect_tx(&bars[Q_QDO], 2 * TILE_BYTES);
      load_tile_q<128>(smem + BqSmem::Q, &tq, &bars[Q_QDO], jh, g, sq.q0 + q0);
      load_tile_q<128>(smem + BqSmem::DO, &tdo, &bars[Q_QDO], jh, g, sq.q0 + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % 3, vs = j & 1;
        if (!mbar_wait(&bars[Q_K_EMPTY + ks], ((j / 3) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[Q_K_FULL + ks], TILE_BYTES);
        load_tile_kv<128>(smem + BqSmem::K + ks * TILE_BYTES, &tk, &bars[Q_K_FULL + ks], g, sq.k0 + j * 128);
        if (!mbar_wait(&bars[Q_V_EMPTY + vs], ((j >> 1) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_arrive_expect_tx(&bars[Q_V_FULL + vs], TILE_BYTES);
        load_tile_kv<128>(smem + BqSmem::V + vs * TILE_BYTES, &tv, &bars[Q_V_FULL + vs], g, sq.k0 + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t sqa = smem_u32(smem + BqSmem::Q), sdo = smem_u32(smem + BqSmem::DO);
      const uint32_t sk = smem_u32(smem + BqSmem::K), sv = smem_u32(smem + BqSmem::V);
      bool ok = mbar_wait(&bars[Q_QDO], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[Q_K_FULL + 0], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[Q_V_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        mma_ss_kmajor<128>(t_s0, sqa, sk, false);   // S[0]
        mma_ss_kmajor<128>(t_dp, sdo, sv, false);   // dP[0]
        tc_commit(&bars[Q_V_EMPTY + 0]);
        tc_commit(&bars[Q_S_FULL]);
        if (n_kv > 1) {
          ok = mbar_wait(&bars[Q_K_FULL + 1], 0, abort_flag);
          if (ok) {
            tc_fence_after_sync();
            mma_ss_kmajor<128>(t_s0 + 128, sqa, sk + TILE_BYTES, false);  // S[1]
          }
        }
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int b = j & 1;
        ok = mbar_wait(&bars[Q_DS_FULL], j & 1, abort_flag);  // math of block j done: dS[j] ready, dP free
        if (!ok) break;
        tc_fence_after_sync();
        if (j + 1 < n_kv) {
          const int vs1 = (j + 1) & 1;
          ok = mbar_wait(&bars[Q_V_FULL + vs1], ((j + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          mma_ss_kmajor<128>(t_dp, sdo, sv + vs1 * TILE_BYTES, false);  // dP[j+1]
          tc_commit(&bars[Q_V_EMPTY + vs1]);
          tc_commit(&bars[Q_S_FULL]);  // S[j+1], dP[j+1] ready
        }
        mma_ts_bmn<8, 2>(t_dq, t_s0 + b * 128, sk + (j % 3) * TILE_BYTES, j > 0);  // dQ += dS[j] K[j]
        tc_commit(&bars[Q_K_EMPTY + (j % 3)]);
        tc_commit(&bars[Q_ACC_DONE]);
        if (j + 2 < n_kv) {
          const int ks2 = (j + 2) % 3;
          ok = mbar_wait(&bars[Q_K_FULL + ks2], ((j + 2) / 3) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          mma_ss_kmajor<128>(t_s0 + b * 128, sqa, sk + ks2 * TILE_BYTES, false);  // S[j+2] over dS[j]
        }
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int cbeg = half * 64;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + row;
    const bool q_valid = qi < sq.qn;
    const long long tok = sq.q0 + qi;
    float lse = q_valid ? p.lse[static_cast<long long>(head) * p.Tq + tok] : INFINITY;
    const float dlt = q_valid ? p.delta[static_cast<long long>(head) * p.Tq + tok] : 0.f;
    // invalid rows and rows that saw no key get probability 0
    const float neg_lse2 = (lse == -INFINITY || !q_valid) ? -INFINITY : -lse * LOG2E;
    const int row_lim = q_valid ? min(sq.kn, p.causal ? qi + off + 1 : sq.kn) : 0;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int kv0 = j * 128;
      ok = math_wait(&bars[Q_S_FULL], j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const int lim = row_lim - kv0;  // score columns [0, lim) of this row are kept
      const uint32_t t_s = t_s0 + (j & 1) * 128 + lane_off;
      uint32_t rs0[32], rd0[32], rs1[32], rd1[32];
      tmem_ld_32x32b_x32(t_s + cbeg, rs0);
      tmem_ld_32x32b_x32(t_dp + lane_off + cbeg, rd0);
      tmem_ld_32x32b_x32(t_s + cbeg + 32, rs1);
      tmem_ld_32x32b_x32(t_dp + lane_off + cbeg + 32, rd1);
      tmem_ld_wait();
      uint32_t pk0[16], pk1[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float a = exp2f(fmaf(__uint_as_float(rs0[2 * i]), p.scale_log2, neg_lse2));
        float b = exp2f(fmaf(__uint_as_float(rs0[2 * i + 1]), p.scale_log2, neg_lse2));
        if (cbeg + 2 * i >= lim) a = 0.f;
        if (cbeg + 2 * i + 1 >= lim) b = 0.f;
        pk0[i] = pack_bf16x2(a * (__uint_as_float(rd0[2 * i]) - dlt) * p.scale,
                             b * (__uint_as_float(rd0[2 * i + 1]) - dlt) * p.scale);
        float c = exp2f(fmaf(__uint_as_float(rs1[2 * i]), p.scale_log2, neg_lse2));
        float d = exp2f(fmaf(__uint_as_float(rs1[2 * i + 1]), p.scale_log2, neg_lse2));
        if (cbeg + 32 + 2 * i >= lim) c = 0.f;
        if (cbeg + 32 + 2 * i + 1 >= lim) d = 0.f;
        pk1[i] = pack_bf16x2(c * (__uint_as_float(rd1[2 * i]) - dlt) * p.scale,
                             d * (__uint_as_float(rd1[2 * i + 1]) - dlt) * p.scale);
      }
      tmem_st_32x32b_x16(t_s + cbeg, pk0);
      tmem_st_32x32b_x16(t_s + cbeg + 16, pk1);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[Q_DS_FULL]);
    }
    if (ok && n_kv > 0) ok = math_wait(&bars[Q_ACC_DONE], (n_kv - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      __nv_bfloat16* dqrow = p.dq + tok * p.dq_ts + static_cast<long long>(g) * p.dq_gs + jh * p.dq_hs;
#pragma unroll 1
      for (int c0 = cbeg; c0 < cbeg + 64 && c0 < p.D; c0 += 32) {
        uint32_t a[32];
        if (n_kv > 0) {
          tmem_ld_32x32b_x32(t_dq + lane_off + c0, a);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = 0u;
        }
        if (q_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (c0 + i < p.D) {
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

// 4-D map (d, head-in-group, group, token) with box (64, 1, 1, rows). The inner extent is the true head dim: the
// part of a 64-wide box past it is zero-filled.
static int make_map_q(CUtensorMap* m, const void* ptr, int T, int D, int groups, int R, long long ts, long long gs,
                      long long hs, int box_rows) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ts % 8) || (gs % 8) || (hs % 8)) return -2;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(R), static_cast<cuuint64_t>(groups),
                        static_cast<cuuint64_t>(T)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(hs) * 2, static_cast<cuuint64_t>(gs) * 2,
                           static_cast<cuuint64_t>(ts) * 2};
  // a degenerate dimension of extent 1 may carry any (16-byte aligned, non-zero) stride
  if (R == 1) strides[0] = 256;
  if (groups == 1) strides[1] = strides[0] * (R > 1 ? R : 1);
  cuuint32_t box[4] = {64, 1, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t es[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}
// 3-D map (d, head, token) with box (64, 1, rows).
static int make_map_kv(CUtensorMap* m, const void* ptr, int T, int D, int heads, long long ts, long long hs,
                       int box_rows) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ts % 8) || (hs % 8)) return -2;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(T)};
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
  p.Tq = a.Tq; p.Tk = a.Tk; p.Hq = a.Hq; p.Hkv = a.Hkv; p.R = a.Hq / a.Hkv; p.D = a.D;
  p.scale = a.scale;
  p.scale_log2 = a.scale * LOG2E;
  p.causal = a.causal ? 1 : 0;
  p.cu_q = a.cu_seqlens_q;
  p.cu_k = a.cu_seqlens_k ? a.cu_seqlens_k : a.cu_seqlens_q;
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

static int check_common(const AttnArgs& a) {
  if (a.Hkv <= 0 || a.Hq % a.Hkv) return -2;
  if (a.D < 8 || a.D > 128 || (a.D % 8)) return -2;
  if (a.cu_seqlens_q == nullptr && a.cu_seqlens_k != nullptr) return -2;
  return 0;
}

// every sequence may add one partial block
static int max_blocks(int T, int rows, const AttnArgs& a) {
  return (T + rows - 1) / rows + (a.cu_seqlens_q ? a.num_seqs : 0);
}

// Per-device, once: opt in to the large dynamic shared memory of the three kernels.
static int ensure_attrs() {
  constexpr int kMaxDev = 64;
  static bool done[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -4;
  if (done[dev]) return 0;
  if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem::BYTES) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BkvSmem::BYTES) !=
          cudaSuccess ||
      cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BqSmem::BYTES) !=
          cudaSuccess)
    return -4;
  done[dev] = true;
  return 0;
}

int attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.Tq == 0) return 0;
  int rc;
  if ((rc = check_common(a))) return rc;
  if ((a.o_ts % 8) || (a.o_hs % 8)) return -2;
  const int R = a.Hq / a.Hkv;
  CUtensorMap tq, tk, tv;
  if ((rc = make_map_q(&tq, a.q, a.Tq, a.D, a.Hkv, R, a.q_ts, a.q_gs, a.q_hs, 128))) return rc;
  if ((rc = make_map_kv(&tk, a.k, a.Tk, a.D, a.Hkv, a.k_ts, a.k_hs, 128))) return rc;
  if ((rc = make_map_kv(&tv, a.v, a.Tk, a.D, a.Hkv, a.v_ts, a.v_hs, 128))) return rc;
  if ((rc = ensure_attrs())) return rc;
  const AttnParams p = make_params(a);
  dim3 grid(max_blocks(a.Tq, 256, a), a.Hq);
  attn_fwd_kernel<<<grid, FWD_THREADS, FwdSmem::BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int attn_bwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.Tq == 0) return 0;
  int rc;
  if ((rc = check_common(a))) return rc;
  const int R = a.Hq / a.Hkv;
  if ((a.do_ts % 8) || (a.do_hs % 8) || (a.dq_ts % 8) || (a.dq_gs % 8) || (a.dq_hs % 8) || (a.dk_ts % 8) ||
      (a.dk_hs % 8) || (a.dv_ts % 8) || (a.dv_hs % 8))
    return -2;
  CUtensorMap tq, tk, tv, tdo, tq64, tdo64;
  if ((rc = make_map_q(&tq, a.q, a.Tq, a.D, a.Hkv, R, a.q_ts, a.q_gs, a.q_hs, 128))) return rc;
  if ((rc = make_map_q(&tq64, a.q, a.Tq, a.D, a.Hkv, R, a.q_ts, a.q_gs, a.q_hs, 64))) return rc;
  if ((rc = make_map_kv(&tk, a.k, a.Tk, a.D, a.Hkv, a.k_ts, a.k_hs, 128))) return rc;
  if ((rc = make_map_kv(&tv, a.v, a.Tk, a.D, a.Hkv, a.v_ts, a.v_hs, 128))) return rc;
  // dO is [Tq, Hq, D]: group stride R * head stride
  if ((rc = make_map_q(&tdo, a.dout, a.Tq, a.D, a.Hkv, R, a.do_ts, a.do_hs * R, a.do_hs, 128))) return rc;
  if ((rc = make_map_q(&tdo64, a.dout, a.Tq, a.D, a.Hkv, R, a.do_ts, a.do_hs * R, a.do_hs, 64))) return rc;
  if ((rc = ensure_attrs())) return rc;
  const AttnParams p = make_params(a);
  const long long warps = static_cast<long long>(a.Tq) * a.Hq;
  attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a.dout), static_cast<const __nv_bfloat16*>(a.o), a.delta, a.Tq, a.Hq, a.D,
      a.do_ts, a.do_hs, a.o_ts, a.o_hs);
  if (a.Tk > 0) {
    dim3 grid_kv(max_blocks(a.Tk, 128, a), a.Hkv);
    attn_bwd_dkdv_kernel<<<grid_kv, BWD_THREADS, BkvSmem::BYTES, stream>>>(tq64, tk, tv, tdo64, p);
  }
  dim3 grid_q(max_blocks(a.Tq, 128, a), a.Hq);
  attn_bwd_dq_kernel<<<grid_q, BWD_THREADS, BqSmem::BYTES, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
