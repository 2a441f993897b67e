// DeepSeek sparse attention (DSA) on the absorbed multi-latent form, forward, for sm_100a.
//
//   o[t, h, :512] = softmax_k( q[t, h, :576] . kv[idx[t, k], :576] * scale ) @ kv[idx[t, k], :512]
//
// q [m, H <= 128, 576] bf16 (latent 512 + rope 64), kv [n, 576] bf16 shared by all heads, idx [m, topk] int32 with -1
// for empty slots. For one query token the H heads share the same gathered rows, so the heads are the M = 128 rows of
// the tensor-core tile:
//   S[128 heads x 64 keys]  = Q_t K_blk^T        (36 k-steps over the 576 dims)
//   O[128 heads x 256]     += P K_blk[:, half]   (A = P packed bf16 in TMEM over the columns of S, B = the gathered
//                                                 block read MN-major)
// The fp32 accumulator of all 512 value dims would fill the 512 TMEM columns by itself, so one CTA owns ONE HALF of the
// value dims of one query token (grid = tokens x 2) and recomputes the scores.
//
// Where the operands live. Score MMAs narrower than 64 keys run far below the tensor core's rate (a cycle probe
// showed ~75 cycles for a 128 x 32 x 16 MMA against 64 for 128 x 128 x 16), so a block is 64 gathered keys, and
// shared memory goes to two 72 KB gather stages rather than to Q: the first 256 dims of the Q tile sit in TMEM (128
// columns, written once per CTA by the softmax warps from a TMA-staged copy) and feed the score product as a TMEM A
// operand; the other 320 dims stay in shared memory (80 KB). The stages are filled by 128 producer threads with
// 16-byte cp.async copies straight into the 128-byte-swizzled tile layout. TMEM: O 256 | S[2] 2 x 64 | Q 128 = 512
// columns. Issue order of the MMA thread per block: O += P[j] V[j], then S[j+1]: the gather of block j + 2 (into the
// stage that product has just released) then has a whole block of tensor work and softmax to land in. The softmax
// uses the lazily rescaled running maximum of the dense attention kernel; a per-block bit mask of live slots comes
// from the producers. Every wait is bounded.
//
// Replaces the TileLang kernel of the reference (ops/tilelang_ops/sparse_mla_fwd.py:11-181; oracle :218-265).
#include "sm100_ptx.cuh"
#include "dsa_sm100.h"

namespace lf {

static constexpr int SM_DK = 576, SM_NB = 64;                      // key dims, gathered rows per block
static constexpr int SM_QBOX = 128 * 64 * 2;                       // one [128 heads x 64 dims] box of Q: 16 KB
static constexpr int SM_QT_BOXES = 4;                              // Q boxes that move to TMEM (256 dims = 128 columns)
static constexpr int SM_QS_BYTES = 5 * SM_QBOX;                    // Q boxes that stay in shared memory: 80 KB
static constexpr int SM_KBOX = SM_NB * 64 * 2;                     // one [64 rows x 64 dims] box: 8 KB
static constexpr int SM_KV_BYTES = 9 * SM_KBOX;                    // 72 KB per stage
static constexpr int SM_STAGES = 2;
static constexpr int SM_KV0 = SM_QS_BYTES;                         // gather stages (first used to stage Q for TMEM)
static constexpr int SM_CTL = SM_KV0 + SM_STAGES * SM_KV_BYTES;
static constexpr int SM_SMEM = SM_CTL + 1280 + 1024;  // control block (barriers, masks, head-sum scratch) + alignment slack
static constexpr int SM_THREADS = 288;  // 4 gather warps, 1 MMA warp, 4 softmax warps
static constexpr float SM_LOG2E = 1.4426950408889634f;
static constexpr int BOXK = 128 * 64 * 2;  // one [128 rows x 64 dims] box of the indexer's key tile

struct SmlaParams {
  const __nv_bfloat16* kv;
  long long kv_ts;
  const int* idx;
  int topk, m, H, n_kv;
  float scale_log2;
  __nv_bfloat16* o;
  long long o_ts, o_hs;
  float* lse;  // [m, H]
  float* pmean;  // PROBS pass: [m, topk] head-mean attention probabilities (lse is an input there)
  int* status;
};

enum { S_Q = 0, S_QT = 1, S_KV_FULL = 2, S_KV_EMPTY = 4, S_S_FULL = 6, S_P_FULL = 8, S_O_DONE = 10, S_PART_FULL = 11,
       S_PART_EMPTY = 12 };

struct SmlaCtl {
  uint64_t bars[16];
  uint32_t tmem_slot;
  int abort_flag;
  uint32_t live[4][2];  // [block & 3]: bit i of word w: slot 32 w + i of the block holds a key (four entries: a stage is
                        // refilled before the softmax warps are done with the mask of its previous block)
  float part[4][SM_NB];         // PROBS pass: per-warp head sums of one block
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// PROBS = false: the attention forward above. PROBS = true: a second pass that, given the forward's log-sum-exp, writes
// the head-averaged attention probability of every selected slot, pmean[m, s] = (1 / H) sum_h exp(scale s_h - lse_h)
// (the target distribution of the indexer loss, reference dsa_fused_kernels.py:1844-1955). Same gather, same score
// MMAs, no value product: one CTA per token; the softmax warps turn scores into probabilities, sum over their 32
// heads with a transposing butterfly of warp shuffles (62 shuffles for 64 columns) and over the four warps through
// shared memory in a fixed order.
template <bool PROBS>
__global__ void __launch_bounds__(SM_THREADS, 1)
sparse_mla_fwd_kernel(const __grid_constant__ CUtensorMap tq, const SmlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmlaCtl* ctl = reinterpret_cast<SmlaCtl*>(smem + SM_CTL);
  uint64_t* bars = ctl->bars;
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = PROBS ? blockIdx.x : (blockIdx.x >> 1), half = PROBS ? 0 : (blockIdx.x & 1);
  const int nb = (p.topk + SM_NB - 1) / SM_NB;
  const int* my_idx = p.idx + static_cast<long long>(tok) * p.topk;

  if (threadIdx.x == 0) {
    mbar_init(&bars[S_Q], 1);
    mbar_init(&bars[S_QT], 4);
    for (int s = 0; s < SM_STAGES; ++s) {
      mbar_init(&bars[S_KV_FULL + s], 128);
      mbar_init(&bars[S_KV_EMPTY + s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars[S_S_FULL + b], 1);
      mbar_init(&bars[S_P_FULL + b], 4);
    }
    mbar_init(&bars[S_O_DONE], 1);
    mbar_init(&bars[S_PART_FULL], 4);
    mbar_init(&bars[S_PART_EMPTY], 4);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t t_o = tmem, t_s = tmem + 256, t_q = tmem + 384;  // O 256 | S[2] 2 x 64 | Q 128

  if (warp < 4) {
    // ------------------------------------------------------------ gather producers
    if (threadIdx.x == 0) {
      // Q: boxes 0..3 are staged in the (still unused) gather area for the copy into TMEM, boxes 4..8 stay resident
      mbar_arrive_expect_tx(&bars[S_Q], 9 * SM_QBOX);
      for (int b = 0; b < SM_QT_BOXES; ++b) tma_load_3d(smem + SM_KV0 + b * SM_QBOX, &tq, &bars[S_Q], b * 64, 0, tok);
      for (int b = SM_QT_BOXES; b < 9; ++b)
        tma_load_3d(smem + (b - SM_QT_BOXES) * SM_QBOX, &tq, &bars[S_Q], b * 64, 0, tok);
    }
    // Thread t copies row t / 2 of every block: the 16-byte chunks 2 i + (t % 2), so two neighbouring lanes read 32
    // contiguous bytes. Only one stage is ever free at a time (the other holds the block whose scores are running),
    // so a producer issues a block, waits for it to land, publishes it (after a proxy fence) and then waits for the
    // next stage to be released.
    const int row = threadIdx.x >> 1, hd = threadIdx.x & 1;
    // the gather area is free once the softmax warps have moved the staged part of Q into TMEM
    bool ok = mbar_wait(&bars[S_QT], 0, abort_flag);
    for (int j = 0; j < nb && ok; ++j) {
      const int s = j % SM_STAGES;
      ok = mbar_wait(&bars[S_KV_EMPTY + s], ((j / SM_STAGES) & 1) ^ 1, abort_flag);
      if (!ok) break;
      uint8_t* stage = smem + SM_KV0 + s * SM_KV_BYTES;
      if (warp < 2) {  // warp w publishes the live bits of slots 32 w .. 32 w + 31
        const int sl = j * SM_NB + warp * 32 + lane;
        const int idl = sl < p.topk ? my_idx[sl] : -1;
        const unsigned m = __ballot_sync(0xffffffffu, idl >= 0 && idl < p.n_kv);
        if (lane == 0) ctl->live[j & 3][warp] = m;
      }
      const int slot = j * SM_NB + row;
      const int id = slot < p.topk ? my_idx[slot] : -1;
      uint8_t* drow = stage + (row >> 3) * 1024 + (row & 7) * 128;
      if (id >= 0 && id < p.n_kv) {
        const __nv_bfloat16* src = p.kv + static_cast<long long>(id) * p.kv_ts;
#pragma unroll
        for (int i = 0; i < 36; ++i) {
          const int col16 = i * 2 + hd;
          cp_async16(smem_u32(drow + (col16 >> 3) * SM_KBOX + (((col16 & 7) ^ (row & 7)) << 4)), src + col16 * 8);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 36; ++i) {
          const int col16 = i * 2 + hd;
          *reinterpret_cast<uint4*>(drow + (col16 >> 3) * SM_KBOX + (((col16 & 7) ^ (row & 7)) << 4)) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        if (id >= p.n_kv) atomicCAS(p.status, 0, LF_ERR_BAD_INDEX);
      }
      cp_async_wait_all();
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
      mbar_arrive(&bars[S_KV_FULL + s]);
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
  } else if (warp == 4) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t sq = smem_u32(smem), skv = smem_u32(smem + SM_KV0);
      constexpr uint32_t idesc_s = make_idesc(1, 1, false, false, 128, SM_NB);
      constexpr uint32_t idesc_o = make_idesc(1, 1, false, true, 128, 256);
      auto issue_s = [&](int j) {
        const int s = j % SM_STAGES, b = j & 1;
        const uint32_t kb = skv + s * SM_KV_BYTES;
        // dims 0..255: Q from TMEM (8 columns per k-step); dims 256..575: Q from shared memory
#pragma unroll 4
        for (int kk = 0; kk < 4 * SM_QT_BOXES; ++kk) {
          const uint64_t db = make_smem_desc_sw128(kb + (kk >> 2) * SM_KBOX + (kk & 3) * 32, 16, 1024);
          tc_mma_f16_ts(t_s + b * SM_NB, t_q + kk * 8, db, idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll 4
        for (int kk = 4 * SM_QT_BOXES; kk < 36; ++kk) {
          const uint64_t da = make_smem_desc_sw128(sq + ((kk >> 2) - SM_QT_BOXES) * SM_QBOX + (kk & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(kb + (kk >> 2) * SM_KBOX + (kk & 3) * 32, 16, 1024);
          tc_mma_f16_ss(t_s + b * SM_NB, da, db, idesc_s, 1u);
        }
        tc_commit(&bars[S_S_FULL + b]);
      };
      bool ok = mbar_wait(&bars[S_Q], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars[S_QT], 0, abort_flag);
      if constexpr (PROBS) {
        for (int j = 0; j < nb && ok; ++j) {
          const int s = j % SM_STAGES, b = j & 1;
          ok = mbar_wait(&bars[S_KV_FULL + s], (j / SM_STAGES) & 1, abort_flag);
          // the softmax warps have read the scores of block j - 2 out of this buffer
          if (ok && j >= 2) ok = mbar_wait(&bars[S_P_FULL + b], ((j - 2) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(j);
          tc_commit(&bars[S_KV_EMPTY + s]);
        }
        if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
        ok = false;  // nothing of the forward's loop below runs
      }
      if (ok && nb > 0) {
        ok = mbar_wait(&bars[S_KV_FULL + 0], 0, abort_flag);
        if (ok) {
          tc_fence_after_sync();
          issue_s(0);
        }
      }
      for (int j = 0; j < nb && ok; ++j) {
        const int s = j % SM_STAGES, b = j & 1;
        ok = mbar_wait(&bars[S_P_FULL + b], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        // O += P[j] V[j]: 64 gathered rows = 4 k-steps; B = this half's four 64-dim boxes read MN-major
        const uint32_t vb = skv + s * SM_KV_BYTES + half * 4 * SM_KBOX;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t db = make_smem_desc_sw128(vb + kk * 2048, SM_KBOX, 1024);
          tc_mma_f16_ts(t_o, t_s + b * SM_NB + kk * 8, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&bars[S_KV_EMPTY + s]);  // the producers refill this stage with block j + 2 ...
        tc_commit(&bars[S_O_DONE]);
        if (j + 1 < nb) {  // ... while the scores of block j + 1 (other stage, other S buffer) run
          ok = mbar_wait(&bars[S_KV_FULL + ((j + 1) % SM_STAGES)], ((j + 1) / SM_STAGES) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(j + 1);
        }
      }
      if (!PROBS && !ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    // ------------------------------------------------------------ softmax warps: one thread per head
    const int quarter = warp & 3;
    const int h = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = mbar_wait(&bars[S_Q], 0, abort_flag);
    if (ok) {
      // move dims 0..255 of this head's Q row from the staged (swizzled) boxes into TMEM: two bf16 per column
      const uint8_t* qst = smem + SM_KV0;
#pragma unroll 1
      for (int b = 0; b < SM_QT_BOXES; ++b) {
        const uint8_t* rowp = qst + b * SM_QBOX + (h >> 3) * 1024 + (h & 7) * 128;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {  // 16 columns = 32 dims = four 16-byte chunks
          uint32_t r[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + (((hh * 4 + c) ^ (h & 7)) << 4));
            r[c * 4] = v.x; r[c * 4 + 1] = v.y; r[c * 4 + 2] = v.z; r[c * 4 + 3] = v.w;
          }
          tmem_st_32x32b_x16(t_q + lane_off + b * 32 + hh * 16, r);
        }
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[S_QT]);
    }
    if constexpr (PROBS) {
      const float lse_n = h < p.H ? p.lse[static_cast<long long>(tok) * p.H + h] : -INFINITY;
      const float neg_lse2 = lse_n == -INFINITY ? -INFINITY : -lse_n * SM_LOG2E;
      const float inv_h = 1.f / static_cast<float>(p.H);
      const int st_tid = threadIdx.x - 5 * 32;  // 0..127 over the softmax warps
      for (int j = 0; j < nb && ok; ++j) {
        const int b = j & 1;
        // No wait on the stage's "full" barrier here: in this pass a stage is released as soon as its scores are
        // done, so that barrier can complete the phase of block j + 2 before these warps have looked at it for block
        // j, and a parity wait two phases late would never return. The scores' barrier orders the mask as well: the
        // MMA thread saw the stage full before it issued the scores.
        ok = mbar_wait(&bars[S_S_FULL + b], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t live0 = *reinterpret_cast<volatile uint32_t*>(&ctl->live[j & 3][0]);
        const uint32_t live1 = *reinterpret_cast<volatile uint32_t*>(&ctl->live[j & 3][1]);
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(t_s + b * SM_NB + lane_off, r0);
        tmem_ld_32x32b_x32(t_s + b * SM_NB + lane_off + 32, r1);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[S_P_FULL + b]);  // the score buffer may be overwritten
        float v[64];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          v[i] = ((live0 >> i) & 1u) && neg_lse2 != -INFINITY
                     ? exp2f(fmaf(__uint_as_float(r0[i]), p.scale_log2, neg_lse2)) : 0.f;
          v[32 + i] = ((live1 >> i) & 1u) && neg_lse2 != -INFINITY
                          ? exp2f(fmaf(__uint_as_float(r1[i]), p.scale_log2, neg_lse2)) : 0.f;
        }
        // transposing butterfly: after the step with distance d a lane keeps the half of its columns that its bit d
        // selects, summed with the partner's; at the end lane L holds the 32-head sums of columns 2 L and 2 L + 1
#pragma unroll
        for (int d = 16, n = 32; d >= 1; d >>= 1, n >>= 1) {
          const bool up = (lane & d) != 0;
#pragma unroll
          for (int i = 0; i < n; ++i) {
            const float send = up ? v[i] : v[i + n];
            const float recv = __shfl_xor_sync(0xffffffffu, send, d);
            v[i] = (up ? v[i + n] : v[i]) + recv;
          }
        }
        // the four warps meet through two mbarriers (bounded waits, like every other wait of this kernel)
        if (j >= 1) ok = mbar_wait(&bars[S_PART_EMPTY], (j - 1) & 1, abort_flag);  // previous block's sums were read
        if (!ok) break;
        ctl->part[quarter][2 * lane] = v[0];
        ctl->part[quarter][2 * lane + 1] = v[1];
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[S_PART_FULL]);
        ok = mbar_wait(&bars[S_PART_FULL], j & 1, abort_flag);
        if (!ok) break;
        if (st_tid < SM_NB) {
          const int slot = j * SM_NB + st_tid;
          if (slot < p.topk)
            p.pmean[static_cast<long long>(tok) * p.topk + slot] =
                (ctl->part[0][st_tid] + ctl->part[1][st_tid] + ctl->part[2][st_tid] + ctl->part[3][st_tid]) * inv_h;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[S_PART_EMPTY]);
      }
      if (!ok && lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
      ok = false;  // skip the forward's loop and epilogue below
    }
    for (int j = 0; j < nb && ok; ++j) {
      const int s = j % SM_STAGES, b = j & 1;
      ok = mbar_wait(&bars[S_KV_FULL + s], (j / SM_STAGES) & 1, abort_flag);  // the producers' mask is visible
      if (ok) ok = mbar_wait(&bars[S_S_FULL + b], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t live0 = ctl->live[j & 3][0], live1 = ctl->live[j & 3][1];
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(t_s + b * SM_NB + lane_off, r0);
      tmem_ld_32x32b_x32(t_s + b * SM_NB + lane_off + 32, r1);
      tmem_ld_wait();
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (!((live0 >> i) & 1u)) r0[i] = 0xff800000u;  // empty slots (-1) are masked
        if (!((live1 >> i) & 1u)) r1[i] = 0xff800000u;
        mx0 = fmaxf(mx0, __uint_as_float(r0[i]));
        mx1 = fmaxf(mx1, __uint_as_float(r1[i]));
      }
      const float mx = fmaxf(mx0, mx1) * p.scale_log2;
      float m_new = m_ref;
      if (mx > m_ref + 8.f || m_ref == -INFINITY) m_new = fmaxf(mx, m_ref);
      const bool rescale = (m_new != m_ref) && (j > 0);
      const unsigned any = __ballot_sync(0xffffffffu, rescale);
      const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
      if (any) {
        ok = mbar_wait(&bars[S_O_DONE], (j - 1) & 1, abort_flag);  // O += P[j-1] V[j-1] retired
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 16) {
          uint32_t q[16];
          tmem_ld_32x32b_x16(t_o + lane_off + c0, q);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) q[i] = __float_as_uint(__uint_as_float(q[i]) * alpha);
          tmem_st_32x32b_x16(t_o + lane_off + c0, q);
        }
      }
      l_sum *= alpha;
      m_ref = m_new;
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      float la = 0.f, lb = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float a = exp2f(fmaf(__uint_as_float(r0[2 * i]), p.scale_log2, neg_m));
        const float b2 = exp2f(fmaf(__uint_as_float(r0[2 * i + 1]), p.scale_log2, neg_m));
        la += a; lb += b2;
        pk[i] = pack_bf16x2(a, b2);
      }
      tmem_st_32x32b_x16(t_s + b * SM_NB + lane_off, pk);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float a = exp2f(fmaf(__uint_as_float(r1[2 * i]), p.scale_log2, neg_m));
        const float b2 = exp2f(fmaf(__uint_as_float(r1[2 * i + 1]), p.scale_log2, neg_m));
        la += a; lb += b2;
        pk[i] = pack_bf16x2(a, b2);
      }
      tmem_st_32x32b_x16(t_s + b * SM_NB + lane_off + 16, pk);
      l_sum += la + lb;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[S_P_FULL + b]);
    }
    if (ok && nb > 0) ok = mbar_wait(&bars[S_O_DONE], (nb - 1) & 1, abort_flag);
    if (PROBS) {
      // nothing more to do in the probabilities pass
    } else if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
    } else {
      tc_fence_after_sync();
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      // every lane takes part in the warp-collective TMEM loads; only lanes that map to a head store
      const bool live = h < p.H;
      __nv_bfloat16* orow = p.o + static_cast<long long>(tok) * p.o_ts + static_cast<long long>(live ? h : 0) * p.o_hs +
                            half * 256;
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 32) {
        uint32_t q[32];
        if (nb > 0) {
          tmem_ld_32x32b_x32(t_o + lane_off + c0, q);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) q[i] = 0u;
        }
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(q[i]) * inv, __uint_as_float(q[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(q[i + 2]) * inv, __uint_as_float(q[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(q[i + 4]) * inv, __uint_as_float(q[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(q[i + 6]) * inv, __uint_as_float(q[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + i) = w;
          }
        }
      }
      if (live && half == 0)
        p.lse[static_cast<long long>(tok) * p.H + h] = l_sum > 0.f ? (m_ref + log2f(l_sum)) * (1.f / SM_LOG2E) : -INFINITY;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn dsa_encode_fn() {
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

static int sparse_mla_launch(const SparseMlaArgs& a, bool probs, cudaStream_t stream);
int sparse_mla_fwd(const SparseMlaArgs& a, cudaStream_t stream) { return sparse_mla_launch(a, false, stream); }
int sparse_mla_probs(const SparseMlaArgs& a, cudaStream_t stream) { return sparse_mla_launch(a, true, stream); }

static int sparse_mla_launch(const SparseMlaArgs& a, bool probs, cudaStream_t stream) {
  if (a.m <= 0) return 0;
  if (probs && (a.pmean == nullptr || a.lse == nullptr)) return -2;
  if (a.H < 1 || a.H > 128 || a.topk < 1) return -2;
  if ((a.q_ts % 8) || (a.q_hs % 8) || (a.kv_ts % 8) || (!probs && ((a.o_ts % 8) || (a.o_hs % 8)))) return -2;
  if ((reinterpret_cast<uintptr_t>(a.q) & 15) || (reinterpret_cast<uintptr_t>(a.kv) & 15) ||
      (!probs && (reinterpret_cast<uintptr_t>(a.o) & 15)))
    return -2;
  EncodeTiledFn fn = dsa_encode_fn();
  if (!fn) return -1;
  // (dim, head, token) map of q with box (64, 128, 1); heads past H are zero-filled
  CUtensorMap tq;
  cuuint64_t dims[3] = {SM_DK, static_cast<cuuint64_t>(a.H), static_cast<cuuint64_t>(a.m)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(a.q_hs) * 2, static_cast<cuuint64_t>(a.q_ts) * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t es[3] = {1, 1, 1};
  if (fn(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(a.q), dims, strides, box, es,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -3;
  constexpr int kMaxDev = 64;
  static bool attr[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -4;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(sparse_mla_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_SMEM) !=
            cudaSuccess ||
        cudaFuncSetAttribute(sparse_mla_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_SMEM) !=
            cudaSuccess)
      return -4;
    attr[dev] = true;
  }
  SmlaParams p;
  p.kv = static_cast<const __nv_bfloat16*>(a.kv);
  p.kv_ts = a.kv_ts;
  p.idx = a.idx;
  p.topk = a.topk; p.m = a.m; p.H = a.H; p.n_kv = a.n_kv;
  p.scale_log2 = a.scale * SM_LOG2E;
  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.o_ts = a.o_ts; p.o_hs = a.o_hs;
  p.lse = a.lse;
  p.pmean = a.pmean;
  p.status = a.status;
  if (probs)
    sparse_mla_fwd_kernel<true><<<a.m, SM_THREADS, SM_SMEM, stream>>>(tq, p);
  else
    sparse_mla_fwd_kernel<false><<<2 * a.m, SM_THREADS, SM_SMEM, stream>>>(tq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}


// =========================================================================== lightning indexer: logits
//   logits[m, n] = sum_h w[m, h] * relu(q[m, h, :] . k[n, :])        (Hi index heads of 128 dims, k shared by the heads)
// computed TRANSPOSED so that the key row is the TMEM lane and the head sum stays inside one thread:
//   S^T[128 keys x 256] = K_blk (A, shared memory) x Q_grp^T (B: the 256 / Hi query tokens of this CTA, all heads)
// One CTA owns a group of 256 / Hi consecutive query tokens, keeps their Q tile resident and streams the key blocks
// its tokens may see (a contiguous range per token, [k_start, k_end)); the epilogue warps apply relu and the per-head
// weights from shared memory and write one fp32 logit per (token, key). Entries outside a token's range are left
// unwritten: the selection kernel below reads ranges only. Two S^T accumulators (2 x 256 TMEM columns) let the
// tensor core run one key block ahead of the epilogue.
// Replaces the TileLang indexer kernel of the reference (ops/tilelang_ops/lightning_indexer.py:82-139; oracle :12-32).
static constexpr int IX_KSTAGES = 4;
static constexpr int IX_Q_BYTES = 256 * 128 * 2;  // 64 KB: two [256 x 64] boxes
static constexpr int IX_K_BYTES = 128 * 128 * 2;  // 32 KB: two [128 x 64] boxes
static constexpr int IX_W = IX_Q_BYTES + IX_KSTAGES * IX_K_BYTES;  // 256 fp32 head weights
static constexpr int IX_CTL = IX_W + 1024;
static constexpr int IX_SMEM = IX_CTL + 256 + 1024;
static constexpr int IX_THREADS = 192;
enum { I_Q = 0, I_K_FULL = 1, I_K_EMPTY = 5, I_S_FULL = 9, I_S_EMPTY = 11 };

struct IndexerParams {
  const float* w;       // [m, Hi]
  const int* k_start;   // [m]
  const int* k_end;     // [m] exclusive
  float* logits;        // [m, ld]
  long long ld;
  int m, n, Hi;
  int* status;
};

struct IxCtl {
  uint64_t bars[16];
  uint32_t tmem_slot;
  int abort_flag;
  int blk_lo, blk_hi;
};

__global__ void __launch_bounds__(IX_THREADS, 1)
indexer_logits_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                      const IndexerParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  IxCtl* ctl = reinterpret_cast<IxCtl*>(smem + IX_CTL);
  uint64_t* bars = ctl->bars;
  volatile int* abort_flag = &ctl->abort_flag;
  float* ws = reinterpret_cast<float*>(smem + IX_W);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tpc = 256 / p.Hi;               // query tokens per CTA
  const int t0 = blockIdx.x * tpc;          // first token of the group
  // head weights of the group (zero for tokens past the end) and the union of the tokens' key ranges
  for (int i = threadIdx.x; i < 256; i += IX_THREADS) {
    const int t = t0 + i / p.Hi;
    ws[i] = t < p.m ? p.w[static_cast<long long>(t) * p.Hi + (i % p.Hi)] : 0.f;
  }
  if (threadIdx.x == 0) {
    int lo = 0x7fffffff, hi = 0;
    for (int t = t0; t < min(t0 + tpc, p.m); ++t) {
      if (p.k_end[t] > p.k_start[t]) {
        lo = min(lo, p.k_start[t]);
        hi = max(hi, p.k_end[t]);
      }
    }
    ctl->blk_lo = hi > 0 ? lo / 128 : 0;
    ctl->blk_hi = hi > 0 ? (min(hi, p.n) + 127) / 128 : 0;
    mbar_init(&bars[I_Q], 1);
    for (int s = 0; s < IX_KSTAGES; ++s) {
      mbar_init(&bars[I_K_FULL + s], 1);
      mbar_init(&bars[I_K_EMPTY + s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars[I_S_FULL + b], 1);
      mbar_init(&bars[I_S_EMPTY + b], 4);
    }
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&ctl->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const int blk_lo = ctl->blk_lo, nblk = ctl->blk_hi - ctl->blk_lo;

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      mbar_arrive_expect_tx(&bars[I_Q], IX_Q_BYTES);
      for (int b = 0; b < 2; ++b) tma_load_2d(smem + b * (256 * 128), &tq, &bars[I_Q], b * 64, t0 * p.Hi);
      for (int j = 0; j < nblk; ++j) {
        const int s = j % IX_KSTAGES;
        if (!mbar_wait(&bars[I_K_EMPTY + s], ((j / IX_KSTAGES) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
          break;
        }
        uint8_t* dst = smem + IX_Q_BYTES + s * IX_K_BYTES;
        mbar_arrive_expect_tx(&bars[I_K_FULL + s], IX_K_BYTES);
        for (int b = 0; b < 2; ++b) tma_load_2d(dst + b * BOXK, &tk, &bars[I_K_FULL + s], b * 64, (blk_lo + j) * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, false, false, 128, 256);
      const uint32_t sq = smem_u32(smem), sk = smem_u32(smem + IX_Q_BYTES);
      bool ok = mbar_wait(&bars[I_Q], 0, abort_flag);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j % IX_KSTAGES, b = j & 1;
        ok = mbar_wait(&bars[I_K_FULL + s], (j / IX_KSTAGES) & 1, abort_flag);
        if (ok) ok = mbar_wait(&bars[I_S_EMPTY + b], ((j >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t ka = sk + s * IX_K_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t da = make_smem_desc_sw128(ka + (kk >> 2) * BOXK + (kk & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sq + (kk >> 2) * (256 * 128) + (kk & 3) * 32, 16, 1024);
          tc_mma_f16_ss(tmem + b * 256, da, db, idesc, kk > 0 ? 1u : 0u);
        }
        tc_commit(&bars[I_K_EMPTY + s]);
        tc_commit(&bars[I_S_FULL + b]);
      }
      if (!ok) atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // key row inside the block
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float4* w4 = reinterpret_cast<const float4*>(ws);
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int b = j & 1;
      ok = mbar_wait(&bars[I_S_FULL + b], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const int key = (blk_lo + j) * 128 + row;
      float acc = 0.f;
      int col = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + b * 256 + lane_off + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 w = w4[(c0 + i) >> 2];
          acc = fmaf(fmaxf(__uint_as_float(r[i]), 0.f), w.x, acc);
          acc = fmaf(fmaxf(__uint_as_float(r[i + 1]), 0.f), w.y, acc);
          acc = fmaf(fmaxf(__uint_as_float(r[i + 2]), 0.f), w.z, acc);
          acc = fmaf(fmaxf(__uint_as_float(r[i + 3]), 0.f), w.w, acc);
        }
        col += 32;
        if (col % p.Hi == 0) {  // a token's heads are complete (Hi is 32, 64, 128 or 256)
          const int t = t0 + (c0 + 32) / p.Hi - 1;
          if (t < p.m && key < p.n) p.logits[static_cast<long long>(t) * p.ld + key] = acc;
          acc = 0.f;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[I_S_EMPTY + b]);
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// =========================================================================== top-k selection over a range of a row
// One CTA per query row: the fp32 logits of the row's key range are loaded into shared memory once as order-preserving
// unsigned keys, an MSB-first radix select (four 8-bit passes over shared memory) finds the k-th largest key exactly,
// and a last pass writes the indices above it plus as many ties as are needed. The output order is unspecified
// (a set), -1 pads rows with fewer than k candidates. Rows longer than TK_MAX_ROW are refused on the host.
static constexpr int TK_THREADS = 512;
static constexpr int TK_MAX_ROW = 49152;  // 192 KB of keys

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(TK_THREADS) topk_range_kernel(const float* __restrict__ logits, long long ld,
                                                                const int* __restrict__ k_start,
                                                                const int* __restrict__ k_end, int* __restrict__ out,
                                                                int topk) {
  extern __shared__ uint32_t keys[];
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_need, s_above, s_ties;
  const int rowi = blockIdx.x;
  const int ks = k_start[rowi];
  const int len = max(k_end[rowi] - ks, 0);
  int* o = out + static_cast<long long>(rowi) * topk;
  if (len <= topk) {  // everything is selected
    for (int i = threadIdx.x; i < topk; i += TK_THREADS) o[i] = i < len ? ks + i : -1;
    return;
  }
  const float* src = logits + static_cast<long long>(rowi) * ld + ks;
  for (int i = threadIdx.x; i < len; i += TK_THREADS) keys[i] = order_key(src[i]);
  if (threadIdx.x == 0) {
    s_prefix = 0u;
    s_mask = 0u;
    s_need = topk;
  }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += TK_THREADS) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = threadIdx.x; i < len; i += TK_THREADS) {
      const uint32_t kx = keys[i];
      if ((kx & mask) == prefix) atomicAdd(&hist[(kx >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {  // walk down from the largest digit
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_need = need;  // how many of the chosen digit's keys are still wanted
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_mask = mask | (255u << shift);
    }
    __syncthreads();
  }
  // s_prefix is now the exact k-th largest key; s_need of the keys equal to it are taken
  if (threadIdx.x == 0) {
    s_above = 0;
    s_ties = 0;
  }
  __syncthreads();
  const uint32_t thr = s_prefix;
  const int need = s_need, n_above = topk - need;
  for (int i = threadIdx.x; i < len; i += TK_THREADS) {
    const uint32_t kx = keys[i];
    if (kx > thr) {
      const int pos = atomicAdd(&s_above, 1);
      if (pos < n_above) o[pos] = ks + i;
    } else if (kx == thr) {
      const int pos = atomicAdd(&s_ties, 1);
      if (pos < need) o[n_above + pos] = ks + i;
    }
  }
}

static int make_map_2d(CUtensorMap* m, const void* ptr, long long rows, long long ld, int box_rows) {
  EncodeTiledFn fn = dsa_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld % 8)) return -2;
  cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t es[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}

int indexer_logits(const IndexerArgs& a, cudaStream_t stream) {
  if (a.m <= 0 || a.n <= 0) return 0;
  if (!(a.Hi == 32 || a.Hi == 64 || a.Hi == 128 || a.Hi == 256) || (a.ld % 4)) return -2;
  CUtensorMap tq, tk;
  int rc;
  // q viewed as [m * Hi, 128] rows; rows past the end are zero-filled by TMA
  if ((rc = make_map_2d(&tq, a.q, static_cast<long long>(a.m) * a.Hi, 128, 256))) return rc;
  if ((rc = make_map_2d(&tk, a.k, a.n, a.k_ld, 128))) return rc;
  constexpr int kMaxDev = 64;
  static bool attr[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -4;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(indexer_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IX_SMEM) !=
            cudaSuccess ||
        cudaFuncSetAttribute(topk_range_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_MAX_ROW * 4) !=
            cudaSuccess)
      return -4;
    attr[dev] = true;
  }
  IndexerParams p;
  p.w = a.w; p.k_start = a.k_start; p.k_end = a.k_end;
  p.logits = a.logits; p.ld = a.ld;
  p.m = a.m; p.n = a.n; p.Hi = a.Hi;
  p.status = a.status;
  const int tpc = 256 / a.Hi;
  indexer_logits_kernel<<<(a.m + tpc - 1) / tpc, IX_THREADS, IX_SMEM, stream>>>(tq, tk, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int topk_range(const float* logits, long long ld, const int* k_start, const int* k_end, int* out, int m, int topk,
               int max_len, cudaStream_t stream) {
  if (m <= 0) return 0;
  if (max_len > TK_MAX_ROW || topk < 1) return -2;
  constexpr int kMaxDev = 64;
  static bool attr[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -4;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(topk_range_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_MAX_ROW * 4) !=
        cudaSuccess)
      return -4;
    attr[dev] = true;
  }
  const size_t smem = static_cast<size_t>(max_len > 0 ? max_len : 1) * 4;
  topk_range_kernel<<<m, TK_THREADS, smem, stream>>>(logits, ld, k_start, k_end, out, topk);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace lf
