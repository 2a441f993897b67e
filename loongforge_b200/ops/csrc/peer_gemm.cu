// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
// ag_gemm  (sequence-parallel all-gather -> GEMM; replaces all_gather + TE LayerNormColumnParallelLinear
//           GEMM, and the reference's closest analogue, TE userbuffers overlap,
//           loongforge/train/initialize.py:349-351):
//   One launch = a few COPY CTAs + the persistent tcgen05 GEMM CTAs.
//   Every rank keeps a symmetric [T, K] gather buffer and has written its OWN rows into it before the
//   launch. Copy CTAs pull the peers' rows through NVLink with SM-issued bulk copies (peer global ->
//   shared -> local global, several 32 KB copies in flight per CTA) into the same rows of the local
//   buffer, one 128-row block at a time, and publish `chunk_flags[block] = epoch`. The GEMM CTAs start
//   on their own rows at once (nothing to wait for) and their TMA producer waits (bounded) on the flag
//   of a remote block only when it reaches it, so the transfer overlaps the math of the own rows. Every
//   remote byte crosses NVLink exactly once and is then re-read by the N/256 column tiles from local
//   memory / L2.
//
// gemm_rs  (GEMM -> reduce-scatter (+ residual); replaces TE RowParallelLinear + reduce_scatter):
//   Tiles whose rows belong to a peer are computed FIRST and their bf16 partial sums are stored
//   straight from the TMEM epilogue into the peer's receive buffer (posted NVLink writes), followed
//   by a release-increment of that tile's counter on the peer. Tiles whose rows this rank owns are
//   computed last; their epilogue waits (bounded) for the peers' counters, adds the received
//   partials (fixed order: deterministic) and the residual, and writes the final output once.
//   Receive buffers are double buffered by call parity, which makes a cross-rank barrier unnecessary.
//
// Peers are only touched with plain (single-destination) bulk copies,
// vector stores and scalar flag operations.
#include "sm100_ptx.cuh"
#include "gemm_sm100.h"
#include "peer_gemm.h"
#include "wait_budget.h"

namespace lf {

static constexpr int PG_BM = 128, PG_BN = 256, PG_BK = 64, PG_UMMA_K = 16, PG_STAGES = 4;
static constexpr int PG_THREADS = 192;
static constexpr int PG_A_BYTES = PG_BM * PG_BK * 2, PG_B_BYTES = PG_BN * PG_BK * 2;
static constexpr int PG_STAGE_BYTES = PG_A_BYTES + PG_B_BYTES;
static constexpr int PG_STG_ROW = 144;  // bytes per staged row: 64 bf16 + 16 bytes of padding (conflict-free 16-byte stores)
static constexpr int PG_STG_BYTES = 4 * 32 * PG_STG_ROW;  // one [32 rows x 64 columns] patch per epilogue warp
static constexpr int PG_SMEM_BYTES = PG_STAGES * PG_STAGE_BYTES + PG_STG_BYTES + 1024 + 256;
static constexpr int CP_PIECE = 32 * 1024;  // bytes per bulk copy
static constexpr int CP_STAGES = 5;         // 160 KB of the same dynamic shared memory

struct PeerParams {
  int M, N, K, tiles_m, tiles_n, tiles_per_rank_m;
  int rank, world, rows_per_rank;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  int* status;
  // ag
  const uint8_t* peer_x[kMaxPeers];
  int* peer_sync[kMaxPeers];
  uint8_t* x_full;
  int* chunk_flags;
  int epoch;
  int copy_ctas;
  // rs
  __nv_bfloat16* peer_recv[kMaxPeers];
  int* peer_tile_flags[kMaxPeers];
  int parity;
  int expect;
  long long wait_cycles;  // budget of every wait that depends on a peer GPU (wait_budget.h)
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded spin on a global flag until it reaches `target`. Returns false on timeout.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const int* p, int target, long long budget) {
  if ((SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p)) >= target) return true;
  const long long t0 = clock64();
  while (true) {
    if ((SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p)) >= target) return true;
    __nanosleep(40);
    if (clock64() - t0 > budget) return false;
  }
}

__device__ __forceinline__ void pg_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % rows);
  tn = r / rows;
}

// ------------------------------------------------------------------ copy CTA (ag mode)
__device__ void ag_copy_cta(const PeerParams& p, uint8_t* smem, uint64_t* bars) {
  // one thread drives everything; bars[0..CP_STAGES) = load-complete barriers
  if (threadIdx.x != 0) return;
  const int c = blockIdx.x;
  for (int s = 0; s < CP_STAGES; ++s) mbar_init(&bars[s], 1);
  fence_mbar_init();
  // cross-rank arrival: every rank's X shard is final once that rank has reached this kernel
  if (c == 0) {
    for (int r = 0; r < p.world; ++r)
      if (r != p.rank) st_release_sys(p.peer_sync[r] + p.rank, p.epoch);
  }
  bool ok = true;
  for (int r = 0; r < p.world && ok; ++r)
    if (r != p.rank) ok = wait_flag_ge<true>(p.peer_sync[p.rank] + r, p.epoch, p.wait_cycles);
  if (!ok) {
    atomicCAS(p.status, 0, LF_ERR_WAIT_PEER);
    return;
  }
  const long long block_bytes = static_cast<long long>(PG_BM) * p.K * 2;
  const int pieces = static_cast<int>((block_bytes + CP_PIECE - 1) / CP_PIECE);
  uint32_t issued = 0;  // pieces whose load has been issued (stage = issued % CP_STAGES)
  // only the peers' rows move: this rank's own rows were written into the buffer before the launch
  const int remote_blocks = p.tiles_m - p.tiles_per_rank_m;
  for (int vb = c; vb < remote_blocks; vb += p.copy_ctas) {
    // visiting order: rank+1's shard first, then rank+2, ... (the order in which the GEMM CTAs reach them)
    const int b = ((p.rank + 1) * p.tiles_per_rank_m + vb) % p.tiles_m;
    const int src_rank = b / p.tiles_per_rank_m;
    // every rank's buffer has the same layout: block b sits at the same offset on its owner
    const uint8_t* src = p.peer_x[src_rank] + static_cast<long long>(b) * block_bytes;
    uint8_t* dst = p.x_full + static_cast<long long>(b) * block_bytes;
    int loaded = 0, stored = 0;
    const uint32_t base = issued;
    while (stored < pieces) {
      // keep up to CP_STAGES loads in flight
      while (loaded < pieces && loaded - stored < CP_STAGES) {
        const uint32_t it = base + loaded;
        const int s = it % CP_STAGES;
        // the bulk store that last read this stage must have finished reading shared memory
        tma_store_wait_read<0>();
        const long long off = static_cast<long long>(loaded) * CP_PIECE;
        const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(CP_PIECE), block_bytes - off));
        mbar_arrive_expect_tx(&bars[s], bytes);
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_u32(smem + s * CP_PIECE)),
            "l"(src + off), "r"(bytes), "r"(smem_u32(&bars[s]))
            : "memory");
        ++loaded;
      }
      const uint32_t it = base + stored;
      const int s = it % CP_STAGES;
      int dummy_abort = 0;
      if (!mbar_wait(&bars[s], (it / CP_STAGES) & 1, &dummy_abort)) {
        atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
        return;
      }
      const long long off = static_cast<long long>(stored) * CP_PIECE;
      const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(CP_PIECE), block_bytes - off));
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + off),
                   "r"(smem_u32(smem + s * CP_PIECE)), "r"(bytes)
                   : "memory");
      tma_store_commit();
      ++stored;
    }
    issued = base + pieces;
    tma_store_wait<0>();      // all bytes of this row block are in local global memory
    fence_proxy_async_all();  // order the async-proxy writes before the flag
    st_release_gpu(p.chunk_flags + b, p.epoch);
  }
}

// ------------------------------------------------------------------ the kernel
template <bool B_MN, int MODE>  // MODE 0: all-gather -> GEMM, MODE 1: GEMM -> reduce-scatter
__global__ void __launch_bounds__(PG_THREADS, 1)
peer_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const PeerParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* stage_base = smem + PG_STAGES * PG_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_base + PG_STG_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + PG_STAGES;
  uint64_t* tmem_full = bars + 2 * PG_STAGES;
  uint64_t* tmem_empty = bars + 2 * PG_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PG_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  int cta = blockIdx.x;
  int num_ctas = gridDim.x;
  if (MODE == 0) {
    if (cta < p.copy_ctas) {
      ag_copy_cta(p, smem, bars);
      return;
    }
    cta -= p.copy_ctas;
    num_ctas -= p.copy_ctas;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + PG_BK - 1) / PG_BK;
  // row-block rotation: AG visits own rows first, RS visits own rows last
  const int rot = (MODE == 0 ? p.rank : (p.rank + 1) % p.world) * p.tiles_per_rank_m;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PG_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * PG_BN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int ready_block = -1;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        int vm, tn;
        pg_tile_coords(tile, p.tiles_m, p.tiles_n, vm, tn);
        const int tm = (vm + rot) % p.tiles_m;
        if (MODE == 0 && tm != ready_block && tm / p.tiles_per_rank_m != p.rank) {
          if (!wait_flag_ge<false>(p.chunk_flags + tm, p.epoch, p.wait_cycles)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_PEER);
            *abort_flag = 1;
            ok = false;
            break;
          }
          fence_proxy_async_all();  // the block was written through the async proxy by a copy CTA
          ready_block = tm;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % PG_STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / PG_STAGES) & 1) ^ 1, abort_flag, p.wait_cycles)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = tiles + s * PG_STAGE_BYTES;
          uint8_t* sb = sa + PG_A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], PG_STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[s], kb * PG_BK, tm * PG_BM);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < PG_BN / 64; ++j)
              tma_load_2d(sb + j * (PG_BK * 128), &tmap_b, &full_bar[s], tn * PG_BN + j * 64, kb * PG_BK);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[s], kb * PG_BK, tn * PG_BN);
          }
        }
      }
      if (*abort_flag) {
        const uint32_t first = it > PG_STAGES ? it - PG_STAGES : 0;
        for (uint32_t j = first; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[j % PG_STAGES], (j / PG_STAGES) & 1))
            if (clock64() - t0 > (LF_WAIT_BUDGET_CYCLES >> 4)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, false, B_MN, PG_BM, PG_BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas, ++acc_it) {
        const uint32_t acc = acc_it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.wait_cycles)) {
          atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * PG_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % PG_STAGES;
          if (!mbar_wait(&full_bar[s], (it / PG_STAGES) & 1, abort_flag, p.wait_cycles)) {
            atomicCAS(p.status, 0, LF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + s * PG_STAGE_BYTES);
          const uint32_t sb = sa + PG_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < PG_BK / PG_UMMA_K; ++kk) {
            const uint64_t da = make_smem_desc_sw128(sa + kk * (PG_UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * (PG_UMMA_K * 128), PG_BK * 128, 1024)
                                     : make_smem_desc_sw128(sb + kk * (PG_UMMA_K * 2), 16, 1024);
            tc_mma_f16_ss(tmem_d, da, db, idesc, (kb | kk) != 0);
          }
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = cta; tile < num_tiles && ok; tile += num_ctas, ++acc_it) {
      int vm, tn;
      pg_tile_coords(tile, p.tiles_m, p.tiles_n, vm, tn);
      const int tm = (vm + rot) % p.tiles_m;
      const uint32_t acc = acc_it & 1;
      if (!mbar_wait_warp(&tmem_full[acc], (acc_it >> 1) & 1, abort_flag, p.wait_cycles)) {
        if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * PG_BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * PG_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int owner = (MODE == 1) ? tm / p.tiles_per_rank_m : p.rank;
      const int local_tile = (tm - owner * p.tiles_per_rank_m) * p.tiles_n + tn;
      const int tiles_per_rank = p.tiles_per_rank_m * p.tiles_n;
      __nv_bfloat16* drow;
      if (MODE == 1 && owner != p.rank) {
        // partial sums go straight into the owner's receive slot for (parity, this rank)
        const long long slot = static_cast<long long>(p.parity) * p.world + p.rank;
        drow = p.peer_recv[owner] + (slot * p.rows_per_rank + (row - owner * p.rows_per_rank)) * p.N;
      } else if (MODE == 1) {
        drow = p.out + static_cast<long long>(row - owner * p.rows_per_rank) * p.ldo;
        // wait for every peer's partial of this tile (4 epilogue warps each bump the counter once)
        bool got = true;
        if (lane == 0) {
          for (int src = 0; src < p.world && got; ++src)
            if (src != p.rank)
              got = wait_flag_ge<true>(
                  p.peer_tile_flags[p.rank] + (static_cast<long long>(p.parity) * p.world + src) * tiles_per_rank +
                      local_tile,
                  p.expect, p.wait_cycles);
        }
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (!got) {
          if (lane == 0) atomicCAS(p.status, 0, LF_ERR_WAIT_PEER);
          *abort_flag = 1;
          ok = false;
        }
      } else {
        drow = p.out + static_cast<long long>(row) * p.ldo;
      }
      if (ok) {
        uint8_t* stg = stage_base + (warp & 3) * (32 * PG_STG_ROW);
        // first row of this warp's 32-row patch in the destination, and the destination's row pitch
        __nv_bfloat16* dwarp = drow - static_cast<long long>(lane) * ((MODE == 1) ? (owner != p.rank ? p.N : p.ldo) : p.ldo);
        const long long dpitch = (MODE == 1) ? (owner != p.rank ? p.N : p.ldo) : p.ldo;
#pragma unroll 1
        for (int c0 = 0; c0 < PG_BN; c0 += 64) {
          const int col = tn * PG_BN + c0;
          if (col >= p.N) break;
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(taddr + c0, r0);
          tmem_ld_32x32b_x32(taddr + c0 + 32, r1);
          tmem_ld_wait();
          float v[64];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r0[j]);
            v[32 + j] = __uint_as_float(r1[j]);
          }
          if (p.bias != nullptr && (MODE == 0)) {
#pragma unroll
            for (int j = 0; j < 64; ++j)
              if (col + j < p.N) v[j] += __bfloat162float(p.bias[col + j]);
          }
          if (MODE == 1 && owner == p.rank) {
            const int lrow = row - owner * p.rows_per_rank;
            for (int src = 0; src < p.world; ++src) {
              if (src == p.rank) continue;
              const __nv_bfloat16* rr =
                  p.peer_recv[p.rank] +
                  ((static_cast<long long>(p.parity) * p.world + src) * p.rows_per_rank + lrow) * p.N + col;
#pragma unroll
              for (int j = 0; j < 64; j += 8) {
                if (col + j + 8 <= p.N) {
                  const uint4 q = __ldcv(reinterpret_cast<const uint4*>(rr + j));
                  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                  for (int t = 0; t < 4; ++t) {
                    const float2 f = __bfloat1622float2(h[t]);
                    v[j + 2 * t] += f.x;
                    v[j + 2 * t + 1] += f.y;
                  }
                }
              }
            }
            if (p.residual != nullptr) {
              const __nv_bfloat16* rs = p.residual + static_cast<long long>(lrow) * p.ldr + col;
#pragma unroll
              for (int j = 0; j < 64; j += 8) {
                if (col + j + 8 <= p.N) {
                  const uint4 q = *reinterpret_cast<const uint4*>(rs + j);
                  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                  for (int t = 0; t < 4; ++t) {
                    const float2 f = __bfloat1622float2(h[t]);
                    v[j + 2 * t] += f.x;
                    v[j + 2 * t + 1] += f.y;
                  }
                }
              }
            }
          }
          // transpose through shared memory: each thread parks its row's 128 bytes, then the warp writes four rows
          // per instruction as full 128-byte segments (efficient NVLink packets for the remote tiles)
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(v[j], v[j + 1]);
            o.y = pack_bf16x2(v[j + 2], v[j + 3]);
            o.z = pack_bf16x2(v[j + 4], v[j + 5]);
            o.w = pack_bf16x2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(stg + lane * PG_STG_ROW + j * 2) = o;
          }
          __syncwarp();
          const int piece = lane & 7;
          if (col + piece * 8 + 8 <= p.N) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3);
              const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * PG_STG_ROW + piece * 16);
              *reinterpret_cast<uint4*>(dwarp + rr * dpitch + col + piece * 8) = o;
            }
          }
        }
        if (MODE == 1 && owner != p.rank) {
          // make this warp's stores visible at the peer, then count the warp in
          __threadfence_system();
          __syncwarp();
          if (lane == 0)
            red_release_sys_add(p.peer_tile_flags[owner] +
                                    (static_cast<long long>(p.parity) * p.world + p.rank) * tiles_per_rank + local_tile,
                                1);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * PG_BN);
  }
}

// ---------------------------------------------------------------------- host
static int pg_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <bool B_MN, int MODE>
static int pg_launch(const CUtensorMap& ta, const CUtensorMap& tb, const PeerParams& p, int grid, cudaStream_t stream) {
  auto kern = peer_gemm_kernel<B_MN, MODE>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PG_SMEM_BYTES) != cudaSuccess) return -4;
    attr = true;
  }
  kern<<<grid, PG_THREADS, PG_SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ag_gemm(const AgGemmArgs& a, cudaStream_t stream) {
  const int T = a.rows_per_rank * a.world;
  if (a.world < 1 || a.world > kMaxPeers || a.rows_per_rank % PG_BM || (a.K % 8) || (a.N % 8) || (a.ldo % 8) ||
      (a.ldb % 8))
    return -2;
  if ((static_cast<long long>(PG_BM) * a.K * 2) % 16) return -2;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_bf16_2d(&ta, a.x_full, T, a.K, a.K, PG_BM, PG_BK))) return rc;
  if (a.b_mn_major)
    rc = make_tmap_bf16_2d(&tb, a.B, a.K, a.N, a.ldb, PG_BK, 64);
  else
    rc = make_tmap_bf16_2d(&tb, a.B, a.N, a.K, a.ldb, PG_BN, PG_BK);
  if (rc) return rc;
  PeerParams p = {};
  p.M = T; p.N = a.N; p.K = a.K;
  p.tiles_m = T / PG_BM;
  p.tiles_n = (a.N + PG_BN - 1) / PG_BN;
  p.tiles_per_rank_m = a.rows_per_rank / PG_BM;
  p.rank = a.rank; p.world = a.world; p.rows_per_rank = a.rows_per_rank;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.ldo = a.ldo;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.status = a.status;
  for (int r = 0; r < a.world; ++r) {
    p.peer_x[r] = static_cast<const uint8_t*>(a.peer_x[r]);
    p.peer_sync[r] = a.peer_sync[r];
  }
  p.x_full = static_cast<uint8_t*>(a.x_full);
  p.chunk_flags = a.chunk_flags;
  p.epoch = a.epoch;
  p.wait_cycles = g_peer_wait_cycles;
  const int sms = pg_sms();
  int copy = a.copy_ctas;
  if (copy < 1) copy = 1;
  if (copy > p.tiles_m) copy = p.tiles_m;
  if (copy > sms / 4) copy = sms / 4;
  p.copy_ctas = copy;
  const int tiles = p.tiles_m * p.tiles_n;
  int gemm_ctas = sms - copy;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  // every CTA of the grid must be resident at once (GEMM CTAs wait on copy CTAs): grid <= #SMs
  const int grid = copy + gemm_ctas;
  return a.b_mn_major ? pg_launch<true, 0>(ta, tb, p, grid, stream) : pg_launch<false, 0>(ta, tb, p, grid, stream);
}

int gemm_rs(const GemmRsArgs& a, cudaStream_t stream) {
  if (a.world < 1 || a.world > kMaxPeers || a.T % (PG_BM * a.world) || (a.K % 8) || (a.N % 8) || (a.ldo % 8) ||
      (a.lda % 8) || (a.ldb % 8) || (a.residual && (a.ldr % 8)))
    return -2;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_bf16_2d(&ta, a.A, a.T, a.K, a.lda, PG_BM, PG_BK))) return rc;
  if (a.b_mn_major)
    rc = make_tmap_bf16_2d(&tb, a.B, a.K, a.N, a.ldb, PG_BK, 64);
  else
    rc = make_tmap_bf16_2d(&tb, a.B, a.N, a.K, a.ldb, PG_BN, PG_BK);
  if (rc) return rc;
  PeerParams p = {};
  p.M = a.T; p.N = a.N; p.K = a.K;
  p.tiles_m = a.T / PG_BM;
  p.tiles_n = (a.N + PG_BN - 1) / PG_BN;
  p.rows_per_rank = a.T / a.world;
  p.tiles_per_rank_m = p.rows_per_rank / PG_BM;
  p.rank = a.rank; p.world = a.world;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.ldo = a.ldo;
  p.residual = static_cast<const __nv_bfloat16*>(a.residual);
  p.ldr = a.ldr;
  p.status = a.status;
  for (int r = 0; r < a.world; ++r) {
    p.peer_recv[r] = static_cast<__nv_bfloat16*>(a.peer_recv[r]);
    p.peer_tile_flags[r] = a.peer_tile_flags[r];
  }
  p.parity = a.call_index & 1;
  p.wait_cycles = g_peer_wait_cycles;
  p.expect = 4 * (a.call_index / 2 + 1);
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = pg_sms();
  if (grid > tiles) grid = tiles;
  return a.b_mn_major ? pg_launch<true, 1>(ta, tb, p, grid, stream) : pg_launch<false, 1>(ta, tb, p, grid, stream);
}

}  // namespace lf
