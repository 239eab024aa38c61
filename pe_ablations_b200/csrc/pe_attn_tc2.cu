// CTA-pair variant of the tcgen05 fused PE-attention forward (bf16, d_v = 128).
//
// Two CTAs on neighbouring SMs (a cluster of 2) own 512 query rows of one (batch, head) and
// share every K/V tile: each CTA loads and transforms only HALF of a 128-key tile (64 keys of
// K, 64 value columns of V), and the leader CTA issues `tcgen05.mma.cta_group::2` instructions
// that span both SMs (M = 256: 128 rows in each CTA's TMEM; N = 128 taken half from each CTA's
// shared memory).  Compared with the single-CTA kernel this halves the shared-memory operand
// traffic per MMA (the QK product is no longer port-bound), the L2 -> SM traffic, and the
// positional transform work per FLOP, and doubles the keys per synchronisation step.
//
// Per CTA: two 128-row query tiles.  "Pair tile" i is the 256 rows made of tile i of both CTAs
// (CTA rank r holds rows m0 + (2 i + r) * 128 ...).  TMEM per CTA: S_i / P_i at columns
// i * 128 (P, packed bf16, overwrites its own S tile chunk by chunk), O_i at 256 + i * 128.
//
// Warp roles per CTA as in the single-CTA kernel (0: Q/K TMA, 1: MMA issue -- leader only,
// 2: TMEM, 3: V TMA, 4-7 / 8-11: softmax of tile 0 / 1, 12-15: K transform).  Barriers that
// gate MMA issue (q_full, k_full, v_full, p_ready) live in the leader's shared memory and
// collect arrivals from both CTAs; barriers signalled by MMA completion (s_full, k_empty,
// v_empty, o_done) exist in both CTAs and are signalled together by one multicast commit.
// Issue order of the leader, per key tile j:  PV_0(j)  QK_0(j+1)  PV_1(j)  QK_1(j+1), so the
// tensor pipe works on one pair tile while the softmax warps work on the other.
//
// Few-wave grids: a pair works through one 512-row block at the pace of its dependency chain,
// and the longest block of a causal problem needs as many steps as there are key tiles.  When
// a launch has fewer than about three blocks per pair slot, the longest blocks of every
// (batch, head) are therefore cut in two along the KEYS: two pairs attend the same rows to the
// first and the second half of the key tiles, write normalised fp32 partial outputs and
// logsumexps to a caller-provided workspace, and ``pair_merge_kernel`` combines them.  Work
// items (parts and whole blocks) are handed out longest first.
//
// Every wait is bounded; a CTA that gives up reports through the status word and both CTAs
// still meet at the final cluster barrier before releasing TMEM.
#include <cuda.h>

#include <array>
#include <map>
#include <mutex>
#include <queue>
#include <vector>

#include "pe_attn_tc_common.cuh"

// How the K-transform warps tell the leader's MMA warp that their rows of a K tile are in shared
// memory.  Every lane has run fence.proxy.async after its stores and the warp has synchronised
// before lane 0 arrives, so the rows are in this SM's shared memory (there is no cache between
// the stores and the tensor core's reads) when the arrival leaves; the arrival itself is
// relaxed because a release at cluster scope costs about 600 clocks per arrival, which sat on
// the K-ready path of the variants that transform whole K rows (configuration 3: 678 -> 750
// TFLOP/s).  -DPE_TC2_KFULL_ARRIVE=mbar_arrive_cluster restores the release.
#ifndef PE_TC2_P_PARTS
#define PE_TC2_P_PARTS 4   // 1, 2 or 4
#endif
#ifndef PE_TC2_KFULL_ARRIVE
#define PE_TC2_KFULL_ARRIVE mbar_arrive_cluster_relaxed
#endif

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

constexpr int BLOCK_M = 128;     // query rows per tile per CTA (TMEM lanes)
constexpr int Q_TILES = 2;       // query tiles per CTA
constexpr int PAIR_ROWS = 512;   // query rows per CTA pair
constexpr int BLOCK_N = 128;     // keys per tile (64 held by each CTA)
constexpr int HALF_N = 64;
constexpr int DV = 128;
constexpr int KV_STAGES = 2;
constexpr int NTHREADS = 512;
constexpr int TMEM_COLS = 512;
constexpr int TAIL_BYTES = 1024;
// workspace of one split block: fp32 [2 parts][512 rows][128] partial outputs, then [2][512] logsumexps
constexpr int SPLIT_ITEM_FLOATS = 2 * PAIR_ROWS * DV + 2 * PAIR_ROWS;

// key tiles the LAST row tile of 512-row block ``sblk`` needs (the block's step count)
__host__ __device__ __forceinline__ int block_tiles(int sblk, int Sk, int causal_off) {
  int kend = sblk * PAIR_ROWS + PAIR_ROWS + causal_off;
  if (kend > Sk) kend = Sk;
  return (kend + BLOCK_N - 1) / BLOCK_N;
}

constexpr int MAX_K_STAGES = 4;
enum : int {
  BAR_QFULL = 0, BAR_VFULL = 2, BAR_VEMPTY = 4, BAR_SFULL = 6, BAR_PREADY = 8, BAR_ODONE = 10, BAR_MMADONE = 12,
  BAR_PHALF = 13,    // up to three partial hand-offs x two tiles
  BAR_KFULL = 19, BAR_KEMPTY = BAR_KFULL + MAX_K_STAGES, NUM_BARS = BAR_KEMPTY + MAX_K_STAGES
};
static_assert(NUM_BARS * 8 <= 256, "the barriers share the first 256 bytes of the tail");

template <int DC, int DR>
struct Cfg2 {
  static constexpr int DQK = DC + 2 * DR;
  static constexpr int NCHUNK = DQK / 64;
  static constexpr int NCC = DC / 64;
  static constexpr int Q_CHUNK_BYTES = BLOCK_M * 128;
  static constexpr int K_CHUNK_BYTES = HALF_N * 128;
  static constexpr int Q_TILE_BYTES = NCHUNK * Q_CHUNK_BYTES;
  static constexpr int K_STAGE_BYTES = NCHUNK * K_CHUNK_BYTES;   // this CTA's 64 keys
  static constexpr int V_STAGE_BYTES = BLOCK_N * 128;            // 128 keys x this CTA's 64 value columns
  // K tiles in flight: two where d_qk = 192 / 256 fills the shared memory, four below that -- a
  // K tile built by the transform warps (wake-up on "stage free", eight passes, proxy fence, an
  // arrival at the leader's barrier) then has three steps instead of one before the MMA warp
  // wants it, which at d_qk = 128 (short steps) it did not always make
  static constexpr int K_STAGES = DQK <= 128 ? MAX_K_STAGES : 2;
  static constexpr int Q_OFF = TAIL_BYTES;
  static constexpr int K_OFF = Q_OFF + Q_TILES * Q_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + K_STAGES * K_STAGE_BYTES;
  static constexpr int SMEM_USED = V_OFF + KV_STAGES * V_STAGE_BYTES;
  static constexpr int SMEM_BYTES = SMEM_USED + 1024;
  static_assert(DQK % 64 == 0 && DQK >= 64 && DQK <= 256, "d_qk must be 64..256 in steps of 64");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
};

template <int DC, int DR, int MODE, bool ALIBI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
pe_attn_tc2_kernel(const KParams p, const int bh_group, const int n_top, float* const split_ws,
                   const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV) {
  using C = Cfg2<DC, DR>;
  constexpr bool HAS_TMA_QK = (MODE == MODE_PLAIN) || (MODE == MODE_POPE && DC > 0);
  constexpr bool HAS_XFORM = MODE != MODE_PLAIN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 256);
  volatile uint32_t* abort_slot = reinterpret_cast<volatile uint32_t*>(smem + 260);
  float* freq_s = reinterpret_cast<float*>(smem + 512);
  float* delta_s = reinterpret_cast<float*>(smem + 768);
  auto bar = [&](int idx) -> uint32_t { return smem_base + 8u * (uint32_t)idx; };

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  auto lbar = [&](int idx) -> uint32_t { return mapa(bar(idx), 0); };  // the leader's copy of a barrier
  // stage and barrier phase of key tile j in the ring of K stages
  auto ks = [](int j) -> int { return j & (C::K_STAGES - 1); };
  auto kph = [](int j) -> uint32_t { return (uint32_t)((j / C::K_STAGES) & 1); };

  // pair (cluster) index -> work item of a (batch, head), longest first within head groups.
  // Items per (batch, head): the n_top longest blocks as two parts each, the others whole.
  const int n_sblk = (p.Sq + PAIR_ROWS - 1) / PAIR_ROWS;
  const int n_bh = p.B * p.H;
  const int pair = (int)(blockIdx.x >> 1);
  const int per_group = bh_group * (n_sblk + n_top);
  const int grp = pair / per_group, in_grp = pair % per_group;
  const int g_first = grp * bh_group;
  const int g_size = (n_bh - g_first) < bh_group ? (n_bh - g_first) : bh_group;
  const int item_rank = in_grp / g_size;   // 0 = the longest item
  const int bh = g_first + in_grp % g_size;
  const int h = bh % p.H, b = bh / p.H;
  const int hk = h / p.groups;
  int sblk = n_sblk - 1 - item_rank, part = -1;   // part -1: a whole block
  if (n_top > 0) {
    // merge of two descending lists (parts of the longest blocks, whole shorter blocks) up to
    // this item's rank: one thread walks it, everybody reads the answer
    volatile int* decode_slot = reinterpret_cast<volatile int*>(smem + 264);
    if (tid == 0) {
      int ia = 0, ib = n_sblk - n_top - 1, found_blk = 0, found_part = -1;
      for (int r = 0;; ++r) {
        int size_a = -1, size_b = -1;
        if (ia < 2 * n_top) {
          const int t = block_tiles(n_sblk - 1 - (ia >> 1), p.Sk, p.causal_off);
          size_a = (ia & 1) ? t - t / 2 : t / 2;
        }
        if (ib >= 0) size_b = block_tiles(ib, p.Sk, p.causal_off);
        const bool take_a = size_a >= size_b;
        if (r == item_rank) {
          found_blk = take_a ? n_sblk - 1 - (ia >> 1) : ib;
          found_part = take_a ? (ia & 1) : -1;
          break;
        }
        if (take_a) ++ia; else --ib;
      }
      decode_slot[0] = found_blk;
      decode_slot[1] = found_part;
    }
    __syncthreads();
    sblk = decode_slot[0];
    part = decode_slot[1];
  }
  const int m0 = sblk * PAIR_ROWS;

  // key tiles pair tile i needs: keys [0, min(Sk, last row of the pair tile + 1 + off)); a part
  // of a split block takes the first half of the block's tiles or the rest.  ``jb`` is the
  // first tile, nt[i] the number of tiles from there on: loops count from 0, the tile they
  // address is jb + j.
  int nt[Q_TILES], jb = 0;
  {
    const int cut = block_tiles(sblk, p.Sk, p.causal_off) / 2;
    if (part == 1) jb = cut;
#pragma unroll
    for (int i = 0; i < Q_TILES; ++i) {
      const int first = m0 + i * 2 * BLOCK_M;
      int kend = first + 2 * BLOCK_M + p.causal_off;
      if (kend > p.Sk) kend = p.Sk;
      int n = first < p.Sq ? (kend + BLOCK_N - 1) / BLOCK_N : 0;
      if (part == 0) n = n < cut ? n : cut;
      if (part == 1) n = n > cut ? n - cut : 0;
      nt[i] = n;
    }
  }
  const int n_tiles = nt[1] > nt[0] ? nt[1] : nt[0];
  // partial results of a part: [512 rows][128] fp32, then the block's logsumexps [2][512]
  float* const ws_out = part < 0 ? nullptr
                                 : split_ws + (size_t)(bh * n_top + (n_sblk - 1 - sblk)) * SPLIT_ITEM_FLOATS +
                                       (size_t)part * PAIR_ROWS * DV;
  float* const ws_lse = part < 0 ? nullptr
                                 : split_ws + (size_t)(bh * n_top + (n_sblk - 1 - sblk)) * SPLIT_ITEM_FLOATS +
                                       (size_t)2 * PAIR_ROWS * DV + (size_t)part * PAIR_ROWS;

  auto fail = [&](int code) {
    if (p.status != nullptr) atomicOr(p.status, code);
  };

  if (tid == 0) {
    *abort_slot = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
    const uint32_t n_xf = HAS_XFORM ? 4u : 0u;
    const uint32_t n_tma = HAS_TMA_QK ? 1u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_QFULL + i), 2 * (n_tma + n_xf));   // both CTAs report to the leader's copy
      mbar_init(bar(BAR_VFULL + i), 2);
      mbar_init(bar(BAR_PREADY + i), 8);                   // 4 softmax warps x 2 CTAs
      for (int part = 0; part < 3; ++part) mbar_init(bar(BAR_PHALF + 2 * part + i), 8);   // ... for the earlier parts of P
      mbar_init(bar(BAR_VEMPTY + i), 1);
      mbar_init(bar(BAR_SFULL + i), 1);
      mbar_init(bar(BAR_ODONE + i), 1);
    }
    for (int i = 0; i < C::K_STAGES; ++i) {
      mbar_init(bar(BAR_KFULL + i), 2 * (n_tma + n_xf));
      mbar_init(bar(BAR_KEMPTY + i), 1);
    }
    mbar_init(bar(BAR_MMADONE), 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  if constexpr (MODE == MODE_POPE) {
    // eight lanes per frequency column (whole warps: 8 DR is a multiple of 32)
    if (tid < 8 * DR) {
      const float f = effective_freq_lanes<8>(p, tid >> 3, tid & 7);
      if ((tid & 7) == 0) {
        freq_s[tid >> 3] = f;
        delta_s[tid >> 3] = clamped_delta(p, tid >> 3);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool run = *abort_slot == 0;

  const uint32_t q_smem = smem_base + C::Q_OFF;
  const uint32_t k_smem = smem_base + C::K_OFF;
  const uint32_t v_smem = smem_base + C::V_OFF;

  // Register budget per warpgroup (24 / 160 / 160 / 168 x 128 threads = 64 K registers: the K
  // transform at d_r = 64 keeps 64 table values per thread and spilled at 152); each role sits
  // inside the branch that sets its budget.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
  if (!run) {
    // nothing to do
  } else if (warp == 0) {
    // ===================== TMA producer: content halves of this CTA's Q tiles and K half-tiles
    if constexpr (HAS_TMA_QK) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
      }
      for (int i = 0; i < Q_TILES; ++i) {
        if (nt[i] == 0) continue;
        if (elect_one()) {
          const uint32_t qb = lbar(BAR_QFULL + i);
          mbar_arrive_expect_tx_cluster_relaxed(qb, C::NCC * C::Q_CHUNK_BYTES);
#pragma unroll
          for (int c = 0; c < C::NCC; ++c)
            tma_load_4d_pair(q_smem + i * C::Q_TILE_BYTES + c * C::Q_CHUNK_BYTES, &tmQ, qb, c * 64,
                             m0 + (2 * i + (int)rank) * BLOCK_M, h, b);
        }
        __syncwarp();
      }
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int s = ks(j);
        const uint32_t ph = kph(j);
        if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1u))) { fail(ST_WAIT_KEMPTY); break; }
        if (elect_one()) {
          const uint32_t kb = lbar(BAR_KFULL + s);
          mbar_arrive_expect_tx_cluster_relaxed(kb, C::NCC * C::K_CHUNK_BYTES);
#pragma unroll
          for (int c = 0; c < C::NCC; ++c)
            tma_load_4d_pair(k_smem + s * C::K_STAGE_BYTES + c * C::K_CHUNK_BYTES, &tmK, kb, c * 64,
                             (jb + j) * BLOCK_N + (int)rank * HALF_N, hk, b);
        }
        __syncwarp();
      }
    }
  } else if (warp == 3) {
    // ===================== TMA producer: this CTA's 64 value columns of every V tile
    if (elect_one()) tma_prefetch_desc(&tmV);
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_VEMPTY + s), ph ^ 1u))) { fail(ST_WAIT_VEMPTY); break; }
      if (elect_one()) {
        const uint32_t vb = lbar(BAR_VFULL + s);
        mbar_arrive_expect_tx_cluster_relaxed(vb, C::V_STAGE_BYTES);
        tma_load_4d_pair(v_smem + s * C::V_STAGE_BYTES, &tmV, vb, (int)rank * 64, (jb + j) * BLOCK_N, hk, b);
      }
      __syncwarp();
    }
  } else if (warp == 1 && rank == 0) {
    // ===================== MMA issuer (leader CTA only) =====================
    constexpr uint32_t IDESC_QK = make_idesc_bf16(2 * BLOCK_M, BLOCK_N, false);
    constexpr uint32_t IDESC_PV = make_idesc_bf16(2 * BLOCK_M, DV, true);
    constexpr uint16_t BOTH = 3;
    const uint64_t qdesc0 = make_smem_desc(q_smem, 16, 1024);
    const uint64_t kdesc0 = make_smem_desc(k_smem, 16, 1024);
    const uint64_t vdesc0 = make_smem_desc(v_smem, 16, 1024);
    bool ok = true;
    for (int i = 0; i < Q_TILES && ok; ++i)
      if (nt[i] > 0 && !__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_QFULL + i), 0))) { fail(ST_WAIT_QFULL); ok = false; }

    // S_i = Q_i K(j)^T for pair tile i, then tell both CTAs' softmax warps
    auto issue_qk = [&](int i, int j) {
      if (elect_one()) {
        const uint32_t d = tmem_base + (uint32_t)(i * BLOCK_N);
        uint64_t qd = advance_smem_desc(qdesc0, (uint32_t)(i * C::Q_TILE_BYTES));
        uint64_t kd = advance_smem_desc(kdesc0, (uint32_t)(ks(j) * C::K_STAGE_BYTES));
#pragma unroll 1
        for (int c = 0; c < C::NCHUNK; ++c) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_ss_pair(d, advance_smem_desc(qd, (uint32_t)(k4 * 32)), advance_smem_desc(kd, (uint32_t)(k4 * 32)),
                        IDESC_QK, (c > 0 || k4 > 0) ? 1u : 0u);
          qd = advance_smem_desc(qd, C::Q_CHUNK_BYTES);
          kd = advance_smem_desc(kd, C::K_CHUNK_BYTES);
        }
        tc_commit_pair(bar(BAR_SFULL + i), BOTH);
      }
      __syncwarp();
    };
    auto wait_k = [&](int j) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_KFULL + ks(j)), kph(j)))) {
        fail(ST_WAIT_KFULL);
        return false;
      }
      tc_fence_after_sync();
      return true;
    };

    if (ok && n_tiles > 0) {
      ok = wait_k(0);
      if (ok) {
        for (int i = 0; i < Q_TILES; ++i)
          if (nt[i] > 0) issue_qk(i, 0);
        if (elect_one()) tc_commit_pair(bar(BAR_KEMPTY + 0), BOTH);
        __syncwarp();
      }
    }
#pragma unroll 1
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_VFULL + s), ph))) { fail(ST_WAIT_VFULL); ok = false; break; }
      bool have_k = false;
      const uint64_t vd = advance_smem_desc(vdesc0, (uint32_t)(s * C::V_STAGE_BYTES));
#pragma unroll
      for (int i = 0; i < Q_TILES; ++i) {
        if (j < nt[i]) {
          // P arrives in PE_TC2_P_PARTS parts: the PV MMAs of a part run under the exponentials
          // of the next one
          const uint32_t d = tmem_base + 256u + (uint32_t)(i * DV);
          const uint32_t a = tmem_base + (uint32_t)(i * BLOCK_N);
          constexpr int KK_PART = (BLOCK_N / 16) / PE_TC2_P_PARTS;   // MMAs (16 keys each) per part of P
#pragma unroll
          for (int part = 0; part + 1 < PE_TC2_P_PARTS; ++part) {
            if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PHALF + 2 * part + i), (uint32_t)(j & 1)))) {
              fail(ST_WAIT_PREADY);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (elect_one()) {
#pragma unroll
              for (int kk = part * KK_PART; kk < (part + 1) * KK_PART; ++kk)
                mma_ts_pair(d, a + (uint32_t)(kk * 8), advance_smem_desc(vd, (uint32_t)(kk * 16 * 128)), IDESC_PV,
                            (j > 0 || kk > 0) ? 1u : 0u);
            }
            __syncwarp();
          }
          if (!ok) break;
          if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PREADY + i), (uint32_t)(j & 1)))) {
            fail(ST_WAIT_PREADY);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (elect_one()) {
#pragma unroll
            for (int kk = (PE_TC2_P_PARTS - 1) * KK_PART; kk < BLOCK_N / 16; ++kk)
              mma_ts_pair(d, a + (uint32_t)(kk * 8), advance_smem_desc(vd, (uint32_t)(kk * 16 * 128)), IDESC_PV,
                          (j > 0 || kk > 0) ? 1u : 0u);
            tc_commit_pair(bar(BAR_ODONE + i), BOTH);
          }
          __syncwarp();
        }
        if (j + 1 < nt[i]) {
          if (!have_k) {
            if (!wait_k(j + 1)) { ok = false; break; }
            have_k = true;
          }
          issue_qk(i, j + 1);   // overwrites S_i / P_i: ordered after PV_i(j) by the in-order tensor pipe
        }
      }
      if (!ok) break;
      if (elect_one()) {
        tc_commit_pair(bar(BAR_VEMPTY + s), BOTH);
        if (j + 1 < n_tiles) tc_commit_pair(bar(BAR_KEMPTY + ks(j + 1)), BOTH);
      }
      __syncwarp();
    }
    if (elect_one()) tc_commit_pair(bar(BAR_MMADONE), 1);
    __syncwarp();
    if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_MMADONE), 0))) fail(ST_WAIT_MMADONE);
  }
  } else if (warp < 12) {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
  if (run) {
    // ===================== softmax warpgroups =====================
    const int i = (warp - 4) >> 2;
    const int tg = tid - 128 - i * BLOCK_M;
    const int ntile = nt[i];
    const int row0 = m0 + (2 * i + (int)rank) * BLOCK_M;   // first query row of this CTA's tile i
    if (ntile > 0) {
      if constexpr (HAS_XFORM) {
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const int r0 = row0 + half * 64;
          build_slab<DC, DR, MODE>(p, q_smem + i * C::Q_TILE_BYTES + half * 64 * 128, C::Q_CHUNK_BYTES, p.q, p.qr, b,
                                   h, r0, p.Sq, p.q_pos0 + r0, false, freq_s, delta_s, tg);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lbar(BAR_QFULL + i));
      }
      const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
      const int row = row0 + tg;
      const int row_lim = row + p.causal_off;
      const float c2 = p.scale * 1.4426950408889634f;
      float slope2 = 0.f;
      if constexpr (ALIBI) slope2 = p.slopes[h] * 1.4426950408889634f;
      const float kf = ALIBI ? 1.0f : c2;
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;
      const uint32_t s_addr = tmem_base + lane_sel + (uint32_t)(i * BLOCK_N);
      const uint32_t o_addr = tmem_base + lane_sel + 256u + (uint32_t)(i * DV);
      const uint32_t pready = lbar(BAR_PREADY + i);
      const uint32_t ppart = lbar(BAR_PHALF + i);   // part k's barrier is 2 * k barriers (16 bytes each step) further

#pragma unroll 1
      for (int j = 0; j < ntile; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_SFULL + i), (uint32_t)(j & 1)));
        if (!ok) { fail(ST_WAIT_SFULL); break; }
        tc_fence_after_sync();
        const int key0 = (jb + j) * BLOCK_N;
        const bool need_mask = (key0 + BLOCK_N - 1 > row0 + p.causal_off) || (key0 + BLOCK_N > p.Sk);
        float base_bias = 0.f;
        if constexpr (ALIBI) base_bias = slope2 * (float)(key0 - row_lim);

        // ---- the whole S row (128 fp32) into registers with one wait, bias / mask in place
        uint32_t sr[4][32];
        tmem_ld32(s_addr, sr[0]);
        tmem_ld32(s_addr + 32, sr[1]);
        tmem_ld32(s_addr + 64, sr[2]);
        tmem_ld32(s_addr + 96, sr[3]);
        tmem_wait_ld();
        float t[BLOCK_N];
#pragma unroll
        for (int c = 0; c < BLOCK_N; ++c) t[c] = __uint_as_float(sr[c >> 5][c & 31]);
        if constexpr (ALIBI) {
#pragma unroll
          for (int c = 0; c < BLOCK_N; c += 2) {
            // two columns per packed FMA (same roundings as fmaf(t, c2, fmaf(c, slope2, base)) each)
            const float2 bias = __ffma2_rn(make_float2((float)c, (float)(c + 1)), make_float2(slope2, slope2),
                                           make_float2(base_bias, base_bias));
            const float2 r = __ffma2_rn(make_float2(t[c], t[c + 1]), make_float2(c2, c2), bias);
            t[c] = r.x;
            t[c + 1] = r.y;
          }
        }
        if (need_mask) {
          // columns past the row's last visible key (causal limit, end of the keys): one compare each
          const int last = (row_lim < p.Sk - 1 ? row_lim : p.Sk - 1) - key0;
#pragma unroll
          for (int c = 0; c < BLOCK_N; ++c)
            if (c > last) t[c] = -INFINITY;
        }
        float mx0 = fmax3(t[0], t[1], t[2]), mx1 = fmax3(t[3], t[4], t[5]), mx2 = fmax3(t[6], t[7], t[8]),
              mx3 = fmax3(t[9], t[10], t[11]);
#pragma unroll
        for (int c = 12; c + 8 <= BLOCK_N; c += 8) {
          mx0 = fmax3(mx0, t[c], t[c + 1]);
          mx1 = fmax3(mx1, t[c + 2], t[c + 3]);
          mx2 = fmax3(mx2, t[c + 4], t[c + 5]);
          mx3 = fmax3(mx3, t[c + 6], t[c + 7]);
        }
        // 12 + 14 * 8 = 124: the last four columns
        mx0 = fmax3(mx0, t[BLOCK_N - 4], t[BLOCK_N - 3]);
        mx1 = fmax3(mx1, t[BLOCK_N - 2], t[BLOCK_N - 1]);
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));

        // ---- lazy rescale of the running output
        const bool need = (mx - m_used) * kf > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? ex2_approx((m_used - mx) * kf) : 1.0f;
          if (j > 0) {
            ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_ODONE + i), (uint32_t)((j - 1) & 1)));
            if (!ok) { fail(ST_WAIT_PVDONE); break; }
            tc_fence_after_sync();
            // rare path, and the whole S row is live in registers: 16 columns at a time
#pragma unroll 1
            for (int cb = 0; cb < DV / 16; ++cb) {
              uint32_t orow[16];
              tmem_ld16(o_addr + cb * 16, orow);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 16; ++c) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
              tmem_st16(o_addr + cb * 16, orow);
            }
            tmem_wait_st();
          }
          l_sum *= alpha;
          if (need) m_used = mx;
        }

        // ---- exponentials, row sum, P as bf16 pairs over the first 64 columns of this S tile
        // (every S value of the row is already in registers)
        // scale-and-shift and the row sum use the packed fp32x2 FMA / ADD of sm_100 (half the
        // issue slots of scalar code); the exponentials stay on the special-function unit
        const float2 kf2 = make_float2(kf, kf), nm2 = make_float2(-m_used * kf, -m_used * kf);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int cb = 0; cb < BLOCK_N / 32; ++cb) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float2 x01 = __ffma2_rn(make_float2(t[cb * 32 + c], t[cb * 32 + c + 1]), kf2, nm2);
            const float2 x23 = __ffma2_rn(make_float2(t[cb * 32 + c + 2], t[cb * 32 + c + 3]), kf2, nm2);
            const float2 p01 = make_float2(ex2_approx(x01.x), ex2_approx(x01.y));
            const float2 p23 = make_float2(ex2_approx(x23.x), ex2_approx(x23.y));
            acc0 = __fadd2_rn(acc0, p01);
            acc1 = __fadd2_rn(acc1, p23);
            pk[c >> 1] = pack_bf16x2(p01.x, p01.y);
            pk[(c >> 1) + 1] = pack_bf16x2(p23.x, p23.y);
          }
          tmem_st16(s_addr + cb * 16, pk);
          // every BLOCK_N / PE_TC2_P_PARTS keys of P that are in TMEM are handed to the MMA warp
          if (PE_TC2_P_PARTS > 1 && cb + 1 < BLOCK_N / 32 && (cb + 1) % (4 / PE_TC2_P_PARTS) == 0) {
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(ppart + 16u * (uint32_t)((cb + 1) / (4 / PE_TC2_P_PARTS) - 1));
          }
        }
        const float a0 = acc0.x, a1 = acc0.y, a2 = acc1.x, a3 = acc1.y;
        l_sum += (a0 + a1) + (a2 + a3);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(pready);
      }

      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_ODONE + i), (uint32_t)((ntile - 1) & 1)));
        if (!ok) fail(ST_WAIT_PVDONE);
      }
      if (ok) {
        tc_fence_after_sync();
        // a part whose keys are all hidden from this row contributes nothing
        const float inv_l = l_sum > 0.f ? 1.0f / l_sum : 0.f;
        const float row_lse = l_sum > 0.f ? m_used * kf * 0.6931471805599453f + logf(l_sum) : -INFINITY;
        if (ws_out != nullptr) ws_lse[row - m0] = row_lse;
        else if (p.lse != nullptr && row < p.Sq) p.lse[((long long)b * p.H + h) * p.Sq + row] = row_lse;
        char* dst = reinterpret_cast<char*>(const_cast<void*>(p.out.ptr)) +
                    2 * ((long long)b * p.out.sb + (long long)h * p.out.sh + (long long)row * p.out.ss);
#pragma unroll 1
        for (int cb = 0; cb < DV / 32; ++cb) {
          uint32_t orow[32];
          tmem_ld32(o_addr + cb * 32, orow);
          tmem_wait_ld();
          if (ws_out != nullptr) {
            float4* wdst = reinterpret_cast<float4*>(ws_out + (size_t)(row - m0) * DV + cb * 32);
#pragma unroll
            for (int v = 0; v < 8; ++v)
              wdst[v] = make_float4(__uint_as_float(orow[v * 4 + 0]) * inv_l, __uint_as_float(orow[v * 4 + 1]) * inv_l,
                                    __uint_as_float(orow[v * 4 + 2]) * inv_l, __uint_as_float(orow[v * 4 + 3]) * inv_l);
          } else if (row < p.Sq) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(orow[v * 8 + 0]) * inv_l, __uint_as_float(orow[v * 8 + 1]) * inv_l);
              o.y = pack_bf16x2(__uint_as_float(orow[v * 8 + 2]) * inv_l, __uint_as_float(orow[v * 8 + 3]) * inv_l);
              o.z = pack_bf16x2(__uint_as_float(orow[v * 8 + 4]) * inv_l, __uint_as_float(orow[v * 8 + 5]) * inv_l);
              o.w = pack_bf16x2(__uint_as_float(orow[v * 8 + 6]) * inv_l, __uint_as_float(orow[v * 8 + 7]) * inv_l);
              *reinterpret_cast<uint4*>(dst + (cb * 32 + v * 8) * 2) = o;
            }
          }
        }
      }
    }
  }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
  if (run) {
    // ===================== positional transform of this CTA's 64 keys of every K tile ===========
    const int tg = tid - 384;
    if constexpr (MODE == MODE_POPE) {
      constexpr int VPR = DR / 8, RPP = 128 / VPR, PASSES = HALF_N / RPP;
      const int cv = tg % VPR, r_in = tg / VPR;
      float th[8], tcs[PASSES][8], tsn[PASSES][8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        th[e] = freq_s[cv * 8 + e];
        const float dl = delta_s[cv * 8 + e];
#pragma unroll
        for (int k = 0; k < PASSES; ++k)
          sincos_reduced(__fadd_rn(__fmul_rn((float)(r_in + k * RPP), th[e]), dl), &tsn[k][e], &tcs[k][e]);
      }
      const char* src = reinterpret_cast<const char*>(p.kr.ptr) +
                        2 * ((long long)b * p.kr.sb + (long long)hk * p.kr.sh + (long long)cv * 8);
      const int col_c = DC + cv * 8, col_s = DC + DR + cv * 8;
      const uint32_t off_c = (uint32_t)((col_c / 64) * C::K_CHUNK_BYTES), off_s = (uint32_t)((col_s / 64) * C::K_CHUNK_BYTES);
      const int slot_c = (col_c % 64) / 8, slot_s = (col_s % 64) / 8;
      const int rbase = (int)rank * HALF_N;   // this CTA's keys inside a tile
      uint4 nxt[PASSES];
#pragma unroll
      for (int k = 0; k < PASSES; ++k) {
        const int grow = jb * BLOCK_N + rbase + r_in + k * RPP;
        nxt[k] = grow < p.Sk ? ldg_nc_v4(src + 2 * (long long)grow * p.kr.ss) : make_uint4(0, 0, 0, 0);
      }
      const uint32_t kfull = lbar(BAR_KFULL);
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int s = ks(j);
        uint4 cur[PASSES];
#pragma unroll
        for (int k = 0; k < PASSES; ++k) cur[k] = nxt[k];
        if (j + 1 < n_tiles) {
#pragma unroll
          for (int k = 0; k < PASSES; ++k) {
            const int grow = (jb + j + 1) * BLOCK_N + rbase + r_in + k * RPP;
            nxt[k] = grow < p.Sk ? ldg_nc_v4(src + 2 * (long long)grow * p.kr.ss) : make_uint4(0, 0, 0, 0);
          }
        }
        float cb[8], sb[8];
        const float pos0 = (float)(p.k_pos0 + (jb + j) * BLOCK_N + rbase);
#pragma unroll
        for (int e = 0; e < 8; ++e) sincos_reduced(__fmul_rn(pos0, th[e]), &sb[e], &cb[e]);
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), kph(j) ^ 1u));
        if (!ok) { fail(ST_WAIT_KEMPTY); break; }
        const uint32_t kb = k_smem + s * C::K_STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < PASSES; ++k) {
          const int r = r_in + k * RPP;
          const uint32_t w[4] = {cur[k].x, cur[k].y, cur[k].z, cur[k].w};
          float oc[8], os[8];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            // two columns at a time with the packed fp32x2 FMA / MUL / ADD
            const float2 x = make_float2(bf16_lo(w[e >> 1]), bf16_hi(w[e >> 1]));
            const float2 ex = __fmul2_rn(make_float2(-fabsf(x.x), -fabsf(x.y)), make_float2(1.4426950408889634f, 1.4426950408889634f));
            const float2 on = __fadd2_rn(make_float2(ex2_approx(ex.x), ex2_approx(ex.y)), make_float2(1.0f, 1.0f));
            const float2 mu = __ffma2_rn(make_float2(lg2_approx(on.x), lg2_approx(on.y)),
                                         make_float2(0.6931471805599453f, 0.6931471805599453f),
                                         make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f)));
            const float2 mc = __fmul2_rn(mu, make_float2(cb[e], cb[e + 1]));
            const float2 ms = __fmul2_rn(mu, make_float2(sb[e], sb[e + 1]));
            const float2 tc2 = make_float2(tcs[k][e], tcs[k][e + 1]), ts2 = make_float2(tsn[k][e], tsn[k][e + 1]);
            // cos(a + b) = ca cb - sa sb ; sin(a + b) = sa cb + ca sb
            const float2 c2v = __ffma2_rn(mc, tc2, __fmul2_rn(make_float2(-ms.x, -ms.y), ts2));
            const float2 s2v = __ffma2_rn(ms, tc2, __fmul2_rn(mc, ts2));
            oc[e] = c2v.x; oc[e + 1] = c2v.y;
            os[e] = s2v.x; os[e + 1] = s2v.y;
          }
          sts_v4(kb + off_c + swz(r, slot_c), make_uint4(pack_bf16x2(oc[0], oc[1]), pack_bf16x2(oc[2], oc[3]),
                                                         pack_bf16x2(oc[4], oc[5]), pack_bf16x2(oc[6], oc[7])));
          sts_v4(kb + off_s + swz(r, slot_s), make_uint4(pack_bf16x2(os[0], os[1]), pack_bf16x2(os[2], os[3]),
                                                         pack_bf16x2(os[4], os[5]), pack_bf16x2(os[6], os[7])));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) PE_TC2_KFULL_ARRIVE(kfull + 8u * (uint32_t)s);
      }
    } else if constexpr (MODE == MODE_XFORM) {
      // raw rows and table entries of the next tile are requested before the wait for its stage
      XformRegs<DC> xr;
      const int rbase = (int)rank * HALF_N;
      XformCursor<DC> cur;
      xform_cursor_init<DC>(p, cur, p.k, b, hk, jb * BLOCK_N + rbase, p.k_pos0 + jb * BLOCK_N + rbase, BLOCK_N, tg);
      if (n_tiles > 0) xform_load_next<DC>(p, xr, cur, p.Sk, BLOCK_N);
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int s = ks(j);
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), kph(j) ^ 1u));
        if (!ok) { fail(ST_WAIT_KEMPTY); break; }
        xform_finish<DC>(p, xr, k_smem + s * C::K_STAGE_BYTES, C::K_CHUNK_BYTES, (jb + j) * BLOCK_N + rbase, p.Sk, tg);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) PE_TC2_KFULL_ARRIVE(lbar(BAR_KFULL + s));
        if (j + 1 < n_tiles) xform_load_next<DC>(p, xr, cur, p.Sk, BLOCK_N);
      }
    }
  }
  }  // register-budget branch

  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
  }
  // neither CTA may release shared memory or TMEM while the other one's MMAs, copies or
  // barrier arrivals can still touch them
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// Combine the two parts of every split block: out = sum_p w_p O_p with w_p = exp(lse_p - lse),
// lse = log(sum_p exp(lse_p)).  One warp per row (8 rows per CTA), four output columns per lane.
constexpr int MERGE_ROWS = 8;
__global__ void __launch_bounds__(32 * MERGE_ROWS) pair_merge_kernel(const KParams p, const int n_top, const float* const ws) {
  const int n_sblk = (p.Sq + PAIR_ROWS - 1) / PAIR_ROWS;
  const int item = blockIdx.y, r = blockIdx.x * MERGE_ROWS + (threadIdx.x >> 5), c = (threadIdx.x & 31) * 4;
  const int bh = item / n_top, sblk = n_sblk - 1 - item % n_top;
  const int row = sblk * PAIR_ROWS + r;
  if (row >= p.Sq) return;
  const int h = bh % p.H, b = bh / p.H;
  const float* base = ws + (size_t)item * SPLIT_ITEM_FLOATS;
  const float l0 = base[2 * PAIR_ROWS * DV + r], l1 = base[2 * PAIR_ROWS * DV + PAIR_ROWS + r];
  const float lm = fmaxf(l0, l1);
  const float e0 = lm == -INFINITY ? 0.f : expf(l0 - lm), e1 = lm == -INFINITY ? 0.f : expf(l1 - lm);
  const float inv = (e0 + e1) > 0.f ? 1.0f / (e0 + e1) : 0.f;
  const float w0 = e0 * inv, w1 = e1 * inv;
  const float4 a = *reinterpret_cast<const float4*>(base + (size_t)r * DV + c);
  const float4 d = *reinterpret_cast<const float4*>(base + (size_t)(PAIR_ROWS + r) * DV + c);
  uint2 o;
  o.x = pack_bf16x2(a.x * w0 + d.x * w1, a.y * w0 + d.y * w1);
  o.y = pack_bf16x2(a.z * w0 + d.z * w1, a.w * w0 + d.w * w1);
  char* dst = reinterpret_cast<char*>(const_cast<void*>(p.out.ptr)) +
              2 * ((long long)b * p.out.sb + (long long)h * p.out.sh + (long long)row * p.out.ss + c);
  *reinterpret_cast<uint2*>(dst) = o;
  if (p.lse != nullptr && c == 0) p.lse[((long long)b * p.H + h) * p.Sq + row] = lm + logf(e0 + e1);
}

// Key tiles the greedy hand-out of the work items (longest first, as the kernel orders them) takes
// on ``pair_slots`` CTA-pair slots when the ``n_top`` longest blocks are cut in two; every item
// also pays ``fixed`` tiles' worth of prologue and epilogue.
double split_makespan(const KParams& p, int n_top, int pair_slots, double fixed) {
  const int n_sblk = (p.Sq + PAIR_ROWS - 1) / PAIR_ROWS;
  const long long n_bh = (long long)p.B * p.H;
  std::priority_queue<double, std::vector<double>, std::greater<double>> free_at;
  for (int i = 0; i < pair_slots; ++i) free_at.push(0.0);
  double end = 0.0;
  int ia = 0, ib = n_sblk - n_top - 1;
  while (ia < 2 * n_top || ib >= 0) {
    int size_a = -1, size_b = -1;
    if (ia < 2 * n_top) {
      const int t = block_tiles(n_sblk - 1 - (ia >> 1), p.Sk, p.causal_off);
      size_a = (ia & 1) ? t - t / 2 : t / 2;
    }
    if (ib >= 0) size_b = block_tiles(ib, p.Sk, p.causal_off);
    const bool take_a = size_a >= size_b;
    const int size = take_a ? size_a : size_b;
    if (take_a) ++ia; else --ib;
    for (long long k = 0; k < n_bh; ++k) {
      const double t = free_at.top() + size + fixed;
      free_at.pop();
      free_at.push(t);
      if (t > end) end = t;
    }
  }
  return end;
}

// How many of the longest blocks of every (batch, head) to cut in two.  A launch with many
// blocks per pair slot balances by itself; for one with fewer than three per slot the hand-out
// is simulated for every count and the best one is taken if it beats the unsplit launch by
// 15 % or more.  Smaller predicted gains do not materialise: the configuration-4 problem on
// two heads x two batches (128 blocks for 74 slots) was predicted 6 % faster with six blocks
// split and measured 3 % slower -- the merge pass and the partial results cost time, and an
// unsplit launch runs its long tail at a higher clock because most SMs are idle by then.
// Plans are cached.
int plan_split(const KParams& p, int pair_slots) {
  const int n_sblk = (p.Sq + PAIR_ROWS - 1) / PAIR_ROWS;
  const long long n_bh = (long long)p.B * p.H;
  if (n_sblk < 4 || n_bh * n_sblk >= 3ll * pair_slots) return 0;
  static std::mutex mu;
  static std::map<std::array<long long, 5>, int> cache;
  const std::array<long long, 5> key = {p.Sq, p.Sk, p.causal_off, n_bh, pair_slots};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  const double base = split_makespan(p, 0, pair_slots, 2.0);
  double best = base;
  int best_n = 0;
  for (int n = 1; n < n_sblk; ++n) {
    if (block_tiles(n_sblk - n, p.Sk, p.causal_off) < 8) break;   // a part keeps a few tiles of its own
    const double t = split_makespan(p, n, pair_slots, 2.0);
    if (t < best) { best = t; best_n = n; }
  }
  if (best > 0.85 * base) best_n = 0;
  if (cache.size() > 256) cache.clear();
  cache[key] = best_n;
  return best_n;
}

int pair_slots_of_device() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms / 2;
}

template <int DC, int DR, int MODE, bool ALIBI>
int launch_instance2(const KParams& p, cudaStream_t stream) {
  using C = Cfg2<DC, DR>;
  auto kern = pe_attn_tc2_kernel<DC, DR, MODE, ALIBI>;
  static PerDeviceOnce configured;
  int cfg_dev;
  if (configured.pending(&cfg_dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(%d bytes) failed: %s", C::SMEM_BYTES, cudaGetErrorString(e));
      return PE_ATTN_ERR_LAUNCH;
    }
    configured.mark(cfg_dev);
  }
  CUtensorMap tmQ, tmK, tmV;
  memset(&tmQ, 0, sizeof(tmQ));
  memset(&tmK, 0, sizeof(tmK));
  if (!encode_map(&tmV, p.v, DV, p.Sk, p.Hkv, p.B, BLOCK_N)) {
    set_error("cuTensorMapEncodeTiled failed for v");
    return PE_ATTN_ERR_LAUNCH;
  }
  if constexpr (MODE == MODE_PLAIN || (MODE == MODE_POPE && DC > 0)) {
    if (!encode_map(&tmQ, p.q, DC, p.Sq, p.H, p.B, BLOCK_M) || !encode_map(&tmK, p.k, DC, p.Sk, p.Hkv, p.B, HALF_N)) {
      set_error("cuTensorMapEncodeTiled failed for q / k");
      return PE_ATTN_ERR_LAUNCH;
    }
  }
  const int n_sblk = (p.Sq + PAIR_ROWS - 1) / PAIR_ROWS;
  int n_top = plan_split(p, pair_slots_of_device());
  if ((size_t)n_top * p.B * p.H * SPLIT_ITEM_FLOATS * sizeof(float) > p.workspace_bytes || p.workspace == nullptr) n_top = 0;
  const long long kv_bytes_per_head = 2ll * p.Sk * (DC + DR + DV);
  const int bh_group = balanced_bh_group((long long)p.B * p.H, kv_bytes_per_head, p.groups);
  dim3 grid((unsigned)(2ll * (n_sblk + n_top) * p.H * p.B)), block(NTHREADS);
  kern<<<grid, block, C::SMEM_BYTES, stream>>>(p, bh_group, n_top, p.workspace, tmQ, tmK, tmV);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && n_top > 0) {
    pair_merge_kernel<<<dim3(PAIR_ROWS / MERGE_ROWS, (unsigned)(n_top * p.H * p.B)), 32 * MERGE_ROWS, 0, stream>>>(
        p, n_top, p.workspace);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_error("tcgen05 CTA-pair kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

template <int DC, int DR, int MODE>
int launch_alibi2(const KParams& p, cudaStream_t stream) {
  if (p.variant == PE_ATTN_ALIBI) return launch_instance2<DC, DR, MODE, true>(p, stream);
  return launch_instance2<DC, DR, MODE, false>(p, stream);
}

}  // namespace

// The CTA-pair kernel covers d_v = 128 (each CTA then owns one 64-column, 128-byte chunk of V).
bool tc2_supports(const KParams& p) {
  if (p.d_v != 128) return false;
  if (p.variant == PE_ATTN_POPE)
    return (p.d_c == 128 && (p.d_r == 64 || p.d_r == 32)) || (p.d_c == 0 && p.d_r == 64);
  return p.d_c == 128;
}

// Workspace that lets the pair kernel split the longest blocks of a few-wave launch (0: no split planned).
size_t tc2_workspace_bytes(const KParams& p) {
  return (size_t)plan_split(p, pair_slots_of_device()) * p.B * p.H * SPLIT_ITEM_FLOATS * sizeof(float);
}

int launch_tc2(const KParams& p, cudaStream_t stream) {
  if (p.variant == PE_ATTN_POPE) {
    if (p.d_c == 128 && p.d_r == 64) return launch_instance2<128, 64, MODE_POPE, false>(p, stream);
    if (p.d_c == 128 && p.d_r == 32) return launch_instance2<128, 32, MODE_POPE, false>(p, stream);
    return launch_instance2<0, 64, MODE_POPE, false>(p, stream);
  }
  const bool xform = p.variant == PE_ATTN_ROTARY || (p.flags & PE_ATTN_QK_NORM);
  return xform ? launch_alibi2<128, 0, MODE_XFORM>(p, stream) : launch_alibi2<128, 0, MODE_PLAIN>(p, stream);
}

}  // namespace pe_attn
