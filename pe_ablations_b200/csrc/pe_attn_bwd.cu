// Causal attention BACKWARD on the 5th-generation tensor cores (sm_100a): gradients of
//   out = softmax_causal(scale * Q K^T + bias) V
// with respect to Q, K and V, for bf16 operands that already carry their positional transform
// (the [q_c | mu cos | mu sin] rows of the PoPE family, rotated rows of the rotary family, plain
// rows otherwise; bias = ALiBi's -slope * distance or nothing).  It is the part of the
// reference's training step that autograd derives from F.scaled_dot_product_attention
// (src/model/attention.py:91-96, src/model/fpope_attention.py:171-177, src/model/alibi.py:145-160);
// the transform's own backward stays with the caller.
//
// One CTA owns 128 keys of one key/value head and walks over the query blocks that can see
// them (all query heads of the GQA group in turn).  Scores are formed TRANSPOSED, keys on the
// TMEM lanes and queries along the columns, so that the two probability-shaped operands of
// the key-side products are already where a tensor-core A operand may live:
//     S^T  = K Q^T          dP^T = V dO^T                       (SS MMAs, fp32 in TMEM)
//     P^T  = exp(scale S^T + bias - lse),  dS^T = scale * P^T o (dP^T - D)
//                           (8 warps: thread = key, half of the query columns each; both
//                            written back over S^T / dP^T as packed bf16, dS^T also to
//                            shared memory)
//     dV  += P^T dO         dK += dS^T Q                        (TS MMAs, A from TMEM)
//     dQ   = dS K                                               (SS MMA, A = the shared-memory
//                                                                copy of dS^T read MN-major)
// Q, K, dO and V tiles are loaded once by TMA in the 128-byte-swizzled layout and the same
// bytes serve as K-major operands (S^T, dP^T) and as MN-major ones (dV, dK, dQ); nothing is
// transposed in memory.  Q / dO tiles are double-buffered, so the loads of the next query
// block overlap this block's math.  dK and dV stay in TMEM for the whole CTA.  dQ of each
// block is drained by four warps of their own: TMEM -> registers -> a staging tile in shared
// memory (the dS^T buffer, idle at that time) -> TMA reduction (fp32 add) into the global
// accumulation buffer; the order in which key blocks add is not fixed, so dQ bits vary from
// run to run.  D = rowsum(dO o O) comes from a small kernel that runs first.
//
// TMEM columns: S^T / P^T / dQ [0,128)   dP^T / dS^T [128,256)   dV [256,256+DV)
//               dK [256+DV, 256+DV+DQK).   P^T of query columns [64h, 64h+64) sits in columns
// [64h, 64h+32) (inside the half of S^T its own warps read), dS^T likewise at 128 + ....
// dQ overwrites the S^T / P^T columns: it is issued after the dV product that reads P^T, and
// MMAs of one thread execute in issue order.
// Warps 0-7: softmax-gradient math and epilogues; warps 8-11: dQ drain; warp 12: TMA;
// warp 13: TMEM + MMA issue (14, 15 idle: register budgets are set per warpgroup).
// Every wait is bounded and reports through the device status word.

#include <cuda.h>
#include <string.h>

#include "pe_attn_tc_common.cuh"

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

constexpr int BM = 128;          // query rows per block
constexpr int BN = 128;          // keys per CTA
constexpr int NCOMPUTE = 256;    // 8 warps
constexpr int NDRAIN = 128;      // 4 warps
constexpr int NTHREADS = 512;    // + TMA warp, MMA warp, two idle warps (a full warpgroup for setmaxnreg)
constexpr int CH = 128 * 128;    // bytes of one 128-row x 64-column bf16 chunk
constexpr int TMEM_COLS = 512;
constexpr int TAIL = 2048;       // barriers, TMEM slot, per-block lse / D vectors
constexpr int ST_WAIT_BWD = 1 << 9;

enum : int { BAR_KV = 0, BAR_LDFULL = 1, BAR_LDEMPTY = 3, BAR_S = 5, BAR_P = 6, BAR_DQ = 7, BAR_SFREE = 8, BAR_VEC = 9, BAR_STG = 10, BAR_DRA = 11, BAR_DRB = 12, BAR_PA = 13, NUM_BARS = 16 };   // BAR_PA: three partial hand-offs

template <int DQK, int DV>
struct BCfg {
  static constexpr int NQC = DQK / 64, NVC = DV / 64;
  static constexpr int K_OFF = TAIL;
  static constexpr int V_OFF = K_OFF + NQC * CH;
  static constexpr int Q_OFF = V_OFF + NVC * CH;             // 2 stages
  static constexpr int DO_OFF = Q_OFF + 2 * NQC * CH;        // 2 stages
  static constexpr int DS_OFF = DO_OFF + 2 * NVC * CH;
  // the dQ drain's staging tile: its own 32 KB where shared memory allows (d_v = 64), else the
  // dS^T buffer, which is idle between a block's dQ product and the next block's softmax
  static constexpr bool OWN_STAGING = DS_OFF + 4 * CH + 1024 <= 232448;
  static constexpr int STG_OFF = OWN_STAGING ? DS_OFF + 2 * CH : DS_OFF;
  static constexpr int SMEM_BYTES = STG_OFF + 2 * CH + 1024;  // slack to align the base to 1024
  static_assert(DQK == 64 || DQK == 128, "d_qk must be 64 or 128");
  static_assert(DV == 64 || DV == 128, "d_v must be 64 or 128");
  static_assert(256 + DV + DQK <= TMEM_COLS, "TMEM budget exceeded");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
};

template <int DQK, int DV, bool ALIBI>
__global__ void __launch_bounds__(NTHREADS, 1)
pe_attn_bwd_kernel(const BwdParams p, const int bh_group, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmDQ) {
  using C = BCfg<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 256);
  float* lse_s = reinterpret_cast<float*>(smem + 1024);   // [128] -log2(e) * logsumexp of the query block's rows
  float* dsum_s = reinterpret_cast<float*>(smem + 1536);  // [128] -scale * D of the query block's rows
  auto bar = [&](int idx) -> uint32_t { return smem_base + 8u * (uint32_t)idx; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // 1-D grid: key blocks in ascending order (block 0 sees every query block: longest first)
  // inside groups of ``bh_group`` (batch, K/V head) problems whose Q / dO stay in L2 together
  const int n_kblk = (p.Sk + BN - 1) / BN;
  const int n_bh = p.B * p.Hkv;
  const int per_group = bh_group * n_kblk;
  const int grp = (int)(blockIdx.x / per_group), in_grp = (int)(blockIdx.x % per_group);
  const int g_first = grp * bh_group;
  const int g_size = (n_bh - g_first) < bh_group ? (n_bh - g_first) : bh_group;
  const int bh = g_first + in_grp % g_size;
  const int key0 = (in_grp / g_size) * BN, hk = bh % p.Hkv, b = bh / p.Hkv;
  const int n_qblk = (p.Sq + BM - 1) / BM;
  // query row r sees key s iff s <= r + causal_off: the first block with a row that sees key0
  int first_row = key0 - p.causal_off;
  if (first_row < 0) first_row = 0;
  const int i_first = first_row / BM;
  const int per_head = n_qblk > i_first ? n_qblk - i_first : 0;
  const int n_iter = per_head * p.groups;

  auto fail = [&]() {
    if (p.status != nullptr) atomicOr(p.status, ST_WAIT_BWD);
  };

  if (tid == 0) {
    mbar_init(bar(BAR_KV), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BAR_LDFULL + s), 1);
      mbar_init(bar(BAR_LDEMPTY + s), 1);
    }
    mbar_init(bar(BAR_S), 1);
    mbar_init(bar(BAR_P), NCOMPUTE / 32);
    for (int part = 0; part < 3; ++part) mbar_init(bar(BAR_PA + part), NCOMPUTE / 32);
    mbar_init(bar(BAR_DQ), 1);
    mbar_init(bar(BAR_SFREE), NDRAIN / 32);
    mbar_init(bar(BAR_VEC), NCOMPUTE / 32);
    mbar_init(bar(BAR_STG), 1);
    mbar_init(bar(BAR_DRA), NDRAIN / 32);
    mbar_init(bar(BAR_DRB), 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 13) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t k_smem = smem_base + C::K_OFF, v_smem = smem_base + C::V_OFF, q_smem = smem_base + C::Q_OFF,
                 do_smem = smem_base + C::DO_OFF, ds_smem = smem_base + C::DS_OFF, stg_smem = smem_base + C::STG_OFF;
  constexpr uint32_t Q_STAGE = (uint32_t)(C::NQC * CH), DO_STAGE = (uint32_t)(C::NVC * CH);
  constexpr uint32_t LD_BYTES = Q_STAGE + DO_STAGE;

  // Each role sits inside the branch that sets its register budget:
  // 2 x 128 x 136 (softmax) + 128 x 152 (dQ drain) + 128 x 88 (TMA, MMA) = 64 K registers.
  if (warp >= 12) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (warp == 12) {
    // ===================== TMA producer =====================
    if (n_iter > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        mbar_arrive_expect_tx(bar(BAR_KV), LD_BYTES);
#pragma unroll
        for (int c = 0; c < C::NQC; ++c) tma_load_4d(k_smem + c * CH, &tmK, bar(BAR_KV), c * 64, key0, hk, b);
#pragma unroll
        for (int c = 0; c < C::NVC; ++c) tma_load_4d(v_smem + c * CH, &tmV, bar(BAR_KV), c * 64, key0, hk, b);
      }
      __syncwarp();
#pragma unroll 1
      for (int it = 0; it < n_iter; ++it) {
        const int h = hk * p.groups + it / per_head, i = i_first + it % per_head;
        const int s = it & 1;
        // the products of the block that used this stage two iterations ago have finished
        if (it >= 2 && !__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_LDEMPTY + s), (uint32_t)(((it >> 1) - 1) & 1)))) {
          fail();
          break;
        }
        if (elect_one()) {
          mbar_arrive_expect_tx(bar(BAR_LDFULL + s), LD_BYTES);
#pragma unroll
          for (int c = 0; c < C::NQC; ++c)
            tma_load_4d(q_smem + s * Q_STAGE + c * CH, &tmQ, bar(BAR_LDFULL + s), c * 64, i * BM, h, b);
#pragma unroll
          for (int c = 0; c < C::NVC; ++c)
            tma_load_4d(do_smem + s * DO_STAGE + c * CH, &tmDO, bar(BAR_LDFULL + s), c * 64, i * BM, h, b);
        }
        __syncwarp();
      }
    }
  } else if (warp == 13) {
    // ===================== MMA issuer =====================
    constexpr uint32_t IDESC_ST = make_idesc_bf16_mn(BN, BM, false, false);   // S^T, dP^T: both K-major
    constexpr uint32_t IDESC_DV = make_idesc_bf16_mn(BN, DV, false, true);    // P^T (TMEM) x dO (MN-major)
    constexpr uint32_t IDESC_DK = make_idesc_bf16_mn(BN, DQK, false, true);   // dS^T (TMEM) x Q (MN-major)
    constexpr uint32_t IDESC_DQ = make_idesc_bf16_mn(BM, DQK, true, true);    // dS (MN-major) x K (MN-major)
    // K-major view: 8-row groups 1024 bytes apart, 16 elements (32 bytes) per K step
    const uint64_t k_k = make_smem_desc(k_smem, 16, 1024), v_k = make_smem_desc(v_smem, 16, 1024);
    const uint64_t q_k0 = make_smem_desc(q_smem, 16, 1024), do_k0 = make_smem_desc(do_smem, 16, 1024);
    // MN-major view of the same bytes: 64-wide MN chunks CH bytes apart, 16 K rows = 2048 bytes
    const uint64_t q_mn0 = make_smem_desc(q_smem, CH, 1024), do_mn0 = make_smem_desc(do_smem, CH, 1024);
    const uint64_t ds_mn = make_smem_desc(ds_smem, CH, 1024), k_mn = make_smem_desc(k_smem, CH, 1024);
    const uint32_t t_s = tmem_base, t_dp = tmem_base + 128u, t_dv = tmem_base + 256u,
                   t_dk = tmem_base + 256u + (uint32_t)DV;
    bool ok = n_iter == 0 || __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_KV), 0));
    if (!ok) fail();
    // dP^T = V dO^T of the block in stage ``st`` (the dP^T / dS^T columns).  At d_v = 128 (eight
    // MMAs) the next block's is issued early, see the end of the loop: 820 -> 868 TFLOP/s at
    // S 16384; at d_v = 64 it measured 0 to -4 %.
    constexpr bool EARLY_DP = DV == 128;
    auto issue_dp = [&](int st) {
      if (elect_one()) {
        const uint64_t do_k = advance_smem_desc(do_k0, (uint32_t)st * DO_STAGE);
#pragma unroll
        for (int c = 0; c < C::NVC; ++c)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_ss(t_dp, advance_smem_desc(v_k, (uint32_t)(c * CH + k4 * 32)),
                   advance_smem_desc(do_k, (uint32_t)(c * CH + k4 * 32)), IDESC_ST, (c > 0 || k4 > 0) ? 1u : 0u);
      }
      __syncwarp();
    };
#pragma unroll 1
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t ph = (uint32_t)(it & 1);
      const int s = it & 1;
      // with EARLY_DP later blocks' tiles were checked, and their dP^T issued, at the end of the
      // block before
      if (it == 0 || !EARLY_DP) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_LDFULL + s), (uint32_t)((it >> 1) & 1)));
        if (!ok) { fail(); break; }
        tc_fence_after_sync();
        issue_dp(s);
      }
      // the S^T columns double as dQ: the previous block's dQ has been read out
      if (it > 0) ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_SFREE), ph ^ 1u));
      if (!ok) { fail(); break; }
      tc_fence_after_sync();
      const uint64_t q_k = advance_smem_desc(q_k0, (uint32_t)s * Q_STAGE);
      const uint64_t q_mn = advance_smem_desc(q_mn0, (uint32_t)s * Q_STAGE), do_mn = advance_smem_desc(do_mn0, (uint32_t)s * DO_STAGE);
      if (elect_one()) {
#pragma unroll
        for (int c = 0; c < C::NQC; ++c)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_ss(t_s, advance_smem_desc(k_k, (uint32_t)(c * CH + k4 * 32)),
                   advance_smem_desc(q_k, (uint32_t)(c * CH + k4 * 32)), IDESC_ST, (c > 0 || k4 > 0) ? 1u : 0u);
        tc_commit(bar(BAR_S));   // S^T, and dP^T issued before it
      }
      __syncwarp();
      // P^T and dS^T arrive in two parts -- the first 32 query columns of each half of the block,
      // then the rest: the key-side products of the first part run under the softmax of the second
      auto issue_dv_dk = [&](int kk) {   // 16 query columns per step; packed bf16: 8 TMEM columns
        const uint32_t acc = (it > 0 || kk > 0) ? 1u : 0u;
        const uint32_t a_off = (uint32_t)((kk >> 2) * 64 + (kk & 3) * 8);
        mma_ts(t_dv, t_s + a_off, advance_smem_desc(do_mn, (uint32_t)(kk * 2048)), IDESC_DV, acc);
        mma_ts(t_dk, t_dp + a_off, advance_smem_desc(q_mn, (uint32_t)(kk * 2048)), IDESC_DK, acc);
      };
#pragma unroll
      for (int part = 0; part < 3 && ok; ++part) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PA + part), ph));
        if (!ok) break;
        tc_fence_after_sync();
        if (elect_one()) {
          issue_dv_dk(part);
          issue_dv_dk(4 + part);
        }
        __syncwarp();
      }
      if (!ok) { fail(); break; }
      ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_P), ph));
      if (!ok) { fail(); break; }
      tc_fence_after_sync();
      if (elect_one()) {
        issue_dv_dk(3);
        issue_dv_dk(7);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)     // 16 keys per step
          mma_ss(t_s, advance_smem_desc(ds_mn, (uint32_t)(kk * 2048)), advance_smem_desc(k_mn, (uint32_t)(kk * 2048)),
                 IDESC_DQ, kk > 0 ? 1u : 0u);
        tc_commit(bar(BAR_DQ));
        tc_commit(bar(BAR_LDEMPTY + s));
      }
      __syncwarp();
      // dP^T of the next block now, behind this block's dK product (the last reader of the dS^T
      // columns; MMAs of one thread execute in issue order): it runs while the drain warps read dQ
      // out of the S^T columns, which only the next block's S^T product has to wait for
      if (EARLY_DP && it + 1 < n_iter) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_LDFULL + (s ^ 1)), (uint32_t)(((it + 1) >> 1) & 1)));
        if (!ok) { fail(); break; }
        tc_fence_after_sync();
        issue_dp(s ^ 1);
      }
    }
  }
  } else if (warp >= 8) {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
  {
    // ===================== dQ drain (lanes = query rows) =====================
    // TMEM -> registers -> a staging tile in shared memory -> TMA reduction (fp32 add) into the
    // global accumulation buffer.  Its own warps, so that the drain of block i overlaps the
    // S^T product and the softmax of block i + 1.  Without a staging tile of its own the dS^T
    // buffer serves, idle between this block's dQ product and the next block's softmax stores.
    const int r = tid & 127;
    const bool leader = tid == NCOMPUTE;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    constexpr int HALVES = DQK / 64;       // 64 columns (two 32-column boxes, 32 KB) per pass
    bool dok = true;
    if (leader) tma_prefetch_desc(&tmDQ);
#pragma unroll 1
    for (int it = 0; it < n_iter && dok; ++it) {
      const int h = hk * p.groups + it / per_head, row0 = (i_first + it % per_head) * BM;
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_DQ), (uint32_t)(it & 1)))) { fail(); break; }
      tc_fence_after_sync();
      uint32_t qr[DQK];
#pragma unroll
      for (int cb = 0; cb < DQK / 32; ++cb)
        tmem_ld32(tmem_base + lane_sel + (uint32_t)(cb * 32), *reinterpret_cast<uint32_t(*)[32]>(&qr[cb * 32]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_SFREE));   // the S^T / dQ columns may be overwritten
#pragma unroll
      for (int half = 0; half < HALVES; ++half) {
        const uint32_t ph2 = (uint32_t)((it * HALVES + half) & 1);
#pragma unroll
        for (int bx = 0; bx < 2; ++bx)
#pragma unroll
          for (int sl = 0; sl < 8; ++sl) {
            const int c = half * 64 + bx * 32 + sl * 4;
            sts_v4(stg_smem + (uint32_t)(bx * CH) + swz(r, sl), make_uint4(qr[c], qr[c + 1], qr[c + 2], qr[c + 3]));
          }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_DRA));
        if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_DRA), ph2))) { fail(); dok = false; break; }
        if (leader) {
          tma_reduce_add_4d(&tmDQ, stg_smem, half * 64, row0, h, b);
          tma_reduce_add_4d(&tmDQ, stg_smem + CH, half * 64 + 32, row0, h, b);
          bulk_commit_group();
          bulk_wait_read_all();                       // the tile has been read: it may be rewritten
          mbar_arrive(bar(BAR_DRB));
        }
        if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_DRB), ph2))) { fail(); dok = false; break; }
      }
      if (dok && leader) mbar_arrive(bar(BAR_STG));   // the softmax warps may write dS^T again
    }
    if (leader) bulk_wait_all();                      // every reduction has been performed
  }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 136;");
  {
    // ===================== softmax gradient + epilogues =====================
    // thread = (key lane, half of the query columns)
    const int r = tid & 127, hh = tid >> 7;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    const int key = key0 + r;
    bool ok = true;
    // each thread fetches one entry of the block's vectors, one block ahead: -log2(e) * lse
    // (first half of the threads) or -scale * D (second half), the addends of the two FMAs
    auto fetch_vec = [&](int it) -> float {
      const int h = hk * p.groups + it / per_head, row = (i_first + it % per_head) * BM + r;
      if (row >= p.Sq) return 0.f;
      const long long idx = ((long long)b * p.H + h) * p.Sq + row;
      return hh == 0 ? -p.lse[idx] * 1.4426950408889634f : -p.dvec[idx] * p.scale;
    };
    float vec_next = n_iter > 0 ? fetch_vec(0) : 0.f;
#pragma unroll 1
    for (int it = 0; it < n_iter; ++it) {
      const uint32_t ph = (uint32_t)(it & 1);
      const int h = hk * p.groups + it / per_head, i = i_first + it % per_head;
      const int row0 = i * BM;
      // the vectors of the previous block are dead once all eight warps have handed over its P
      if (it > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_P), ph ^ 1u));
        if (!ok) { fail(); break; }
      }
      (hh == 0 ? lse_s : dsum_s)[r] = vec_next;
      // rendezvous of the eight warps on a barrier with a bounded wait (a plain bar.sync would
      // hang the others if one warp had left after an expired wait)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_VEC));
      ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_VEC), ph));
      if (!ok) { fail(); break; }
      if (it + 1 < n_iter) vec_next = fetch_vec(it + 1);
      float slope2 = 0.f;
      if constexpr (ALIBI) slope2 = p.slopes[h] * 1.4426950408889634f;
      const bool need_mask = (key0 + BN - 1 > row0 + p.causal_off) || (key0 + BN > p.Sk) || (row0 + BM > p.Sq);
      // query column c of this block sees this thread's key iff c >= c_first (causality; no
      // column if the key is past Sk) and c < c_end (rows past Sq)
      const int c_first = key < p.Sk ? key - row0 - p.causal_off : (1 << 30);
      const int c_end = p.Sq - row0;

      ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_S), ph));
      if (!ok) { fail(); break; }
      tc_fence_after_sync();
      // 16 query columns per round, the next round's TMEM loads in flight during the math
      uint32_t sr[2][16], dr[2][16], pp[8], dall[32];
      const uint32_t s_col = tmem_base + lane_sel + (uint32_t)(hh * 64), d_col = s_col + 128u;
      tmem_ld16(s_col, sr[0]);
      tmem_ld16(d_col, dr[0]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        tmem_wait_ld();
        if (j < 3) {
          tmem_ld16(s_col + (uint32_t)((j + 1) * 16), sr[(j + 1) & 1]);
          tmem_ld16(d_col + (uint32_t)((j + 1) * 16), dr[(j + 1) & 1]);
        }
        const int col0 = hh * 64 + j * 16;
#pragma unroll
        for (int c = 0; c < 16; c += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse_s + col0 + c);
          const float4 d4 = *reinterpret_cast<const float4*>(dsum_s + col0 + c);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dsv[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], gv[4];
          // packed fp32x2 FMA / MUL (half the issue slots of scalar code); exponentials on the SFU
          const float2 cc = make_float2(c2, c2), sc = make_float2(p.scale, p.scale);
#pragma unroll
          for (int e = 0; e < 4; e += 2) {
            const int qc = col0 + c + e;
            float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[j & 1][c + e]), __uint_as_float(sr[j & 1][c + e + 1])),
                                  cc, make_float2(lv[e], lv[e + 1]));
            if constexpr (ALIBI) {
              // -slope * (query position - key position), in log2 units
              x.x = fmaf((float)(key - row0 - p.causal_off - qc), slope2, x.x);
              x.y = fmaf((float)(key - row0 - p.causal_off - qc - 1), slope2, x.y);
            }
            float2 pe = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            if (need_mask) {
              if (qc < c_first || qc >= c_end) pe.x = 0.f;
              if (qc + 1 < c_first || qc + 1 >= c_end) pe.y = 0.f;
            }
            const float2 t = __ffma2_rn(make_float2(__uint_as_float(dr[j & 1][c + e]), __uint_as_float(dr[j & 1][c + e + 1])),
                                        sc, make_float2(dsv[e], dsv[e + 1]));
            const float2 gg = __fmul2_rn(pe, t);
            pv[e] = pe.x; pv[e + 1] = pe.y;
            gv[e] = gg.x; gv[e + 1] = gg.y;
          }
          const int o = c >> 1;
          pp[o] = pack_bf16x2(pv[0], pv[1]);
          pp[o + 1] = pack_bf16x2(pv[2], pv[3]);
          dall[j * 8 + (c >> 1)] = pack_bf16x2(gv[0], gv[1]);
          dall[j * 8 + (c >> 1) + 1] = pack_bf16x2(gv[2], gv[3]);
        }
        // packed bf16 back over columns this thread has already read; the round's 16 query
        // columns are one K step of the key-side products: hand them over
        tmem_st8(s_col + (uint32_t)(j * 8), pp);
        tmem_st8(d_col + (uint32_t)(j * 8), *reinterpret_cast<uint32_t(*)[8]>(&dall[j * 8]));
        if (j < 3) {
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(BAR_PA + j));
        }
      }
      // dS^T row ``r`` to shared memory (64 query columns = the eight 16-byte slots of chunk hh),
      // once the drain warps have let go of the buffer they use as their staging tile
      if (it > 0 && !C::OWN_STAGING) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_STG), ph ^ 1u));
        if (!ok) { fail(); break; }
      }
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
        sts_v4(ds_smem + (uint32_t)(hh * CH) + swz(r, sl),
               make_uint4(dall[sl * 4], dall[sl * 4 + 1], dall[sl * 4 + 2], dall[sl * 4 + 3]));
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_P));
    }
    // every MMA has completed once the last block's dQ product has
    if (ok && n_iter > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_DQ), (uint32_t)((n_iter - 1) & 1)));
      if (!ok) fail();
      tc_fence_after_sync();
    }

    // ---- dV and dK of this CTA's keys: thread = (key row, half of the columns).  The last
    // BAR_DQ wait above covered every MMA; with no visible query block the gradients are zero.
    if (ok) {
      const bool key_live = key < p.Sk;
      char* dv_dst = reinterpret_cast<char*>(const_cast<void*>(p.dv.ptr)) +
                     2 * ((long long)b * p.dv.sb + (long long)hk * p.dv.sh + (long long)key * p.dv.ss);
      char* dk_dst = reinterpret_cast<char*>(const_cast<void*>(p.dk.ptr)) +
                     2 * ((long long)b * p.dk.sb + (long long)hk * p.dk.sh + (long long)key * p.dk.ss);
      // tcgen05.ld is warp-collective: every lane loads, live keys store
      auto flush = [&](char* dst, uint32_t taddr, int ncol) {
        const int c_begin = hh * (ncol / 2), c_end = c_begin + ncol / 2;
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
          uint32_t t[32];
          if (n_iter > 0) {
            tmem_ld32(taddr + (uint32_t)c0, t);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) t[c] = 0u;
          }
          if (key_live) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]), __uint_as_float(t[v * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]), __uint_as_float(t[v * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]), __uint_as_float(t[v * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]), __uint_as_float(t[v * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + (c0 + v * 8) * 2) = o;
            }
          }
        }
      };
      flush(dv_dst, tmem_base + lane_sel + 256u, DV);
      flush(dk_dst, tmem_base + lane_sel + 256u + (uint32_t)DV, DQK);
    }
  }
  }  // register-budget branch

  // after a failed wait give copies in flight time to land before shared memory and TMEM go
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 13) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// D[b, h, row] = sum_d dO[b, row, h, d] * O[b, row, h, d]  (fp32).  Memory-bound: 16 bytes per
// thread and tensor, the DV / 8 threads of a row are neighbours in a warp and add up with
// shuffles; rows ordered (batch, position, head) like the tensors.
template <int DV>
__global__ void __launch_bounds__(256) bwd_dvec_kernel(const BwdParams p) {
  constexpr int VPR = DV / 8;
  const long long n = (long long)p.B * p.Sq * p.H * VPR;
  const long long n_pad = (n + 31) / 32 * 32;   // whole warps stay in the loop (shuffles)
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n_pad; idx += stride) {
    const bool live = idx < n;
    const long long r = (live ? idx : n - 1) / VPR;
    const int cv = (int)(idx % VPR);
    const int h = (int)(r % p.H), row = (int)((r / p.H) % p.Sq), b = (int)(r / ((long long)p.H * p.Sq));
    const __nv_bfloat16* o = reinterpret_cast<const __nv_bfloat16*>(p.out.ptr) + (long long)b * p.out.sb +
                             (long long)h * p.out.sh + (long long)row * p.out.ss + cv * 8;
    const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(p.dout.ptr) + (long long)b * p.dout.sb +
                             (long long)h * p.dout.sh + (long long)row * p.dout.ss + cv * 8;
    const uint4 ov = ldg_nc_v4(o), gv = ldg_nc_v4(g);
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc = fmaf(bf16_lo(ow[e]), bf16_lo(gw[e]), fmaf(bf16_hi(ow[e]), bf16_hi(gw[e]), acc));
#pragma unroll
    for (int d = 1; d < VPR; d <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (live && cv == 0) p.dvec[((long long)b * p.H + h) * p.Sq + row] = acc;
  }
}

template <int DQK, int DV, bool ALIBI>
int launch_bwd_instance(const BwdParams& p, cudaStream_t stream) {
  using C = BCfg<DQK, DV>;
  auto kern = pe_attn_bwd_kernel<DQK, DV, ALIBI>;
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
  CUtensorMap tmQ, tmK, tmV, tmDO, tmDQ;
  if (!encode_map(&tmQ, p.q, DQK, p.Sq, p.H, p.B, BM) || !encode_map(&tmK, p.k, DQK, p.Sk, p.Hkv, p.B, BN) ||
      !encode_map(&tmV, p.v, DV, p.Sk, p.Hkv, p.B, BN) || !encode_map(&tmDO, p.dout, DV, p.Sq, p.H, p.B, BM)) {
    set_error("cuTensorMapEncodeTiled failed for a backward operand");
    return PE_ATTN_ERR_LAUNCH;
  }
  if (!encode_map_f32(&tmDQ, p.dq_accum, DQK, p.Sq, p.H, p.B, BM)) {
    set_error("cuTensorMapEncodeTiled failed for dq_accum");
    return PE_ATTN_ERR_LAUNCH;
  }
  cudaError_t e = cudaMemsetAsync(p.dq_accum, 0, sizeof(float) * (size_t)p.B * p.H * p.Sq * DQK, stream);
  if (e != cudaSuccess) {
    set_error("clearing dq_accum failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  long long dblocks = ((long long)p.B * p.H * p.Sq * (DV / 8) + 255) / 256;
  if (dblocks > 148 * 8) dblocks = 148 * 8;
  bwd_dvec_kernel<DV><<<(unsigned)dblocks, 256, 0, stream>>>(p);
  // a CTA streams the Q and dO rows of its K/V head's query heads; heads per group by what L2 holds
  const int bh_group = balanced_bh_group((long long)p.B * p.Hkv, 2ll * p.Sq * (DQK + DV) * p.groups, 1);
  dim3 grid((unsigned)((long long)((p.Sk + BN - 1) / BN) * p.Hkv * p.B)), block(NTHREADS);
  kern<<<grid, block, C::SMEM_BYTES, stream>>>(p, bh_group, tmQ, tmK, tmV, tmDO, tmDQ);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("backward kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

}  // namespace

bool bwd_supports(int d_qk, int d_v) {
  return (d_qk == 64 && d_v == 64) || (d_qk == 128 && d_v == 64) || (d_qk == 128 && d_v == 128);
}

int launch_bwd(const BwdParams& p, int d_qk, int d_v, int dtype, bool alibi, cudaStream_t stream) {
  // fp32 calls, and head dimensions without a tensor-core instantiation (d_qk = 256 above all),
  // run on the CUDA cores
  if (dtype != PE_ATTN_BF16 || !bwd_supports(d_qk, d_v)) return launch_bwd_simt(p, d_qk, d_v, dtype, alibi, stream);
  if (d_qk == 64 && d_v == 64)
    return alibi ? launch_bwd_instance<64, 64, true>(p, stream) : launch_bwd_instance<64, 64, false>(p, stream);
  if (d_qk == 128 && d_v == 64)
    return alibi ? launch_bwd_instance<128, 64, true>(p, stream) : launch_bwd_instance<128, 64, false>(p, stream);
  return alibi ? launch_bwd_instance<128, 128, true>(p, stream) : launch_bwd_instance<128, 128, false>(p, stream);
}

}  // namespace pe_attn
