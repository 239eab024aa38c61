// Four-query-tile variant of the tcgen05 fused PE-attention forward (bf16, d_v = 64).
//
// At head_dim 64 a 64-key step of one query tile is little work (4 + 4 MMAs, 64 exponentials
// per row) next to the fixed latencies around it (S ready -> softmax -> P ready -> MMA), so the
// two-tile kernel leaves both the tensor pipe and the special-function unit mostly idle.  This
// kernel keeps FOUR independent 128-row query tiles in flight per CTA (768 threads, 1 CTA/SM):
// while one tile waits for a hand-off the other three compute, and every K/V tile that is
// loaded and positionally transformed serves 512 query rows instead of 256.
//
// The four tiles of a CTA all read the same K/V head.  With grouped-query attention they are
// (heads of one group) x (row tiles): 4 heads x 128 rows, 2 heads x 256 rows, or 1 head x 512
// rows, so that tiles of equal row range -- equal causal trip count -- run side by side.
//
//   warp 0        TMA producer: content halves of Q and K (128B-swizzled tiles)
//   warp 1        MMA issuer:   S_i = Q_i K^T (SS, M128 N64), O_i += P_i V (TS, P from TMEM)
//   warp 2        TMEM allocation / release (512 columns)
//   warp 3        TMA producer: V tiles
//   warps 4-19    softmax of query tiles 0..3 (one warpgroup each, one row per thread); each
//                 warpgroup also builds the positional part of its own Q tile once
//   warps 20-23   positional transform of every K tile into the swizzled K-major operand
//
// A second instantiation keeps TWO tiles per CTA and no transform warps (384 threads, half the
// TMEM and shared memory) so that two CTAs share an SM: the same four tiles in flight per SM,
// in units of 256 rows.  It serves the variants without a positional transform (NoPE, plain
// ALiBi) of models without grouped heads, where nothing is gained by sharing a K tile between
// more rows and the finer units balance the causal triangle better.
//
// TMEM map (columns), NT tiles: S_i / P_i at 64 i (P, packed bf16, overwrites the first 32
// columns of its own S tile), O_i at 64 NT + 64 i.  S is single-buffered: QK_i(j+1) is issued right behind
// PV_i(j) on the in-order tensor pipe, which is what frees S_i.
//
// Every mbarrier wait is bounded; on expiry the CTA ORs a code into the caller's status word,
// lets its copies land, frees its TMEM and returns.
#include <cuda.h>

#include "pe_attn_tc_common.cuh"

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

constexpr int BLOCK_M = 128;   // query rows per tile (TMEM lanes)
constexpr int MAX_TILES = 4;   // query tiles per CTA: 4, or 2 in the two-CTAs-per-SM instantiation
constexpr int BLOCK_N = 64;    // keys per tile
constexpr int DV = 64;
constexpr int KV_STAGES = 3;
constexpr int threads_for(int nt) { return 128 + nt * 128 + (nt == 4 ? 128 : 0); }
constexpr int TAIL_BYTES = 1024;  // barriers, TMEM base, frequency / phase-bias vectors

enum : int {
  BAR_QFULL = 0, BAR_KFULL = 4, BAR_KEMPTY = 7, BAR_VFULL = 10, BAR_VEMPTY = 13, BAR_SFULL = 16, BAR_PREADY = 20,
  BAR_ODONE = 24, BAR_MMADONE = 28, NUM_BARS = 29,
  BAR_PHALF = 34   // four more behind the TMEM / abort words at bytes 256..263: the first 32 keys of P are ready
};

// Register budgets per warpgroup (see the kernel body): control / softmax / K-transform warps of
// the four-tile instantiation, control / softmax warps of the two-tile one.
#ifndef PE_TC4_REGS_CTRL
#define PE_TC4_REGS_CTRL 24
#define PE_TC4_REGS_SOFTMAX 88
#define PE_TC4_REGS_XFORM 104
#define PE_TC4_XFORM_GROUP 4
#endif
#define PE_TC2_REGS_CTRL 24
#define PE_TC2_REGS_SOFTMAX 104
#define PE_STR2(x) #x
#define PE_STR(x) PE_STR2(x)
static_assert(4 * PE_TC4_REGS_CTRL + 16 * PE_TC4_REGS_SOFTMAX + 4 * PE_TC4_REGS_XFORM == 24 * 80,
              "the budgets must add up to the 24 warps x 80 registers the kernel is launched with");
static_assert(4 * PE_TC2_REGS_CTRL + 8 * PE_TC2_REGS_SOFTMAX <= 12 * 80,
              "the two-tile budgets must fit the 12 warps x 80 registers that instantiation is launched with");


template <int DC, int DR, int NT>
struct Cfg4 {
  static constexpr int DQK = DC + 2 * DR;
  static constexpr int NCHUNK = DQK / 64;  // 64-column (128-byte) operand chunks
  static constexpr int NCC = DC / 64;      // chunks that are plain content (TMA-loaded)
  static constexpr int Q_CHUNK_BYTES = BLOCK_M * 128;
  static constexpr int K_CHUNK_BYTES = BLOCK_N * 128;
  static constexpr int Q_TILE_BYTES = NCHUNK * Q_CHUNK_BYTES;
  static constexpr int K_STAGE_BYTES = NCHUNK * K_CHUNK_BYTES;
  static constexpr int V_STAGE_BYTES = BLOCK_N * 128;
  static constexpr int Q_OFF = TAIL_BYTES;
  static constexpr int K_OFF = Q_OFF + NT * Q_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * K_STAGE_BYTES;
  static constexpr int SMEM_USED = V_OFF + KV_STAGES * V_STAGE_BYTES;
  static constexpr int SMEM_BYTES = SMEM_USED + 1024;  // slack to align the base to 1024
  static_assert(DQK == 64 || DQK == 128, "d_qk must be 64 or 128");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
};

template <int DC, int DR, int MODE, bool ALIBI, int NT>
__global__ void __launch_bounds__(threads_for(NT), NT == 4 ? 1 : 2)
pe_attn_tc4_kernel(const KParams p, const int heads_per_cta, const int bh_group, const __grid_constant__ CUtensorMap tmQ,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
  using C = Cfg4<DC, DR, NT>;
  static_assert(NT == 4 || (NT == 2 && MODE == MODE_PLAIN), "two tiles per CTA: no transform warps");
  constexpr int TMEM_COLS = NT * (BLOCK_N + DV);
  constexpr uint32_t O_COL0 = NT * BLOCK_N;
  constexpr bool HAS_TMA_QK = (MODE == MODE_PLAIN) || (MODE == MODE_POPE && DC > 0);
  constexpr bool HAS_XFORM = MODE != MODE_PLAIN;
  // hand P to the MMA warp in two halves, except where it measured slower (the PoPE instantiations:
  // 699 against 680 TFLOP/s at head_dim 64 + 2 x 32, S 4096; the others gain 1-3 %)
  constexpr int P_PARTS = MODE == MODE_POPE ? 1 : 2;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 256);
  volatile uint32_t* abort_slot = reinterpret_cast<volatile uint32_t*>(smem + 260);
  float* freq_s = reinterpret_cast<float*>(smem + 512);   // [<= 64]
  float* delta_s = reinterpret_cast<float*>(smem + 768);  // [<= 64]
  auto bar = [&](int idx) -> uint32_t { return smem_base + 8u * (uint32_t)idx; };

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);

  // Work decomposition.  A CTA owns ``heads_per_cta`` (1, 2 or 4) query heads of one K/V head and
  // NT / heads_per_cta consecutive 128-row tiles of each.  1-D grid, longest row blocks first
  // within groups of ``bh_group`` (batch, head-set) problems whose K/V stay in L2 together.
  const int row_tiles = NT / heads_per_cta;
  const int rows_per_cta = row_tiles * BLOCK_M;
  const int n_rblk = (p.Sq + rows_per_cta - 1) / rows_per_cta;
  const int n_hset = p.H / heads_per_cta;
  const int n_bh = p.B * n_hset;
  const int per_group = bh_group * n_rblk;
  const int grp = (int)(blockIdx.x / per_group), in_grp = (int)(blockIdx.x % per_group);
  const int g_first = grp * bh_group;
  const int g_size = (n_bh - g_first) < bh_group ? (n_bh - g_first) : bh_group;
  const int rblk = n_rblk - 1 - in_grp / g_size;
  const int bh = g_first + in_grp % g_size;
  const int hset = bh % n_hset, b = bh / n_hset;
  const int h_first = hset * heads_per_cta;
  const int hk = h_first / p.groups;
  const int m0 = rblk * rows_per_cta;

  // tile i = (head h_first + i % heads_per_cta, rows m0 + (i / heads_per_cta) * 128 ...): key tiles
  // it needs (causal): keys [0, min(Sk, last row + 1 + off)); 0 for a tile past the last query row
  int nt[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int first = m0 + (i / heads_per_cta) * BLOCK_M;
    int kend = first + BLOCK_M + p.causal_off;
    if (kend > p.Sk) kend = p.Sk;
    nt[i] = first < p.Sq ? (kend + BLOCK_N - 1) / BLOCK_N : 0;
  }
  int n_tiles = 0;
#pragma unroll
  for (int i = 0; i < NT; ++i) n_tiles = nt[i] > n_tiles ? nt[i] : n_tiles;

  auto fail = [&](int code) {
    if (p.status != nullptr) atomicOr(p.status, code);
  };

  if (tid == 0) {
    // a CTA that starts after another one reported a failure does no work
    *abort_slot = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
    const uint32_t n_xf = HAS_XFORM ? 4u : 0u;
    const uint32_t n_tma = HAS_TMA_QK ? 1u : 0u;
    for (int i = 0; i < NT; ++i) {
      mbar_init(bar(BAR_QFULL + i), n_tma + n_xf);
      mbar_init(bar(BAR_SFULL + i), 1);
      mbar_init(bar(BAR_PREADY + i), 4);
      mbar_init(bar(BAR_PHALF + i), 4);
      mbar_init(bar(BAR_ODONE + i), 1);
    }
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar(BAR_KFULL + s), n_tma + n_xf);
      mbar_init(bar(BAR_KEMPTY + s), 1);
      mbar_init(bar(BAR_VFULL + s), 1);
      mbar_init(bar(BAR_VEMPTY + s), 1);
    }
    mbar_init(bar(BAR_MMADONE), 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
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
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool run = *abort_slot == 0;

  const uint32_t q_smem = smem_base + C::Q_OFF;
  const uint32_t k_smem = smem_base + C::K_OFF;
  const uint32_t v_smem = smem_base + C::V_OFF;

  // Register budgets per warpgroup.  setmaxnreg only moves registers around inside the CTA's own
  // allocation -- 24 warps x the 80 registers per thread the kernel is launched with = 1920
  // warp-registers -- and an increase beyond what the other warps have given back blocks for
  // good, so the budgets add up to exactly that: 4 x 24 + 16 x 88 + 4 x 104 = 1920.
  // The role code sits inside the branch that sets its budget.
  if (warp < 4) {
  if constexpr (NT == 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 " PE_STR(PE_TC4_REGS_CTRL) ";");
  else asm volatile("setmaxnreg.dec.sync.aligned.u32 " PE_STR(PE_TC2_REGS_CTRL) ";");
  if (!run) {
    // nothing to do
  } else if (warp == 0) {
    // ===================== TMA producer: content halves of Q and K =====================
    if constexpr (HAS_TMA_QK) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
      }
      for (int i = 0; i < NT; ++i) {
        if (nt[i] == 0) continue;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar(BAR_QFULL + i), C::NCC * C::Q_CHUNK_BYTES);
#pragma unroll
          for (int c = 0; c < C::NCC; ++c)
            tma_load_4d(q_smem + i * C::Q_TILE_BYTES + c * C::Q_CHUNK_BYTES, &tmQ, bar(BAR_QFULL + i), c * 64,
                        m0 + (i / heads_per_cta) * BLOCK_M, h_first + i % heads_per_cta, b);
        }
        __syncwarp();
      }
      int s = 0;
      uint32_t ph = 0;
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1u))) { fail(ST_WAIT_KEMPTY); break; }
        if (elect_one()) {
          mbar_arrive_expect_tx(bar(BAR_KFULL + s), C::NCC * C::K_CHUNK_BYTES);
#pragma unroll
          for (int c = 0; c < C::NCC; ++c)
            tma_load_4d(k_smem + s * C::K_STAGE_BYTES + c * C::K_CHUNK_BYTES, &tmK, bar(BAR_KFULL + s), c * 64,
                        j * BLOCK_N, hk, b);
        }
        __syncwarp();
        if (++s == KV_STAGES) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 3) {
    // ===================== TMA producer: V tiles =====================
    if (elect_one()) tma_prefetch_desc(&tmV);
    int s = 0;
    uint32_t ph = 0;
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_VEMPTY + s), ph ^ 1u))) { fail(ST_WAIT_VEMPTY); break; }
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(BAR_VFULL + s), C::V_STAGE_BYTES);
        tma_load_4d(v_smem + s * C::V_STAGE_BYTES, &tmV, bar(BAR_VFULL + s), 0, j * BLOCK_N, hk, b);
      }
      __syncwarp();
      if (++s == KV_STAGES) { s = 0; ph ^= 1u; }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    // The whole warp runs the loop converged; one elected lane issues the tcgen05 instructions.
    constexpr uint32_t IDESC_QK = make_idesc_bf16(BLOCK_M, BLOCK_N, false);
    constexpr uint32_t IDESC_PV = make_idesc_bf16(BLOCK_M, DV, true);
    const uint64_t qdesc0 = make_smem_desc(q_smem, 16, 1024);
    const uint64_t kdesc0 = make_smem_desc(k_smem, 16, 1024);
    const uint64_t vdesc0 = make_smem_desc(v_smem, C::V_STAGE_BYTES, 1024);
    bool ok = true;
    for (int i = 0; i < NT && ok; ++i)
      if (nt[i] > 0 && !__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_QFULL + i), 0))) { fail(ST_WAIT_QFULL); ok = false; }

    // S_i = Q_i K(stage ks)^T, then tell tile i's softmax warps
    auto issue_qk = [&](int i, int ks) {
      if (elect_one()) {
        const uint32_t d = tmem_base + (uint32_t)(i * BLOCK_N);
        uint64_t qd = advance_smem_desc(qdesc0, (uint32_t)(i * C::Q_TILE_BYTES));
        uint64_t kd = advance_smem_desc(kdesc0, (uint32_t)(ks * C::K_STAGE_BYTES));
#pragma unroll
        for (int c = 0; c < C::NCHUNK; ++c) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_ss(d, advance_smem_desc(qd, (uint32_t)(k4 * 32)), advance_smem_desc(kd, (uint32_t)(k4 * 32)), IDESC_QK,
                   (c > 0 || k4 > 0) ? 1u : 0u);
          qd = advance_smem_desc(qd, C::Q_CHUNK_BYTES);
          kd = advance_smem_desc(kd, C::K_CHUNK_BYTES);
        }
        tc_commit(bar(BAR_SFULL + i));
      }
      __syncwarp();
    };
    auto wait_k = [&](int ks, uint32_t kph) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_KFULL + ks), kph))) {
        fail(ST_WAIT_KFULL);
        return false;
      }
      tc_fence_after_sync();
      return true;
    };

    if (ok && n_tiles > 0) {
      ok = wait_k(0, 0);
      if (ok) {
        for (int i = 0; i < NT; ++i)
          if (nt[i] > 0) issue_qk(i, 0);
        if (elect_one()) tc_commit(bar(BAR_KEMPTY + 0));
        __syncwarp();
      }
    }
    int s = 0;            // stage of K(j) / V(j)
    uint32_t ph = 0;
#pragma unroll 1
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s1 = (s + 1 == KV_STAGES) ? 0 : s + 1;              // stage of K(j+1)
      const uint32_t ph1 = (s + 1 == KV_STAGES) ? (ph ^ 1u) : ph;
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_VFULL + s), ph))) { fail(ST_WAIT_VFULL); ok = false; break; }
      const uint64_t vd = advance_smem_desc(vdesc0, (uint32_t)(s * C::V_STAGE_BYTES));
      bool have_k = false;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        if (j < nt[i]) {
          // P arrives in two halves of 32 keys (P_PARTS == 2): the first half's PV runs under the
          // second half's exponentials
          const uint32_t d = tmem_base + O_COL0 + (uint32_t)(i * DV);
          const uint32_t a = tmem_base + (uint32_t)(i * BLOCK_N);
          if constexpr (P_PARTS == 2) {
            if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PHALF + i), (uint32_t)(j & 1)))) {
              fail(ST_WAIT_PREADY);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < BLOCK_N / 32; ++kk)
                mma_ts(d, a + (uint32_t)(kk * 8), advance_smem_desc(vd, (uint32_t)(kk * 16 * 128)), IDESC_PV,
                       (j > 0 || kk > 0) ? 1u : 0u);
            }
            __syncwarp();
          }
          if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PREADY + i), (uint32_t)(j & 1)))) {
            fail(ST_WAIT_PREADY);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (elect_one()) {
#pragma unroll
            for (int kk = P_PARTS == 2 ? BLOCK_N / 32 : 0; kk < BLOCK_N / 16; ++kk)
              mma_ts(d, a + (uint32_t)(kk * 8), advance_smem_desc(vd, (uint32_t)(kk * 16 * 128)), IDESC_PV,
                     (j > 0 || kk > 0) ? 1u : 0u);
            tc_commit(bar(BAR_ODONE + i));
          }
          __syncwarp();
        }
        if (j + 1 < nt[i]) {
          if (!have_k) {
            if (!wait_k(s1, ph1)) { ok = false; break; }
            have_k = true;
          }
          issue_qk(i, s1);   // overwrites S_i / P_i: ordered behind PV_i(j) by the in-order tensor pipe
        }
      }
      if (!ok) break;
      if (elect_one()) {
        tc_commit(bar(BAR_VEMPTY + s));
        if (j + 1 < n_tiles) tc_commit(bar(BAR_KEMPTY + s1));
      }
      __syncwarp();
      s = s1;
      ph = ph1;
    }
    // every MMA, and with it every barrier arrival they trigger, has landed before the CTA exits
    if (elect_one()) tc_commit(bar(BAR_MMADONE));
    __syncwarp();
    if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_MMADONE), 0))) fail(ST_WAIT_MMADONE);
  }
  } else if (warp < 4 + 4 * NT) {
  if constexpr (NT == 4) asm volatile("setmaxnreg.inc.sync.aligned.u32 " PE_STR(PE_TC4_REGS_SOFTMAX) ";");
  else asm volatile("setmaxnreg.inc.sync.aligned.u32 " PE_STR(PE_TC2_REGS_SOFTMAX) ";");
  if (run) {
    // ===================== softmax warpgroups =====================
    const int i = (warp - 4) >> 2;
    const int tg = tid - 128 - i * BLOCK_M;
    const int ntile = nt[i];
    const int h = h_first + i % heads_per_cta;
    const int row0 = m0 + (i / heads_per_cta) * BLOCK_M;
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
        if (lane == 0) mbar_arrive(bar(BAR_QFULL + i));
      }
      const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
      const int row = row0 + tg;
      const int row_lim = row + p.causal_off;  // last visible key
      const float c2 = p.scale * 1.4426950408889634f;
      float slope2 = 0.f;
      if constexpr (ALIBI) slope2 = p.slopes[h] * 1.4426950408889634f;
      const float kf = ALIBI ? 1.0f : c2;      // with ALiBi the logits are put into log2 units up front
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;
      const uint32_t s_addr = tmem_base + lane_sel + (uint32_t)(i * BLOCK_N);
      const uint32_t o_addr = tmem_base + lane_sel + O_COL0 + (uint32_t)(i * DV);

#pragma unroll 1
      for (int j = 0; j < ntile; ++j) {
        // up to sixteen warps wait here at a time: the suspending wait, not a polling loop that
        // would take issue slots from the warps that have work (measured: 1-2 % apart)
        ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_SFULL + i), (uint32_t)(j & 1)));
        if (!ok) { fail(ST_WAIT_SFULL); break; }
        tc_fence_after_sync();
        uint32_t sr[2][32];
        tmem_ld32(s_addr, sr[0]);
        tmem_ld32(s_addr + 32, sr[1]);
        tmem_wait_ld();

        float t[64];
#pragma unroll
        for (int c = 0; c < 64; ++c) t[c] = __uint_as_float(sr[c >> 5][c & 31]);
        const int key0 = j * BLOCK_N;
        if constexpr (ALIBI) {
          // logit (log2 units) = s * c2 - slope2 * (row_lim - key)
          const float base = slope2 * (float)(key0 - row_lim);
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            // two columns per packed FMA (same roundings as fmaf(t, c2, fmaf(c, slope2, base)) each)
            const float2 bias = __ffma2_rn(make_float2((float)c, (float)(c + 1)), make_float2(slope2, slope2),
                                           make_float2(base, base));
            const float2 r = __ffma2_rn(make_float2(t[c], t[c + 1]), make_float2(c2, c2), bias);
            t[c] = r.x;
            t[c + 1] = r.y;
          }
        }
        const bool need_mask = (key0 + BLOCK_N - 1 > row0 + p.causal_off) || (key0 + BLOCK_N > p.Sk);
        if (need_mask) {
          // columns past the row's last visible key (causal limit, end of the keys): one compare each
          const int last = (row_lim < p.Sk - 1 ? row_lim : p.Sk - 1) - key0;
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c > last) t[c] = -INFINITY;
        }
        float mx0 = fmax3(t[0], t[1], t[2]), mx1 = fmax3(t[3], t[4], t[5]), mx2 = fmax3(t[6], t[7], t[8]),
              mx3 = fmax3(t[9], t[10], t[11]);
#pragma unroll
        for (int c = 12; c + 8 <= 64; c += 8) {
          mx0 = fmax3(mx0, t[c], t[c + 1]);
          mx1 = fmax3(mx1, t[c + 2], t[c + 3]);
          mx2 = fmax3(mx2, t[c + 4], t[c + 5]);
          mx3 = fmax3(mx3, t[c + 6], t[c + 7]);
        }
        mx0 = fmax3(mx0, t[60], t[61]);   // 12 + 6 * 8 = 60: the last four columns
        mx1 = fmax3(mx1, t[62], t[63]);
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // lazy rescale: move the reference maximum only when it grows by more than 2^8
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
        // packed fp32x2 FMA / ADD for scale-and-shift and the row sum; exponentials on the SFU;
        // P as bf16 pairs over the first 32 columns of this S tile, 16 columns per store so that
        // the packed words need not all be live at once
        const float2 kf2 = make_float2(kf, kf), nm2 = make_float2(-m_used * kf, -m_used * kf);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
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
          if (P_PARTS == 2 && cb == 0) {
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BAR_PHALF + i));
          }
        }
        l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_PREADY + i));
      }

      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_ODONE + i), (uint32_t)((ntile - 1) & 1)));
        if (!ok) fail(ST_WAIT_PVDONE);
      }
      if (ok) {
        tc_fence_after_sync();
        const float inv_l = 1.0f / l_sum;
        if (p.lse != nullptr && row < p.Sq)
          p.lse[((long long)b * p.H + h) * p.Sq + row] = m_used * kf * 0.6931471805599453f + logf(l_sum);
        char* dst = reinterpret_cast<char*>(const_cast<void*>(p.out.ptr)) +
                    2 * ((long long)b * p.out.sb + (long long)h * p.out.sh + (long long)row * p.out.ss);
#pragma unroll
        for (int cb = 0; cb < DV / 32; ++cb) {
          uint32_t orow[32];
          tmem_ld32(o_addr + cb * 32, orow);
          tmem_wait_ld();
          if (row < p.Sq) {
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
  asm volatile("setmaxnreg.inc.sync.aligned.u32 " PE_STR(PE_TC4_REGS_XFORM) ";");
  if (run) {
    // ===================== K-tile positional transform =====================
    const int tg = tid - 640;
    if constexpr (MODE == MODE_POPE) {
      // Thread (r_in, cv) owns columns [8 cv, 8 cv + 8) of rows r_in + k * RPP of every key tile.
      // cos / sin of (row-in-tile * freq + delta) for those cells are computed once and kept in
      // registers; per tile only the tile's base angle pos0 * freq needs the special-function
      // unit, and each cell is rotated by it with four FMAs:
      //   cos(pos0 w + (r w + d)) = cb Tc - sb Ts,  sin(...) = sb Tc + cb Ts.
      constexpr int VPR = DR / 8, RPP = 128 / VPR, PASSES = BLOCK_N / RPP;
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
      uint4 nxt[PASSES];
#pragma unroll
      for (int k = 0; k < PASSES; ++k) {
        const int grow = r_in + k * RPP;
        nxt[k] = grow < p.Sk ? ldg_nc_v4(src + 2 * (long long)grow * p.kr.ss) : make_uint4(0, 0, 0, 0);
      }
      int s = 0;
      uint32_t ph = 0;
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        uint4 cur[PASSES];
#pragma unroll
        for (int k = 0; k < PASSES; ++k) cur[k] = nxt[k];
        if (j + 1 < n_tiles) {
#pragma unroll
          for (int k = 0; k < PASSES; ++k) {
            const int grow = (j + 1) * BLOCK_N + r_in + k * RPP;
            nxt[k] = grow < p.Sk ? ldg_nc_v4(src + 2 * (long long)grow * p.kr.ss) : make_uint4(0, 0, 0, 0);
          }
        }
        float cb[8], sb[8];
        const float pos0 = (float)(p.k_pos0 + j * BLOCK_N);
#pragma unroll
        for (int e = 0; e < 8; ++e) sincos_reduced(__fmul_rn(pos0, th[e]), &sb[e], &cb[e]);
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1u));
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
        if (lane == 0) mbar_arrive(bar(BAR_KFULL + s));
        if (++s == KV_STAGES) { s = 0; ph ^= 1u; }
      }
    } else if constexpr (MODE == MODE_XFORM) {
      // raw rows and table entries of the next tile are requested before the wait for its stage
      XformRegs<DC> xr;
      XformCursor<DC> cur;
      xform_cursor_init<DC>(p, cur, p.k, b, hk, 0, p.k_pos0, BLOCK_N, tg);
      if (n_tiles > 0) xform_load_next<DC>(p, xr, cur, p.Sk, BLOCK_N);
      int s = 0;
      uint32_t ph = 0;
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1u));
        if (!ok) { fail(ST_WAIT_KEMPTY); break; }
        xform_finish<DC, PE_TC4_XFORM_GROUP>(p, xr, k_smem + s * C::K_STAGE_BYTES, C::K_CHUNK_BYTES, j * BLOCK_N, p.Sk, tg);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_KFULL + s));
        if (j + 1 < n_tiles) xform_load_next<DC>(p, xr, cur, p.Sk, BLOCK_N);
        if (++s == KV_STAGES) { s = 0; ph ^= 1u; }
      }
    }
  }
  }  // register-budget branch

  // common exit: after a failed wait give copies in flight time to land before the
  // shared memory and TMEM are released
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// heads of one K/V head that share a CTA: the largest of 4, 2, 1 that divides the GQA ratio
int heads_per_cta_for(const KParams& p) { return (p.groups % 4 == 0) ? 4 : (p.groups % 2 == 0) ? 2 : 1; }

// Two tiles per CTA, two CTAs per SM: the variants without a positional transform when no heads
// share K/V (the four-tile CTA would then be 512 consecutive rows of one head).
bool two_tile_ctas(const KParams& p) {
  const bool plain = p.variant != PE_ATTN_POPE && p.variant != PE_ATTN_ROTARY && !(p.flags & PE_ATTN_QK_NORM);
  return plain && p.groups % 2 != 0;
}

// ---- host side --------------------------------------------------------------------------
template <int DC, int DR, int MODE, bool ALIBI, int NT>
int launch_instance4(const KParams& p, cudaStream_t stream) {
  using C = Cfg4<DC, DR, NT>;
  auto kern = pe_attn_tc4_kernel<DC, DR, MODE, ALIBI, NT>;
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
    if (!encode_map(&tmQ, p.q, DC, p.Sq, p.H, p.B, BLOCK_M) || !encode_map(&tmK, p.k, DC, p.Sk, p.Hkv, p.B, BLOCK_N)) {
      set_error("cuTensorMapEncodeTiled failed for q / k");
      return PE_ATTN_ERR_LAUNCH;
    }
  }
  const int hpc = NT == 4 ? heads_per_cta_for(p) : 1;
  const int rows_per_cta = (NT / hpc) * BLOCK_M;
  const int n_rblk = (p.Sq + rows_per_cta - 1) / rows_per_cta;
  const long long n_bh = (long long)p.B * (p.H / hpc);
  // (batch, head-set) problems per scheduling group: equal groups whose K/V stay in L2 together
  const long long kv_bytes_per_head = 2ll * p.Sk * (DC + DR + DV);
  const int bh_group = balanced_bh_group(n_bh, kv_bytes_per_head, 1);
  dim3 grid((unsigned)(n_rblk * n_bh)), block(threads_for(NT));
  kern<<<grid, block, C::SMEM_BYTES, stream>>>(p, hpc, bh_group, tmQ, tmK, tmV);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("tcgen05 four-tile kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

template <int DC, int DR, int MODE, int NT>
int launch_alibi4(const KParams& p, cudaStream_t stream) {
  if (p.variant == PE_ATTN_ALIBI) return launch_instance4<DC, DR, MODE, true, NT>(p, stream);
  return launch_instance4<DC, DR, MODE, false, NT>(p, stream);
}

}  // namespace

// The four-tile kernel covers d_v = 64 (head_dim 64 models) once a CTA's four tiles are mostly
// real: more query rows than half of what one CTA owns.
bool tc4_supports(const KParams& p) {
  if (p.d_v != 64) return false;
  const bool shape = (p.variant == PE_ATTN_POPE) ? ((p.d_c == 64 && p.d_r == 32) || (p.d_c == 0 && p.d_r == 32))
                                                 : (p.d_c == 64);
  if (!shape) return false;
  const int rows_per_cta = two_tile_ctas(p) ? 2 * BLOCK_M : (MAX_TILES / heads_per_cta_for(p)) * BLOCK_M;
  return p.Sq > rows_per_cta / 2;
}

int launch_tc4(const KParams& p, cudaStream_t stream) {
  if (p.variant == PE_ATTN_POPE) {
    if (p.d_c == 64) return launch_instance4<64, 32, MODE_POPE, false, 4>(p, stream);
    return launch_instance4<0, 32, MODE_POPE, false, 4>(p, stream);
  }
  const bool xform = p.variant == PE_ATTN_ROTARY || (p.flags & PE_ATTN_QK_NORM);
  if (xform) return launch_alibi4<64, 0, MODE_XFORM, 4>(p, stream);
  return two_tile_ctas(p) ? launch_alibi4<64, 0, MODE_PLAIN, 2>(p, stream) : launch_alibi4<64, 0, MODE_PLAIN, 4>(p, stream);
}

}  // namespace pe_attn
