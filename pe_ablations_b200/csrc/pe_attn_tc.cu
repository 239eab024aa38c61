// tcgen05 / TMEM / TMA fused PE-attention forward for bf16 tensors (sm_100a).
//
// One CTA (512 threads, 1 per SM) owns 256 query rows of one (batch, head) as two
// 128-row tiles and streams 64-key tiles through a 2-stage shared-memory ring:
//
//   warp 0        TMA producer: content halves of Q and K as 128B-swizzled tiles
//   warp 3        TMA producer: V tiles
//   warp 1        MMA issuer:   S_i = Q_i K^T  (SS, M128 N64 K16 x d_qk/16) into TMEM,
//                               O_i += P_i V   (TS: P read from TMEM, V from smem, N = d_v)
//   warp 2        TMEM allocation / release (512 columns)
//   warps 4-7     softmax of query tile 0: TMEM -> registers, running max / sum, P (bf16)
//   warps 8-11    softmax of query tile 1          back into TMEM over its own S buffer
//   warps 12-15   positional transform of every K tile, written straight into the
//                 swizzled K-major operand layout the MMA reads
// The softmax warpgroups also build the positional part of their own Q tile once.
//
// Nothing positional ever goes to global memory: RoPE-family rotation (from the (cos, sin)
// table), QKNorm, and the PoPE expansion [softplus(x) cos(phi), softplus(x) sin(phi)] with
// phi = pos * freq (+ clamped key phase bias) are computed in registers from the raw
// projections and stored as bf16 MMA operands in shared memory.  The FoPE frequency mix
// and floor clipping run in the kernel prologue.
//
// TMEM map (columns): S/P buffers (tile i, buffer b) at (2 i + b) * 64, 64 fp32 columns
// each (P reuses the first 32 as packed bf16 pairs); O_i at 256 + i * d_v.
//
// Every mbarrier wait is bounded; on expiry the CTA ORs a code into the caller's status
// word, lets its copies land, frees its TMEM and returns.
#include <cuda.h>

#include "pe_attn_tc_common.cuh"

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

constexpr int BLOCK_M = 128;   // query rows per tile (TMEM lanes)
constexpr int Q_TILES = 2;     // query tiles per CTA
constexpr int BLOCK_N = 64;    // keys per tile
constexpr int KV_STAGES = 2;
constexpr int NTHREADS = 512;
constexpr int TMEM_COLS = 512;
constexpr int TAIL_BYTES = 1024;  // barriers, TMEM base, frequency / phase-bias vectors


enum : int {
  BAR_QFULL = 0, BAR_KFULL = 2, BAR_KEMPTY = 4, BAR_VFULL = 6, BAR_VEMPTY = 8, BAR_SFULL = 10, BAR_PREADY = 14,
  BAR_PVDONE = 18 /* one per query tile, completes once */, BAR_MMADONE = 22, NUM_BARS = 23
};

template <int DC, int DR, int DV>
struct Cfg {
  static constexpr int DQK = DC + 2 * DR;
  static constexpr int NCHUNK = DQK / 64;  // 64-column (128-byte) operand chunks
  static constexpr int NCC = DC / 64;      // chunks that are plain content (TMA-loaded)
  static constexpr int VCH = DV / 64;
  static constexpr int Q_CHUNK_BYTES = BLOCK_M * 128;
  static constexpr int K_CHUNK_BYTES = BLOCK_N * 128;
  static constexpr int V_CHUNK_BYTES = BLOCK_N * 128;
  static constexpr int Q_TILE_BYTES = NCHUNK * Q_CHUNK_BYTES;
  static constexpr int K_STAGE_BYTES = NCHUNK * K_CHUNK_BYTES;
  static constexpr int V_STAGE_BYTES = VCH * V_CHUNK_BYTES;
  static constexpr int Q_OFF = TAIL_BYTES;
  static constexpr int K_OFF = Q_OFF + Q_TILES * Q_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * K_STAGE_BYTES;
  static constexpr int SMEM_USED = V_OFF + KV_STAGES * V_STAGE_BYTES;
  static constexpr int SMEM_BYTES = SMEM_USED + 1024;  // slack to align the base to 1024
  static_assert(DQK % 64 == 0 && DQK >= 64 && DQK <= 256, "d_qk must be 64..256 in steps of 64");
  static_assert(DV == 64 || DV == 128, "d_v must be 64 or 128");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
};

template <int DC, int DR, int DV, int MODE, bool ALIBI>
__global__ void __launch_bounds__(NTHREADS, 1)
pe_attn_tc_kernel(const KParams p, const int bh_group, const __grid_constant__ CUtensorMap tmQ,
                  const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
  using C = Cfg<DC, DR, DV>;
  constexpr bool HAS_TMA_QK = (MODE == MODE_PLAIN) || (MODE == MODE_POPE && DC > 0);
  constexpr bool HAS_XFORM = MODE != MODE_PLAIN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base;                       // NUM_BARS x 8 bytes
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 256);
  volatile uint32_t* abort_slot = reinterpret_cast<volatile uint32_t*>(smem + 260);
  float* freq_s = reinterpret_cast<float*>(smem + 512);   // [64]
  float* delta_s = reinterpret_cast<float*>(smem + 768);  // [64]
  auto bar = [&](int idx) -> uint32_t { return bars + 8u * (uint32_t)idx; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // 1-D grid, longest query blocks first within groups of ``bh_group`` (batch, head) problems.
  // Block ids are handed out in increasing order, so a group's last (longest) query blocks
  // start first; the group is sized so that the K/V of the heads in flight stay in L2.
  const int n_qblk = (p.Sq + Q_TILES * BLOCK_M - 1) / (Q_TILES * BLOCK_M);
  const int n_bh = p.B * p.H;
  const int per_group = bh_group * n_qblk;
  const int grp = (int)(blockIdx.x / per_group), in_grp = (int)(blockIdx.x % per_group);
  const int g_first = grp * bh_group;
  const int g_size = (n_bh - g_first) < bh_group ? (n_bh - g_first) : bh_group;
  const int qblk = n_qblk - 1 - in_grp / g_size;
  const int bh = g_first + in_grp % g_size;
  const int h = bh % p.H, b = bh / p.H;
  const int hk = h / p.groups;
  const int m0 = qblk * Q_TILES * BLOCK_M;

  // key tiles each query tile needs (causal): keys [0, min(Sk, last row + 1 + off))
  int nt[Q_TILES];
#pragma unroll
  for (int i = 0; i < Q_TILES; ++i) {
    const int first = m0 + i * BLOCK_M;
    int kend = first + BLOCK_M + p.causal_off;
    if (kend > p.Sk) kend = p.Sk;
    nt[i] = first < p.Sq ? (kend + BLOCK_N - 1) / BLOCK_N : 0;
  }
  const int n_tiles = nt[1] > nt[0] ? nt[1] : nt[0];

  auto fail = [&](int code) {
    if (p.status != nullptr) atomicOr(p.status, code);
  };

  if (tid == 0) {
    // a CTA that starts after another one reported a failure does no work
    *abort_slot = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
    const uint32_t n_xf = HAS_XFORM ? 4u : 0u;
    const uint32_t n_tma = HAS_TMA_QK ? 1u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_QFULL + i), n_tma + n_xf);
      mbar_init(bar(BAR_KFULL + i), n_tma + n_xf);
      mbar_init(bar(BAR_KEMPTY + i), 1);
      mbar_init(bar(BAR_VFULL + i), 1);
      mbar_init(bar(BAR_VEMPTY + i), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(BAR_SFULL + i), 1);
      mbar_init(bar(BAR_PREADY + i), 4);
      mbar_init(bar(BAR_PVDONE + i), 1);
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

  // Register budget: the producer / MMA / allocator warpgroup gives registers back, the
  // softmax and transform warpgroups take them (4 x 128 x 56 + 12 x 128 x 152 = 64 K).

  const uint32_t q_smem = smem_base + C::Q_OFF;
  const uint32_t k_smem = smem_base + C::K_OFF;
  const uint32_t v_smem = smem_base + C::V_OFF;

  // The role code sits inside the branch that sets its register budget, so that the
  // budget is unambiguous along every path.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (!run) {
    // nothing to do
  } else if (warp == 0) {
    // ===================== TMA producer =====================
    // The whole warp runs the loop (waits included); one elected lane issues the copies.
    if constexpr (HAS_TMA_QK) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
      }
    }
    if constexpr (HAS_TMA_QK) {
      for (int i = 0; i < Q_TILES; ++i) {
        if (nt[i] == 0) continue;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar(BAR_QFULL + i), C::NCC * C::Q_CHUNK_BYTES);
#pragma unroll
          for (int c = 0; c < C::NCC; ++c)
            tma_load_4d(q_smem + i * C::Q_TILE_BYTES + c * C::Q_CHUNK_BYTES, &tmQ, bar(BAR_QFULL + i), c * 64,
                        m0 + i * BLOCK_M, h, b);
        }
        __syncwarp();
      }
    }
    if constexpr (HAS_TMA_QK) {
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1u))) { fail(ST_WAIT_KEMPTY); break; }
        if (elect_one()) {
          mbar_arrive_expect_tx(bar(BAR_KFULL + s), C::NCC * C::K_CHUNK_BYTES);
#pragma unroll
          for (int c = 0; c < C::NCC; ++c)
            tma_load_4d(k_smem + s * C::K_STAGE_BYTES + c * C::K_CHUNK_BYTES, &tmK, bar(BAR_KFULL + s), c * 64,
                        j * BLOCK_N, hk, b);
        }
        __syncwarp();
      }
    }
  } else if (warp == 3) {
    // ===================== TMA producer for V (its own warp: K and V stages are released at
    // different times, and one warp waiting on both in turn would issue each copy late)
    if (elect_one()) tma_prefetch_desc(&tmV);
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_VEMPTY + s), ph ^ 1u))) { fail(ST_WAIT_VEMPTY); break; }
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(BAR_VFULL + s), C::V_STAGE_BYTES);
#pragma unroll
        for (int c = 0; c < C::VCH; ++c)
          tma_load_4d(v_smem + s * C::V_STAGE_BYTES + c * C::V_CHUNK_BYTES, &tmV, bar(BAR_VFULL + s), c * 64,
                      j * BLOCK_N, hk, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    // The whole warp runs the loop; descriptors are warp-uniform values and one elected lane
    // issues the tcgen05 instructions.
    constexpr uint32_t IDESC_QK = make_idesc_bf16(BLOCK_M, BLOCK_N, false);
    constexpr uint32_t IDESC_PV = make_idesc_bf16(BLOCK_M, DV, true);
    const uint64_t qdesc0 = make_smem_desc(q_smem, 16, 1024);
    const uint64_t kdesc0 = make_smem_desc(k_smem, 16, 1024);
    const uint64_t vdesc0 = make_smem_desc(v_smem, C::V_CHUNK_BYTES, 1024);
    bool ok = true;
    for (int i = 0; i < Q_TILES && ok; ++i)
      if (nt[i] > 0 && !__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_QFULL + i), 0))) { fail(ST_WAIT_QFULL); ok = false; }

    auto issue_qk = [&](int j) -> bool {
      const int s = j & 1;
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_KFULL + s), (uint32_t)((j >> 1) & 1)))) {
        fail(ST_WAIT_KFULL);
        return false;
      }
      tc_fence_after_sync();
      if (elect_one()) {
        const uint64_t kd = advance_smem_desc(kdesc0, (uint32_t)(s * C::K_STAGE_BYTES));
#pragma unroll
        for (int i = 0; i < Q_TILES; ++i) {
          if (j < nt[i]) {
            const uint32_t d = tmem_base + (uint32_t)((2 * i + (j & 1)) * BLOCK_N);
            uint64_t qd = advance_smem_desc(qdesc0, (uint32_t)(i * C::Q_TILE_BYTES));
            uint64_t kc = kd;
#pragma unroll 1
            for (int c = 0; c < C::NCHUNK; ++c) {
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4)
                mma_ss(d, advance_smem_desc(qd, (uint32_t)(k4 * 32)), advance_smem_desc(kc, (uint32_t)(k4 * 32)),
                       IDESC_QK, (c > 0 || k4 > 0) ? 1u : 0u);
              qd = advance_smem_desc(qd, C::Q_CHUNK_BYTES);
              kc = advance_smem_desc(kc, C::K_CHUNK_BYTES);
            }
            tc_commit(bar(BAR_SFULL + 2 * i + (j & 1)));
          }
        }
        tc_commit(bar(BAR_KEMPTY + s));
      }
      __syncwarp();
      return true;
    };
    auto issue_pv = [&](int j) -> bool {
      const int s = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_VFULL + s), ph))) { fail(ST_WAIT_VFULL); return false; }
      const uint64_t vd = advance_smem_desc(vdesc0, (uint32_t)(s * C::V_STAGE_BYTES));
#pragma unroll
      for (int i = 0; i < Q_TILES; ++i) {
        if (j < nt[i]) {
          if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PREADY + 2 * i + (j & 1)), ph))) {
            fail(ST_WAIT_PREADY);
            return false;
          }
          tc_fence_after_sync();
          if (elect_one()) {
            const uint32_t d = tmem_base + 256u + (uint32_t)(i * DV);
            const uint32_t a = tmem_base + (uint32_t)((2 * i + (j & 1)) * BLOCK_N);
#pragma unroll
            for (int kk = 0; kk < BLOCK_N / 16; ++kk)
              mma_ts(d, a + (uint32_t)(kk * 8), advance_smem_desc(vd, (uint32_t)(kk * 16 * 128)), IDESC_PV,
                     (j > 0 || kk > 0) ? 1u : 0u);
            if (j == nt[i] - 1) tc_commit(bar(BAR_PVDONE + i));  // this tile's output is final
          }
          __syncwarp();
        }
      }
      if (elect_one()) tc_commit(bar(BAR_VEMPTY + s));
      __syncwarp();
      return true;
    };

    if (ok && n_tiles > 0) ok = issue_qk(0);
#pragma unroll 1
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) ok = issue_qk(j + 1);
      if (ok) ok = issue_pv(j);
    }
    // every MMA, and with it every barrier arrival they trigger, has landed before the CTA exits
    if (elect_one()) tc_commit(bar(BAR_MMADONE));
    __syncwarp();
    if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_MMADONE), 0))) fail(ST_WAIT_MMADONE);
  }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
  if (!run) {
    // nothing to do
  } else if (warp < 12) {
    // ===================== softmax warpgroups =====================
    const int i = (warp - 4) >> 2;
    const int tg = tid - 128 - i * BLOCK_M;
    const int ntile = nt[i];
    if (ntile > 0) {
      if constexpr (MODE == MODE_XFORM && DC <= 64) {
        // both 64-row halves of the query tile: all loads first, then the math (two register
        // sets: affordable at head_dim 64 only)
        const int r0 = m0 + i * BLOCK_M;
        XformRegs<DC> xa, xb;
        xform_load<DC>(p, xa, p.q, b, h, r0, p.Sq, p.q_pos0 + r0, tg);
        xform_load<DC>(p, xb, p.q, b, h, r0 + 64, p.Sq, p.q_pos0 + r0 + 64, tg);
        xform_finish<DC>(p, xa, q_smem + i * C::Q_TILE_BYTES, C::Q_CHUNK_BYTES, r0, p.Sq, tg);
        xform_finish<DC>(p, xb, q_smem + i * C::Q_TILE_BYTES + 64 * 128, C::Q_CHUNK_BYTES, r0 + 64, p.Sq, tg);
      } else if constexpr (HAS_XFORM) {
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const int r0 = m0 + i * BLOCK_M + half * 64;
          build_slab<DC, DR, MODE>(p, q_smem + i * C::Q_TILE_BYTES + half * 64 * 128, C::Q_CHUNK_BYTES, p.q, p.qr, b,
                                   h, r0, p.Sq, p.q_pos0 + r0, false, freq_s, delta_s, tg);
        }
      }
      if constexpr (HAS_XFORM) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_QFULL + i));
      }
      const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
      const int row = m0 + i * BLOCK_M + tg;
      const int row_lim = row + p.causal_off;  // last visible key
      const float c2 = p.scale * 1.4426950408889634f;
      float slope2 = 0.f;
      if constexpr (ALIBI) slope2 = p.slopes[h] * 1.4426950408889634f;
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;

#pragma unroll 1
      for (int j = 0; j < ntile; ++j) {
        const int bsel = 2 * i + (j & 1);
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_SFULL + bsel), ph));
        if (!ok) { fail(ST_WAIT_SFULL); break; }
        tc_fence_after_sync();
        const uint32_t s_addr = tmem_base + lane_sel + (uint32_t)(bsel * BLOCK_N);
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
        const bool need_mask = (key0 + BLOCK_N - 1 > m0 + i * BLOCK_M + p.causal_off) || (key0 + BLOCK_N > p.Sk);
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
        const float kf = ALIBI ? 1.0f : c2;  // t is already in log2 units with ALiBi
        // lazy rescale: move the reference maximum only when it grows by more than 2^8
        const bool need = (mx - m_used) * kf > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? ex2_approx((m_used - mx) * kf) : 1.0f;
          if (j > 0) {
            // PV(j-1) of both query tiles is complete once its V stage has been released
            ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_VEMPTY + ((j - 1) & 1)), (uint32_t)(((j - 1) >> 1) & 1)));
            if (!ok) { fail(ST_WAIT_PVDONE); break; }
            tc_fence_after_sync();
            const uint32_t o_addr = tmem_base + lane_sel + 256u + (uint32_t)(i * DV);
#pragma unroll
            for (int cb = 0; cb < DV / 32; ++cb) {
              uint32_t orow[32];
              tmem_ld32(o_addr + cb * 32, orow);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
              tmem_st32(o_addr + cb * 32, orow);
            }
            tmem_wait_st();
          }
          l_sum *= alpha;
          if (need) m_used = mx;
        }
        // packed fp32x2 FMA / ADD for scale-and-shift and the row sum; exponentials on the SFU
        const float2 kf2 = make_float2(kf, kf), nm2 = make_float2(-m_used * kf, -m_used * kf);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          const float2 x01 = __ffma2_rn(make_float2(t[c], t[c + 1]), kf2, nm2);
          const float2 x23 = __ffma2_rn(make_float2(t[c + 2], t[c + 3]), kf2, nm2);
          const float2 p01 = make_float2(ex2_approx(x01.x), ex2_approx(x01.y));
          const float2 p23 = make_float2(ex2_approx(x23.x), ex2_approx(x23.y));
          acc0 = __fadd2_rn(acc0, p01);
          acc1 = __fadd2_rn(acc1, p23);
          pk[c >> 1] = pack_bf16x2(p01.x, p01.y);
          pk[(c >> 1) + 1] = pack_bf16x2(p23.x, p23.y);
        }
        const float a0 = acc0.x, a1 = acc0.y, a2 = acc1.x, a3 = acc1.y;
        l_sum += (a0 + a1) + (a2 + a3);
        tmem_st32(s_addr, pk);  // P over the first 32 columns of this S buffer
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_PREADY + bsel));
      }

      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(BAR_PVDONE + i), 0));
        if (!ok) fail(ST_WAIT_PVDONE);
      }
      if (ok) {
        tc_fence_after_sync();
        const float inv_l = 1.0f / l_sum;
        if (p.lse != nullptr && row < p.Sq)
          p.lse[((long long)b * p.H + h) * p.Sq + row] =
              m_used * (ALIBI ? 1.0f : c2) * 0.6931471805599453f + logf(l_sum);
        const uint32_t o_addr = tmem_base + lane_sel + 256u + (uint32_t)(i * DV);
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
  } else {
    // ===================== K-tile positional transform =====================
    const int tg = tid - 384;
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
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
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
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), (uint32_t)(((j >> 1) & 1) ^ 1)));
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
      }
    } else if constexpr (MODE == MODE_XFORM) {
      // raw rows and table entries of the next tile are requested before the wait for its stage
      XformRegs<DC> xr;
      XformCursor<DC> cur;
      xform_cursor_init<DC>(p, cur, p.k, b, hk, 0, p.k_pos0, BLOCK_N, tg);
      if (n_tiles > 0) xform_load_next<DC>(p, xr, cur, p.Sk, BLOCK_N);
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_KEMPTY + s), (uint32_t)(((j >> 1) & 1) ^ 1)));
        if (!ok) { fail(ST_WAIT_KEMPTY); break; }
        xform_finish<DC>(p, xr, k_smem + s * C::K_STAGE_BYTES, C::K_CHUNK_BYTES, j * BLOCK_N, p.Sk, tg);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_KFULL + s));
        if (j + 1 < n_tiles) xform_load_next<DC>(p, xr, cur, p.Sk, BLOCK_N);
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

// ---- host side --------------------------------------------------------------------------
template <int DC, int DR, int DV, int MODE, bool ALIBI>
int launch_instance(const KParams& p, cudaStream_t stream) {
  using C = Cfg<DC, DR, DV>;
  auto kern = pe_attn_tc_kernel<DC, DR, DV, MODE, ALIBI>;
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
  const int n_qblk = (p.Sq + Q_TILES * BLOCK_M - 1) / (Q_TILES * BLOCK_M);
  // (batch, head) problems per scheduling group: enough blocks to fill the GPU twice over, but
  // no more heads than keep their K/V (about 48 MB) resident in the 126 MB L2
  const long long kv_bytes_per_head = 2ll * p.Sk * (DC + DR + DV);
  const int bh_group = balanced_bh_group((long long)p.B * p.H, kv_bytes_per_head, p.groups);
  dim3 grid((unsigned)((long long)n_qblk * p.H * p.B)), block(NTHREADS);
  kern<<<grid, block, C::SMEM_BYTES, stream>>>(p, bh_group, tmQ, tmK, tmV);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("tcgen05 kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

template <int DC, int DR, int DV, int MODE>
int launch_alibi(const KParams& p, cudaStream_t stream) {
  if (p.variant == PE_ATTN_ALIBI) return launch_instance<DC, DR, DV, MODE, true>(p, stream);
  return launch_instance<DC, DR, DV, MODE, false>(p, stream);
}

}  // namespace

bool tc_supports(const KParams& p) {
  if (p.variant == PE_ATTN_POPE) {
    return (p.d_c == 64 && p.d_r == 32 && p.d_v == 64) || (p.d_c == 128 && p.d_r == 64 && p.d_v == 128) ||
           (p.d_c == 128 && p.d_r == 32 && p.d_v == 128) || (p.d_c == 0 && p.d_r == 32 && p.d_v == 64) ||
           (p.d_c == 0 && p.d_r == 64 && p.d_v == 128);
  }
  return (p.d_c == 64 && p.d_v == 64) || (p.d_c == 128 && p.d_v == 128);
}

int launch_tc(const KParams& p, cudaStream_t stream) {
  // long sequences at d_v = 128 go to the CTA-pair kernel (two CTAs share every K/V tile)
  if (tc2_supports(p) && p.Sq > 256 && !(p.flags & PE_ATTN_SINGLE_CTA)) return launch_tc2(p, stream);
  // head_dim 64: four query tiles per CTA once there are enough query rows to fill them
  if (tc4_supports(p) && !(p.flags & PE_ATTN_SINGLE_CTA)) return launch_tc4(p, stream);
  if (p.variant == PE_ATTN_POPE) {
    if (p.d_c == 64 && p.d_r == 32) return launch_instance<64, 32, 64, MODE_POPE, false>(p, stream);
    if (p.d_c == 128 && p.d_r == 64) return launch_instance<128, 64, 128, MODE_POPE, false>(p, stream);
    if (p.d_c == 128 && p.d_r == 32) return launch_instance<128, 32, 128, MODE_POPE, false>(p, stream);
    if (p.d_c == 0 && p.d_r == 32) return launch_instance<0, 32, 64, MODE_POPE, false>(p, stream);
    return launch_instance<0, 64, 128, MODE_POPE, false>(p, stream);
  }
  const bool xform = p.variant == PE_ATTN_ROTARY || (p.flags & PE_ATTN_QK_NORM);
  if (p.d_c == 64) {
    return xform ? launch_alibi<64, 0, 64, MODE_XFORM>(p, stream) : launch_alibi<64, 0, 64, MODE_PLAIN>(p, stream);
  }
  return xform ? launch_alibi<128, 0, 128, MODE_XFORM>(p, stream) : launch_alibi<128, 0, 128, MODE_PLAIN>(p, stream);
}

}  // namespace pe_attn
