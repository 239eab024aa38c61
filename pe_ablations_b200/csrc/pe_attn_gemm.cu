// The two GEMMs of the evaluation path whose results never need to exist in HBM, as one
// persistent tcgen05 kernel with fused epilogues.
//
//   C[M, N] = A[M, K] * B[N, K]^T      (bf16 operands, K contiguous; fp32 accumulation in TMEM)
//
// * EPI_CE: the language-model head followed by the cross-entropy
//   (src/model/transformer.py:358-371).  The epilogue rounds a 256 x 256 tile of logits to
//   bf16 (what the head's autocast output holds), reduces it to (max, sum of exp) per row and
//   picks the target's logit; a second small kernel merges the tiles' partial results, forms
//   the row losses and adds them up in a fixed order.  The [tokens, vocab] logits are never
//   written.
// * EPI_SWIGLU: the feed-forward's two input projections followed by SwiGLU
//   (src/model/ffn.py:30-68): CTA 0 of a pair stages the gate weight's rows, CTA 1 the up
//   weight's, so accumulator columns [0, 128) hold the gate and [128, 256) the up projection of
//   the same 128 output columns; the epilogue writes cast(cast(silu(cast(g))) * cast(u)).
// * EPI_STORE: plain C as bf16.
//
// Layout of the work: a cluster of two CTAs (one per SM) owns a 256 x 256 accumulator tile:
// `tcgen05.mma.cta_group::2` M256 N256 K16, each CTA holding 128 rows of A and 128 rows of B
// per 64-wide K step (32 KB per stage, six TMA stages).  One launch runs 74 pairs; pair p takes
// tiles p, p + 74, ... with the M block changing fastest, so the tiles in flight at one time
// share one or two B tiles and A (67 MB at the 1B shape) stays in L2.  The accumulator is
// double-buffered in TMEM (2 x 256 columns): the epilogue warps of tile t run under the MMAs
// of tile t + 1.
//
// Warps: 0 TMA producer (each CTA loads its own halves; byte counts go to the leader's
// barrier), 1 MMA issuer (leader CTA only), 2-5 epilogue (one TMEM lane = one row per thread).
// Every wait is bounded; an expired wait sets the status word and all roles leave.
#include <cuda.h>

#include "pe_attn_tc_common.cuh"

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

constexpr int G_BM = 128;                          // rows of A per CTA (256 per pair)
constexpr int G_BN = 256;                          // accumulator columns of a tile
constexpr int G_BK = 64;                           // one 128-byte swizzled row of bf16
#ifndef PE_GEMM_STAGES
#define PE_GEMM_STAGES 7
#endif
constexpr int G_STAGES = PE_GEMM_STAGES;
constexpr int G_A_BYTES = G_BM * G_BK * 2;         // 16 KB
constexpr int G_B_BYTES = (G_BN / 2) * G_BK * 2;   // 16 KB: this CTA's half of the B tile
constexpr int G_STAGE_BYTES = G_A_BYTES + G_B_BYTES;
constexpr int G_SMEM = 1024 + G_STAGES * G_STAGE_BYTES + 1024;
static_assert(G_SMEM <= 232448, "more shared memory than a CTA can have");
constexpr int G_THREADS = 192;
constexpr uint32_t G_TMEM_COLS = 512;
enum { GB_FULL = 0, GB_EMPTY = G_STAGES, GB_ACCFULL = 2 * G_STAGES, GB_ACCEMPTY = 2 * G_STAGES + 2 };
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_CE = 2 };

#ifndef PE_GEMM_PRODUCER_WAIT
#define PE_GEMM_PRODUCER_WAIT mbar_wait_spin
#endif

constexpr float kLog2e = 1.4426950408889634f;

struct GemmParams {
  int M, N, K;                  // N: accumulator columns (EPI_SWIGLU: twice the output columns)
  int n_mblk, n_ntile;          // tiles of 256 rows / 256 accumulator columns
  int gm, pn, rounds, n_iter;   // tile order, see tile_of()
  __nv_bfloat16* out;           // EPI_STORE [M, N], EPI_SWIGLU [M, N / 2]
  long long out_stride;         // elements
  const __nv_bfloat16* residual; // EPI_STORE, optional [M, N]: C = cast(cast(A B^T) + residual)
  long long res_stride;
  const long long* targets;     // EPI_CE [M]
  int vocab;                    // EPI_CE: columns >= vocab are padding
  float2* part;                 // EPI_CE [n_ntile][m_pad]: (max, sum of exp(x - max)) per row and tile
  float* tgt_logit;             // EPI_CE [m_pad]
  int m_pad;
  int* status;
};

// Tile order.  Pair (i, j) = (pair % gm, pair / gm) works on row block sb * gm + i for one
// super-block sb after the other, and inside a super-block on column tiles j, j + pn, ...: it
// re-reads its own A rows (1 MB at K = 2048) tile after tile, so they stay in the half of L2
// next to it, and the gm pairs that share j read the same B tile at the same time.  (With the
// row block changing fastest instead, every tile streamed A through L2 and three in ten sectors
// came from the far half: 0.75 PFLOP/s, whatever the number of stages.)
__device__ __forceinline__ bool tile_of(const GemmParams& p, int pair, int it, int& mb, int& nb) {
  if (p.gm == 0) {   // round robin over all pairs, row block fastest
    const int t = pair + it * p.pn;
    mb = t % p.n_mblk;
    nb = t / p.n_mblk;
    return t < p.n_mblk * p.n_ntile;
  }
  const int i = pair % p.gm, j = pair / p.gm;
  const int sb = it / p.rounds, r = it - sb * p.rounds;
  mb = sb * p.gm + i;
  nb = r * p.pn + j;
  return j < p.pn && mb < p.n_mblk && nb < p.n_ntile;
}

// 32-byte store (one full sector per thread)
__device__ __forceinline__ void stg_v8(void* ptr, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

#ifdef PE_GEMM_TRACE
__device__ long long g_trace[148 * 16];
#define TR_ADD(slot, v) do { if (lane == 0) g_trace[blockIdx.x * 16 + (slot)] += (v); } while (0)
#define TR_T() clock64()
#else
#define TR_ADD(slot, v) do { } while (0)
#define TR_T() 0ll
#endif

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G_THREADS, 1)
pe_gemm_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmB2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 256);
  volatile uint32_t* abort_slot = reinterpret_cast<volatile uint32_t*>(smem + 260);
  auto bar = [&](int idx) -> uint32_t { return smem_base + 8u * (uint32_t)idx; };
  auto lbar = [&](int idx) -> uint32_t { return mapa(bar(idx), 0); };   // the leader's copy
  const uint32_t stage0 = smem_base + 1024u;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const uint32_t rank = cluster_ctarank();
  const int pair = (int)(blockIdx.x >> 1);
  const int k_steps = (p.K + G_BK - 1) / G_BK;

  auto fail = [&](int code) {
    if (p.status != nullptr) atomicOr(p.status, code);
  };

  if (tid == 0) {
    *abort_slot = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
    for (int s = 0; s < G_STAGES; ++s) {
      mbar_init(bar(GB_FULL + s), 2);     // one arrive.expect_tx from each CTA's producer
      mbar_init(bar(GB_EMPTY + s), 1);    // tcgen05.commit, multicast to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(GB_ACCFULL + b), 1);
      mbar_init(bar(GB_ACCEMPTY + b), 8);  // 4 epilogue warps x 2 CTAs, on the leader's copy
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), G_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool run = *abort_slot == 0;

  if (!run) {
    // an earlier kernel on this status word reported an expired wait: do nothing
  } else if (warp == 0) {
    // ===================== TMA producer =====================
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if constexpr (EPI == EPI_SWIGLU) tma_prefetch_desc(&tmB2);
    }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    [[maybe_unused]] const long long tr0 = TR_T();
#pragma unroll 1
    for (int ti = 0; ti < p.n_iter && ok; ++ti) {
      int mb, nb;
      if (!tile_of(p, pair, ti, mb, nb)) continue;
      const int a_row = mb * 2 * G_BM + (int)rank * G_BM;
      // EPI_SWIGLU: the leader stages the gate weight's rows, the other CTA the up weight's
      const CUtensorMap* mapB = (EPI == EPI_SWIGLU && rank == 1) ? &tmB2 : &tmB;
      const int b_row = EPI == EPI_SWIGLU ? nb * (G_BN / 2) : nb * G_BN + (int)rank * (G_BN / 2);
#pragma unroll 1
      for (int ks = 0; ks < k_steps; ++ks) {
        [[maybe_unused]] const long long tw0 = TR_T();
        // polled, not suspended: a late refill shortens the pipeline by the wake-up time
        if (!__all_sync(0xffffffffu, PE_GEMM_PRODUCER_WAIT(bar(GB_EMPTY + s), ph ^ 1u))) { fail(ST_WAIT_KEMPTY); ok = false; break; }
        [[maybe_unused]] const long long tw1 = TR_T();
        TR_ADD(1, tw1 - tw0);
        if (elect_one()) {
          const uint32_t fb = lbar(GB_FULL + s);
          const uint32_t dst = stage0 + (uint32_t)(s * G_STAGE_BYTES);
          // relaxed: the arrival publishes nothing this thread wrote (the tile comes through the
          // async proxy and its complete_tx); with .release each arrival cost about 600 clocks
#ifdef PE_GEMM_RELEASE_ARRIVE   // the slow form, kept so that the measurement can be repeated
          mbar_arrive_expect_tx_cluster(fb, G_STAGE_BYTES);
#else
          mbar_arrive_expect_tx_cluster_relaxed(fb, G_STAGE_BYTES);
#endif
          tma_load_4d_pair(dst, &tmA, fb, ks * G_BK, a_row, 0, 0);
          tma_load_4d_pair(dst + G_A_BYTES, mapB, fb, ks * G_BK, b_row, 0, 0);
        }
        __syncwarp();
        TR_ADD(2, TR_T() - tw1);
        if (++s == G_STAGES) { s = 0; ph ^= 1u; }
      }
    }
    TR_ADD(0, TR_T() - tr0);
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA only) =====================
    if (rank == 0) {
      constexpr uint32_t IDESC = make_idesc_bf16(2 * G_BM, G_BN, false);
      constexpr uint16_t BOTH = 3;
      int s = 0, it = 0;
      uint32_t ph = 0;
      bool ok = true;
      [[maybe_unused]] const long long tr0 = TR_T();
#pragma unroll 1
      for (int ti = 0; ti < p.n_iter && ok; ++ti) {
        int mb, nb;
        if (!tile_of(p, pair, ti, mb, nb)) continue;
        const int buf = it & 1;
        [[maybe_unused]] const long long ta0 = TR_T();
        // the epilogue warps of both CTAs have read this accumulator's previous tile
        if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(GB_ACCEMPTY + buf), (uint32_t)(((it >> 1) & 1) ^ 1)))) {
          fail(ST_WAIT_PVDONE);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        TR_ADD(5, TR_T() - ta0);
        const uint32_t d = tmem_base + (uint32_t)(buf * G_BN);
#pragma unroll 1
        for (int ks = 0; ks < k_steps; ++ks) {
          [[maybe_unused]] const long long tf0 = TR_T();
          if (!__all_sync(0xffffffffu, mbar_wait_spin(bar(GB_FULL + s), ph))) { fail(ST_WAIT_KFULL); ok = false; break; }
          tc_fence_after_sync();
          TR_ADD(4, TR_T() - tf0);
          if (elect_one()) {
            const uint32_t a_s = stage0 + (uint32_t)(s * G_STAGE_BYTES);
            const uint64_t ad = make_smem_desc(a_s, 16, 1024);
            const uint64_t bd = make_smem_desc(a_s + G_A_BYTES, 16, 1024);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
              mma_ss_pair(d, advance_smem_desc(ad, (uint32_t)(k4 * 32)), advance_smem_desc(bd, (uint32_t)(k4 * 32)), IDESC,
                          (ks > 0 || k4 > 0) ? 1u : 0u);
            tc_commit_pair(bar(GB_EMPTY + s), BOTH);
          }
          __syncwarp();
          if (++s == G_STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit_pair(bar(GB_ACCFULL + buf), BOTH);
        __syncwarp();
        ++it;
      }
      TR_ADD(3, TR_T() - tr0);
    }
  } else {
    // ===================== epilogue: TMEM lane = row, 4 warps cover the CTA's 128 rows ==========
    const int quarter = warp & 3;                        // the TMEM lanes this warp may read
    const int row_in_cta = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    int it = 0;
    bool ok = true;
    [[maybe_unused]] const long long tr0 = TR_T();
#pragma unroll 1
    for (int ti = 0; ti < p.n_iter && ok; ++ti) {
      int mb, nb;
      if (!tile_of(p, pair, ti, mb, nb)) continue;
      const int buf = it & 1;
      [[maybe_unused]] const long long te0 = TR_T();
      const int row = mb * 2 * G_BM + (int)rank * G_BM + row_in_cta;
      const bool row_ok = row < p.M;
      if (!__all_sync(0xffffffffu, mbar_wait(bar(GB_ACCFULL + buf), (uint32_t)((it >> 1) & 1)))) {
        fail(ST_WAIT_SFULL);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      if (warp == 2) TR_ADD(7, TR_T() - te0);
      const uint32_t acc = lane_addr + (uint32_t)(buf * G_BN);

      if constexpr (EPI == EPI_CE) {
        const int n0 = nb * G_BN;
        const bool ragged = n0 + G_BN > p.vocab;
        long long tgt = -1;
        if (row_ok) tgt = p.targets[row];
        const int rel = (tgt >= n0 && tgt < (long long)n0 + G_BN) ? (int)(tgt - n0) : -1;
        float mx = -INFINITY, sum = 0.f, picked = 0.f;
#pragma unroll 1
        for (int c = 0; c < G_BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(acc + (uint32_t)(c * 32), r);
          tmem_wait_ld();
          float x[32];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint32_t w = pack_bf16x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            x[i] = bf16_lo(w);
            x[i + 1] = bf16_hi(w);
          }
          if (ragged) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + c * 32 + i >= p.vocab) x[i] = -INFINITY;
          }
          if ((unsigned)(rel - c * 32) < 32u) {
            const int want = rel - c * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i == want) picked = x[i];
          }
          float cm = x[0];
#pragma unroll
          for (int i = 1; i < 31; i += 2) cm = fmax3(cm, x[i], x[i + 1]);
          cm = fmaxf(cm, x[31]);
          const float m_new = fmaxf(mx, cm);
          if (m_new != -INFINITY) {      // all -inf so far: nothing to add (and -inf - -inf is NaN)
            const float base = m_new * kLog2e;
            float acc_s = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) acc_s += ex2_approx(fmaf(x[i], kLog2e, -base));
            sum = sum * ex2_approx(fmaf(mx, kLog2e, -base)) + acc_s;
            mx = m_new;
          }
        }
        if (row_ok) {
          p.part[(size_t)nb * p.m_pad + row] = make_float2(mx, sum);
          if (rel >= 0) p.tgt_logit[row] = picked;
        }
      } else {
        constexpr int OUT_COLS = EPI == EPI_SWIGLU ? G_BN / 2 : G_BN;
        const int c0 = nb * OUT_COLS;
        const int n_out = EPI == EPI_SWIGLU ? p.N / 2 : p.N;
        __nv_bfloat16* orow = p.out + (size_t)(row_ok ? row : 0) * p.out_stride + c0;
        const bool wide = ((reinterpret_cast<uintptr_t>(p.out) | (uintptr_t)(p.out_stride * 2)) & 31u) == 0;  // 32-byte rows
#pragma unroll 1
        for (int c = 0; c < OUT_COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(acc + (uint32_t)(c * 32), r);
          uint32_t w[16];
          if constexpr (EPI == EPI_SWIGLU) {
            uint32_t u[32];
            tmem_ld32(acc + (uint32_t)(G_BN / 2 + c * 32), u);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              // gate and up as the bf16 values the two projections would have written
              const uint32_t gw = pack_bf16x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
              const uint32_t uw = pack_bf16x2(__uint_as_float(u[i]), __uint_as_float(u[i + 1]));
              const float g0 = bf16_lo(gw), g1 = bf16_hi(gw);
              const float s0 = round_bf16(g0 / (1.0f + __expf(-g0))), s1 = round_bf16(g1 / (1.0f + __expf(-g1)));
              w[i >> 1] = pack_bf16x2(s0 * bf16_lo(uw), s1 * bf16_hi(uw));
            }
          } else {
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 2) w[i >> 1] = pack_bf16x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            if (p.residual != nullptr && row_ok && c0 + c * 32 + 32 <= n_out) {
              // the residual stream's add (h = x + wo(..), out = h + w2(..)), rounded like the
              // bf16 add of the projection's bf16 output it replaces
              const uint4* rp = reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.res_stride + c0 + c * 32);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const uint4 rv = __ldg(rp + q4);
                const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const uint32_t cw = w[q4 * 4 + e];
                  w[q4 * 4 + e] = pack_bf16x2(bf16_lo(cw) + bf16_lo(rr[e]), bf16_hi(cw) + bf16_hi(rr[e]));
                }
              }
            } else if (p.residual != nullptr && row_ok) {
              for (int i = 0; i < 32 && c0 + c * 32 + i < n_out; ++i) {
                const float rv = __bfloat162float(p.residual[(size_t)row * p.res_stride + c0 + c * 32 + i]);
                const uint32_t cw = w[i >> 1];
                const float cv = (i & 1) ? bf16_hi(cw) : bf16_lo(cw);
                const uint32_t nv = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(cv + rv));
                w[i >> 1] = (i & 1) ? ((cw & 0xFFFFu) | (nv << 16)) : ((cw & 0xFFFF0000u) | nv);
              }
            }
          }
          if (row_ok) {
            const int col = c0 + c * 32;
            if (col + 32 <= n_out && wide) {
              stg_v8(orow + c * 32, w);
              stg_v8(orow + c * 32 + 16, w + 8);
            } else if (col + 32 <= n_out) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            } else {
              for (int i = 0; i < 32 && col + i < n_out; ++i) {
                const uint32_t ww = w[i >> 1];
                reinterpret_cast<uint16_t*>(orow + c * 32)[i] = (uint16_t)((i & 1) ? (ww >> 16) : (ww & 0xFFFFu));
              }
            }
          }
        }
      }
      // this warp is done with the accumulator: let the leader's MMA warp reuse it
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(lbar(GB_ACCEMPTY + buf));   // TMEM reads, ordered by the tcgen05 fence
      ++it;
    }
    if (warp == 2) TR_ADD(6, TR_T() - tr0);
  }

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
    tmem_dealloc_pair(tmem_base, G_TMEM_COLS);
  }
}

// Row losses from the tiles' partial results, then their sum in a fixed order by the last CTA
// to finish (as the stand-alone cross-entropy kernel does).
constexpr int FIN_THREADS = 256;
__global__ void __launch_bounds__(FIN_THREADS)
head_ce_finalize_kernel(const GemmParams p, const int ignore_index, float* row_loss, unsigned int* counter, double* out) {
  __shared__ bool is_last;
  __shared__ double red_a[FIN_THREADS], red_c[FIN_THREADS];
  const int tid = threadIdx.x;
  const int row = blockIdx.x * FIN_THREADS + tid;
  if (row < p.M) {
    const long long tgt = p.targets[row];
    float loss = -INFINITY;   // not scored
    if (tgt != ignore_index) {
      float m = -INFINITY, s = 0.f;
      for (int nb = 0; nb < p.n_ntile; ++nb) {
        const float2 ps = p.part[(size_t)nb * p.m_pad + row];
        const float mm = fmaxf(m, ps.x);
        if (mm != -INFINITY) {
          s = s * __expf(m - mm) + ps.y * __expf(ps.x - mm);
          m = mm;
        }
      }
      loss = (tgt >= 0 && tgt < p.vocab) ? (m + logf(s)) - p.tgt_logit[row] : __int_as_float(0x7fc00000);
    }
    row_loss[row] = loss;
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned done = atomicAdd(counter, 1u);
    is_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  double acc = 0.0, cnt = 0.0;
  for (int r = tid; r < p.M; r += FIN_THREADS) {
    const float l = reinterpret_cast<volatile float*>(row_loss)[r];
    if (l != -INFINITY) { acc += (double)l; cnt += 1.0; }
  }
  red_a[tid] = acc;
  red_c[tid] = cnt;
  __syncthreads();
  for (int w = FIN_THREADS / 2; w > 0; w >>= 1) {
    if (tid < w) { red_a[tid] += red_a[tid + w]; red_c[tid] += red_c[tid + w]; }
    __syncthreads();
  }
  if (tid == 0) {
    out[0] += red_a[0];
    out[1] += red_c[0];
    *counter = 0u;
  }
}

// [rows, K] bf16 matrix, rows ``stride`` elements apart, as a TMA tensor with a (64 x 128) box
bool encode_matrix(CUtensorMap* map, const void* ptr, long long stride, int rows, int K) {
  TensorRef t{ptr, stride * (long long)rows, stride * (long long)rows, stride};
  return encode_map(map, t, K, rows, 1, 1, G_BM);
}

template <int EPI>
int launch_gemm(const GemmParams& p, const void* a, long long a_stride, const void* b, long long b_stride, const void* b2,
                int b_rows, cudaStream_t stream) {
  auto kern = pe_gemm_pair_kernel<EPI>;
  static PerDeviceOnce configured;
  int cfg_dev;
  if (configured.pending(&cfg_dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(%d bytes) failed: %s", G_SMEM, cudaGetErrorString(e));
      return PE_ATTN_ERR_LAUNCH;
    }
    configured.mark(cfg_dev);
  }
  CUtensorMap tmA, tmB, tmB2;
  if (!encode_matrix(&tmA, a, a_stride, p.M, p.K) || !encode_matrix(&tmB, b, b_stride, b_rows, p.K) ||
      !encode_matrix(&tmB2, b2 != nullptr ? b2 : b, b_stride, b_rows, p.K)) {
    set_error("cuTensorMapEncodeTiled failed for a GEMM operand");
    return PE_ATTN_ERR_LAUNCH;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  // rows of pairs (gm) x columns of pairs (pn): the fewest iterations, then the largest gm (B is
  // read from HBM once per super-block of gm row blocks)
  GemmParams q = p;
  long long best = -1;
  for (int gm = 1; gm <= pairs && gm <= p.n_mblk; ++gm) {
    const int pn = pairs / gm;
    const int rounds = (p.n_ntile + pn - 1) / pn;
    const long long iters = (long long)((p.n_mblk + gm - 1) / gm) * rounds;
    if (best < 0 || iters <= best) {
      best = iters;
      q.gm = gm;
      q.pn = pn;
      q.rounds = rounds;
      q.n_iter = (int)iters;
    }
  }
  // The grid of pairs leaves pairs idle when the column tiles do not divide (8 column tiles at
  // N = 2048 use 64 of 74 pairs): beyond 8 % more iterations than a plain round robin over all
  // tiles (row block fastest), take the round robin.  Where both fit, the grid is faster (the
  // SwiGLU GEMM: 1 479 against 1 271 TFLOP/s), where it does not, the round robin is (N = 2048:
  // 1 424 against 1 324).
  const long long linear_iters = ((long long)p.n_mblk * p.n_ntile + pairs - 1) / pairs;
  if (best * 100 > linear_iters * 108) {
    q.gm = 0;
    q.pn = pairs;
    q.rounds = 1;
    q.n_iter = (int)linear_iters;
  }
  kern<<<dim3((unsigned)(2 * pairs)), G_THREADS, G_SMEM, stream>>>(q, tmA, tmB, tmB2);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("tcgen05 GEMM launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

int check_matrix(const char* name, const void* ptr, long long stride, int K) {
  if (ptr == nullptr) {
    set_error("%s is null", name);
    return PE_ATTN_ERR_NULL;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) || stride < K || (stride % 8) != 0) {
    set_error("%s must be 16-byte aligned with a row stride that is a multiple of 8 elements and >= K", name);
    return PE_ATTN_ERR_ALIGNMENT;
  }
  return PE_ATTN_OK;
}

inline size_t align256(size_t x) { return (x + 255u) & ~(size_t)255u; }

}  // namespace
}  // namespace pe_attn

extern "C" {

using namespace pe_attn;

size_t pe_lm_head_ce_workspace_bytes(int n_rows, int vocab) {
  if (n_rows < 1 || vocab < 1) return 0;
  const size_t m_pad = (size_t)((n_rows + 255) / 256) * 256;
  const size_t n_ntile = (size_t)(vocab + G_BN - 1) / G_BN;
  // counter block, row losses, target logits, per-tile (max, sum) pairs
  return 256 + align256(m_pad * 4) + align256(m_pad * 4) + n_ntile * m_pad * sizeof(float2);
}

int pe_lm_head_ce_loss_sums(const void* hidden, int64_t hidden_stride, const void* weight, int64_t weight_stride,
                            const int64_t* targets, int n_rows, int hidden_dim, int vocab, int ignore_index,
                            void* workspace, size_t workspace_bytes, double* out, int32_t* device_status, void* stream) {
  if (targets == nullptr || out == nullptr || workspace == nullptr) {
    set_error("targets, out or workspace is null");
    return PE_ATTN_ERR_NULL;
  }
  if (n_rows < 1 || vocab < 1 || hidden_dim < 64 || (hidden_dim % 8) != 0) {
    set_error("need n_rows >= 1, vocab >= 1 and hidden_dim >= 64, a multiple of 8 (got %d, %d, %d)", n_rows, vocab,
              hidden_dim);
    return PE_ATTN_ERR_SHAPE;
  }
  int rc = check_matrix("hidden", hidden, hidden_stride, hidden_dim);
  if (rc == PE_ATTN_OK) rc = check_matrix("weight", weight, weight_stride, hidden_dim);
  if (rc != PE_ATTN_OK) return rc;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || (reinterpret_cast<uintptr_t>(out) & 7u)) {
    set_error("workspace must be 256-byte aligned and out 8-byte aligned");
    return PE_ATTN_ERR_ALIGNMENT;
  }
  if (workspace_bytes < pe_lm_head_ce_workspace_bytes(n_rows, vocab)) {
    set_error("workspace of %zu bytes is smaller than pe_lm_head_ce_workspace_bytes() = %zu", workspace_bytes,
              pe_lm_head_ce_workspace_bytes(n_rows, vocab));
    return PE_ATTN_ERR_SHAPE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GemmParams p{};
  p.M = n_rows;
  p.N = vocab;
  p.K = hidden_dim;
  p.n_mblk = (n_rows + 255) / 256;
  p.n_ntile = (vocab + G_BN - 1) / G_BN;
  p.m_pad = p.n_mblk * 256;
  p.targets = reinterpret_cast<const long long*>(targets);
  p.vocab = vocab;
  char* ws = reinterpret_cast<char*>(workspace);
  unsigned int* counter = reinterpret_cast<unsigned int*>(ws);
  float* row_loss = reinterpret_cast<float*>(ws + 256);
  p.tgt_logit = reinterpret_cast<float*>(ws + 256 + align256((size_t)p.m_pad * 4));
  p.part = reinterpret_cast<float2*>(ws + 256 + 2 * align256((size_t)p.m_pad * 4));
  p.status = device_status;
  if (cudaMemsetAsync(counter, 0, 256, st) != cudaSuccess) {
    set_error("clearing the workspace's counter block failed");
    return PE_ATTN_ERR_LAUNCH;
  }
  rc = launch_gemm<EPI_CE>(p, hidden, hidden_stride, weight, weight_stride, nullptr, vocab, st);
  if (rc != PE_ATTN_OK) return rc;
  head_ce_finalize_kernel<<<(unsigned)((n_rows + FIN_THREADS - 1) / FIN_THREADS), FIN_THREADS, 0, st>>>(
      p, ignore_index, row_loss, counter, out);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("loss finalisation kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

int pe_swiglu_gemm(const void* x, int64_t x_stride, const void* w_gate, const void* w_up, int64_t w_stride, void* y,
                   int64_t y_stride, int n_rows, int hidden_dim, int ffn_dim, int32_t* device_status, void* stream) {
  if (y == nullptr) {
    set_error("y is null");
    return PE_ATTN_ERR_NULL;
  }
  if (n_rows < 1 || ffn_dim < 8 || (ffn_dim % 8) != 0 || hidden_dim < 64 || (hidden_dim % 8) != 0) {
    set_error("need n_rows >= 1, ffn_dim >= 8, hidden_dim >= 64, both multiples of 8 (got %d, %d, %d)", n_rows, hidden_dim,
              ffn_dim);
    return PE_ATTN_ERR_SHAPE;
  }
  int rc = check_matrix("x", x, x_stride, hidden_dim);
  if (rc == PE_ATTN_OK) rc = check_matrix("w_gate", w_gate, w_stride, hidden_dim);
  if (rc == PE_ATTN_OK) rc = check_matrix("w_up", w_up, w_stride, hidden_dim);
  if (rc == PE_ATTN_OK) rc = check_matrix("y", y, y_stride, ffn_dim);
  if (rc != PE_ATTN_OK) return rc;
  GemmParams p{};
  p.M = n_rows;
  p.N = 2 * ffn_dim;
  p.K = hidden_dim;
  p.n_mblk = (n_rows + 255) / 256;
  p.n_ntile = (ffn_dim + G_BN / 2 - 1) / (G_BN / 2);
  p.out = reinterpret_cast<__nv_bfloat16*>(y);
  p.out_stride = y_stride;
  p.status = device_status;
  return launch_gemm<EPI_SWIGLU>(p, x, x_stride, w_gate, w_stride, w_up, ffn_dim, static_cast<cudaStream_t>(stream));
}

#ifdef PE_GEMM_TRACE
int pe_gemm_trace_read(long long* host, int clear) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host, g_trace, sizeof(long long) * 148 * 16);
  if (clear) {
    static long long zeros[148 * 16];
    cudaMemcpyToSymbol(g_trace, zeros, sizeof(zeros));
  }
  return 0;
}
#endif

int pe_gemm_nt(const void* a, int64_t a_stride, const void* b, int64_t b_stride, void* c, int64_t c_stride,
               const void* residual, int64_t residual_stride, int m, int n, int k, int32_t* device_status, void* stream) {
  if (c == nullptr) {
    set_error("c is null");
    return PE_ATTN_ERR_NULL;
  }
  if (m < 1 || n < 8 || (n % 8) != 0 || k < 64 || (k % 8) != 0) {
    set_error("need m >= 1, n >= 8, k >= 64 (one 128-byte TMA row), n and k multiples of 8 (got %d, %d, %d)", m, n, k);
    return PE_ATTN_ERR_SHAPE;
  }
  int rc = check_matrix("a", a, a_stride, k);
  if (rc == PE_ATTN_OK) rc = check_matrix("b", b, b_stride, k);
  if (rc == PE_ATTN_OK) rc = check_matrix("c", c, c_stride, n);
  if (rc == PE_ATTN_OK && residual != nullptr) rc = check_matrix("residual", residual, residual_stride, n);
  if (rc != PE_ATTN_OK) return rc;
  GemmParams p{};
  p.M = m;
  p.N = n;
  p.K = k;
  p.n_mblk = (m + 255) / 256;
  p.n_ntile = (n + G_BN - 1) / G_BN;
  p.out = reinterpret_cast<__nv_bfloat16*>(c);
  p.out_stride = c_stride;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.res_stride = residual_stride;
  p.status = device_status;
  return launch_gemm<EPI_STORE>(p, a, a_stride, b, b_stride, nullptr, n, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
