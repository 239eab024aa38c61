// Split-KV forward for decode steps: a handful of query rows against a long cached K/V.
//
// With one to eight query rows per K/V head (one new token, or a short chunk, times the GQA
// ratio) the work is a single pass over the cache: HBM-bound, no tensor-core shape.  The
// query-tiled kernels give such a call one CTA per head; this one cuts the keys of every
// (batch, K/V head) into splits so that about two CTAs per SM stream the cache, each keeping
// its own running maximum, sum and un-normalised output, and a second small kernel merges the
// splits (the same logsumexp algebra as between key tiles).
//
// One CTA = 256 threads, tiles of 64 keys, 2-4 TMA stages (raw K halves and V, 128-byte
// swizzle; 64-byte swizzle for a 32-column positional half).  Warp w owns keys 8w..8w+7 of
// every tile, start to end, with its own running maximum, sum and output, so the warps never
// wait for each other inside a tile:
//   scores   lane = (key, quarter of the 16-byte column slots): reads its key's slots from the
//            swizzled tile (conflict-free: 8 consecutive keys per quarter-warp), applies the
//            positional transform in registers (rotation / L2 norm factor / softplus magnitude
//            and phase), multiplies with the query rows held in shared memory as fp32 (already
//            transformed, scaled by scale * log2 e); two shuffles join the quarters
//   softmax  maximum over the warp's 8 keys by shuffles, rescale, probabilities in registers
//   values   lane = 4 (or 2) value columns: O_w += p_j * V_j for the 8 keys, p_j by shuffle
// A warp that is done with a tile adds one to the stage's counter; the warp that brings it to
// eight issues the TMA refill of that stage (no producer warp, no block-wide barrier in the
// loop).  After the last tile the eight warps' (max, sum, output) are merged through shared
// memory and written as the split's partial result.
//
// The transforms restate src/model/rope.py:35-57, src/model/normalization.py:44-56,
// src/model/pope.py:124-183 and src/model/fpope.py:266-338 of the reference; the call is what
// its cache modules do per generated token (src/model/fpope_attention.py:180-271).
#include <cstring>

#include "pe_attn_tc_common.cuh"

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

constexpr int TK = 64;             // keys per tile
constexpr int NT = 256;            // threads per CTA
constexpr int NWARP = NT / 32;
constexpr int MAX_ROWS = 8;        // query rows per K/V head (GQA ratio x Sq)
constexpr int MAX_SPLITS = 64;
constexpr int TARGET_CTAS = 296;   // two co-resident CTAs on each of 148 SMs
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeParams {
  int rows, n_splits, tiles_per_split;
  float* part_o;    // [B*H*Sq, n_splits, d_v]
  float2* part_ml;  // [B*H*Sq, n_splits] (running maximum in log2 units, sum)
};

template <int DC, int DR, int DV, int R_T>
struct DCfg {
  static constexpr int DQK = DC + 2 * DR;
  static constexpr int K_BYTES = TK * DC * 2;
  static constexpr int V_BYTES = TK * DV * 2;
  static constexpr int KR_BYTES = TK * DR * 2;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES + KR_BYTES;
  static constexpr int NSTAGE = STAGE_BYTES >= 32768 ? 2 : (STAGE_BYTES >= 20480 ? 3 : 4);
  static constexpr int RED_BYTES = NWARP * R_T * (DV + 2) * 4;   // end-of-kernel merge, reuses the stages
  static_assert(RED_BYTES <= NSTAGE * STAGE_BYTES, "reduction buffer must fit the stages");
  static_assert(STAGE_BYTES % 1024 == 0, "stages keep the 1024-byte swizzle alignment");
  // after the stages: query rows, per-row slope and causal limit, frequencies, stage counters, barriers
  static constexpr int OFF_Q = NSTAGE * STAGE_BYTES;
  static constexpr int OFF_ROW = OFF_Q + R_T * DQK * 4;
  static constexpr int OFF_FREQ = (OFF_ROW + 2 * R_T * 4 + 15) & ~15;   // read as float4
  // frequency, phase bias, cos / sin of one tile's advance (PoPE); or the (cos, sin) of one tile's
  // advance of every rotary column pair (DC floats)
  static constexpr int OFF_CNT = OFF_FREQ + (4 * (DR > 0 ? DR : 4) * 4 > DC * 4 ? 4 * (DR > 0 ? DR : 4) * 4 : DC * 4);
  static constexpr int OFF_BAR = (OFF_CNT + NSTAGE * 4 + 7) & ~7;
  static constexpr int SMEM_BYTES = OFF_BAR + NSTAGE * 8 + 1024;   // + slack for the 1024-byte alignment
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = bf16_lo(w[e]);
    f[2 * e + 1] = bf16_hi(w[e]);
  }
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
  return x;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}

// One query row, transformed as the forward kernels transform it (rounded to bf16 once), times
// scale * log2 e, as fp32 in shared memory.  One warp per row.
template <int DC, int DR, int MODE>
__device__ void build_query_row(const KParams& p, float* dst, int b, int h, int qi, const float* freq_s, int lane) {
  const float sc = p.scale * kLog2e;
  const int pos = p.q_pos0 + qi;
  if constexpr (DC > 0) {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.q.ptr) + (long long)b * p.q.sb +
                               (long long)h * p.q.sh + (long long)qi * p.q.ss;
    constexpr int PPL = DC / 64;   // pairs per lane
    float o[PPL][2];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PPL; ++i) {
      const int pr = lane + 32 * i;
      float x0 = __bfloat162float(src[2 * pr]), x1 = __bfloat162float(src[2 * pr + 1]);
      if (MODE == MODE_XFORM && p.variant == PE_ATTN_ROTARY) {
        const float2 cs = reinterpret_cast<const float2*>(p.table)[(size_t)(pos - p.table_pos0) * (DC / 2) + pr];
        const float r0 = x0 * cs.x - x1 * cs.y, r1 = x0 * cs.y + x1 * cs.x;
        x0 = r0 * p.mscale;
        x1 = r1 * p.mscale;
      }
      o[i][0] = x0;
      o[i][1] = x1;
      ss = fmaf(x0, x0, fmaf(x1, x1, ss));
    }
    float inv = 1.0f;
    if (MODE == MODE_XFORM && (p.flags & PE_ATTN_QK_NORM)) inv = 1.0f / (sqrtf(warp_sum(ss)) + p.eps);
#pragma unroll
    for (int i = 0; i < PPL; ++i) {
      const int pr = lane + 32 * i;
      dst[2 * pr] = round_bf16(o[i][0] * inv) * sc;
      dst[2 * pr + 1] = round_bf16(o[i][1] * inv) * sc;
    }
  }
  if constexpr (MODE == MODE_POPE) {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.qr.ptr) + (long long)b * p.qr.sb +
                               (long long)h * p.qr.sh + (long long)qi * p.qr.ss;
    for (int c = lane; c < DR; c += 32) {
      const float mu = softplus_fast(__bfloat162float(src[c]));
      float sn, cs;
      sincos_reduced(__fmul_rn((float)pos, freq_s[c]), &sn, &cs);   // queries carry no phase bias
      dst[DC + c] = round_bf16(mu * cs) * sc;
      dst[DC + DR + c] = round_bf16(mu * sn) * sc;
    }
  }
}

template <int DC, int DR, int DV, int MODE, int R_T>
__global__ void __launch_bounds__(NT, 2)
pe_attn_decode_kernel(const KParams p, const DecodeParams dp, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmKR, const __grid_constant__ CUtensorMap tmV) {
  using C = DCfg<DC, DR, DV, R_T>;
  constexpr int DQK = C::DQK;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw_u32);
  float* sQ = reinterpret_cast<float*>(gen + C::OFF_Q);
  float* sSlope = reinterpret_cast<float*>(gen + C::OFF_ROW);
  int* sLim = reinterpret_cast<int*>(sSlope + R_T);
  int* sCnt = reinterpret_cast<int*>(gen + C::OFF_CNT);
  float* freq_s = reinterpret_cast<float*>(gen + C::OFF_FREQ);
  float* delta_s = freq_s + (DR > 0 ? DR : 4);
  float* rot_c = delta_s + (DR > 0 ? DR : 4);
  float* rot_s = rot_c + (DR > 0 ? DR : 4);
  const uint32_t bar0 = base + C::OFF_BAR;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int R = dp.rows;
  const int tile0 = split * dp.tiles_per_split;
  int n_tiles = (p.Sk + TK - 1) / TK - tile0;
  if (n_tiles > dp.tiles_per_split) n_tiles = dp.tiles_per_split;
  if (n_tiles < 0) n_tiles = 0;

  auto issue = [&](int t) {   // one thread
    const int stage = t % C::NSTAGE;
    const uint32_t dst = base + stage * C::STAGE_BYTES, bar = bar0 + stage * 8;
    const int row = (tile0 + t) * TK;
    mbar_arrive_expect_tx(bar, C::STAGE_BYTES);
#pragma unroll
    for (int c = 0; c < DC / 64; ++c) tma_load_4d(dst + c * 8192, &tmK, bar, c * 64, row, hk, b);
#pragma unroll
    for (int c = 0; c < DV / 64; ++c) tma_load_4d(dst + C::K_BYTES + c * 8192, &tmV, bar, c * 64, row, hk, b);
    if constexpr (DR > 0) tma_load_4d(dst + C::K_BYTES + C::V_BYTES, &tmKR, bar, 0, row, hk, b);
  };

  if (tid == 0) {
    for (int s = 0; s < C::NSTAGE; ++s) {
      mbar_init(bar0 + s * 8, 1);
      sCnt[s] = 0;
    }
    mbar_fence_init();
    for (int t = 0; t < C::NSTAGE && t < n_tiles; ++t) issue(t);
  }
  if constexpr (MODE == MODE_POPE) {
    if (tid < 4 * DR) {   // four threads per column (whole warps: 4 DR is 128 or 256)
      const int c = tid >> 2;
      const float f = effective_freq_lanes<4>(p, c, tid & 3);
      if ((tid & 3) == 0) {
        freq_s[c] = f;
        delta_s[c] = clamped_delta(p, c);
        sincos_reduced(__fmul_rn((float)TK, f), &rot_s[c], &rot_c[c]);   // the phase advances TK * freq per tile
      }
    }
  }
  if constexpr (MODE == MODE_XFORM) {
    // geometric rotary table: (cos, sin) of TK positions per column pair = row (first key of the
    // split's second tile) x conj(row (its first key)); both rows exist when the split has two tiles
    if (p.variant == PE_ATTN_ROTARY && (p.flags & PE_ATTN_TABLE_GEOMETRIC) && n_tiles > 1 && tid < DC / 2) {
      const long long row_a = (long long)tile0 * TK + p.k_pos0 - p.table_pos0;
      const float2 a = reinterpret_cast<const float2*>(p.table)[row_a * (DC / 2) + tid];
      const float2 bq = reinterpret_cast<const float2*>(p.table)[(row_a + TK) * (DC / 2) + tid];
      reinterpret_cast<float2*>(freq_s)[tid] = make_float2(bq.x * a.x + bq.y * a.y, bq.y * a.x - bq.x * a.y);
    }
  }
  if (tid < R_T) {
    const int r = tid;
    const int g = r / p.Sq, qi = r - g * p.Sq;
    sSlope[r] = (p.variant == PE_ATTN_ALIBI && r < R) ? p.slopes[hk * p.groups + g] * kLog2e : 0.f;
    sLim[r] = r < R ? qi + p.causal_off : -1;   // last visible key of the row
  }
  __syncthreads();
  for (int r = warp; r < R_T; r += NWARP) {
    if (r < R) {
      const int g = r / p.Sq, qi = r - g * p.Sq;
      build_query_row<DC, DR, MODE>(p, sQ + r * DQK, b, hk * p.groups + g, qi, freq_s, lane);
    } else {
      for (int c = lane; c < DQK; c += 32) sQ[r * DQK + c] = 0.f;
    }
  }

  // scores: this thread's key and column quarter
  const int part = lane >> 3, key_local = warp * 8 + (lane & 7);
  // PoPE: (cos, sin) of this lane's key's phase for its columns, advanced from tile to tile by a
  // rotation (the key position grows by TK per tile) and recomputed from the position every
  // RESEED tiles, which bounds the accumulated rounding to about RESEED * 5e-7 rad -- well under
  // the rounding of fl(pos * freq) itself at long contexts
  constexpr int NRS = DR > 0 ? DR / 32 : 1, RESEED = 16;
  [[maybe_unused]] float2 ph_c[NRS][4], ph_s[NRS][4];
  const bool rotary = MODE == MODE_XFORM && p.variant == PE_ATTN_ROTARY;
  const bool norm = MODE == MODE_XFORM && (p.flags & PE_ATTN_QK_NORM);
  const bool alibi = p.variant == PE_ATTN_ALIBI;

  // values: this thread's columns
  constexpr int CPT = DV / 32;
  float2 acc_o[R_T][CPT / 2];
#pragma unroll
  for (int r = 0; r < R_T; ++r)
#pragma unroll
    for (int c = 0; c < CPT / 2; ++c) acc_o[r][c] = make_float2(0.f, 0.f);
  float m_run[R_T], l_lane[R_T];   // maximum over the warp's keys so far; this lane's key's share of the sum
#pragma unroll
  for (int r = 0; r < R_T; ++r) {
    m_run[r] = -INFINITY;
    l_lane[r] = 0.f;
  }
  const uint32_t v_lane_off = DV == 128 ? (uint32_t)((lane >> 4) * 8192 + (lane & 1) * 8) : (uint32_t)((lane & 3) * 4);
  const int v_slot = DV == 128 ? ((lane & 15) >> 1) : (lane >> 2);

  __syncthreads();   // query rows complete
  bool bad = false;

  // rotary: the (cos, sin) table entries of this lane's key and columns.
  // For a table that is geometric in the position (row i = angles i * angle_c: every table the
  // reference builds) the entries are only FETCHED every RESEED tiles and advanced in between
  // by the rotation of TK positions, like the PoPE phases above: the fp32 table is twice the
  // bytes of the bf16 keys it rotates, and reading all of it made this path L2-bound.
  constexpr int NCS = DC > 0 ? DC / 32 : 1;
  [[maybe_unused]] float4 tab_cur[NCS][2];
  const bool recur = rotary && (p.flags & PE_ATTN_TABLE_GEOMETRIC) && n_tiles > 1;
  auto load_table = [&](int t) {
    const int kg_t = (tile0 + t) * TK + key_local;
    const long long krow = (long long)(kg_t < p.Sk ? kg_t : p.Sk - 1) + p.k_pos0 - p.table_pos0;
#pragma unroll
    for (int i = 0; i < NCS; ++i) {
      const float4* tp = reinterpret_cast<const float4*>(p.table + (krow * (DC / 2) + (part + 4 * i) * 4) * 2);
      tab_cur[i][0] = __ldg(tp);
      tab_cur[i][1] = __ldg(tp + 1);
    }
  };
  for (int t = 0; t < n_tiles; ++t) {
    if constexpr (MODE == MODE_XFORM) {
      if (rotary) {
        if (!recur || (t % RESEED) == 0) {
          load_table(t);   // issued before the wait for the tile's stage; every tile only for a table that is not geometric
        } else {
          // (c, s) <- (c cs - s ss, s cs + c ss) for the four pairs of each slot
#pragma unroll
          for (int i = 0; i < NCS; ++i) {
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
              const float4 c = tab_cur[i][hlf];
              const float4 st = *reinterpret_cast<const float4*>(freq_s + ((part + 4 * i) * 4 + 2 * hlf) * 2);
              tab_cur[i][hlf] = make_float4(c.x * st.x - c.y * st.y, c.y * st.x + c.x * st.y,
                                            c.z * st.z - c.w * st.w, c.w * st.z + c.z * st.w);
            }
          }
        }
      }
    }
    const int stage = t % C::NSTAGE;
    const uint32_t sb = base + stage * C::STAGE_BYTES;
    const bool ok = bad ? mbar_wait_for(bar0 + stage * 8, (t / C::NSTAGE) & 1, 100000)
                        : mbar_wait(bar0 + stage * 8, (t / C::NSTAGE) & 1);
    if (!ok && !bad) {
      bad = true;
      if (p.status != nullptr) atomicOr(p.status, ST_WAIT_KFULL);
    }
    const int kg = (tile0 + t) * TK + key_local;
    float2 acc2[R_T];   // even / odd columns
#pragma unroll
    for (int r = 0; r < R_T; ++r) acc2[r] = make_float2(0.f, 0.f);
    float nrm2 = 0.f;

    if constexpr (DC > 0) {
#pragma unroll
      for (int i = 0; i < DC / 32; ++i) {
        const int slot_g = part + 4 * i;
        const int chunk = slot_g >> 3, slot = slot_g & 7;
        float kf[8];
        unpack8(lds_v4(sb + chunk * 8192 + key_local * 128 + ((slot ^ (key_local & 7)) << 4)), kf);
        if constexpr (MODE == MODE_XFORM) {
          if (rotary) {
            const float4 t0 = tab_cur[i][0], t1 = tab_cur[i][1];
            const float cs[4] = {t0.x, t0.z, t1.x, t1.z}, sn[4] = {t0.y, t0.w, t1.y, t1.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // (x0 c - x1 s, x0 s + x1 c)
              const float x0 = kf[2 * e], x1 = kf[2 * e + 1];
              const float2 o = __ffma2_rn(make_float2(x0, x0), make_float2(cs[e], sn[e]),
                                          __fmul2_rn(make_float2(-x1, x1), make_float2(sn[e], cs[e])));
              kf[2 * e] = o.x;
              kf[2 * e + 1] = o.y;
            }
          }
          if (norm) {
#pragma unroll
            for (int e = 0; e < 8; ++e) nrm2 = fmaf(kf[e], kf[e], nrm2);
          }
        }
#pragma unroll
        for (int r = 0; r < R_T; ++r) {
          const float4 q0 = *reinterpret_cast<const float4*>(sQ + r * DQK + slot_g * 8);
          const float4 q1 = *reinterpret_cast<const float4*>(sQ + r * DQK + slot_g * 8 + 4);
          float2 a = acc2[r];
          a = __ffma2_rn(make_float2(q0.x, q0.y), make_float2(kf[0], kf[1]), a);
          a = __ffma2_rn(make_float2(q0.z, q0.w), make_float2(kf[2], kf[3]), a);
          a = __ffma2_rn(make_float2(q1.x, q1.y), make_float2(kf[4], kf[5]), a);
          a = __ffma2_rn(make_float2(q1.z, q1.w), make_float2(kf[6], kf[7]), a);
          acc2[r] = a;
        }
      }
    }
    if constexpr (MODE == MODE_POPE) {
      const uint32_t sbr = sb + C::K_BYTES + C::V_BYTES;
      const bool reseed = (t % RESEED) == 0;
      const float pos = (float)(p.k_pos0 + kg);
#pragma unroll
      for (int i = 0; i < DR / 32; ++i) {
        const int rs = part + 4 * i;
        const uint32_t addr = DR == 64 ? sbr + key_local * 128 + ((rs ^ (key_local & 7)) << 4)
                                       : sbr + key_local * 64 + ((rs ^ ((key_local >> 1) & 3)) << 4);
        const uint4 raw = lds_v4(addr);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        if (reseed) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // phase = fl(fl(pos * freq) + delta), the reference's rounding order
            const int c = rs * 8 + 2 * e;
            sincos_reduced(__fadd_rn(__fmul_rn(pos, freq_s[c]), delta_s[c]), &ph_s[i][e].x, &ph_c[i][e].x);
            sincos_reduced(__fadd_rn(__fmul_rn(pos, freq_s[c + 1]), delta_s[c + 1]), &ph_s[i][e].y, &ph_c[i][e].y);
          }
        } else {
          const float4 c01 = *reinterpret_cast<const float4*>(rot_c + rs * 8), c23 = *reinterpret_cast<const float4*>(rot_c + rs * 8 + 4);
          const float4 s01 = *reinterpret_cast<const float4*>(rot_s + rs * 8), s23 = *reinterpret_cast<const float4*>(rot_s + rs * 8 + 4);
          const float2 rc[4] = {make_float2(c01.x, c01.y), make_float2(c01.z, c01.w), make_float2(c23.x, c23.y), make_float2(c23.z, c23.w)};
          const float2 rsn[4] = {make_float2(s01.x, s01.y), make_float2(s01.z, s01.w), make_float2(s23.x, s23.y), make_float2(s23.z, s23.w)};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 c0 = ph_c[i][e], s0 = ph_s[i][e];
            ph_c[i][e] = __ffma2_rn(c0, rc[e], __fmul2_rn(make_float2(-s0.x, -s0.y), rsn[e]));
            ph_s[i][e] = __ffma2_rn(s0, rc[e], __fmul2_rn(c0, rsn[e]));
          }
        }
        float2 kc[4], ks[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // magnitude: softplus of the raw position half, two columns per instruction
          const float2 x = make_float2(bf16_lo(w[e]), bf16_hi(w[e]));
          const float2 tt = __fmul2_rn(x, make_float2(kLog2e, kLog2e));
          const float2 u = __fadd2_rn(make_float2(ex2_approx(-fabsf(tt.x)), ex2_approx(-fabsf(tt.y))), make_float2(1.0f, 1.0f));
          const float2 mu = __ffma2_rn(make_float2(lg2_approx(u.x), lg2_approx(u.y)), make_float2(kLn2, kLn2),
                                       make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f)));
          kc[e] = __fmul2_rn(mu, ph_c[i][e]);
          ks[e] = __fmul2_rn(mu, ph_s[i][e]);
        }
#pragma unroll
        for (int r = 0; r < R_T; ++r) {
          const float* qc = sQ + r * DQK + DC + rs * 8;
          const float* qs = qc + DR;
          const float4 c0 = *reinterpret_cast<const float4*>(qc), c1 = *reinterpret_cast<const float4*>(qc + 4);
          const float4 s0 = *reinterpret_cast<const float4*>(qs), s1 = *reinterpret_cast<const float4*>(qs + 4);
          float2 a = acc2[r];
          a = __ffma2_rn(make_float2(c0.x, c0.y), kc[0], a);
          a = __ffma2_rn(make_float2(c0.z, c0.w), kc[1], a);
          a = __ffma2_rn(make_float2(c1.x, c1.y), kc[2], a);
          a = __ffma2_rn(make_float2(c1.z, c1.w), kc[3], a);
          a = __ffma2_rn(make_float2(s0.x, s0.y), ks[0], a);
          a = __ffma2_rn(make_float2(s0.z, s0.w), ks[1], a);
          a = __ffma2_rn(make_float2(s1.x, s1.y), ks[2], a);
          a = __ffma2_rn(make_float2(s1.z, s1.w), ks[3], a);
          acc2[r] = a;
        }
      }
    }
    float acc[R_T];
#pragma unroll
    for (int r = 0; r < R_T; ++r) acc[r] = acc2[r].x + acc2[r].y;
    // join the four column quarters of a key (lanes l, l^8, l^16, l^24)
#pragma unroll
    for (int r = 0; r < R_T; ++r) {
      acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 8);
      acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 16);
    }
    float kfac = 1.0f;
    if constexpr (MODE == MODE_XFORM) {
      kfac = p.mscale;   // k' = mscale * rot(k), then k' / (|k'| + eps)
      if (norm) {
        nrm2 += __shfl_xor_sync(0xffffffffu, nrm2, 8);
        nrm2 += __shfl_xor_sync(0xffffffffu, nrm2, 16);
        float nr;
        asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(nr) : "f"(nrm2));
        kfac = __fdividef(p.mscale, fmaf(p.mscale, nr, p.eps));
      }
    }
    // online softmax over the warp's 8 keys (every lane of a quarter holds the same values)
    float pr[R_T];
#pragma unroll
    for (int r = 0; r < R_T; ++r) {
      const int lim = sLim[r];
      float sc = acc[r] * kfac;
      if (alibi) sc = fmaf(-sSlope[r], (float)(lim - kg), sc);
      sc = kg <= lim ? sc : -INFINITY;
      float tmax = sc;
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
      const float m_new = fmaxf(m_run[r], tmax);
      const bool empty = m_new == -INFINITY;
      const float alpha = empty ? 1.f : ex2_approx(m_run[r] - m_new);
      pr[r] = empty ? 0.f : ex2_approx(sc - m_new);
      l_lane[r] = fmaf(l_lane[r], alpha, pr[r]);
      m_run[r] = m_new;
#pragma unroll
      for (int c = 0; c < CPT / 2; ++c) acc_o[r][c] = __fmul2_rn(acc_o[r][c], make_float2(alpha, alpha));
    }

    const uint32_t sbv = sb + C::K_BYTES + v_lane_off;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int j = warp * 8 + jj;
      float2 vv[CPT / 2];
      if constexpr (DV == 128) {
        const uint2 w = lds_v2(sbv + j * 128 + ((v_slot ^ (j & 7)) << 4));
        vv[0] = make_float2(bf16_lo(w.x), bf16_hi(w.x));
        vv[1] = make_float2(bf16_lo(w.y), bf16_hi(w.y));
      } else {
        const uint32_t w = lds_u32(sbv + j * 128 + ((v_slot ^ (j & 7)) << 4));
        vv[0] = make_float2(bf16_lo(w), bf16_hi(w));
      }
#pragma unroll
      for (int r = 0; r < R_T; ++r) {
        const float pj = __shfl_sync(0xffffffffu, pr[r], jj);
#pragma unroll
        for (int c = 0; c < CPT / 2; ++c) acc_o[r][c] = __ffma2_rn(make_float2(pj, pj), vv[c], acc_o[r][c]);
      }
    }

    // this warp has left the stage; the last of the eight refills it
    __threadfence_block();
    __syncwarp();
    if (lane == 0) {
      if (atomicAdd(&sCnt[stage], 1) == NWARP - 1) {
        sCnt[stage] = 0;
        if (t + C::NSTAGE < n_tiles) {
          fence_proxy_async_smem();
          issue(t + C::NSTAGE);
        }
      }
    }
  }

  // merge the eight warps' (max, sum, output); the stages are idle: every issued tile was waited for
  __syncthreads();
  float* red = reinterpret_cast<float*>(gen);
  float2* red_ml = reinterpret_cast<float2*>(red + NWARP * R_T * DV);
#pragma unroll
  for (int r = 0; r < R_T; ++r) {
#pragma unroll
    for (int c = 0; c < CPT / 2; ++c)
      *reinterpret_cast<float2*>(red + (warp * R_T + r) * DV + lane * CPT + 2 * c) = acc_o[r][c];
    float l = l_lane[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    if (lane == 0) red_ml[warp * R_T + r] = make_float2(m_run[r], l);
  }
  __syncthreads();
  for (int idx = tid; idx < R * DV; idx += NT) {
    const int r = idx / DV, col = idx - r * DV;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) M = fmaxf(M, red_ml[w * R_T + r].x);
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      const float2 ml = red_ml[w * R_T + r];
      const float wt = ml.x == -INFINITY ? 0.f : ex2_approx(ml.x - M);
      l = fmaf(wt, ml.y, l);
      o = fmaf(wt, red[(w * R_T + r) * DV + col], o);
    }
    const int g = r / p.Sq, qi = r - g * p.Sq;
    const long long row = ((long long)b * p.H + hk * p.groups + g) * p.Sq + qi;
    dp.part_o[(row * dp.n_splits + split) * DV + col] = o;
    if (col == 0) dp.part_ml[row * dp.n_splits + split] = make_float2(M, l);
  }
}

// out = sum_i 2^(m_i - M) O_i / sum_i 2^(m_i - M) l_i per (batch, head, query row)
template <int DV>
__global__ void __launch_bounds__(DV) decode_merge_kernel(const KParams p, const DecodeParams dp) {
  __shared__ float wt[MAX_SPLITS];
  __shared__ float inv_l, lse2;
  const long long row = blockIdx.x;
  const int col = threadIdx.x, ns = dp.n_splits;
  if (col < 32) {   // one warp: weights of the splits (n_splits <= 64)
    const float2 a = col < ns ? dp.part_ml[row * ns + col] : make_float2(-INFINITY, 0.f);
    const float2 c = col + 32 < ns ? dp.part_ml[row * ns + col + 32] : make_float2(-INFINITY, 0.f);
    float M = fmaxf(a.x, c.x);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
    const float wa = a.x == -INFINITY ? 0.f : ex2_approx(a.x - M), wc = c.x == -INFINITY ? 0.f : ex2_approx(c.x - M);
    wt[col] = wa;
    wt[col + 32] = wc;
    const float L = warp_sum(wa * a.y + wc * c.y);
    if (col == 0) {
      inv_l = 1.0f / L;
      lse2 = M + log2f(L);
    }
  }
  __syncthreads();
  const float* po = dp.part_o + row * ns * DV + col;
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;   // four loads in flight
  int i = 0;
  for (; i + 4 <= ns; i += 4) {
    const float x0 = po[(long long)i * DV], x1 = po[(long long)(i + 1) * DV], x2 = po[(long long)(i + 2) * DV],
                x3 = po[(long long)(i + 3) * DV];
    o0 = fmaf(wt[i], x0, o0);
    o1 = fmaf(wt[i + 1], x1, o1);
    o2 = fmaf(wt[i + 2], x2, o2);
    o3 = fmaf(wt[i + 3], x3, o3);
  }
  for (; i < ns; ++i) o0 = fmaf(wt[i], po[(long long)i * DV], o0);
  const int qi = (int)(row % p.Sq);
  const int h = (int)((row / p.Sq) % p.H), b = (int)(row / ((long long)p.Sq * p.H));
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.out.ptr)) + (long long)b * p.out.sb +
                       (long long)h * p.out.sh + (long long)qi * p.out.ss;
  out[col] = __float2bfloat16_rn(((o0 + o1) + (o2 + o3)) * inv_l);
  if (p.lse != nullptr && col == 0) p.lse[row] = lse2 * kLn2;
}

// tensor map of a [B, H, S, d] bf16 tensor with a (cols x 64 rows) box
bool encode_box(CUtensorMap* map, const TensorRef& t, int d, int S, int H, int B, int box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)t.ss * 2, (cuuint64_t)t.sh * 2, (cuuint64_t)t.sb * 2};
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || strides[i] % 16 != 0) strides[i] = (cuuint64_t)d * 2;   // size-1 dimensions
  cuuint32_t box[4] = {(cuuint32_t)box_cols, TK, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(t.ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// How many splits: with few (batch, K/V head) problems, as many as fill the 296 CTA slots once
// (at least two tiles each); with many, splits of at least MIN_TILES tiles chosen so that the
// CTA count comes close to a whole number of waves -- short CTAs keep the last wave's idle
// time small and a new CTA's prologue runs under its neighbour's streaming.
void plan(const KParams& p, DecodeParams* dp) {
  constexpr int MIN_TILES = 16;
  const int total = (p.Sk + TK - 1) / TK;
  const long long problems = (long long)p.B * p.Hkv;
  int by_len = total / MIN_TILES;
  if (by_len > MAX_SPLITS) by_len = MAX_SPLITS;
  if (by_len < 1) by_len = 1;
  int want;
  if (problems * by_len <= TARGET_CTAS) {
    long long w = TARGET_CTAS / problems;
    if (w > MAX_SPLITS) w = MAX_SPLITS;
    if (w > total / 2) w = total / 2;   // at least two tiles per split
    want = w < 1 ? 1 : (int)w;
  } else {
    want = 1;
    double best = 0.0;
    for (int n = 1; n <= by_len; ++n) {
      const long long ctas = problems * n;
      const long long waves = (ctas + TARGET_CTAS - 1) / TARGET_CTAS;
      // occupied share of the waves, with a mild preference for more, shorter CTAs
      const double eff = (double)ctas / (double)(waves * TARGET_CTAS) + 1e-3 * n;
      if (eff > best) {
        best = eff;
        want = n;
      }
    }
  }
  dp->tiles_per_split = (total + want - 1) / want;
  dp->n_splits = (total + dp->tiles_per_split - 1) / dp->tiles_per_split;
  dp->rows = p.groups * p.Sq;
}

template <int DC, int DR, int DV, int MODE, int R_T>
int launch_instance(const KParams& p, const DecodeParams& dp, cudaStream_t stream) {
  using C = DCfg<DC, DR, DV, R_T>;
  auto kern = pe_attn_decode_kernel<DC, DR, DV, MODE, R_T>;
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
  CUtensorMap tmK, tmKR, tmV;
  memset(&tmK, 0, sizeof(tmK));
  memset(&tmKR, 0, sizeof(tmKR));
  bool ok = encode_box(&tmV, p.v, DV, p.Sk, p.Hkv, p.B, 64);
  if (DC > 0) ok = ok && encode_box(&tmK, p.k, DC, p.Sk, p.Hkv, p.B, 64);
  if (DR > 0) ok = ok && encode_box(&tmKR, p.kr, DR, p.Sk, p.Hkv, p.B, DR);
  if (!ok) {
    set_error("cuTensorMapEncodeTiled failed for the cached k / k_r / v");
    return PE_ATTN_ERR_LAUNCH;
  }
  dim3 grid(dp.n_splits, p.Hkv, p.B);
  kern<<<grid, NT, C::SMEM_BYTES, stream>>>(p, dp, tmK, tmKR, tmV);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    decode_merge_kernel<DV><<<(unsigned)((long long)p.B * p.H * p.Sq), DV, 0, stream>>>(p, dp);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_error("split-KV kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

template <int DC, int DR, int DV, int MODE>
int launch_rows(const KParams& p, const DecodeParams& dp, cudaStream_t stream) {
  if (dp.rows <= 1) return launch_instance<DC, DR, DV, MODE, 1>(p, dp, stream);
  if (dp.rows <= 2) return launch_instance<DC, DR, DV, MODE, 2>(p, dp, stream);
  if (dp.rows <= 4) return launch_instance<DC, DR, DV, MODE, 4>(p, dp, stream);
  return launch_instance<DC, DR, DV, MODE, 8>(p, dp, stream);
}

}  // namespace

bool decode_supports(const KParams& p) {
  return tc_supports(p) && (long long)p.groups * p.Sq <= MAX_ROWS;
}

size_t decode_workspace_bytes(const KParams& p) {
  DecodeParams dp;
  plan(p, &dp);
  return (size_t)p.B * p.H * p.Sq * dp.n_splits * (p.d_v + 2) * sizeof(float);
}

int launch_decode(const KParams& p, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  DecodeParams dp;
  plan(p, &dp);
  const size_t rows = (size_t)p.B * p.H * p.Sq;
  if (workspace_bytes < decode_workspace_bytes(p)) {
    set_error("workspace of %zu bytes is smaller than the %zu this call needs", workspace_bytes, decode_workspace_bytes(p));
    return PE_ATTN_ERR_TOO_LARGE;
  }
  dp.part_ml = reinterpret_cast<float2*>(workspace);
  dp.part_o = reinterpret_cast<float*>(workspace) + rows * dp.n_splits * 2;
  if (p.variant == PE_ATTN_POPE) {
    if (p.d_c == 64 && p.d_r == 32) return launch_rows<64, 32, 64, MODE_POPE>(p, dp, stream);
    if (p.d_c == 128 && p.d_r == 64) return launch_rows<128, 64, 128, MODE_POPE>(p, dp, stream);
    if (p.d_c == 128 && p.d_r == 32) return launch_rows<128, 32, 128, MODE_POPE>(p, dp, stream);
    if (p.d_c == 0 && p.d_r == 32) return launch_rows<0, 32, 64, MODE_POPE>(p, dp, stream);
    return launch_rows<0, 64, 128, MODE_POPE>(p, dp, stream);
  }
  const bool xform = p.variant == PE_ATTN_ROTARY || (p.flags & PE_ATTN_QK_NORM);
  if (p.d_c == 64)
    return xform ? launch_rows<64, 0, 64, MODE_XFORM>(p, dp, stream) : launch_rows<64, 0, 64, MODE_PLAIN>(p, dp, stream);
  return xform ? launch_rows<128, 0, 128, MODE_XFORM>(p, dp, stream) : launch_rows<128, 0, 128, MODE_PLAIN>(p, dp, stream);
}

}  // namespace pe_attn
