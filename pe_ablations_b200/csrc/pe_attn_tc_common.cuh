// Pieces shared by the tcgen05 attention kernels (single-CTA and CTA-pair variants): the
// positional transforms that build MMA operands in shared memory, and the host-side TMA
// descriptor encoding.
#pragma once

#include <cuda.h>

#include "pe_attn_common.cuh"
#include "pe_attn_ptx.cuh"

namespace pe_attn {
namespace tc {

using namespace ptx;

constexpr int SLAB_ROWS = 64;  // rows one build_slab call produces

enum Mode { MODE_PLAIN = 0, MODE_XFORM = 1, MODE_POPE = 2 };

// status codes ORed into the caller's device status word
enum : int {
  ST_WAIT_QFULL = 1 << 0, ST_WAIT_KFULL = 1 << 1, ST_WAIT_VFULL = 1 << 2, ST_WAIT_KEMPTY = 1 << 3,
  ST_WAIT_VEMPTY = 1 << 4, ST_WAIT_SFULL = 1 << 5, ST_WAIT_PREADY = 1 << 6, ST_WAIT_PVDONE = 1 << 7,
  ST_WAIT_MMADONE = 1 << 8
};

// softplus with the special-function unit: max(x, 0) + log1p(exp(-|x|))
__device__ __forceinline__ float softplus_fast(float x) {
  const float e = ex2_approx(-fabsf(x) * 1.4426950408889634f);
  return fmaxf(x, 0.f) + lg2_approx(1.0f + e) * 0.6931471805599453f;
}

// sin / cos of a large fp32 angle: two-term Cody-Waite reduction by 2 pi, then MUFU.  The
// rounding to the nearest whole turn is two additions of 1.5 * 2^23 (exact for |turns| < 2^22,
// ties to even like rintf) instead of a round instruction, which would take a slot of the
// special-function pipe beside the four this transform already needs per element.
__device__ __forceinline__ void sincos_reduced(float x, float* s, float* c) {
  const float k = __fadd_rn(__fadd_rn(x * 0.15915494309189535f, 12582912.0f), -12582912.0f);
  float r = fmaf(k, -6.2831854820251465f, x);
  r = fmaf(k, 1.7484556000744883e-7f, r);
  *s = __sinf(r);
  *c = __cosf(r);
}

// PoPE expansion of two adjacent position columns at once with the packed fp32x2 instructions
// of sm_100 (one issue slot for two multiplies / adds / FMAs): magnitude mu = softplus(x),
// phase = fl(fl(pos * freq) + bias), result (mu cos, mu sin).  Same operations and roundings as
// softplus_fast and sincos_reduced element by element; about 29 instructions per pair against 42.
__device__ __forceinline__ void pope_pair(float2 x, float pos, float2 freq, float2 bias, float2* kc, float2* ks) {
  const float2 t = __fmul2_rn(x, make_float2(1.4426950408889634f, 1.4426950408889634f));
  const float2 u = __fadd2_rn(make_float2(ex2_approx(-fabsf(t.x)), ex2_approx(-fabsf(t.y))), make_float2(1.0f, 1.0f));
  const float2 mu = __ffma2_rn(make_float2(lg2_approx(u.x), lg2_approx(u.y)),
                               make_float2(0.6931471805599453f, 0.6931471805599453f),
                               make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f)));
  const float2 ph = __fadd2_rn(__fmul2_rn(make_float2(pos, pos), freq), bias);
  const float2 turns = __fmul2_rn(ph, make_float2(0.15915494309189535f, 0.15915494309189535f));
  const float2 k = __fadd2_rn(__fadd2_rn(turns, make_float2(12582912.0f, 12582912.0f)),
                              make_float2(-12582912.0f, -12582912.0f));
  float2 r = __ffma2_rn(k, make_float2(-6.2831854820251465f, -6.2831854820251465f), ph);
  r = __ffma2_rn(k, make_float2(1.7484556000744883e-7f, 1.7484556000744883e-7f), r);
  *kc = __fmul2_rn(mu, make_float2(__cosf(r.x), __cosf(r.y)));
  *ks = __fmul2_rn(mu, make_float2(__sinf(r.x), __sinf(r.y)));
}

// byte offset of the 16-byte slot ``slot`` (0..7) of row ``r`` inside a 128B-swizzled chunk
__device__ __forceinline__ uint32_t swz(int r, int slot) { return (uint32_t)(r * 128 + ((slot ^ (r & 7)) << 4)); }

// Rotary family / QKNorm operand rows in two steps, so that a K-tile loop can issue the loads
// of the next tile before it waits for the stage to become free: the raw rows and their
// (cos, sin) table entries for the 64-row slab, then rotation, mscale, L2 normalisation and the
// swizzled stores.  Thread (r_in, cv) owns columns [8 cv, 8 cv + 8) of rows r_in + k * RPP.
template <int DC>
struct XformRegs {
  static constexpr int VPR = DC / 8, RPP = 128 / VPR, PASSES = SLAB_ROWS / RPP;
  uint4 raw[PASSES];
  float4 t0[PASSES], t1[PASSES];
};

template <int DC>
__device__ __forceinline__ void xform_load(const KParams& p, XformRegs<DC>& x, const TensorRef& content, int b,
                                           int head, int row0, int n_rows, int pos_row0, int tg) {
  using X = XformRegs<DC>;
  const int cv = tg % X::VPR, r_in = tg / X::VPR;
  const bool rotary = p.variant == PE_ATTN_ROTARY;
  const char* src = reinterpret_cast<const char*>(content.ptr) +
                    2 * ((long long)b * content.sb + (long long)head * content.sh + (long long)cv * 8);
#pragma unroll
  for (int k = 0; k < X::PASSES; ++k) {
    const int r = r_in + k * X::RPP;
    const bool live = (row0 + r) < n_rows;
    x.raw[k] = live ? ldg_nc_v4(src + 2 * (long long)(row0 + r) * content.ss) : make_uint4(0, 0, 0, 0);
    x.t0[k] = x.t1[k] = make_float4(1.f, 0.f, 1.f, 0.f);
    if (rotary && live) {
      const int trow = pos_row0 + r - p.table_pos0;
      const float4* tp = reinterpret_cast<const float4*>(p.table + ((size_t)trow * (DC / 2) + cv * 4) * 2);
      x.t0[k] = __ldg(tp);
      x.t1[k] = __ldg(tp + 1);
    }
  }
}

// The same loads for a walk over consecutive slabs of one (batch, head): the addresses are
// worked out once and advanced by constants, which leaves about ten instructions per pass
// (the four warps that build K tiles get few issue slots beside the softmax warps).
template <int DC>
struct XformCursor {
  const char* raw;      // this thread's 8 columns of its first row of the current slab
  const float4* tab;    // the matching (cos, sin) table entries
  long long raw_step, raw_slab;   // bytes between a thread's rows / between slabs
  int row;              // global index of the thread's first row in the current slab
};

template <int DC>
__device__ __forceinline__ void xform_cursor_init(const KParams& p, XformCursor<DC>& c, const TensorRef& content, int b,
                                                  int head, int row0, int pos_row0, int slab_stride_rows, int tg) {
  using X = XformRegs<DC>;
  const int cv = tg % X::VPR, r_in = tg / X::VPR;
  c.raw = reinterpret_cast<const char*>(content.ptr) +
          2 * ((long long)b * content.sb + (long long)head * content.sh + (long long)cv * 8 +
               (long long)(row0 + r_in) * content.ss);
  c.raw_step = 2 * (long long)X::RPP * content.ss;
  c.raw_slab = 2 * (long long)slab_stride_rows * content.ss;
  c.tab = p.table == nullptr ? nullptr
                             : reinterpret_cast<const float4*>(p.table) +
                                   ((long long)(pos_row0 + r_in - p.table_pos0) * (DC / 2) + cv * 4) / 2;
  c.row = row0 + r_in;
}

// loads the current slab and moves the cursor ``slab_stride_rows`` rows on
template <int DC>
__device__ __forceinline__ void xform_load_next(const KParams& p, XformRegs<DC>& x, XformCursor<DC>& c, int n_rows,
                                                int slab_stride_rows) {
  using X = XformRegs<DC>;
  const bool rotary = p.variant == PE_ATTN_ROTARY;
#pragma unroll
  for (int k = 0; k < X::PASSES; ++k) {
    const bool live = c.row + k * X::RPP < n_rows;
    x.raw[k] = live ? ldg_nc_v4(c.raw + k * c.raw_step) : make_uint4(0, 0, 0, 0);
    x.t0[k] = x.t1[k] = make_float4(1.f, 0.f, 1.f, 0.f);
    if (rotary && live) {
      const float4* tp = c.tab + (long long)k * X::RPP * (DC / 4);
      x.t0[k] = __ldg(tp);
      x.t1[k] = __ldg(tp + 1);
    }
  }
  c.raw += c.raw_slab;
  if (rotary) c.tab += (long long)slab_stride_rows * (DC / 4);
  c.row += slab_stride_rows;
}

template <int DC, int GROUP = 4>   // GROUP: rows (passes) in flight at a time, bounds the live registers
__device__ __forceinline__ void xform_finish(const KParams& p, XformRegs<DC>& x, uint32_t base, uint32_t chunk_stride,
                                             int row0, int n_rows, int tg) {
  // Rotation, mscale and normalisation in fp32 with the packed fp32x2 FMA / MUL of sm_100 (a
  // quarter of the issue slots of the scalar, round-after-every-step version this replaces: the
  // four warps that build K tiles were the bottleneck of the rotary / QKNorm variants at
  // head_dim 64); one rounding to bf16 at the end.
  using X = XformRegs<DC>;
  const int cv = tg % X::VPR, r_in = tg / X::VPR;
  const bool rotary = p.variant == PE_ATTN_ROTARY;
  const bool norm = (p.flags & PE_ATTN_QK_NORM) != 0;
  const float2 ms2 = make_float2(p.mscale, p.mscale);
  static_assert(X::PASSES % GROUP == 0, "passes per slab must be a multiple of the group size");
#pragma unroll
  for (int k0 = 0; k0 < X::PASSES; k0 += GROUP) {
    float2 v[GROUP][4];
    float ss[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const int k = k0 + g;
      const uint32_t w[4] = {x.raw[k].x, x.raw[k].y, x.raw[k].z, x.raw[k].w};
      const float cs[4] = {x.t0[k].x, x.t0[k].z, x.t1[k].x, x.t1[k].z};
      const float sn[4] = {x.t0[k].y, x.t0[k].w, x.t1[k].y, x.t1[k].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x0 = bf16_lo(w[e]), x1 = bf16_hi(w[e]);
        float2 o = make_float2(x0, x1);
        if (rotary) {
          // (x0 c - x1 s, x0 s + x1 c)
          o = __ffma2_rn(make_float2(x0, x0), make_float2(cs[e], sn[e]),
                         __fmul2_rn(make_float2(-x1, x1), make_float2(sn[e], cs[e])));
          if (p.mscale != 1.0f) o = __fmul2_rn(o, ms2);
        }
        v[g][e] = o;
      }
      float2 acc = __fmul2_rn(v[g][0], v[g][0]);
#pragma unroll
      for (int e = 1; e < 4; ++e) acc = __ffma2_rn(v[g][e], v[g][e], acc);
      ss[g] = acc.x + acc.y;
    }
    if (norm) {
      // row sum of squares across the VPR lanes that share a row (warp-level reduction)
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
#pragma unroll
        for (int d = 1; d < X::VPR; d <<= 1) ss[g] += __shfl_xor_sync(0xffffffffu, ss[g], d);
      }
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const int r = r_in + (k0 + g) * X::RPP;
      if (norm) {
        // special-function-unit square root and reciprocal: 2 ulp, far inside a bf16 rounding
        float nrm;
        asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(nrm) : "f"(ss[g]));
        const float inv = __fdividef(1.0f, nrm + p.eps);
        const float2 inv2 = make_float2(inv, inv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[g][e] = __fmul2_rn(v[g][e], inv2);
      }
      const int col = cv * 8;
      sts_v4(base + (col / 64) * chunk_stride + swz(r, (col % 64) / 8),
             make_uint4(pack_bf16x2(v[g][0].x, v[g][0].y), pack_bf16x2(v[g][1].x, v[g][1].y),
                        pack_bf16x2(v[g][2].x, v[g][2].y), pack_bf16x2(v[g][3].x, v[g][3].y)));
    }
  }
}

// Build 64 operand rows (positional / transformed columns only) in shared memory with a
// group of 128 threads (tg = 0..127).  ``base`` is the shared address of chunk 0 at the
// slab's first row (1024-byte aligned), chunks are ``chunk_stride`` bytes apart.
//   MODE_POPE : columns [DC, DC + 2 DR): softplus magnitude x (cos, sin) of the phase
//   MODE_XFORM: columns [0, DC): optional pair rotation, mscale, optional L2 normalisation
template <int DC, int DR, int MODE>
__device__ __forceinline__ void build_slab(const KParams& p, uint32_t base, uint32_t chunk_stride,
                                           const TensorRef& content, const TensorRef& posi, int b, int head,
                                           int row0, int n_rows, int pos_row0, bool is_key, const float* freq_s,
                                           const float* delta_s, int tg) {
  if constexpr (MODE == MODE_POPE) {
    constexpr int VPR = DR / 8;            // 16-byte vectors per row
    constexpr int RPP = 128 / VPR;         // rows per pass
    constexpr int PASSES = SLAB_ROWS / RPP;
    const int cv = tg % VPR, r_in = tg / VPR;
    float f[8], dl[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      f[e] = freq_s[cv * 8 + e];
      dl[e] = is_key ? delta_s[cv * 8 + e] : 0.f;
    }
    const char* src = reinterpret_cast<const char*>(posi.ptr) +
                      2 * ((long long)b * posi.sb + (long long)head * posi.sh + (long long)cv * 8);
    uint4 raw[PASSES];
#pragma unroll
    for (int k = 0; k < PASSES; ++k) {
      const int grow = row0 + r_in + k * RPP;
      raw[k] = make_uint4(0, 0, 0, 0);
      if (grow < n_rows) raw[k] = ldg_nc_v4(src + 2 * (long long)grow * posi.ss);
    }
#pragma unroll
    for (int k = 0; k < PASSES; ++k) {
      const int r = r_in + k * RPP;
      const bool live = (row0 + r) < n_rows;
      const float pos = (float)(pos_row0 + r);
      const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
      float oc[8], os[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // phase = fl(fl(pos * freq) + delta), the reference's rounding order
        float2 c2, s2;
        pope_pair(make_float2(bf16_lo(w[e]), bf16_hi(w[e])), pos, make_float2(f[2 * e], f[2 * e + 1]),
                  make_float2(dl[2 * e], dl[2 * e + 1]), &c2, &s2);
        oc[2 * e] = live ? c2.x : 0.f;
        oc[2 * e + 1] = live ? c2.y : 0.f;
        os[2 * e] = live ? s2.x : 0.f;
        os[2 * e + 1] = live ? s2.y : 0.f;
      }
      const uint4 vc = make_uint4(pack_bf16x2(oc[0], oc[1]), pack_bf16x2(oc[2], oc[3]), pack_bf16x2(oc[4], oc[5]),
                                  pack_bf16x2(oc[6], oc[7]));
      const uint4 vs = make_uint4(pack_bf16x2(os[0], os[1]), pack_bf16x2(os[2], os[3]), pack_bf16x2(os[4], os[5]),
                                  pack_bf16x2(os[6], os[7]));
      const int col_c = DC + cv * 8, col_s = DC + DR + cv * 8;
      sts_v4(base + (col_c / 64) * chunk_stride + swz(r, (col_c % 64) / 8), vc);
      sts_v4(base + (col_s / 64) * chunk_stride + swz(r, (col_s % 64) / 8), vs);
    }
  } else if constexpr (MODE == MODE_XFORM) {
    XformRegs<DC> x;
    xform_load<DC>(p, x, content, b, head, row0, n_rows, pos_row0, tg);
    xform_finish<DC>(p, x, base, chunk_stride, row0, n_rows, tg);
  }
}

// ---- host side --------------------------------------------------------------------------

// (batch, head) problems per scheduling group of a launch whose blocks are handed out longest
// first inside each group: as many as keep their K/V in L2 together (about 48 MB of the 126 MB),
// in groups of EQUAL size, a multiple of ``min_group`` (query heads that share a K/V head).  A
// short last group starts its longest blocks when the rest of the GPU is draining: a list
// schedule of configuration 2 (96 problems x 4 blocks on 148 SMs) takes 128 us with groups of
// 74 + 22 and 105 us with 48 + 48 (a single group: 105, the bound 96).
inline int balanced_bh_group(long long n_bh, long long kv_bytes_per_head, int min_group) {
  long long cap = (48ll << 20) / (kv_bytes_per_head > 0 ? kv_bytes_per_head : 1);
  if (cap < min_group) cap = min_group;
  if (cap < 1) cap = 1;
  if (cap > n_bh) cap = n_bh;
  const long long n_groups = (n_bh + cap - 1) / cap;
  long long g = (n_bh + n_groups - 1) / n_groups;
  if (min_group > 1) g = ((g + min_group - 1) / min_group) * min_group;
  if (g > n_bh) g = n_bh;
  return (int)(g < 1 ? 1 : g);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// [B, H, S, d] bf16 tensor viewed as a 4-D TMA tensor (d, S, H, B) with a (64 x rows) box,
// 128-byte swizzle, zero fill outside the tensor.
inline bool encode_map(CUtensorMap* map, const TensorRef& t, int d, int S, int H, int B, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)t.ss * 2, (cuuint64_t)t.sh * 2, (cuuint64_t)t.sb * 2};
  // a size-1 dimension may carry any stride; TMA still wants a multiple of 16 bytes
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || strides[i] % 16 != 0) strides[i] = (cuuint64_t)d * 2;
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(t.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Contiguous fp32 [B, S, H, d] tensor as a 4-D TMA tensor (d, S, H, B) with a (32 x rows) box
// (128-byte rows), 128-byte swizzle: the target of TMA reductions.
inline bool encode_map_f32(CUtensorMap* map, float* ptr, int d, int S, int H, int B, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)d * 4 * H, (cuuint64_t)d * 4, (cuuint64_t)d * 4 * S * H};
  cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace pe_attn
