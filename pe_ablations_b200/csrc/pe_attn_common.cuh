// Shared definitions of the PE-attention kernels: the device-side argument block
// and the positional-encoding math both kernel families use.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/pe_attn.h"

namespace pe_attn {

// A [B, H, S, d] tensor addressed by element strides, innermost contiguous.
struct TensorRef {
  const void* ptr;
  long long sb, sh, ss;
};

// Device-side copy of the validated arguments (passed to kernels by value).
struct KParams {
  int variant;
  unsigned flags;
  int B, H, Hkv, groups;
  int Sq, Sk;
  int d_c, d_r, d_v, d_qk;
  int q_pos0, k_pos0;
  int causal_off;  // key s visible to query row r iff s <= r + causal_off
  float scale, eps, mscale;
  TensorRef q, k, v, out, qr, kr;
  const float* table;
  int table_pos0, table_rows;
  const float* slopes;
  const float* freqs;
  const float* delta;
  const float* coeffs;
  int n_fourier;
  float floor_freq, ceil_freq;
  int* status;
  float* lse;  // optional [B, H, Sq] logsumexp output
  float* workspace;        // optional scratch of the forward (pe_attn_forward_workspace_bytes)
  size_t workspace_bytes;
};

// Device-side arguments of the attention backward (operands already transformed).
struct BwdParams {
  int B, H, Hkv, groups;
  int Sq, Sk;
  int causal_off;          // key s visible to query row r iff s <= r + causal_off
  float scale;
  TensorRef q, k, v, out, dout, dk, dv;
  const float* lse;        // [B, H, Sq] from the forward
  const float* slopes;     // ALiBi, or null
  float* dq_accum;         // [B, Sq, H, d_qk] fp32, cleared by the launch
  float* dvec;             // [B, H, Sq] fp32 workspace
  int* status;
};

constexpr float kTwoPi = 6.283185307179586f;

// Effective frequency of PoPE dimension c.  Without FOURIER_MIX this is freqs[c].
// With it, the FoPE collapse of the reference (src/model/fpope.py:116-146):
//   eff = base * sum_j a^_j * j + base,  a^ = a / (sum_j |a_j| + 1e-8) when normalising,
//   |eff| < floor -> 0, optional clamp to +-ceil.
// The sum is accumulated in fp64 and rounded once, which lands within an ulp of any
// fp32 summation order.
__device__ __forceinline__ float effective_freq(const KParams& p, int c) {
  const float base = p.freqs[c];
  if (!(p.flags & PE_ATTN_FOURIER_MIX)) return base;
  const float* a = p.coeffs + (size_t)c * p.n_fourier;
  float denom = 1.0f;
  if (p.flags & PE_ATTN_FOURIER_NORMALIZE) {
    double s = 0.0;
    for (int j = 0; j < p.n_fourier; ++j) s += fabs((double)a[j]);
    denom = __fadd_rn((float)s, 1e-8f);
  }
  double acc = 0.0;
  for (int j = 0; j < p.n_fourier; ++j) {
    const float an = (p.flags & PE_ATTN_FOURIER_NORMALIZE) ? __fdiv_rn(a[j], denom) : a[j];
    const float sj = __fmul_rn(base, (float)(j + 1));
    acc += (double)__fmul_rn(an, sj);
  }
  float eff = __fadd_rn((float)acc, base);
  if (fabsf(eff) < p.floor_freq) eff = 0.0f;
  if (p.flags & PE_ATTN_FOURIER_CEILING) eff = fminf(fmaxf(eff, -p.ceil_freq), p.ceil_freq);
  return eff;
}

// The same value with the Fourier terms of column c dealt to LANES neighbouring lanes of a warp
// (term j to lane j mod LANES) and the fp64 partial sums joined by shuffles: a chain of
// 2 n_fourier / LANES dependent fp64 additions instead of 2 n_fourier, for kernel prologues that
// nothing hides.  Every lane of the warp must make the call (full-mask shuffles); the LANES lanes
// of a group pass the same c and their index ``sub`` in the group, and all get the result.  The
// terms are fp32 values and their fp64 sum is exact at these counts, so the rounded result does
// not depend on the order: bit for bit the value effective_freq() returns.
template <int LANES>
__device__ __forceinline__ float effective_freq_lanes(const KParams& p, int c, int sub) {
  static_assert(LANES == 2 || LANES == 4 || LANES == 8 || LANES == 16 || LANES == 32, "LANES: a power of two <= 32");
  const float base = p.freqs[c];
  if (!(p.flags & PE_ATTN_FOURIER_MIX)) return base;
  const float* a = p.coeffs + (size_t)c * p.n_fourier;
  const bool normalize = (p.flags & PE_ATTN_FOURIER_NORMALIZE) != 0;
  float denom = 1.0f;
  if (normalize) {
    double s = 0.0;
    for (int j = sub; j < p.n_fourier; j += LANES) s += fabs((double)a[j]);
#pragma unroll
    for (int d = 1; d < LANES; d <<= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    denom = __fadd_rn((float)s, 1e-8f);
  }
  double acc = 0.0;
  for (int j = sub; j < p.n_fourier; j += LANES) {
    const float an = normalize ? __fdiv_rn(a[j], denom) : a[j];
    acc += (double)__fmul_rn(an, __fmul_rn(base, (float)(j + 1)));
  }
#pragma unroll
  for (int d = 1; d < LANES; d <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  float eff = __fadd_rn((float)acc, base);
  if (fabsf(eff) < p.floor_freq) eff = 0.0f;
  if (p.flags & PE_ATTN_FOURIER_CEILING) eff = fminf(fmaxf(eff, -p.ceil_freq), p.ceil_freq);
  return eff;
}

// Key phase bias as used: clamp(delta, -2 pi, 0) (src/model/pope.py:172, src/model/fpope.py:328).
__device__ __forceinline__ float clamped_delta(const KParams& p, int c) {
  if (p.delta == nullptr) return 0.0f;
  return fminf(fmaxf(p.delta[c], -kTwoPi), 0.0f);
}

// softplus with torch's defaults (beta 1, threshold 20), accurate libm calls.
__device__ __forceinline__ float softplus_accurate(float x) {
  return x > 20.0f ? x : log1pf(expf(x));
}

int launch_simt(const KParams& p, int dtype, cudaStream_t stream);
size_t simt_key_scratch_bytes(const KParams& p);   // fp32 calls: scratch for keys transformed once, or 0
int launch_tc(const KParams& p, cudaStream_t stream);
bool tc_supports(const KParams& p);
int launch_tc2(const KParams& p, cudaStream_t stream);  // CTA-pair (cta_group::2) variant, d_v = 128
bool tc2_supports(const KParams& p);
size_t tc2_workspace_bytes(const KParams& p);
int launch_tc4(const KParams& p, cudaStream_t stream);  // four query tiles per CTA, d_v = 64
bool tc4_supports(const KParams& p);
int launch_ce(const void* logits, int dtype, long long row_stride, const long long* targets, int n_rows, int vocab,
              int ignore_index, float* row_loss, unsigned int* counter, double* out, cudaStream_t stream);

bool decode_supports(const KParams& p);   // split-KV path: bf16 shapes of the tcgen05 kernels, <= 8 rows per K/V head
size_t decode_workspace_bytes(const KParams& p);
int launch_decode(const KParams& p, void* workspace, size_t workspace_bytes, cudaStream_t stream);

bool bwd_supports(int d_qk, int d_v);        // tensor-core backward kernel
bool bwd_simt_supports(int d_qk, int d_v, int dtype);   // FFMA backward: d_qk <= 256, d_v <= 128 in steps of 8 whose tiles fit shared memory
int launch_bwd_simt(const BwdParams& p, int d_qk, int d_v, int dtype, bool alibi, cudaStream_t stream);
int launch_bwd(const BwdParams& p, int d_qk, int d_v, int dtype, bool alibi, cudaStream_t stream);

void set_error(const char* fmt, ...);

// Function attributes (the dynamic shared-memory limit) are per device, so "already set" is
// remembered per device ordinal: one bit each for devices 0..63, always set again beyond that.
struct PerDeviceOnce {
  std::atomic<unsigned long long> done{0ull};
  // true when the current device still needs its one-time setup; *dev receives its ordinal
  bool pending(int* dev) const {
    *dev = 0;
    if (cudaGetDevice(dev) != cudaSuccess || *dev < 0 || *dev >= 64) return true;
    return !((done.load(std::memory_order_acquire) >> *dev) & 1ull);
  }
  void mark(int dev) {
    if (dev >= 0 && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  }
};

}  // namespace pe_attn
