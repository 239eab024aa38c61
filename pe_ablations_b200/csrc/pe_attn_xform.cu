// PoPE-family positional transform as stand-alone kernels, for the training path: the
// backward pass needs the transformed operands in memory (the backward kernel reads them by
// TMA) and the transform's own gradient.
//
//   expand:    [x_c | x_r]  ->  [x_c | mu cos(phi) | mu sin(phi)],  mu = softplus(x_r),
//              phi = fl(fl(pos * omega) + clamp(delta, -2 pi, 0))         (bf16 in, bf16 out)
//   backward:  g = d/d(expanded row)  ->  d x_c = g_c,
//              d x_r = (g_cos cos + g_sin sin) * sigmoid(x_r),
//              d phi = mu (g_sin cos - g_cos sin);  d omega_c += sum pos * d phi,
//              d delta~_c += sum d phi   (delta~ the clamped phase bias)
//
// They restate src/model/pope.py:124-183 and src/model/fpope.py:266-338 of the reference
// (forward) and what autograd derives from them (backward).  Memory-bound: every input is
// read once and every output written once, 16 bytes per thread and access; thread =
// (row, group of 8 position columns), rows ordered (batch, position, head).  The two
// parameter gradients are reduced per warp with shuffles, per block in shared memory and
// across blocks with fp64 atomics (d_r values each), so their bits do not depend on the
// block schedule beyond fp64 rounding.

#include "pe_attn_tc_common.cuh"

namespace pe_attn {
namespace {

using namespace ptx;
using namespace tc;

struct XfParams {
  int B, S, H, d_c, pos0;
  TensorRef xc, xr, out, grad, dxc, dxr;
  const float* omega;
  const float* delta;   // raw phase bias or null (queries)
  double* d_omega;      // [d_r], accumulated
  double* d_delta;      // [d_r], accumulated; null for queries
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = (e & 1) ? bf16_hi(w[e >> 1]) : bf16_lo(w[e >> 1]);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ long long row_offset(const TensorRef& t, int b, int h, int s) {
  return (long long)b * t.sb + (long long)h * t.sh + (long long)s * t.ss;
}

template <int DR>
__global__ void __launch_bounds__(256) pope_expand_kernel(const XfParams p) {
  constexpr int VPR = DR / 8;
  const long long n = (long long)p.B * p.S * p.H * VPR;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cv = (int)(idx % VPR);
  float om[8], dl[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    om[e] = p.omega[cv * 8 + e];
    dl[e] = p.delta != nullptr ? fminf(fmaxf(p.delta[cv * 8 + e], -kTwoPi), 0.0f) : 0.0f;
  }
  for (; idx < n; idx += stride) {
    const long long row = idx / VPR;
    const int h = (int)(row % p.H), s = (int)((row / p.H) % p.S), b = (int)(row / ((long long)p.H * p.S));
    const __nv_bfloat16* xr = reinterpret_cast<const __nv_bfloat16*>(p.xr.ptr) + row_offset(p.xr, b, h, s);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.out.ptr)) + row_offset(p.out, b, h, s);
    float x[8], oc[8], os[8];
    unpack8(ldg_nc_v4(xr + cv * 8), x);
    const float pos = (float)(p.pos0 + s);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float mu = softplus_fast(x[e]);
      float sn, cs;
      sincos_reduced(__fadd_rn(__fmul_rn(pos, om[e]), dl[e]), &sn, &cs);
      oc[e] = mu * cs;
      os[e] = mu * sn;
    }
    *reinterpret_cast<uint4*>(out + p.d_c + cv * 8) = pack8(oc);
    *reinterpret_cast<uint4*>(out + p.d_c + DR + cv * 8) = pack8(os);
    if (p.d_c > 0) {
      const __nv_bfloat16* xc = reinterpret_cast<const __nv_bfloat16*>(p.xc.ptr) + row_offset(p.xc, b, h, s);
      for (int cg = cv; cg < p.d_c / 8; cg += VPR) *reinterpret_cast<uint4*>(out + cg * 8) = ldg_nc_v4(xc + cg * 8);
    }
  }
}

template <int DR, bool GRAD_F32>
// Three CTAs per SM (80 registers) and a grid of exactly the CTAs that fit at once: a thread then
// walks about nine rows, and the per-CTA reduction of the two parameter gradients (shared-memory
// and global fp64 atomics) happens 444 times instead of 1184 (training shape: 61 -> 51 us for the
// query side, 38 -> 29 us for the key side).
__global__ void __launch_bounds__(256, 3) pope_expand_backward_kernel(const XfParams p) {
  constexpr int VPR = DR / 8;
  __shared__ double sum_w[DR], sum_d[DR];
  for (int i = threadIdx.x; i < DR; i += blockDim.x) sum_w[i] = sum_d[i] = 0.0;
  __syncthreads();
  const long long n = (long long)p.B * p.S * p.H * VPR;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cv = (int)(idx % VPR);
  float om[8], dl[8], acc_w[8], acc_d[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    om[e] = p.omega[cv * 8 + e];
    dl[e] = p.delta != nullptr ? fminf(fmaxf(p.delta[cv * 8 + e], -kTwoPi), 0.0f) : 0.0f;
    acc_w[e] = acc_d[e] = 0.f;
  }
  auto load_grad8 = [&](const void* base, long long off, float (&g)[8]) {
    if constexpr (GRAD_F32) {
      const float4* gp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
      const float4 a = __ldg(gp), c = __ldg(gp + 1);
      g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = c.x; g[5] = c.y; g[6] = c.z; g[7] = c.w;
    } else {
      unpack8(ldg_nc_v4(reinterpret_cast<const __nv_bfloat16*>(base) + off), g);
    }
  };
  for (; idx < n; idx += stride) {
    const long long row = idx / VPR;
    const int h = (int)(row % p.H), s = (int)((row / p.H) % p.S), b = (int)(row / ((long long)p.H * p.S));
    const long long goff = row_offset(p.grad, b, h, s);
    const __nv_bfloat16* xr = reinterpret_cast<const __nv_bfloat16*>(p.xr.ptr) + row_offset(p.xr, b, h, s);
    __nv_bfloat16* dxr = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.dxr.ptr)) + row_offset(p.dxr, b, h, s);
    float x[8], gc[8], gs[8], dx[8];
    unpack8(ldg_nc_v4(xr + cv * 8), x);
    load_grad8(p.grad.ptr, goff + p.d_c + cv * 8, gc);
    load_grad8(p.grad.ptr, goff + p.d_c + DR + cv * 8, gs);
    const float pos = (float)(p.pos0 + s);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      // special-function-unit logarithm and division: 2 ulp, against bf16 outputs and sums of
      // thousands of terms (the accurate log1pf and IEEE division were a fifth of the kernel)
      const float ex = __expf(-fabsf(x[e]));                       // exp(-|x|)
      const float mu = fmaxf(x[e], 0.f) + __logf(1.0f + ex);
      const float sig = __fdividef(x[e] >= 0.f ? 1.0f : ex, 1.0f + ex);   // sigmoid(x) = d softplus / dx
      float sn, cs;
      sincos_reduced(__fadd_rn(__fmul_rn(pos, om[e]), dl[e]), &sn, &cs);
      dx[e] = (gc[e] * cs + gs[e] * sn) * sig;
      const float dphi = mu * (gs[e] * cs - gc[e] * sn);
      acc_w[e] = fmaf(dphi, pos, acc_w[e]);
      acc_d[e] += dphi;
    }
    *reinterpret_cast<uint4*>(dxr + cv * 8) = pack8(dx);
    if (p.d_c > 0) {
      __nv_bfloat16* dxc = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.dxc.ptr)) + row_offset(p.dxc, b, h, s);
      for (int cg = cv; cg < p.d_c / 8; cg += VPR) {
        float g[8];
        load_grad8(p.grad.ptr, goff + cg * 8, g);
        *reinterpret_cast<uint4*>(dxc + cg * 8) = pack8(g);
      }
    }
  }
  // lanes with the same column group: lane % VPR
#pragma unroll
  for (int e = 0; e < 8; ++e) {
#pragma unroll
    for (int off = 16; off >= VPR; off >>= 1) {
      acc_w[e] += __shfl_xor_sync(0xffffffffu, acc_w[e], off);
      acc_d[e] += __shfl_xor_sync(0xffffffffu, acc_d[e], off);
    }
  }
  if ((threadIdx.x & 31) < VPR) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      atomicAdd(&sum_w[cv * 8 + e], (double)acc_w[e]);
      atomicAdd(&sum_d[cv * 8 + e], (double)acc_d[e]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < DR; i += blockDim.x) {
    atomicAdd(p.d_omega + i, sum_w[i]);
    // gradient of the RAW bias: clamp(delta, -2 pi, 0) passes it on inside the interval only
    if (p.d_delta != nullptr && p.delta != nullptr && p.delta[i] >= -kTwoPi && p.delta[i] <= 0.0f)
      atomicAdd(p.d_delta + i, sum_d[i]);
  }
}

// ---- rotary family / QKNorm --------------------------------------------------------------
// expand:   y = normalise(mscale * rotate(x)) with the forward kernel's rounding order (bf16
//           after the rotation, after mscale and after the normalisation); rotation and
//           normalisation are both optional (src/model/rope.py:35-57, rope.py:216-217,
//           src/model/normalization.py:44-56).
// backward: with r the rotated, scaled row and n = |r|_2,
//           d r = g / (n + eps) - r (r . g) / (n (n + eps)^2),   d x = mscale * rotate^T(d r);
//           the roundings are treated as the identity, as autograd treats the casts.
// thread = (row, 8 columns = 4 rotation pairs); the D/8 threads of a row are neighbours in a
// warp and reduce the two row sums with shuffles.
struct RnParams {
  int B, S, H, row0, qk_norm, grad_bf16;
  float mscale, eps;
  TensorRef x, out, grad, dx;
  const float* table;   // [rows, D/2, 2] (cos, sin) or null: no rotation
};

template <int D>
__device__ __forceinline__ void rotated_row(const RnParams& p, const uint4& raw, int s, int cv, float (&r)[8],
                                            float (&cs)[4], float (&sn)[4]) {
  uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if (p.table != nullptr) {
    const float4* tp = reinterpret_cast<const float4*>(p.table + ((size_t)(p.row0 + s) * (D / 2) + cv * 4) * 2);
    const float4 t0 = __ldg(tp), t1 = __ldg(tp + 1);
    cs[0] = t0.x; sn[0] = t0.y; cs[1] = t0.z; sn[1] = t0.w; cs[2] = t1.x; sn[2] = t1.y; cs[3] = t1.z; sn[3] = t1.w;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x0 = bf16_lo(w[e]), x1 = bf16_hi(w[e]);
      w[e] = pack_bf16x2(x0 * cs[e] - x1 * sn[e], x0 * sn[e] + x1 * cs[e]);
      if (p.mscale != 1.0f) w[e] = pack_bf16x2(bf16_lo(w[e]) * p.mscale, bf16_hi(w[e]) * p.mscale);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    r[2 * e] = bf16_lo(w[e]);
    r[2 * e + 1] = bf16_hi(w[e]);
  }
}

template <int D, bool BACKWARD>
__global__ void __launch_bounds__(256) rotary_norm_kernel(const RnParams p) {
  constexpr int VPR = D / 8;
  const long long n = (long long)p.B * p.S * p.H * VPR;
  // whole warps stay in the loop together (the shuffles below need all lanes of a row)
  const long long n_pad = (n + 31) / 32 * 32;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n_pad; idx += stride) {
    const bool live = idx < n;
    const long long row = (live ? idx : n - 1) / VPR;
    const int cv = (int)(idx % VPR);
    const int h = (int)(row % p.H), s = (int)((row / p.H) % p.S), b = (int)(row / ((long long)p.H * p.S));
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x.ptr) + row_offset(p.x, b, h, s);
    float r[8], cs[4], sn[4];
    rotated_row<D>(p, ldg_nc_v4(x + cv * 8), s, cv, r, cs, sn);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(r[e], r[e], ss);
    if constexpr (!BACKWARD) {
      if (p.qk_norm) {
#pragma unroll
        for (int d = 1; d < VPR; d <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
        const float inv = 1.0f / (sqrtf(ss) + p.eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] *= inv;
      }
      if (live) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.out.ptr)) + row_offset(p.out, b, h, s);
        *reinterpret_cast<uint4*>(out + cv * 8) = pack8(r);
      }
    } else {
      // gradient with respect to the normalised row: fp32 [.., D] (queries) or bf16 (keys)
      float g[8];
      const long long goff = row_offset(p.grad, b, h, s) + cv * 8;
      if (p.grad_bf16) {
        unpack8(ldg_nc_v4(reinterpret_cast<const __nv_bfloat16*>(p.grad.ptr) + goff), g);
      } else {
        const float4* gp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.grad.ptr) + goff);
        const float4 a = __ldg(gp), c = __ldg(gp + 1);
        g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = c.x; g[5] = c.y; g[6] = c.z; g[7] = c.w;
      }
      float dr[8];
      if (p.qk_norm) {
        float rg = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) rg = fmaf(r[e], g[e], rg);
#pragma unroll
        for (int d = 1; d < VPR; d <<= 1) {
          ss += __shfl_xor_sync(0xffffffffu, ss, d);
          rg += __shfl_xor_sync(0xffffffffu, rg, d);
        }
        const float nrm = sqrtf(ss), inv = 1.0f / (nrm + p.eps);
        const float coef = nrm > 0.f ? rg * inv * inv / nrm : 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) dr[e] = g[e] * inv - r[e] * coef;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) dr[e] = g[e];
      }
      float dx[8];
      if (p.table != nullptr) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          dx[2 * e] = (dr[2 * e] * cs[e] + dr[2 * e + 1] * sn[e]) * p.mscale;
          dx[2 * e + 1] = (dr[2 * e + 1] * cs[e] - dr[2 * e] * sn[e]) * p.mscale;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) dx[e] = dr[e];
      }
      if (live) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.dx.ptr)) + row_offset(p.dx, b, h, s);
        *reinterpret_cast<uint4*>(out + cv * 8) = pack8(dx);
      }
    }
  }
}

// ---- FoPE frequency mix (src/model/fpope.py:107-146) and its gradient -------------------------
// One thread per position dimension c; d_r and the number of Fourier terms are tens.
// one warp per frequency column
__global__ void fope_freqs_kernel(const KParams p, int d_r, float* omega) {
  const int c = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (c >= d_r) return;
  const float f = effective_freq_lanes<32>(p, c, lane);
  if (lane == 0) omega[c] = f;
}

// eff = base * W / Z + base with W = sum_j a_j j, Z = sum_j |a_j| + 1e-8 (Z = 1 without
// normalisation); zero gradient where the floor clip or the ceiling clamp is active.
__global__ void fope_freqs_backward_kernel(const KParams p, int d_r, const double* d_omega, float* d_coeffs,
                                           float* d_base) {
  // one warp per frequency column, the Fourier terms dealt to its lanes
  const int c = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (c >= d_r) return;
  const float* a = p.coeffs + (size_t)c * p.n_fourier;
  const bool normalize = (p.flags & PE_ATTN_FOURIER_NORMALIZE) != 0;
  double Zs = 0.0, W = 0.0;
  for (int j = lane; j < p.n_fourier; j += 32) {
    Zs += fabs((double)a[j]);
    W += (double)a[j] * (j + 1);
  }
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    Zs += __shfl_xor_sync(0xffffffffu, Zs, d);
    W += __shfl_xor_sync(0xffffffffu, W, d);
  }
  const double Z = normalize ? 1e-8 + Zs : 1.0;
  const double base = p.freqs[c];
  const double eff = base * W / Z + base;
  bool pass = fabs(eff) >= (double)p.floor_freq;
  if ((p.flags & PE_ATTN_FOURIER_CEILING) && fabs(eff) > (double)p.ceil_freq) pass = false;
  const double g = pass ? d_omega[c] : 0.0;
  for (int j = lane; j < p.n_fourier; j += 32) {
    double d = (j + 1) / Z;
    if (normalize) {
      const double sgn = a[j] > 0.f ? 1.0 : (a[j] < 0.f ? -1.0 : 0.0);
      d -= W / (Z * Z) * sgn;
    }
    d_coeffs[(size_t)c * p.n_fourier + j] = (float)(g * base * d);
  }
  if (d_base != nullptr && lane == 0) d_base[c] = (float)(g * (W / Z + 1.0));
}

int check_tensor(const char* name, const void* ptr, const int64_t* s) {
  if (ptr == nullptr) {
    set_error("%s is null", name);
    return PE_ATTN_ERR_NULL;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) {
    set_error("%s is not 16-byte aligned", name);
    return PE_ATTN_ERR_ALIGNMENT;
  }
  for (int i = 0; i < 3; ++i)
    if (s[i] % 8 != 0) {
      set_error("%s stride[%d]=%lld is not a multiple of 8 elements", name, i, (long long)s[i]);
      return PE_ATTN_ERR_ALIGNMENT;
    }
  return PE_ATTN_OK;
}

unsigned grid_for(long long n_threads) {
  long long blocks = (n_threads + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

TensorRef ref_of(const void* ptr, const int64_t* s) { return TensorRef{ptr, s[0], s[1], s[2]}; }

}  // namespace
}  // namespace pe_attn

using namespace pe_attn;

extern "C" int pe_pope_expand(const void* x_c, const int64_t* xc_stride, const void* x_r, const int64_t* xr_stride, void* out,
                              const int64_t* out_stride, int B, int S, int H, int d_c, int d_r, int pos0, const float* omega,
                              const float* delta, void* stream) {
  if (B < 1 || S < 1 || H < 1 || (d_r != 32 && d_r != 64) || d_c < 0 || d_c % 8 != 0) {
    set_error("pe_pope_expand: unsupported shape (d_r must be 32 or 64, d_c a multiple of 8)");
    return PE_ATTN_ERR_SHAPE;
  }
  int rc;
  if ((rc = check_tensor("x_r", x_r, xr_stride)) || (rc = check_tensor("out", out, out_stride))) return rc;
  if (d_c > 0 && (rc = check_tensor("x_c", x_c, xc_stride))) return rc;
  if (omega == nullptr) {
    set_error("omega is null");
    return PE_ATTN_ERR_NULL;
  }
  XfParams p;
  memset(&p, 0, sizeof(p));
  p.B = B; p.S = S; p.H = H; p.d_c = d_c; p.pos0 = pos0;
  if (d_c > 0) p.xc = ref_of(x_c, xc_stride);
  p.xr = ref_of(x_r, xr_stride);
  p.out = ref_of(out, out_stride);
  p.omega = omega; p.delta = delta;
  const unsigned grid = grid_for((long long)B * S * H * (d_r / 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d_r == 32) pope_expand_kernel<32><<<grid, 256, 0, st>>>(p);
  else pope_expand_kernel<64><<<grid, 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("pe_pope_expand launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

extern "C" int pe_pope_expand_backward(const void* grad, int grad_dtype, const int64_t* grad_stride, const void* x_r,
                                       const int64_t* xr_stride, void* dx_c, const int64_t* dxc_stride, void* dx_r,
                                       const int64_t* dxr_stride, int B, int S, int H, int d_c, int d_r, int pos0,
                                       const float* omega, const float* delta, double* d_omega, double* d_delta,
                                       void* stream) {
  if (B < 1 || S < 1 || H < 1 || (d_r != 32 && d_r != 64) || d_c < 0 || d_c % 8 != 0) {
    set_error("pe_pope_expand_backward: unsupported shape (d_r must be 32 or 64, d_c a multiple of 8)");
    return PE_ATTN_ERR_SHAPE;
  }
  if (grad_dtype != PE_ATTN_BF16 && grad_dtype != PE_ATTN_FP32) {
    set_error("grad_dtype must be PE_ATTN_BF16 or PE_ATTN_FP32");
    return PE_ATTN_ERR_VARIANT;
  }
  int rc;
  if ((rc = check_tensor("grad", grad, grad_stride)) || (rc = check_tensor("x_r", x_r, xr_stride)) ||
      (rc = check_tensor("dx_r", dx_r, dxr_stride)))
    return rc;
  if (d_c > 0 && (rc = check_tensor("dx_c", dx_c, dxc_stride))) return rc;
  if (omega == nullptr || d_omega == nullptr) {
    set_error("omega and d_omega are required");
    return PE_ATTN_ERR_NULL;
  }
  XfParams p;
  memset(&p, 0, sizeof(p));
  p.B = B; p.S = S; p.H = H; p.d_c = d_c; p.pos0 = pos0;
  p.grad = ref_of(grad, grad_stride);
  p.xr = ref_of(x_r, xr_stride);
  if (d_c > 0) p.dxc = ref_of(dx_c, dxc_stride);
  p.dxr = ref_of(dx_r, dxr_stride);
  p.omega = omega; p.delta = delta; p.d_omega = d_omega; p.d_delta = d_delta;
  unsigned grid = grid_for((long long)B * S * H * (d_r / 8));
  if (grid > 148u * 3u) grid = 148u * 3u;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f32 = grad_dtype == PE_ATTN_FP32;
  if (d_r == 32) {
    if (f32) pope_expand_backward_kernel<32, true><<<grid, 256, 0, st>>>(p);
    else pope_expand_backward_kernel<32, false><<<grid, 256, 0, st>>>(p);
  } else {
    if (f32) pope_expand_backward_kernel<64, true><<<grid, 256, 0, st>>>(p);
    else pope_expand_backward_kernel<64, false><<<grid, 256, 0, st>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("pe_pope_expand_backward launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

// flags: bit 0 = apply the rotation table, bit 1 = L2-normalise the rows
static int launch_rotary_norm(bool backward, const void* x, const int64_t* x_stride, void* out, const int64_t* out_stride,
                              const void* grad, int grad_dtype, const int64_t* grad_stride, int B, int S, int H, int D,
                              const float* table, int table_row0, int table_rows, float mscale, int qk_norm, float eps,
                              void* stream) {
  if (B < 1 || S < 1 || H < 1 || (D != 64 && D != 128)) {
    set_error("rotary / QKNorm transform: unsupported shape (head dim must be 64 or 128)");
    return PE_ATTN_ERR_SHAPE;
  }
  int rc;
  if ((rc = check_tensor("x", x, x_stride)) || (rc = check_tensor(backward ? "dx" : "out", out, out_stride))) return rc;
  if (backward && (rc = check_tensor("grad", grad, grad_stride))) return rc;
  if (table != nullptr && (table_row0 < 0 || table_row0 + S > table_rows)) {
    set_error("rotary table rows [%d, %d) do not cover the positions in use", table_row0, table_row0 + S);
    return PE_ATTN_ERR_SHAPE;
  }
  RnParams p;
  memset(&p, 0, sizeof(p));
  p.B = B; p.S = S; p.H = H; p.row0 = table_row0;
  p.mscale = table != nullptr ? mscale : 1.0f; p.eps = eps; p.table = table;
  p.x = ref_of(x, x_stride);
  if (backward) {
    p.dx = ref_of(out, out_stride);
    p.grad = ref_of(grad, grad_stride);
    p.qk_norm = qk_norm ? 1 : 0;
    p.grad_bf16 = grad_dtype == PE_ATTN_BF16 ? 1 : 0;
  } else {
    p.out = ref_of(out, out_stride);
    p.qk_norm = qk_norm ? 1 : 0;
  }
  const unsigned grid = grid_for((long long)B * S * H * (D / 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 64) {
    if (backward) rotary_norm_kernel<64, true><<<grid, 256, 0, st>>>(p);
    else rotary_norm_kernel<64, false><<<grid, 256, 0, st>>>(p);
  } else {
    if (backward) rotary_norm_kernel<128, true><<<grid, 256, 0, st>>>(p);
    else rotary_norm_kernel<128, false><<<grid, 256, 0, st>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rotary / QKNorm transform launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

extern "C" int pe_rotary_norm_expand(const void* x, const int64_t* x_stride, void* out, const int64_t* out_stride, int B,
                                     int S, int H, int D, const float* table, int table_row0, int table_rows,
                                     float mscale, int qk_norm, float eps, void* stream) {
  return launch_rotary_norm(false, x, x_stride, out, out_stride, nullptr, 0, nullptr, B, S, H, D, table, table_row0,
                            table_rows, mscale, qk_norm, eps, stream);
}

extern "C" int pe_rotary_norm_expand_backward(const void* grad, int grad_dtype, const int64_t* grad_stride, const void* x,
                                              const int64_t* x_stride, void* dx, const int64_t* dx_stride, int B, int S,
                                              int H, int D, const float* table, int table_row0, int table_rows,
                                              float mscale, int qk_norm, float eps, void* stream) {
  if (grad_dtype != PE_ATTN_BF16 && grad_dtype != PE_ATTN_FP32) {
    set_error("grad_dtype must be PE_ATTN_BF16 or PE_ATTN_FP32");
    return PE_ATTN_ERR_VARIANT;
  }
  return launch_rotary_norm(true, x, x_stride, dx, dx_stride, grad, grad_dtype, grad_stride, B, S, H, D, table,
                            table_row0, table_rows, mscale, qk_norm, eps, stream);
}

static int fope_params(KParams* k, const float* base, const float* coeffs, int d_r, int n_fourier, unsigned flags,
                       float floor_freq, float ceil_freq) {
  if (base == nullptr || coeffs == nullptr) {
    set_error("base frequencies and fourier_coeffs are required");
    return PE_ATTN_ERR_NULL;
  }
  if (d_r < 1 || d_r > 1024 || n_fourier < 1) {
    set_error("unsupported d_r / n_fourier");
    return PE_ATTN_ERR_SHAPE;
  }
  memset(k, 0, sizeof(*k));
  k->flags = PE_ATTN_FOURIER_MIX | (flags & (PE_ATTN_FOURIER_NORMALIZE | PE_ATTN_FOURIER_CEILING));
  k->freqs = base; k->coeffs = coeffs; k->n_fourier = n_fourier;
  k->floor_freq = floor_freq; k->ceil_freq = ceil_freq;
  return PE_ATTN_OK;
}

extern "C" int pe_fope_effective_freqs(const float* base, const float* coeffs, int d_r, int n_fourier, unsigned flags,
                                       float floor_freq, float ceil_freq, float* omega, void* stream) {
  KParams k;
  int rc = fope_params(&k, base, coeffs, d_r, n_fourier, flags, floor_freq, ceil_freq);
  if (rc) return rc;
  if (omega == nullptr) {
    set_error("omega is null");
    return PE_ATTN_ERR_NULL;
  }
  fope_freqs_kernel<<<(d_r * 32 + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(k, d_r, omega);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("pe_fope_effective_freqs launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

extern "C" int pe_fope_effective_freqs_backward(const float* base, const float* coeffs, int d_r, int n_fourier,
                                                unsigned flags, float floor_freq, float ceil_freq, const double* d_omega,
                                                float* d_coeffs, float* d_base, void* stream) {
  KParams k;
  int rc = fope_params(&k, base, coeffs, d_r, n_fourier, flags, floor_freq, ceil_freq);
  if (rc) return rc;
  if (d_omega == nullptr || d_coeffs == nullptr) {
    set_error("d_omega and d_coeffs are required");
    return PE_ATTN_ERR_NULL;
  }
  fope_freqs_backward_kernel<<<(d_r * 32 + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(k, d_r, d_omega, d_coeffs,
                                                                                            d_base);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("pe_fope_effective_freqs_backward launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}
