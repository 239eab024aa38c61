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
__global__ void __launch_bounds__(256) pope_expand_backward_kernel(const XfParams p) {
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
      const float ex = __expf(-fabsf(x[e]));                       // exp(-|x|)
      const float mu = fmaxf(x[e], 0.f) + log1pf(ex);
      const float sig = (x[e] >= 0.f ? 1.0f : ex) / (1.0f + ex);   // sigmoid(x) = d softplus / dx
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
    if (p.d_delta != nullptr) atomicAdd(p.d_delta + i, sum_d[i]);
  }
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
  const unsigned grid = grid_for((long long)B * S * H * (d_r / 8));
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
