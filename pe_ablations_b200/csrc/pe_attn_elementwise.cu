// HBM-bound companions of the attention kernel on the evaluation path: RMSNorm and SwiGLU in
// one pass each.  The eager code they replace makes five to seven passes over the activation
// (upcast, square, mean, rsqrt-multiply, downcast, weight multiply, and one more cast per
// consuming linear layer under autocast), which added up to 40 % of the evaluation's GPU time.
//
//   rmsnorm:  y = cast( cast(x * rsqrt(mean(x^2) + eps)) * w )      x, y: [rows, dim] bf16 or fp32, w fp32
//             (the inner cast is the reference's ``type_as(x)``, the outer one is what the next
//             linear layer's autocast does; for fp32 tensors both are identities)
//   swiglu:   y = cast( cast(silu(g)) * u )                         g, u, y: [n] bf16 or fp32
//
// Algorithmic bytes: rmsnorm 2 * rows * dim * sizeof(T) (+ dim * 4 once), swiglu 3 * n * sizeof(T).
#include "pe_attn_common.cuh"
#include "pe_attn_ptx.cuh"

namespace pe_attn {
namespace {

constexpr int EW_THREADS = 256;

template <bool BF16>
__device__ __forceinline__ void load8(const void* p, float (&x)[8]) {
  if constexpr (BF16) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    x[0] = ptx::bf16_lo(w.x); x[1] = ptx::bf16_hi(w.x); x[2] = ptx::bf16_lo(w.y); x[3] = ptx::bf16_hi(w.y);
    x[4] = ptx::bf16_lo(w.z); x[5] = ptx::bf16_hi(w.z); x[6] = ptx::bf16_lo(w.w); x[7] = ptx::bf16_hi(w.w);
  } else {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
}
template <bool BF16>
__device__ __forceinline__ void store8(void* p, const float (&x)[8]) {
  if constexpr (BF16) {
    uint4 w;
    w.x = ptx::pack_bf16x2(x[0], x[1]); w.y = ptx::pack_bf16x2(x[2], x[3]);
    w.z = ptx::pack_bf16x2(x[4], x[5]); w.w = ptx::pack_bf16x2(x[6], x[7]);
    *reinterpret_cast<uint4*>(p) = w;
  } else {
    reinterpret_cast<float4*>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
  }
}
template <bool BF16>
__device__ __forceinline__ float round_like(float v) {
  if constexpr (BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

// one CTA per row (grid-stride); the row is read twice, the second time from L1/L2
template <bool BF16>
__global__ void __launch_bounds__(EW_THREADS) rmsnorm_kernel(const void* x, const float* w, void* y, int rows, int dim,
                                                             long long x_stride, long long y_stride, float eps) {
  __shared__ float red[EW_THREADS / 32];
  constexpr int ESZ = BF16 ? 2 : 4;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_vec = dim / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const char* xr = reinterpret_cast<const char*>(x) + (size_t)row * x_stride * ESZ;
    char* yr = reinterpret_cast<char*>(y) + (size_t)row * y_stride * ESZ;
    float ss = 0.f;
    for (int v = tid; v < n_vec; v += EW_THREADS) {
      float a[8];
      load8<BF16>(xr + (size_t)v * 8 * ESZ, a);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(a[e], a[e], ss);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < EW_THREADS / 32; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / (float)dim + eps);
    for (int v = tid; v < n_vec; v += EW_THREADS) {
      float a[8], g[8];
      load8<BF16>(xr + (size_t)v * 8 * ESZ, a);
      load8<false>(w + (size_t)v * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = round_like<BF16>(a[e] * rstd) * g[e];
      store8<BF16>(yr + (size_t)v * 8 * ESZ, a);
    }
    __syncthreads();
  }
}

template <bool BF16>
__global__ void __launch_bounds__(EW_THREADS) swiglu_kernel(const void* g, const void* u, void* y, long long n_vec) {
  constexpr int ESZ = BF16 ? 2 : 4;
  for (long long v = (long long)blockIdx.x * EW_THREADS + threadIdx.x; v < n_vec; v += (long long)gridDim.x * EW_THREADS) {
    float a[8], b[8];
    load8<BF16>(reinterpret_cast<const char*>(g) + v * 8 * ESZ, a);
    load8<BF16>(reinterpret_cast<const char*>(u) + v * 8 * ESZ, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = round_like<BF16>(a[e] / (1.0f + expf(-a[e]))) * b[e];
    store8<BF16>(reinterpret_cast<char*>(y) + v * 8 * ESZ, a);
  }
}

int grid_for(long long work_items) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long g = (long long)sms * 8;
  return (int)(work_items < g ? (work_items > 0 ? work_items : 1) : g);
}

}  // namespace
}  // namespace pe_attn

using namespace pe_attn;

extern "C" {

int pe_rmsnorm_forward(const void* x, const float* weight, void* y, int dtype, int rows, int dim, int64_t x_stride,
                       int64_t y_stride, float eps, void* stream) {
  if (x == nullptr || weight == nullptr || y == nullptr) { set_error("x, weight or y is null"); return PE_ATTN_ERR_NULL; }
  if (dtype != PE_ATTN_BF16 && dtype != PE_ATTN_FP32) { set_error("unknown dtype %d", dtype); return PE_ATTN_ERR_VARIANT; }
  if (rows < 1 || dim < 8 || dim % 8 != 0 || x_stride < dim || y_stride < dim) {
    set_error("rmsnorm needs rows >= 1, dim a positive multiple of 8 and strides >= dim (got %d, %d)", rows, dim);
    return PE_ATTN_ERR_SHAPE;
  }
  const int esz = dtype == PE_ATTN_BF16 ? 2 : 4;
  const int need = esz == 2 ? 15 : 31;
  if ((reinterpret_cast<uintptr_t>(x) & need) || (reinterpret_cast<uintptr_t>(y) & need) ||
      (reinterpret_cast<uintptr_t>(weight) & 31) || (x_stride * esz) % (need + 1) || (y_stride * esz) % (need + 1)) {
    set_error("rmsnorm needs %d-byte aligned rows", need + 1);
    return PE_ATTN_ERR_ALIGNMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows);
  if (dtype == PE_ATTN_BF16) rmsnorm_kernel<true><<<grid, EW_THREADS, 0, s>>>(x, weight, y, rows, dim, x_stride, y_stride, eps);
  else rmsnorm_kernel<false><<<grid, EW_THREADS, 0, s>>>(x, weight, y, rows, dim, x_stride, y_stride, eps);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("rmsnorm launch failed: %s", cudaGetErrorString(e)); return PE_ATTN_ERR_LAUNCH; }
  return PE_ATTN_OK;
}

int pe_swiglu_forward(const void* gate, const void* up, void* y, int dtype, int64_t n, void* stream) {
  if (gate == nullptr || up == nullptr || y == nullptr) { set_error("gate, up or y is null"); return PE_ATTN_ERR_NULL; }
  if (dtype != PE_ATTN_BF16 && dtype != PE_ATTN_FP32) { set_error("unknown dtype %d", dtype); return PE_ATTN_ERR_VARIANT; }
  if (n < 8 || n % 8 != 0) { set_error("swiglu needs a positive multiple of 8 elements (got %lld)", (long long)n); return PE_ATTN_ERR_SHAPE; }
  const int need = dtype == PE_ATTN_BF16 ? 15 : 31;
  if ((reinterpret_cast<uintptr_t>(gate) & need) || (reinterpret_cast<uintptr_t>(up) & need) || (reinterpret_cast<uintptr_t>(y) & need)) {
    set_error("swiglu needs %d-byte aligned contiguous tensors", need + 1);
    return PE_ATTN_ERR_ALIGNMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long n_vec = n / 8;
  const int grid = grid_for((n_vec + EW_THREADS - 1) / EW_THREADS);
  if (dtype == PE_ATTN_BF16) swiglu_kernel<true><<<grid, EW_THREADS, 0, s>>>(gate, up, y, n_vec);
  else swiglu_kernel<false><<<grid, EW_THREADS, 0, s>>>(gate, up, y, n_vec);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("swiglu launch failed: %s", cudaGetErrorString(e)); return PE_ATTN_ERR_LAUNCH; }
  return PE_ATTN_OK;
}

}  // extern "C"
