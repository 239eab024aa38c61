// Next-token cross-entropy as loss SUMS for the perplexity evaluation.
//
// For a chunk of logits [n_rows, vocab] and targets [n_rows] this adds
//   out[0] += sum over scored rows of (logsumexp(logits[r, :]) - logits[r, target[r]])
//   out[1] += number of scored rows (target != ignore_index)
// to a caller-owned pair of doubles, which is what a sharded evaluation reduces across
// ranks.  Rows with non-finite losses (NaN or +inf logits) are scored and make the sum
// non-finite, as the eager cross-entropy does; -inf logits count as probability zero; a
// target outside [0, vocab) other than ignore_index makes the sum NaN.  It reads each
// logit exactly once in its stored type (bf16 or fp32); the eager path it replaces upcasts
// the chunk to fp32 and materialises the log-softmax.
//
// One CTA streams one row at a time (grid-stride over rows) with 16-byte loads and an
// online logsumexp per thread, then warp-shuffle and shared-memory reductions.  Row
// losses go to a scratch array; the last CTA to finish adds them up in a fixed order, so
// the result does not depend on the order in which CTAs run.  The scratch is
// [n_rows] floats plus one counter word that must be zero on entry and is left zero.
#include <mutex>

#include "pe_attn_common.cuh"
#include "pe_attn_ptx.cuh"

namespace pe_attn {
namespace {

constexpr int CE_THREADS = 256;

// Scratch of the allocation-free entry point: a counter block followed by one float per
// row.  It is part of the library image, so every GPU that loads the library holds these
// 64.25 KiB until the process exits.
constexpr int CE_STATIC_MAX_ROWS = 16384;
static __device__ __align__(256) unsigned char g_ce_static_scratch[256 + CE_STATIC_MAX_ROWS * sizeof(float)];

struct CeParams {
  const void* logits;
  long long row_stride;  // elements
  const long long* targets;
  int n_rows, vocab, ignore_index;
  float* row_loss;        // scratch [n_rows]
  unsigned int* counter;  // scratch [1], zero on entry
  double* out;            // [2], accumulated
};

__device__ __forceinline__ void online_add(float& m, float& s, float x) {
  // running (max, sum of exp(x - max)); natural base
  if (x > m) {
    s = s * __expf(m - x) + 1.0f;
    m = x;
  } else if (x != -INFINITY) {  // a -inf logit adds nothing (and -inf - -inf would be NaN)
    s += __expf(x - m);
  }
}

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) return;
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

template <bool BF16>
__global__ void __launch_bounds__(CE_THREADS) ce_loss_sums_kernel(const CeParams p) {
  __shared__ float sm_m[CE_THREADS / 32], sm_s[CE_THREADS / 32];
  __shared__ bool is_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int VEC = BF16 ? 8 : 4;  // elements per 16-byte load

  for (int row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
    const long long tgt = p.targets[row];
    const char* base = reinterpret_cast<const char*>(p.logits) + (size_t)row * p.row_stride * (BF16 ? 2 : 4);
    float m = -INFINITY, s = 0.f;
    auto scalar_at = [&](int c) -> float {
      if constexpr (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[c]);
      else return reinterpret_cast<const float*>(base)[c];
    };
    // rows need not start on a 16-byte boundary (e.g. an odd vocabulary size): a scalar
    // head up to the first aligned element, 16-byte vectors, then a scalar tail
    constexpr int ESZ = BF16 ? 2 : 4;
    int lead = (int)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(base) & 15u)) & 15u) / ESZ);
    if (lead > p.vocab) lead = p.vocab;
    const int n_vec = (p.vocab - lead) / VEC;
    if (tid < lead) online_add(m, s, scalar_at(tid));
    const char* vbase = base + (size_t)lead * ESZ;
    for (int v = tid; v < n_vec; v += CE_THREADS) {
      const uint4 w = ptx::ldg_nc_v4(vbase + (size_t)v * 16);
      float x[8];
      if constexpr (BF16) {
        x[0] = ptx::bf16_lo(w.x); x[1] = ptx::bf16_hi(w.x); x[2] = ptx::bf16_lo(w.y); x[3] = ptx::bf16_hi(w.y);
        x[4] = ptx::bf16_lo(w.z); x[5] = ptx::bf16_hi(w.z); x[6] = ptx::bf16_lo(w.w); x[7] = ptx::bf16_hi(w.w);
      } else {
        x[0] = __uint_as_float(w.x); x[1] = __uint_as_float(w.y); x[2] = __uint_as_float(w.z); x[3] = __uint_as_float(w.w);
      }
      float vm = x[0];
#pragma unroll
      for (int e = 1; e < VEC; ++e) vm = fmaxf(vm, x[e]);
      if (vm == -INFINITY) continue;  // eight -inf logits add nothing (NaN is not -inf and goes on)
      if (vm > m) {
        s *= __expf(m - vm);
        m = vm;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) s += __expf(x[e] - m);
    }
    for (int c = lead + n_vec * VEC + tid; c < p.vocab; c += CE_THREADS) online_add(m, s, scalar_at(c));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, d), s2 = __shfl_xor_sync(0xffffffffu, s, d);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) { sm_m[warp] = m; sm_s[warp] = s; }
    __syncthreads();
    if (tid == 0) {
      float mm = sm_m[0], ss = sm_s[0];
      for (int w = 1; w < CE_THREADS / 32; ++w) online_merge(mm, ss, sm_m[w], sm_s[w]);
      // -inf marks an ignored row: a scored row's loss is finite, +inf or NaN, never -inf
      float loss = -INFINITY;
      if (tgt != (long long)p.ignore_index) {
        // a target outside [0, vocab) is an error of the caller: it is scored as NaN, so the
        // sums (and the perplexity) come out NaN instead of silently skipping the row
        loss = (tgt >= 0 && tgt < p.vocab) ? (mm + logf(ss)) - scalar_at((int)tgt) : __int_as_float(0x7fc00000);
      }
      p.row_loss[row] = loss;
    }
    __syncthreads();
  }

  // the last CTA to get here adds the row losses in a fixed order
  if (tid == 0) {
    __threadfence();
    const unsigned done = atomicAdd(p.counter, 1u);
    is_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  double acc = 0.0, cnt = 0.0;
  for (int r = tid; r < p.n_rows; r += CE_THREADS) {
    const float l = reinterpret_cast<volatile float*>(p.row_loss)[r];
    if (l != -INFINITY) { acc += (double)l; cnt += 1.0; }  // NaN and +inf losses reach the sum
  }
  __shared__ double red_a[CE_THREADS], red_c[CE_THREADS];
  red_a[tid] = acc;
  red_c[tid] = cnt;
  __syncthreads();
  for (int w = CE_THREADS / 2; w > 0; w >>= 1) {
    if (tid < w) { red_a[tid] += red_a[tid + w]; red_c[tid] += red_c[tid + w]; }
    __syncthreads();
  }
  if (tid == 0) {
    p.out[0] += red_a[0];
    p.out[1] += red_c[0];
    *p.counter = 0u;  // ready for the next call
  }
}

int check(const void* logits, int dtype, long long row_stride, const long long* targets, int n_rows, int vocab,
          const void* out) {
  if (logits == nullptr || targets == nullptr || out == nullptr) {
    set_error("logits, targets or out is null");
    return PE_ATTN_ERR_NULL;
  }
  if (dtype != PE_ATTN_BF16 && dtype != PE_ATTN_FP32) {
    set_error("unknown dtype %d", dtype);
    return PE_ATTN_ERR_VARIANT;
  }
  if (n_rows < 1 || vocab < 1 || row_stride < vocab) {
    set_error("need n_rows >= 1, vocab >= 1, row_stride >= vocab (got %d, %d, %lld)", n_rows, vocab, row_stride);
    return PE_ATTN_ERR_SHAPE;
  }
  const unsigned esz = dtype == PE_ATTN_BF16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(logits) & (esz - 1)) || (reinterpret_cast<uintptr_t>(out) & 7u)) {
    set_error("logits must be aligned to their element size and out to 8 bytes");
    return PE_ATTN_ERR_ALIGNMENT;
  }
  return PE_ATTN_OK;
}

}  // namespace

int launch_ce(const void* logits, int dtype, long long row_stride, const long long* targets, int n_rows, int vocab,
              int ignore_index, float* row_loss, unsigned int* counter, double* out, cudaStream_t stream) {
  const int rc = check(logits, dtype, row_stride, targets, n_rows, vocab, out);
  if (rc != PE_ATTN_OK) return rc;
  CeParams p{logits, row_stride, targets, n_rows, vocab, ignore_index, row_loss, counter, out};
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms * 8;  // 8 resident CTAs of 256 threads per SM
  if (grid > n_rows) grid = n_rows;
  if (dtype == PE_ATTN_BF16) ce_loss_sums_kernel<true><<<grid, CE_THREADS, 0, stream>>>(p);
  else ce_loss_sums_kernel<false><<<grid, CE_THREADS, 0, stream>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("cross-entropy kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

}  // namespace pe_attn

extern "C" {

size_t pe_ce_scratch_bytes(int n_rows) { return (size_t)(n_rows > 0 ? n_rows : 0) * sizeof(float) + 256; }

int pe_ce_loss_sums(const void* logits, int dtype, int64_t row_stride, const int64_t* targets, int n_rows, int vocab,
                    int ignore_index, void* scratch, double* out, void* stream) {
  if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 255u)) {
    pe_attn::set_error("scratch must be a 256-byte aligned device buffer of pe_ce_scratch_bytes(n_rows) bytes");
    return scratch == nullptr ? PE_ATTN_ERR_NULL : PE_ATTN_ERR_ALIGNMENT;
  }
  // layout: [0, 256) counter word (zero between calls), then the row losses
  unsigned int* counter = reinterpret_cast<unsigned int*>(scratch);
  float* row_loss = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + 256);
  return pe_attn::launch_ce(logits, dtype, row_stride, reinterpret_cast<const long long*>(targets), n_rows, vocab,
                            ignore_index, row_loss, counter, out, static_cast<cudaStream_t>(stream));
}

// Device address of g_ce_static_scratch on the current device.  In host code the array's
// name is only a handle for the runtime, never a device pointer, so the address is asked
// for once per device (with that device current) and remembered for the life of the
// process (a cudaDeviceReset would invalidate it; the library does not support being used
// across one).
static int static_scratch_address(void** ptr) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    pe_attn::set_error("no usable CUDA device is current (%s)", cudaGetErrorString(e));
    return PE_ATTN_ERR_DEVICE;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, pe_attn::g_ce_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      pe_attn::set_error("cudaGetSymbolAddress failed for the static scratch: %s", cudaGetErrorString(e));
      return PE_ATTN_ERR_LAUNCH;
    }
    cached[dev] = p;
  }
  *ptr = cached[dev];
  return PE_ATTN_OK;
}

int pe_ce_static_max_rows(void) { return pe_attn::CE_STATIC_MAX_ROWS; }

int pe_ce_loss_sums_static(const void* logits, int dtype, int64_t row_stride, const int64_t* targets, int n_rows,
                           int vocab, int ignore_index, double* out, void* stream) {
  if (n_rows > pe_attn::CE_STATIC_MAX_ROWS) {
    pe_attn::set_error("n_rows=%d exceeds the %d rows the built-in scratch holds; split the chunk or use "
                       "pe_ce_loss_sums with your own scratch", n_rows, pe_attn::CE_STATIC_MAX_ROWS);
    return PE_ATTN_ERR_TOO_LARGE;
  }
  // every check comes before the shared array is touched: a call that is refused must not
  // disturb a valid call that is using the array on another stream
  int rc = pe_attn::check(logits, dtype, row_stride, reinterpret_cast<const long long*>(targets), n_rows, vocab, out);
  if (rc != PE_ATTN_OK) return rc;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != PE_ATTN_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the counter block must start at zero
  const cudaError_t e = cudaMemsetAsync(scratch, 0, 256, s);
  if (e != cudaSuccess) {
    pe_attn::set_error("clearing the static scratch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  unsigned int* counter = reinterpret_cast<unsigned int*>(scratch);
  float* row_loss = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + 256);
  return pe_attn::launch_ce(logits, dtype, row_stride, reinterpret_cast<const long long*>(targets), n_rows, vocab,
                            ignore_index, row_loss, counter, out, s);
}

}  // extern "C"
