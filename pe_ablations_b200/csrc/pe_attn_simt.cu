// FFMA (CUDA-core) fused PE-attention forward.
//
// This is the fp32 path: every positional transform follows the reference's fp32
// operation order (separately rounded position*frequency product, then the phase
// bias, accurate sin/cos/exp/log1p), because tensor cores at tf32 precision cannot
// hold the 1e-4 tolerance of the fp32 configurations.  Instantiated for bf16
// tensors too, where it serves as an on-device cross-check of the tcgen05 kernel.
//
// One CTA owns 64 query rows of one (batch, head) and streams 64-key tiles:
//   load + transform K tile -> S = Q K^T (4x4 per thread) -> online softmax with
//   16-lane shuffle reductions -> P to shared memory -> O += P V.
// Shared memory: Q and K operands [64][d_qk rounded up to 4, + 4], V [64][d_v rounded up to 4],
// P [64][68], per-dimension frequency / phase-bias vectors.  The row pitches are multiples of
// four floats, so both products read their operands with 16-byte shared-memory loads (four
// steps of the contraction per load; the pitch / 4 is odd at the usual head dims, which keeps
// the 16 rows of a half-warp on different banks); padded columns hold zeros.  The additions
// of every dot product still happen in ascending order of the contraction index.
#include "pe_attn_common.cuh"

namespace pe_attn {
namespace {

constexpr int BM = 64;
constexpr int BN = 64;
constexpr int NTHREADS = 256;
constexpr int MAX_VC = 8;  // d_v <= 128: up to 8 output columns per thread (stride 16)
constexpr int P_LD = BN + 4;

__host__ __device__ constexpr int round4(int x) { return (x + 3) & ~3; }

template <typename T>
__device__ __forceinline__ float load_elem(const void* base, long long off) {
  return static_cast<float>(reinterpret_cast<const T*>(base)[off]);
}
template <>
__device__ __forceinline__ float load_elem<__nv_bfloat16>(const void* base, long long off) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
}

template <bool ROUND>
__device__ __forceinline__ float round_op(float x) {
  if constexpr (ROUND) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

// Fill one 64-row operand tile (Q or K) in shared memory with the transformed rows.
// dst[row][0 .. d_qk) ; rows at or past n_rows are zero.
template <typename T, bool ROUND>
__device__ void build_operand_tile(const KParams& p, float* dst, int ld, const TensorRef& content,
                                   const TensorRef& posi, int b, int head, int row0, int n_rows, int pos0,
                                   bool is_key, const float* freq_s, const float* delta_s) {
  const int tid = threadIdx.x;
  const int d_c = p.d_c, d_r = p.d_r;
  const int n_pad = ld - p.d_qk;   // zero columns behind the operand (at least 4)
  for (int idx = tid; idx < BM * n_pad; idx += NTHREADS) dst[(idx / n_pad) * ld + p.d_qk + idx % n_pad] = 0.f;
  if (p.variant == PE_ATTN_ROTARY) {
    const int half = d_c >> 1;
    for (int idx = tid; idx < BM * half; idx += NTHREADS) {
      const int r = idx / half, i = idx - r * half;
      const int row = row0 + r;
      float o0 = 0.f, o1 = 0.f;
      if (row < n_rows) {
        const long long off = (long long)b * content.sb + (long long)head * content.sh + (long long)row * content.ss;
        const float x0 = load_elem<T>(content.ptr, off + 2 * i);
        const float x1 = load_elem<T>(content.ptr, off + 2 * i + 1);
        const int trow = pos0 + row - p.table_pos0;
        const float2 cs = reinterpret_cast<const float2*>(p.table)[(size_t)trow * half + i];
        // complex product (x0 + i x1)(cos + i sin), each term rounded separately
        o0 = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
        o1 = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
        o0 = round_op<ROUND>(o0);
        o1 = round_op<ROUND>(o1);
        if (p.mscale != 1.0f) {
          o0 = round_op<ROUND>(__fmul_rn(o0, p.mscale));
          o1 = round_op<ROUND>(__fmul_rn(o1, p.mscale));
        }
      }
      dst[r * ld + 2 * i] = o0;
      dst[r * ld + 2 * i + 1] = o1;
    }
  } else {
    // four independent loads in flight per thread before the first store: one at a time, each
    // load's latency would be paid in full (the stores to ``dst`` cannot be moved past them)
    const long long base = (long long)b * content.sb + (long long)head * content.sh;
    for (int idx0 = tid; idx0 < BM * d_c; idx0 += 4 * NTHREADS) {
      float x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * NTHREADS;
        const int r = idx / d_c, c = idx - r * d_c;
        x[u] = (idx < BM * d_c && row0 + r < n_rows) ? load_elem<T>(content.ptr, base + (long long)(row0 + r) * content.ss + c)
                                                     : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * NTHREADS;
        const int r = idx / d_c, c = idx - r * d_c;
        if (idx < BM * d_c) dst[r * ld + c] = x[u];
      }
    }
  }
  if (p.variant == PE_ATTN_POPE) {
    const long long base = (long long)b * posi.sb + (long long)head * posi.sh;
    for (int idx0 = tid; idx0 < BM * d_r; idx0 += 4 * NTHREADS) {
      float xin[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * NTHREADS;
        const int r = idx / d_r, c = idx - r * d_r;
        xin[u] = (idx < BM * d_r && row0 + r < n_rows) ? load_elem<T>(posi.ptr, base + (long long)(row0 + r) * posi.ss + c) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * NTHREADS;
        if (idx >= BM * d_r) break;
        const int r = idx / d_r, c = idx - r * d_r;
        const int row = row0 + r;
        float oc = 0.f, os = 0.f;
        if (row < n_rows) {
          const float mu = softplus_accurate(xin[u]);
          // phase = fl(fl(pos * freq) + delta): product and sum rounded separately, as the
          // reference's tensor ops do
          float phase = __fmul_rn((float)(pos0 + row), freq_s[c]);
          if (is_key) phase = __fadd_rn(phase, delta_s[c]);
          float sn, cs;
          sincosf(phase, &sn, &cs);   // the accurate pair: one argument reduction for both
          oc = round_op<ROUND>(__fmul_rn(mu, cs));
          os = round_op<ROUND>(__fmul_rn(mu, sn));
        }
        dst[r * ld + d_c + c] = oc;
        dst[r * ld + d_c + d_r + c] = os;
      }
    }
  }
  if (p.flags & PE_ATTN_QK_NORM) {
    __syncthreads();
    // x / (||x||_2 + eps) per row, 4 threads per row
    const int r = tid >> 2, q4 = tid & 3;
    float ss = 0.f;
    for (int c = q4; c < p.d_qk; c += 4) {
      const float x = dst[r * ld + c];
      ss = fmaf(x, x, ss);
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const float denom = __fadd_rn(sqrtf(ss), p.eps);
    for (int c = q4; c < p.d_qk; c += 4) dst[r * ld + c] = round_op<ROUND>(__fdiv_rn(dst[r * ld + c], denom));
  }
}

template <typename T>
__device__ __forceinline__ void store_elem(void* base, long long off, float x) {
  reinterpret_cast<T*>(base)[off] = static_cast<T>(x);
}
template <>
__device__ __forceinline__ void store_elem<__nv_bfloat16>(void* base, long long off, float x) {
  reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(x);
}

// VC: output columns per thread (stride 16), the smallest of 2, 4, 8 with 16 VC >= d_v.
// RI: query rows per thread (stride 16): a CTA owns 16 RI query rows, 64 normally, 32 when the
// launch would otherwise leave most SMs without a CTA (configuration 1: 64 CTAs on 148 SMs; the
// longest CTA sets the run time, and half the rows halve its QK and PV work).
// ``k_pre``: null, or the transformed keys of every (batch, K/V head) as written by
// simt_key_pretransform_kernel -- the K tiles are then copied instead of built.
template <typename T, bool ROUND, int VC, int RI>
__global__ void __launch_bounds__(NTHREADS) pe_attn_simt_kernel(const KParams p, const float* const k_pre) {
  constexpr int BMQ = 16 * RI;
  extern __shared__ __align__(16) float smem[];
  const int dqk = p.d_qk, dv = p.d_v;
  const int dqk4 = round4(dqk), ld = dqk4 + 4, dvs = round4(dv);
  float* Qs = smem;
  float* Ks = Qs + BM * ld;
  float* Vs = Ks + BN * ld;
  float* Ps = Vs + BN * dvs;
  float* freq_s = Ps + BM * P_LD;
  float* delta_s = freq_s + (p.d_r > 0 ? p.d_r : 1);

  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  const int n_qblk = (p.Sq + BMQ - 1) / BMQ;
  const int qblk = n_qblk - 1 - (int)blockIdx.x;  // heaviest (last) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / p.groups;
  const int m0 = qblk * BMQ;

  if (p.variant == PE_ATTN_POPE) {
    for (int c = tid; c < p.d_r; c += NTHREADS) {
      freq_s[c] = effective_freq(p, c);
      delta_s[c] = clamped_delta(p, c);
    }
    __syncthreads();
  }
  // rows past this CTA's own are left zero (the tile builder works on 64 rows)
  build_operand_tile<T, ROUND>(p, Qs, ld, p.q, p.qr, b, h, m0, (m0 + BMQ < p.Sq ? m0 + BMQ : p.Sq), p.q_pos0, false, freq_s,
                               delta_s);

  float m_run[RI], l_run[RI], o_acc[RI][VC];
#pragma unroll
  for (int i = 0; i < RI; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) o_acc[i][c] = 0.f;
  }
  const float slope = (p.variant == PE_ATTN_ALIBI) ? p.slopes[h] : 0.f;

  int k_end = m0 + BMQ + p.causal_off;
  if (k_end > p.Sk) k_end = p.Sk;
  for (int n0 = 0; n0 < k_end; n0 += BN) {
    __syncthreads();  // previous tile's reads of Ks / Vs / Ps are done (and Qs is complete)
    if (k_pre != nullptr) {
      const int vec = dqk4 / 4;
      const float4* src = reinterpret_cast<const float4*>(k_pre + ((long long)b * p.Hkv + hk) * p.Sk * dqk4);
      for (int idx0 = tid; idx0 < BN * vec; idx0 += 4 * NTHREADS) {
        float4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = idx0 + u * NTHREADS;
          const int r = idx / vec, c = idx - r * vec;
          x[u] = (idx < BN * vec && n0 + r < p.Sk) ? __ldg(src + (long long)(n0 + r) * vec + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = idx0 + u * NTHREADS;
          const int r = idx / vec, c = idx - r * vec;
          if (idx < BN * vec) *reinterpret_cast<float4*>(&Ks[r * ld + 4 * c]) = x[u];
        }
      }
    } else {
      build_operand_tile<T, ROUND>(p, Ks, ld, p.k, p.kr, b, hk, n0, p.Sk, p.k_pos0, true, freq_s, delta_s);
    }
    {
      const long long vbase = (long long)b * p.v.sb + (long long)hk * p.v.sh;
      for (int idx0 = tid; idx0 < BN * dv; idx0 += 4 * NTHREADS) {
        float x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = idx0 + u * NTHREADS;
          const int r = idx / dv, c = idx - r * dv;
          x[u] = (idx < BN * dv && n0 + r < p.Sk) ? load_elem<T>(p.v.ptr, vbase + (long long)(n0 + r) * p.v.ss + c) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = idx0 + u * NTHREADS;
          const int r = idx / dv, c = idx - r * dv;
          if (idx < BN * dv) Vs[r * dvs + c] = x[u];
        }
      }
    }
    __syncthreads();

    float s[RI][4];
#pragma unroll
    for (int i = 0; i < RI; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int kk = 0; kk < dqk4; kk += 4) {
      float4 a[RI], bb[4];
#pragma unroll
      for (int i = 0; i < RI; ++i) a[i] = *reinterpret_cast<const float4*>(&Qs[(ty + 16 * i) * ld + kk]);
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = *reinterpret_cast<const float4*>(&Ks[(tx + 16 * j) * ld + kk]);
#pragma unroll
      for (int i = 0; i < RI; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float acc = s[i][j];
          acc = fmaf(a[i].x, bb[j].x, acc);
          acc = fmaf(a[i].y, bb[j].y, acc);
          acc = fmaf(a[i].z, bb[j].z, acc);
          acc = fmaf(a[i].w, bb[j].w, acc);
          s[i][j] = acc;
        }
    }

#pragma unroll
    for (int i = 0; i < RI; ++i) {
      const int row = m0 + ty + 16 * i;
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = n0 + tx + 16 * j;
        const int rel = col - (row + p.causal_off);
        float x = s[i][j] * p.scale;
        if (p.variant == PE_ATTN_ALIBI) x = x - slope * fabsf((float)rel);
        if (rel > 0 || col >= p.Sk) x = -INFINITY;
        s[i][j] = x;
        tmax = fmaxf(tmax, x);
      }
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, d));
      const float m_new = fmaxf(m_run[i], tmax);
      const float alpha = (m_new == -INFINITY) ? 1.f : expf(m_run[i] - m_new);
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float pj = (m_new == -INFINITY) ? 0.f : expf(s[i][j] - m_new);
        psum += pj;
        Ps[(ty + 16 * i) * P_LD + tx + 16 * j] = pj;
      }
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, d);
      l_run[i] = l_run[i] * alpha + psum;
      m_run[i] = m_new;
#pragma unroll
      for (int c = 0; c < VC; ++c) o_acc[i][c] *= alpha;
    }
    __syncthreads();

    for (int j = 0; j < BN; j += 4) {
      float4 a[RI];
#pragma unroll
      for (int i = 0; i < RI; ++i) a[i] = *reinterpret_cast<const float4*>(&Ps[(ty + 16 * i) * P_LD + j]);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float vv[VC];
#pragma unroll
        for (int c = 0; c < VC; ++c) {
          const int col = tx + 16 * c;
          vv[c] = col < dv ? Vs[(j + jj) * dvs + col] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < RI; ++i) {
          const float pij = jj == 0 ? a[i].x : jj == 1 ? a[i].y : jj == 2 ? a[i].z : a[i].w;
#pragma unroll
          for (int c = 0; c < VC; ++c) o_acc[i][c] = fmaf(pij, vv[c], o_acc[i][c]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < RI; ++i) {
    const int row = m0 + ty + 16 * i;
    if (row >= p.Sq) continue;
    const float inv = 1.f / l_run[i];
    if (p.lse != nullptr && tx == 0) p.lse[((long long)b * p.H + h) * p.Sq + row] = m_run[i] + logf(l_run[i]);
    const long long off = (long long)b * p.out.sb + (long long)h * p.out.sh + (long long)row * p.out.ss;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
      const int col = tx + 16 * c;
      if (col < dv) store_elem<T>(const_cast<void*>(p.out.ptr), off + col, o_acc[i][c] * inv);
    }
  }
}

// The transformed keys of every (batch, K/V head), once: [B][Hkv][Sk][round4(d_qk)] fp32, built by
// the same code as a K tile inside the attention kernel (bit-identical values).  Every query block
// of a head needs them, and the accurate softplus / sincos of the PoPE transform is 60 % of a key
// tile's instructions: with S / 64 (or S / 32) query blocks per head the attention kernel would
// repeat it that many times.
template <typename T, bool ROUND>
__global__ void __launch_bounds__(NTHREADS) simt_key_pretransform_kernel(const KParams p, float* const k_pre) {
  extern __shared__ __align__(16) float smem[];
  const int dqk4 = round4(p.d_qk), ld = dqk4 + 4;
  float* Ks = smem;
  float* freq_s = Ks + BN * ld;
  float* delta_s = freq_s + (p.d_r > 0 ? p.d_r : 1);
  const int tid = threadIdx.x;
  const int n0 = (int)blockIdx.x * BN, hk = blockIdx.y, b = blockIdx.z;
  if (p.variant == PE_ATTN_POPE) {
    for (int c = tid; c < p.d_r; c += NTHREADS) {
      freq_s[c] = effective_freq(p, c);
      delta_s[c] = clamped_delta(p, c);
    }
    __syncthreads();
  }
  build_operand_tile<T, ROUND>(p, Ks, ld, p.k, p.kr, b, hk, n0, p.Sk, p.k_pos0, true, freq_s, delta_s);
  __syncthreads();
  const int vec = dqk4 / 4;
  float4* dst = reinterpret_cast<float4*>(k_pre + ((long long)b * p.Hkv + hk) * p.Sk * dqk4);
  for (int idx = tid; idx < BN * vec; idx += NTHREADS) {
    const int r = idx / vec, c = idx - r * vec;
    if (n0 + r < p.Sk) dst[(long long)(n0 + r) * vec + c] = *reinterpret_cast<const float4*>(&Ks[r * ld + 4 * c]);
  }
}

}  // namespace

// Scratch for the transformed keys of an fp32 call, or 0 where building K tiles in place is as
// good: no transform to repeat (NoPE / ALiBi without QKNorm), fewer than two query blocks per
// head, or more than 1 GiB.
size_t simt_key_scratch_bytes(const KParams& p) {
  const bool transform = p.variant == PE_ATTN_POPE || p.variant == PE_ATTN_ROTARY || (p.flags & PE_ATTN_QK_NORM);
  if (!transform || p.Sq < 2 * BM) return 0;
  const size_t bytes = (size_t)p.B * p.Hkv * p.Sk * round4(p.d_qk) * sizeof(float);
  return bytes <= ((size_t)1 << 30) ? bytes : 0;
}

size_t simt_smem_bytes(const KParams& p) {
  const size_t ld = round4(p.d_qk) + 4;
  const size_t nfl = 2 * (size_t)BM * ld + (size_t)BN * round4(p.d_v) + (size_t)BM * P_LD + 2 * (size_t)(p.d_r > 0 ? p.d_r : 1);
  return nfl * sizeof(float);
}

namespace {
template <typename T, bool ROUND, int VC, int RI>
cudaError_t launch_simt_instance(const KParams& p, size_t smem, cudaStream_t stream) {
  auto kern = pe_attn_simt_kernel<T, ROUND, VC, RI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  // fp32 calls that were given scratch transform the keys once, in front of the attention kernel
  const float* k_pre = nullptr;
  const size_t need = simt_key_scratch_bytes(p);
  if (!ROUND && need > 0 && p.workspace != nullptr && p.workspace_bytes >= need) {
    auto pre = simt_key_pretransform_kernel<T, ROUND>;
    const size_t pre_smem = ((size_t)BN * (round4(p.d_qk) + 4) + 2 * (size_t)(p.d_r > 0 ? p.d_r : 1)) * sizeof(float);
    e = cudaFuncSetAttribute(pre, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pre_smem);
    if (e != cudaSuccess) return e;
    pre<<<dim3((p.Sk + BN - 1) / BN, p.Hkv, p.B), dim3(NTHREADS), pre_smem, stream>>>(p, p.workspace);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    k_pre = p.workspace;
  }
  dim3 grid((p.Sq + 16 * RI - 1) / (16 * RI), p.H, p.B);
  kern<<<grid, dim3(NTHREADS), smem, stream>>>(p, k_pre);
  return cudaGetLastError();
}
template <typename T, bool ROUND, int VC>
cudaError_t launch_simt_rows(const KParams& p, size_t smem, cudaStream_t stream) {
  // 32-row CTAs when 64-row ones would not give every SM at least one and a half CTAs
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ctas64 = (long long)((p.Sq + BM - 1) / BM) * p.H * p.B;
  if (2 * ctas64 < 3ll * sms) return launch_simt_instance<T, ROUND, VC, 2>(p, smem, stream);
  return launch_simt_instance<T, ROUND, VC, 4>(p, smem, stream);
}
template <typename T, bool ROUND>
cudaError_t launch_simt_dv(const KParams& p, size_t smem, cudaStream_t stream) {
  if (p.d_v <= 32) return launch_simt_rows<T, ROUND, 2>(p, smem, stream);
  if (p.d_v <= 64) return launch_simt_rows<T, ROUND, 4>(p, smem, stream);
  return launch_simt_rows<T, ROUND, MAX_VC>(p, smem, stream);
}
}  // namespace

int launch_simt(const KParams& p, int dtype, cudaStream_t stream) {
  const size_t smem = simt_smem_bytes(p);
  const cudaError_t e = dtype == PE_ATTN_FP32 ? launch_simt_dv<float, false>(p, smem, stream)
                                              : launch_simt_dv<__nv_bfloat16, true>(p, smem, stream);
  if (e != cudaSuccess) {
    set_error("ffma kernel launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

}  // namespace pe_attn
