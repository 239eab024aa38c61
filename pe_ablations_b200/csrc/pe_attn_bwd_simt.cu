// Causal attention BACKWARD on the CUDA cores (FFMA), for the head dimensions the tensor-core
// backward kernel does not have -- above all d_qk = 256 / d_v = 128, the 1B evaluation shape, so
// that every model the forward serves can also be trained through the drop-in modules.
//
// Same contract as the tensor-core kernel: operands that already carry their positional
// transform, the forward's logsumexp, gradients of
//     out = softmax_causal(scale * Q K^T + bias) V
// with respect to Q (fp32 [B,Sq,H,d_qk]), K and V (the operands' type, caller's strides).  The
// kernels are templates over the element type: bf16, and fp32 -- the only backward fp32 calls
// have (the reference's CPU-runnable configuration and its tests run in fp32).  It is the part of
// the reference's training step that autograd derives from F.scaled_dot_product_attention
// (src/model/attention.py:91-96, src/model/fpope_attention.py:171-177, src/model/alibi.py:145-160).
//
// Two kernels, both recomputing the probabilities from Q, K and the logsumexp:
//   * key side:   one CTA owns 64 keys of one K/V head and walks over the query blocks (of every
//                 query head of the group) that see them:  dV += P^T dO,  dK += dS^T Q
//   * query side: one CTA owns 64 query rows of one head and walks over the key blocks it sees:
//                 dQ = dS K
// with P = exp(scale S + bias - lse), dS = scale * P o (dO V^T - D), D = rowsum(dO o O).  Tiles
// are held in shared memory in the operands' type, rows padded by one 16-byte slot, products
// run as 4 x 4 (scores) and 4 x 8 / 4 x 16 (gradients) register tiles in fp32.  Nothing here
// waits on anything but __syncthreads; no atomics, results do not depend on CTA scheduling.
#include <cuda_bf16.h>

#include "pe_attn_common.cuh"

namespace pe_attn {
namespace {

constexpr int BT = 64;          // rows of every tile (queries or keys)
constexpr int NTHREADS = 256;   // 16 x 16 threads
constexpr int P_LD = BT + 4;    // fp32 pitch of the P / dS tiles

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

struct SimtBwdParams {
  BwdParams b;
  int d_qk, d_v;
  int ldq, ldv;   // element pitches of the d_qk- and d_v-wide tiles: width + 16 bytes
};

template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int PAD = 8;   // elements in 16 bytes
  static constexpr bool ONE_BUF = false;
};
template <>
struct Elem<float> {
  static constexpr int PAD = 4;
  static constexpr bool ONE_BUF = true;   // the fp32 operand tiles of d_qk 256 / d_v 128 leave room for one P / dS tile
};

// eight consecutive elements (16-byte aligned) as fp32
__device__ __forceinline__ void load8(const __nv_bfloat16* src, float (&x)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(src);
  x[0] = bf_lo(w.x); x[1] = bf_hi(w.x); x[2] = bf_lo(w.y); x[3] = bf_hi(w.y);
  x[4] = bf_lo(w.z); x[5] = bf_hi(w.z); x[6] = bf_lo(w.w); x[7] = bf_hi(w.w);
}
__device__ __forceinline__ void load8(const float* src, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float (&x)[8]) {
  __align__(16) __nv_bfloat16 o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(x[e]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
}
__device__ __forceinline__ void store8(float* dst, const float (&x)[8]) {
  *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(x[4], x[5], x[6], x[7]);
}

// rows [row0, row0 + 64) of a [B, H, S, d] tensor -> shared memory, 16 bytes per thread and step
template <typename T>
__device__ __forceinline__ void load_tile(T* dst, int ld, const TensorRef& t, int b, int h, int row0, int n_rows, int d) {
  constexpr int EV = 16 / (int)sizeof(T);
  const int vec = d / EV;
  const T* base = reinterpret_cast<const T*>(t.ptr) + (long long)b * t.sb + (long long)h * t.sh;
  for (int idx = threadIdx.x; idx < BT * vec; idx += NTHREADS) {
    const int r = idx / vec, c = idx - r * vec;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row0 + r < n_rows) v = *reinterpret_cast<const uint4*>(base + (long long)(row0 + r) * t.ss + c * EV);
    *reinterpret_cast<uint4*>(dst + r * ld + c * EV) = v;
  }
}

// acc[i][j] += sum_c A[ty + 16 i][c] * B[tx + 16 j][c] over ``d`` columns (16 bytes per step)
__device__ __forceinline__ void dot_tiles(float (&acc)[4][4], const __nv_bfloat16* A, const __nv_bfloat16* Bm, int ld,
                                          int d, int ty, int tx) {
  for (int c = 0; c < d; c += 8) {
    uint4 a[4], bb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const uint4*>(A + (ty + 16 * i) * ld + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) bb[j] = *reinterpret_cast<const uint4*>(Bm + (tx + 16 * j) * ld + c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t bw[4] = {bb[j].x, bb[j].y, bb[j].z, bb[j].w};
        float s = acc[i][j];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s = fmaf(bf_lo(aw[e]), bf_lo(bw[e]), s);
          s = fmaf(bf_hi(aw[e]), bf_hi(bw[e]), s);
        }
        acc[i][j] = s;
      }
    }
  }
}
__device__ __forceinline__ void dot_tiles(float (&acc)[4][4], const float* A, const float* Bm, int ld, int d, int ty,
                                          int tx) {
  for (int c = 0; c < d; c += 4) {
    float4 a[4], bb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(A + (ty + 16 * i) * ld + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) bb[j] = *reinterpret_cast<const float4*>(Bm + (tx + 16 * j) * ld + c);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float s = acc[i][j];
        s = fmaf(a[i].x, bb[j].x, s);
        s = fmaf(a[i].y, bb[j].y, s);
        s = fmaf(a[i].z, bb[j].z, s);
        s = fmaf(a[i].w, bb[j].w, s);
        acc[i][j] = s;
      }
  }
}

// P and dS of one 64 x 64 (query, key) tile from the tiles in shared memory; thread (ty, tx)
// owns queries ty + 16 i and keys tx + 16 j.  Writes both to shared memory ([query][key], fp32).
// PMODE 0: P to ``Ps`` and dS to ``dSs``; 1: P to ``Ps``, dS kept in ``ds_reg`` (the caller writes it
// over P later: fp32, whose operand tiles leave room for one such tile only); 2: dS to ``dSs`` only.
template <typename T, bool ALIBI, int PMODE>
__device__ __forceinline__ void prob_tile(const SimtBwdParams& sp, const T* Qs, const T* Ks, const T* dOs, const T* Vs,
                                          const float* lse_s,
                                          const float* D_s, float* Ps, float* dSs, float (&ds_reg)[4][4], int q0, int k0,
                                          float slope, int ty, int tx) {
  const BwdParams& p = sp.b;
  float s[4][4], dp[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
  dot_tiles(s, Qs, Ks, sp.ldq, sp.d_qk, ty, tx);
  dot_tiles(dp, dOs, Vs, sp.ldv, sp.d_v, ty, tx);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ql = ty + 16 * i, row = q0 + ql;
    const float lse = lse_s[ql], dsum = D_s[ql];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kl = tx + 16 * j, key = k0 + kl;
      const int rel = key - (row + p.causal_off);
      float pr = 0.f;
      if (rel <= 0 && row < p.Sq && key < p.Sk) {
        float x = s[i][j] * p.scale;
        if (ALIBI) x += slope * (float)rel;   // -slope * (distance), rel <= 0
        pr = expf(x - lse);
      }
      const float ds = p.scale * pr * (dp[i][j] - dsum);
      if (PMODE != 2) Ps[ql * P_LD + kl] = pr;
      if (PMODE == 1) ds_reg[i][j] = ds;
      else dSs[ql * P_LD + kl] = ds;
    }
  }
}

// D[b, h, row] = sum_c dO * O: one warp per row
template <typename T>
__global__ void __launch_bounds__(256) rowdot_kernel(const BwdParams p, int d_v) {
  const int warp = (int)((blockIdx.x * 256 + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  const long long n = (long long)p.B * p.H * p.Sq;
  if (warp >= n) return;
  const int row = warp % p.Sq, h = (warp / p.Sq) % p.H, b = warp / ((long long)p.Sq * p.H);
  const T* o = reinterpret_cast<const T*>(p.out.ptr) + (long long)b * p.out.sb + (long long)h * p.out.sh +
               (long long)row * p.out.ss;
  const T* g = reinterpret_cast<const T*>(p.dout.ptr) + (long long)b * p.dout.sb + (long long)h * p.dout.sh +
               (long long)row * p.dout.ss;
  float acc = 0.f;
  for (int c = lane; c < d_v; c += 32) acc = fmaf((float)o[c], (float)g[c], acc);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) p.dvec[((long long)b * p.H + h) * p.Sq + row] = acc;
}

template <typename T, bool ALIBI>
__global__ void __launch_bounds__(NTHREADS) bwd_simt_key_side_kernel(const SimtBwdParams sp) {
  const BwdParams& p = sp.b;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Ks = reinterpret_cast<T*>(smem_raw);
  T* Qs = Ks + BT * sp.ldq;
  T* Vs = Qs + BT * sp.ldq;
  T* dOs = Vs + BT * sp.ldv;
  constexpr bool ONE_BUF = Elem<T>::ONE_BUF;   // fp32: P and dS take turns in one tile
  float* Ps = reinterpret_cast<float*>(dOs + BT * sp.ldv);
  float* dSs = ONE_BUF ? Ps : Ps + BT * P_LD;
  float* lse_s = dSs + BT * P_LD;
  float* D_s = lse_s + BT;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int k0 = (int)blockIdx.x * BT, hk = blockIdx.y, b = blockIdx.z;
  load_tile(Ks, sp.ldq, p.k, b, hk, k0, p.Sk, sp.d_qk);
  load_tile(Vs, sp.ldv, p.v, b, hk, k0, p.Sk, sp.d_v);

  // gradient tiles: keys ty + 16 i, columns 8 (tx + 16 m) .. + 8
  const int n_vg = sp.d_v / 8, n_qg = sp.d_qk / 8;   // 16-byte column groups
  float dv_acc[4][8], dk_acc[2][4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dv_acc[i][e] = dk_acc[0][i][e] = dk_acc[1][i][e] = 0.f;

  int first_row = k0 - p.causal_off;
  if (first_row < 0) first_row = 0;
  const int qb_first = first_row / BT, n_qb = (p.Sq + BT - 1) / BT;
  for (int g = 0; g < p.groups; ++g) {
    const int h = hk * p.groups + g;
    const float slope = ALIBI ? p.slopes[h] : 0.f;
    for (int qb = qb_first; qb < n_qb; ++qb) {
      const int q0 = qb * BT;
      __syncthreads();   // the previous block's reads of Qs / dOs / Ps / dSs are done
      load_tile(Qs, sp.ldq, p.q, b, h, q0, p.Sq, sp.d_qk);
      load_tile(dOs, sp.ldv, p.dout, b, h, q0, p.Sq, sp.d_v);
      if (tid < BT) {
        const int row = q0 + tid;
        lse_s[tid] = row < p.Sq ? p.lse[((long long)b * p.H + h) * p.Sq + row] : 0.f;
        D_s[tid] = row < p.Sq ? p.dvec[((long long)b * p.H + h) * p.Sq + row] : 0.f;
      }
      __syncthreads();
      float ds_reg[4][4];
      prob_tile<T, ALIBI, ONE_BUF ? 1 : 0>(sp, Qs, Ks, dOs, Vs, lse_s, D_s, Ps, dSs, ds_reg, q0, k0, slope, ty, tx);
      __syncthreads();
      // dV[key][c] += sum_q P[q][key] dO[q][c];  dK[key][c] += sum_q dS[q][key] Q[q][c]
      // (one tile for both: first all of dV from P, then dS over it and all of dK)
      for (int pass = 0; pass < (ONE_BUF ? 2 : 1); ++pass) {
      if (ONE_BUF && pass == 1) {
        __syncthreads();   // every thread has read P
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) dSs[(ty + 16 * i) * P_LD + tx + 16 * j] = ds_reg[i][j];
        __syncthreads();
      }
      const bool do_dv = !ONE_BUF || pass == 0, do_dk = !ONE_BUF || pass == 1;
      for (int q = 0; q < BT; ++q) {
        float pq[4], dsq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pq[i] = Ps[q * P_LD + ty + 16 * i];
          dsq[i] = dSs[q * P_LD + ty + 16 * i];
        }
        if (do_dv && tx < n_vg) {
          float x[8];
          load8(dOs + q * sp.ldv + tx * 8, x);
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) dv_acc[i][e] = fmaf(pq[i], x[e], dv_acc[i][e]);
        }
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          if (do_dk && tx + 16 * m < n_qg) {
            float x[8];
            load8(Qs + q * sp.ldq + (tx + 16 * m) * 8, x);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int e = 0; e < 8; ++e) dk_acc[m][i][e] = fmaf(dsq[i], x[e], dk_acc[m][i][e]);
          }
        }
      }
      }  // passes
    }
  }
  // results in the operands' type, 16 bytes per store
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int key = k0 + ty + 16 * i;
    if (key >= p.Sk) continue;
    if (tx < n_vg) {
      store8(reinterpret_cast<T*>(const_cast<void*>(p.dv.ptr)) + (long long)b * p.dv.sb + (long long)hk * p.dv.sh +
                 (long long)key * p.dv.ss + tx * 8,
             dv_acc[i]);
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      if (tx + 16 * m < n_qg) {
        store8(reinterpret_cast<T*>(const_cast<void*>(p.dk.ptr)) + (long long)b * p.dk.sb + (long long)hk * p.dk.sh +
                   (long long)key * p.dk.ss + (tx + 16 * m) * 8,
               dk_acc[m][i]);
      }
    }
  }
}

template <typename T, bool ALIBI>
__global__ void __launch_bounds__(NTHREADS) bwd_simt_query_side_kernel(const SimtBwdParams sp) {
  const BwdParams& p = sp.b;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Ks = reinterpret_cast<T*>(smem_raw);
  T* Qs = Ks + BT * sp.ldq;
  T* Vs = Qs + BT * sp.ldq;
  T* dOs = Vs + BT * sp.ldv;
  constexpr bool ONE_BUF = Elem<T>::ONE_BUF;   // fp32: P and dS take turns in one tile
  float* Ps = reinterpret_cast<float*>(dOs + BT * sp.ldv);
  float* dSs = ONE_BUF ? Ps : Ps + BT * P_LD;
  float* lse_s = dSs + BT * P_LD;
  float* D_s = lse_s + BT;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int n_qb = (p.Sq + BT - 1) / BT;
  const int q0 = (n_qb - 1 - (int)blockIdx.x) * BT, h = blockIdx.y, b = blockIdx.z;   // longest blocks first
  const int hk = h / p.groups;
  const float slope = ALIBI ? p.slopes[h] : 0.f;
  load_tile(Qs, sp.ldq, p.q, b, h, q0, p.Sq, sp.d_qk);
  load_tile(dOs, sp.ldv, p.dout, b, h, q0, p.Sq, sp.d_v);
  if (tid < BT) {
    const int row = q0 + tid;
    lse_s[tid] = row < p.Sq ? p.lse[((long long)b * p.H + h) * p.Sq + row] : 0.f;
    D_s[tid] = row < p.Sq ? p.dvec[((long long)b * p.H + h) * p.Sq + row] : 0.f;
  }
  const int n_qg = sp.d_qk / 8;
  float dq_acc[2][4][8];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) dq_acc[m][i][e] = 0.f;

  int k_end = q0 + BT + p.causal_off;
  if (k_end > p.Sk) k_end = p.Sk;
  for (int k0 = 0; k0 < k_end; k0 += BT) {
    __syncthreads();   // the previous tile's reads are done (and the query-side tiles are complete)
    load_tile(Ks, sp.ldq, p.k, b, hk, k0, p.Sk, sp.d_qk);
    load_tile(Vs, sp.ldv, p.v, b, hk, k0, p.Sk, sp.d_v);
    __syncthreads();
    float ds_unused[4][4];
    prob_tile<T, ALIBI, ONE_BUF ? 2 : 0>(sp, Qs, Ks, dOs, Vs, lse_s, D_s, Ps, dSs, ds_unused, q0, k0, slope, ty, tx);
    __syncthreads();
    // dQ[q][c] += sum_k dS[q][k] K[k][c]: queries ty + 16 i, columns 8 (tx + 16 m) .. + 8
    for (int k = 0; k < BT; ++k) {
      float dsq[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dsq[i] = dSs[(ty + 16 * i) * P_LD + k];
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        if (tx + 16 * m < n_qg) {
          float x[8];
          load8(Ks + k * sp.ldq + (tx + 16 * m) * 8, x);
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) dq_acc[m][i][e] = fmaf(dsq[i], x[e], dq_acc[m][i][e]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = q0 + ty + 16 * i;
    if (row >= p.Sq) continue;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      if (tx + 16 * m < n_qg) {
        float4* dst = reinterpret_cast<float4*>(p.dq_accum + (((long long)b * p.Sq + row) * p.H + h) * sp.d_qk +
                                                (tx + 16 * m) * 8);
        dst[0] = make_float4(dq_acc[m][i][0], dq_acc[m][i][1], dq_acc[m][i][2], dq_acc[m][i][3]);
        dst[1] = make_float4(dq_acc[m][i][4], dq_acc[m][i][5], dq_acc[m][i][6], dq_acc[m][i][7]);
      }
    }
  }
}

size_t simt_bwd_smem(int d_qk, int d_v, size_t elem, int pad, bool one_buf) {
  return (size_t)2 * BT * ((d_qk + pad) + (d_v + pad)) * elem +
         (size_t)((one_buf ? 1 : 2) * BT * P_LD + 2 * BT) * sizeof(float);
}

template <typename T>
int launch_bwd_simt_t(const BwdParams& p, int d_qk, int d_v, bool alibi, cudaStream_t stream) {
  SimtBwdParams sp;
  sp.b = p;
  sp.d_qk = d_qk;
  sp.d_v = d_v;
  sp.ldq = d_qk + Elem<T>::PAD;
  sp.ldv = d_v + Elem<T>::PAD;
  const size_t smem = simt_bwd_smem(d_qk, d_v, sizeof(T), Elem<T>::PAD, Elem<T>::ONE_BUF);
  const long long rows = (long long)p.B * p.H * p.Sq;
  rowdot_kernel<T><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, stream>>>(p, d_v);
  cudaError_t e = cudaGetLastError();
  auto run = [&](auto key_kernel, auto query_kernel) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(key_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(query_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return;
    key_kernel<<<dim3((p.Sk + BT - 1) / BT, p.Hkv, p.B), NTHREADS, smem, stream>>>(sp);
    e = cudaGetLastError();
    if (e != cudaSuccess) return;
    query_kernel<<<dim3((p.Sq + BT - 1) / BT, p.H, p.B), NTHREADS, smem, stream>>>(sp);
    e = cudaGetLastError();
  };
  if (alibi) run(bwd_simt_key_side_kernel<T, true>, bwd_simt_query_side_kernel<T, true>);
  else run(bwd_simt_key_side_kernel<T, false>, bwd_simt_query_side_kernel<T, false>);
  if (e != cudaSuccess) {
    set_error("FFMA backward launch failed: %s", cudaGetErrorString(e));
    return PE_ATTN_ERR_LAUNCH;
  }
  return PE_ATTN_OK;
}

}  // namespace

// d_qk and d_v multiples of 8, d_qk <= 256, d_v <= 128: the four operand tiles of 64 rows then fit
// the 227 KB of shared memory a CTA can have (fp32 at 256 / 128: 214 KB with a single P / dS tile)
bool bwd_simt_supports(int d_qk, int d_v, int dtype) {
  if (!(d_qk >= 8 && d_qk <= 256 && d_qk % 8 == 0 && d_v >= 8 && d_v <= 128 && d_v % 8 == 0)) return false;
  const size_t smem = dtype == PE_ATTN_FP32 ? simt_bwd_smem(d_qk, d_v, 4, Elem<float>::PAD, Elem<float>::ONE_BUF)
                                            : simt_bwd_smem(d_qk, d_v, 2, Elem<__nv_bfloat16>::PAD, Elem<__nv_bfloat16>::ONE_BUF);
  return smem <= 227 * 1024;
}

int launch_bwd_simt(const BwdParams& p, int d_qk, int d_v, int dtype, bool alibi, cudaStream_t stream) {
  return dtype == PE_ATTN_FP32 ? launch_bwd_simt_t<float>(p, d_qk, d_v, alibi, stream)
                               : launch_bwd_simt_t<__nv_bfloat16>(p, d_qk, d_v, alibi, stream);
}

}  // namespace pe_attn
