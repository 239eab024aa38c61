// C ABI of the PE-attention library: argument validation, error reporting and the
// choice between the two kernel families (tcgen05 for bf16, FFMA for fp32).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "pe_attn_common.cuh"
#include "pe_attn_ptx.cuh"

namespace pe_attn {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static TensorRef make_ref(const void* ptr, const int64_t s[3]) { return TensorRef{ptr, s[0], s[1], s[2]}; }

// Checks shared by every entry point; fills the device-side argument block.
static int validate(const pe_attn_args* a, KParams* out) {
  if (a == nullptr) return fail(PE_ATTN_ERR_NULL, "args is null");
  if (a->struct_size != sizeof(pe_attn_args))
    return fail(PE_ATTN_ERR_VARIANT, "struct_size %u does not match this library's %zu", a->struct_size,
                sizeof(pe_attn_args));
  if (a->variant < PE_ATTN_NOPE || a->variant > PE_ATTN_POPE)
    return fail(PE_ATTN_ERR_VARIANT, "unknown variant %d", a->variant);
  if (a->dtype != PE_ATTN_BF16 && a->dtype != PE_ATTN_FP32)
    return fail(PE_ATTN_ERR_VARIANT, "unknown dtype %d", a->dtype);
  if (a->B < 1 || a->H < 1 || a->Hkv < 1 || a->Sq < 1 || a->Sk < 1)
    return fail(PE_ATTN_ERR_SHAPE, "B, H, Hkv, Sq, Sk must be positive (got %d %d %d %d %d)", a->B, a->H, a->Hkv,
                a->Sq, a->Sk);
  if (a->H % a->Hkv != 0) return fail(PE_ATTN_ERR_SHAPE, "H=%d is not a multiple of Hkv=%d", a->H, a->Hkv);
  if (a->Sk < a->Sq) return fail(PE_ATTN_ERR_SHAPE, "Sk=%d < Sq=%d", a->Sk, a->Sq);
  if (a->B > 65535 || a->H > 65535) return fail(PE_ATTN_ERR_SHAPE, "B and H must be <= 65535");
  if (a->d_v < 1 || a->d_v > 128) return fail(PE_ATTN_ERR_SHAPE, "d_v=%d outside [1, 128]", a->d_v);
  if (a->d_c < 0 || a->d_r < 0) return fail(PE_ATTN_ERR_SHAPE, "negative head dim");
  const bool pope = a->variant == PE_ATTN_POPE;
  if (pope) {
    if (a->d_r < 1) return fail(PE_ATTN_ERR_SHAPE, "POPE needs d_r >= 1");
    if (a->q_r == nullptr || a->k_r == nullptr) return fail(PE_ATTN_ERR_NULL, "POPE needs q_r and k_r");
    if (a->freqs == nullptr) return fail(PE_ATTN_ERR_NULL, "POPE needs freqs");
    if (a->flags & PE_ATTN_QK_NORM) return fail(PE_ATTN_ERR_VARIANT, "QK_NORM is not defined for POPE");
    if (a->flags & PE_ATTN_FOURIER_MIX) {
      if (a->fourier_coeffs == nullptr || a->n_fourier < 1)
        return fail(PE_ATTN_ERR_NULL, "FOURIER_MIX needs fourier_coeffs and n_fourier >= 1");
    }
  } else {
    if (a->d_r != 0) return fail(PE_ATTN_ERR_SHAPE, "d_r must be 0 unless the variant is POPE");
    if (a->d_c < 1) return fail(PE_ATTN_ERR_SHAPE, "d_c must be >= 1");
    if (a->flags & PE_ATTN_FOURIER_MIX) return fail(PE_ATTN_ERR_VARIANT, "FOURIER_MIX needs the POPE variant");
  }
  const int d_qk = a->d_c + 2 * a->d_r;
  if (d_qk > 256) return fail(PE_ATTN_ERR_SHAPE, "d_c + 2 d_r = %d exceeds 256", d_qk);
  if (a->d_c > 0 && (a->q == nullptr || a->k == nullptr)) return fail(PE_ATTN_ERR_NULL, "q or k is null");
  if (a->v == nullptr || a->out == nullptr) return fail(PE_ATTN_ERR_NULL, "v or out is null");
  if (a->variant == PE_ATTN_ROTARY) {
    if (a->d_c % 2) return fail(PE_ATTN_ERR_SHAPE, "ROTARY needs an even head dim (got %d)", a->d_c);
    if (a->rotary_table == nullptr) return fail(PE_ATTN_ERR_NULL, "ROTARY needs rotary_table");
    const long long lo = (long long)(a->q_pos0 < a->k_pos0 ? a->q_pos0 : a->k_pos0) - a->table_pos0;
    const long long hq = (long long)a->q_pos0 + a->Sq - a->table_pos0;
    const long long hk = (long long)a->k_pos0 + a->Sk - a->table_pos0;
    if (lo < 0 || hq > a->table_rows || hk > a->table_rows)
      return fail(PE_ATTN_ERR_SHAPE, "rotary_table rows [%d, %d) do not cover the positions in use", a->table_pos0,
                  a->table_pos0 + a->table_rows);
    if (!aligned16(a->rotary_table)) return fail(PE_ATTN_ERR_ALIGNMENT, "rotary_table is not 16-byte aligned");
  }
  if (a->variant == PE_ATTN_ALIBI && a->alibi_slopes == nullptr)
    return fail(PE_ATTN_ERR_NULL, "ALIBI needs alibi_slopes");

  KParams k;
  memset(&k, 0, sizeof(k));
  k.variant = a->variant;
  k.flags = a->flags;
  k.B = a->B; k.H = a->H; k.Hkv = a->Hkv; k.groups = a->H / a->Hkv;
  k.Sq = a->Sq; k.Sk = a->Sk;
  k.d_c = a->d_c; k.d_r = a->d_r; k.d_v = a->d_v; k.d_qk = d_qk;
  k.q_pos0 = a->q_pos0; k.k_pos0 = a->k_pos0;
  k.causal_off = a->Sk - a->Sq;
  k.scale = a->scale; k.eps = a->qk_norm_eps; k.mscale = (a->variant == PE_ATTN_ROTARY) ? a->mscale : 1.0f;
  k.q = make_ref(a->q, a->q_stride);
  k.k = make_ref(a->k, a->k_stride);
  k.v = make_ref(a->v, a->v_stride);
  k.out = make_ref(a->out, a->out_stride);
  k.qr = make_ref(a->q_r, a->qr_stride);
  k.kr = make_ref(a->k_r, a->kr_stride);
  k.table = a->rotary_table; k.table_pos0 = a->table_pos0; k.table_rows = a->table_rows;
  k.slopes = a->alibi_slopes;
  k.freqs = a->freqs; k.delta = a->delta; k.coeffs = a->fourier_coeffs; k.n_fourier = a->n_fourier;
  k.floor_freq = a->floor_freq; k.ceil_freq = a->ceil_freq;
  k.status = a->device_status;
  k.lse = a->lse;
  k.workspace = static_cast<float*>(a->workspace);
  k.workspace_bytes = a->workspace != nullptr ? (size_t)a->workspace_bytes : 0;
  if (a->workspace != nullptr && !aligned16(a->workspace)) return fail(PE_ATTN_ERR_ALIGNMENT, "workspace is not 16-byte aligned");

  const bool use_tc = a->dtype == PE_ATTN_BF16 && !(a->flags & PE_ATTN_SIMT_CHECK);
  if (use_tc) {
    // The tensor-core kernel moves tiles with TMA and 16-byte vector loads.
    struct { const char* name; const void* p; const int64_t* s; bool used; } ts[] = {
        {"q", a->q, a->q_stride, a->d_c > 0},    {"k", a->k, a->k_stride, a->d_c > 0},
        {"v", a->v, a->v_stride, true},          {"out", a->out, a->out_stride, true},
        {"q_r", a->q_r, a->qr_stride, pope},     {"k_r", a->k_r, a->kr_stride, pope}};
    for (auto& t : ts) {
      if (!t.used) continue;
      if (!aligned16(t.p)) return fail(PE_ATTN_ERR_ALIGNMENT, "%s is not 16-byte aligned", t.name);
      for (int i = 0; i < 3; ++i)
        if (t.s[i] % 8 != 0) return fail(PE_ATTN_ERR_ALIGNMENT, "%s stride[%d]=%lld is not a multiple of 8 elements", t.name, i, (long long)t.s[i]);
    }
    if (!tc_supports(k))
      return fail(PE_ATTN_ERR_SHAPE,
                  "bf16 path supports d_c in {0,64,128}, d_r in {0,32,64}, d_v in {64,128} with d_c + 2 d_r in "
                  "{64,128,192,256} (got d_c=%d d_r=%d d_v=%d)", a->d_c, a->d_r, a->d_v);
  }
  if (out) *out = k;
  return PE_ATTN_OK;
}

}  // namespace pe_attn

using namespace pe_attn;

// One warp waits, with the kernels' bounded wait, on a barrier that nothing ever signals.
__global__ void wait_expiry_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  const uint32_t b = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(b, 1);
    ptx::mbar_fence_init();
  }
  __syncthreads();
  const bool ok = ptx::mbar_wait_for(b, 0, limit_cycles);
  if (!ok && threadIdx.x == 0) atomicOr(status, PE_ATTN_SELFTEST_WAIT_EXPIRED);
}

extern "C" {

int pe_attn_selftest_wait_expiry(int32_t* device_status, int64_t limit_cycles, void* stream) {
  if (device_status == nullptr) return fail(PE_ATTN_ERR_NULL, "device_status is null");
  if (limit_cycles < 1000 || limit_cycles > 2000000000ll)
    return fail(PE_ATTN_ERR_SHAPE, "limit_cycles must be in [1e3, 2e9] (got %lld)", (long long)limit_cycles);
  wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_status, limit_cycles);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PE_ATTN_ERR_LAUNCH, "self-test launch failed: %s", cudaGetErrorString(e));
  return PE_ATTN_OK;
}

int pe_attn_backward(const pe_attn_bwd_args* a, void* stream) {
  if (a == nullptr) return fail(PE_ATTN_ERR_NULL, "args is null");
  if (a->struct_size != sizeof(pe_attn_bwd_args))
    return fail(PE_ATTN_ERR_VARIANT, "struct_size %u does not match this library's %zu", a->struct_size,
                sizeof(pe_attn_bwd_args));
  if (a->B < 1 || a->H < 1 || a->Hkv < 1 || a->Sq < 1 || a->Sk < 1)
    return fail(PE_ATTN_ERR_SHAPE, "B, H, Hkv, Sq, Sk must be positive");
  if (a->H % a->Hkv != 0) return fail(PE_ATTN_ERR_SHAPE, "H=%d is not a multiple of Hkv=%d", a->H, a->Hkv);
  if (a->Sk < a->Sq) return fail(PE_ATTN_ERR_SHAPE, "Sk=%d < Sq=%d", a->Sk, a->Sq);
  if (a->B > 65535 || a->Hkv > 65535) return fail(PE_ATTN_ERR_SHAPE, "B and Hkv must be <= 65535");
  if (a->dtype != PE_ATTN_BF16 && a->dtype != PE_ATTN_FP32) return fail(PE_ATTN_ERR_VARIANT, "unknown dtype %d", a->dtype);
  if (!(a->dtype == PE_ATTN_BF16 && bwd_supports(a->d_qk, a->d_v)) && !bwd_simt_supports(a->d_qk, a->d_v, a->dtype))
    return fail(PE_ATTN_ERR_SHAPE,
                "backward supports (d_qk, d_v) in {(64,64), (128,64), (128,128)} on the tensor cores (bf16) and any "
                "multiples of 8 up to (256, 128) on the CUDA cores, bf16 or fp32 (got %d, %d, dtype %d)", a->d_qk, a->d_v,
                a->dtype);
  struct { const char* name; const void* p; const int64_t* s; } ts[] = {
      {"q", a->q, a->q_stride},       {"k", a->k, a->k_stride},   {"v", a->v, a->v_stride},
      {"out", a->out, a->out_stride}, {"dout", a->dout, a->dout_stride},
      {"dk", a->dk, a->dk_stride},    {"dv", a->dv, a->dv_stride}};
  for (auto& t : ts) {
    if (t.p == nullptr) return fail(PE_ATTN_ERR_NULL, "%s is null", t.name);
    if (!aligned16(t.p)) return fail(PE_ATTN_ERR_ALIGNMENT, "%s is not 16-byte aligned", t.name);
    for (int i = 0; i < 3; ++i)
      if (t.s[i] % 8 != 0)
        return fail(PE_ATTN_ERR_ALIGNMENT, "%s stride[%d]=%lld is not a multiple of 8 elements", t.name, i,
                    (long long)t.s[i]);
  }
  if (a->lse == nullptr || a->dq_accum == nullptr || a->dvec == nullptr)
    return fail(PE_ATTN_ERR_NULL, "lse, dq_accum and dvec are required");
  if (!aligned16(a->dq_accum)) return fail(PE_ATTN_ERR_ALIGNMENT, "dq_accum is not 16-byte aligned");
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
      major != 10)
    return fail(PE_ATTN_ERR_DEVICE, "no sm_100 device is current");
  BwdParams p;
  memset(&p, 0, sizeof(p));
  p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.groups = a->H / a->Hkv;
  p.Sq = a->Sq; p.Sk = a->Sk; p.causal_off = a->Sk - a->Sq;
  p.scale = a->scale;
  p.q = make_ref(a->q, a->q_stride);
  p.k = make_ref(a->k, a->k_stride);
  p.v = make_ref(a->v, a->v_stride);
  p.out = make_ref(a->out, a->out_stride);
  p.dout = make_ref(a->dout, a->dout_stride);
  p.dk = make_ref(a->dk, a->dk_stride);
  p.dv = make_ref(a->dv, a->dv_stride);
  p.lse = a->lse; p.slopes = a->alibi_slopes;
  p.dq_accum = a->dq_accum; p.dvec = a->dvec; p.status = a->device_status;
  return launch_bwd(p, a->d_qk, a->d_v, a->dtype, a->alibi_slopes != nullptr, static_cast<cudaStream_t>(stream));
}

int pe_attn_version(void) { return PE_ATTN_ABI_VERSION; }

const char* pe_attn_last_error(void) { return g_error; }

const char* pe_attn_status_string(int status) {
  switch (status) {
    case PE_ATTN_OK: return "ok";
    case PE_ATTN_ERR_NULL: return "null pointer";
    case PE_ATTN_ERR_VARIANT: return "unknown variant, dtype or flag combination";
    case PE_ATTN_ERR_SHAPE: return "unsupported shape";
    case PE_ATTN_ERR_ALIGNMENT: return "misaligned pointer or stride";
    case PE_ATTN_ERR_LAUNCH: return "CUDA launch failure";
    case PE_ATTN_ERR_DEVICE: return "no sm_100 device";
    case PE_ATTN_ERR_TOO_LARGE: return "size exceeds the entry point's limit";
    default: return "unknown status";
  }
}

int pe_attn_validate(const pe_attn_args* args) { return validate(args, nullptr); }

const char* pe_attn_kernel_name(const pe_attn_args* args) {
  if (validate(args, nullptr) != PE_ATTN_OK) return nullptr;
  if (args->dtype != PE_ATTN_BF16 || (args->flags & PE_ATTN_SIMT_CHECK)) return "ffma";
  KParams k;
  validate(args, &k);
  if (tc2_supports(k) && k.Sq > 256 && !(k.flags & PE_ATTN_SINGLE_CTA)) return "tcgen05-pair";
  return (tc4_supports(k) && !(k.flags & PE_ATTN_SINGLE_CTA)) ? "tcgen05-four-tile" : "tcgen05";
}

size_t pe_attn_forward_workspace_bytes(const pe_attn_args* args) {
  KParams k;
  if (validate(args, &k) != PE_ATTN_OK) return 0;
  if (args->dtype == PE_ATTN_FP32) return simt_key_scratch_bytes(k);
  if (args->flags & (PE_ATTN_SIMT_CHECK | PE_ATTN_SINGLE_CTA)) return 0;
  return (tc2_supports(k) && k.Sq > 256) ? tc2_workspace_bytes(k) : 0;
}

double pe_attn_flops(const pe_attn_args* a) {
  if (a == nullptr) return 0.0;
  // causal pairs: row r sees r + 1 + (Sk - Sq) keys
  const double off = (double)a->Sk - a->Sq;
  const double pairs = (double)a->Sq * (off + 1.0) + 0.5 * (double)a->Sq * ((double)a->Sq - 1.0);
  return (double)a->B * a->H * pairs * 2.0 * (a->d_c + 2 * a->d_r + a->d_v);
}

// checks of the decode entry points beyond validate()
static int validate_decode(const pe_attn_args* args, KParams* k) {
  const int rc = validate(args, k);
  if (rc != PE_ATTN_OK) return rc;
  if (args->dtype != PE_ATTN_BF16 || (args->flags & PE_ATTN_SIMT_CHECK))
    return fail(PE_ATTN_ERR_VARIANT, "the split-KV path is bf16 only");
  if (!decode_supports(*k))
    return fail(PE_ATTN_ERR_SHAPE, "the split-KV path takes at most 8 query rows per K/V head (got H/Hkv * Sq = %d)",
                k->groups * k->Sq);
  return PE_ATTN_OK;
}

size_t pe_attn_decode_workspace_bytes(const pe_attn_args* args) {
  KParams k;
  if (validate_decode(args, &k) != PE_ATTN_OK) return 0;
  return decode_workspace_bytes(k);
}

int pe_attn_decode(const pe_attn_args* args, void* workspace, size_t workspace_bytes, void* stream) {
  KParams k;
  const int rc = validate_decode(args, &k);
  if (rc != PE_ATTN_OK) return rc;
  if (workspace == nullptr) return fail(PE_ATTN_ERR_NULL, "workspace is null");
  if (!aligned16(workspace)) return fail(PE_ATTN_ERR_ALIGNMENT, "workspace is not 16-byte aligned");
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
    return fail(PE_ATTN_ERR_DEVICE, "no sm_100 device is current");
  g_error[0] = 0;
  return launch_decode(k, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int pe_attn_forward(const pe_attn_args* args, void* stream) {
  KParams k;
  const int rc = validate(args, &k);
  if (rc != PE_ATTN_OK) return rc;
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return fail(PE_ATTN_ERR_DEVICE, "no CUDA device is current");
  if (major != 10)
    return fail(PE_ATTN_ERR_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
  g_error[0] = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (args->dtype == PE_ATTN_BF16 && !(args->flags & PE_ATTN_SIMT_CHECK)) return launch_tc(k, s);
  return launch_simt(k, args->dtype, s);
}

}  // extern "C"
