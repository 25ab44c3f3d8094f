// C ABI of libintfa.so: argument validation, error reporting, dispatch.
// Nothing here throws or aborts; every entry point returns a status code.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "intfa_internal.h"

namespace intfa {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count_cached() {
  static std::atomic<int> cache[64];     // 0: not asked yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_tma_tensor(const char* name, const void* ptr, const int64_t* st, int esize) {
  if (!ptr) return set_error(INTFA_ERR_INVALID_ARG, "%s is NULL", name);
  if (!aligned16(ptr)) return set_error(INTFA_ERR_INVALID_ARG, "%s must be 16-byte aligned", name);
  for (int i = 0; i < 3; ++i)
    if (st[i] <= 0 || (st[i] * esize) % 16 != 0)
      return set_error(INTFA_ERR_INVALID_ARG, "%s stride[%d]=%lld: byte strides must be positive multiples of 16", name,
                       i, (long long)st[i]);
  return INTFA_OK;
}

}  // namespace intfa

using namespace intfa;

// the head dims of the reference's ops (flash_atten_full_int8.py:193)
static bool head_dim_ok(int D) { return D == 16 || D == 32 || D == 64 || D == 128 || D == 256; }

extern "C" {

int intfa_version(void) { return 100; }

int intfa_last_error(char* buf, size_t len) {
  if (!buf || len == 0) return INTFA_ERR_INVALID_ARG;
  strncpy(buf, g_err, len - 1);
  buf[len - 1] = 0;
  return INTFA_OK;
}

int intfa_sm_count(void) { return sm_count_cached(); }

int intfa_fwd(const IntfaFwdParams* p, void* stream) {
  if (!p) return set_error(INTFA_ERR_INVALID_ARG, "params is NULL");
  if (p->variant != INTFA_VARIANT_FULL && p->variant != INTFA_VARIANT_HALF && p->variant != INTFA_VARIANT_HALF_FP8)
    return set_error(INTFA_ERR_INVALID_ARG, "variant must be INTFA_VARIANT_FULL, INTFA_VARIANT_HALF or INTFA_VARIANT_HALF_FP8");
  const bool full = p->variant == INTFA_VARIANT_FULL;
  if (p->B <= 0 || p->H <= 0 || p->Nq <= 0 || p->Nk <= 0)
    return set_error(INTFA_ERR_INVALID_ARG, "B, H, Nq, Nk must be positive");
  if (!head_dim_ok(p->D))
    return set_error(INTFA_ERR_UNSUPPORTED, "head_dim %d unsupported: 16, 32, 64, 128 or 256", p->D);
  if (p->G != 64 && p->G != 128 && !(p->G == 32 && p->D <= 32 && full))
    return set_error(INTFA_ERR_UNSUPPORTED, "G=%d unsupported: 64 or 128 (32 for full-int8 at head dims 16 and 32)", p->G);
  if (p->D == 256 && p->G == 128 && !full)
    return set_error(INTFA_ERR_UNSUPPORTED, "half-int8 at head_dim 256 runs with G=64 only");
  if (p->p_round != 0 && p->p_round != 1) return set_error(INTFA_ERR_INVALID_ARG, "p_round must be 0 or 1");
  if (p->H_kv < 0 || (p->H_kv > 0 && p->H % p->H_kv != 0))
    return set_error(INTFA_ERR_INVALID_ARG, "H=%d must be a multiple of H_kv=%d", p->H, p->H_kv);
  if (p->o_dtype != INTFA_OUT_FP16 && p->o_dtype != INTFA_OUT_BF16)
    return set_error(INTFA_ERR_INVALID_ARG, "o_dtype must be INTFA_OUT_FP16 or INTFA_OUT_BF16");
  if ((long long)p->B * p->H * (((long long)p->Nq + 127) / 128) * (p->D == 256 ? 2 : 1) > 0x7fffffffLL) return set_error(INTFA_ERR_TOO_LARGE, "too many work items");
  int rc;
  if ((rc = check_tma_tensor("q", p->q, p->q_stride, 1))) return rc;
  if ((rc = check_tma_tensor("k", p->k, p->k_stride, 1))) return rc;
  if ((rc = check_tma_tensor("v", p->v, p->v_stride, p->variant == INTFA_VARIANT_HALF ? 2 : 1))) return rc;
  if (!p->q_scale || !p->k_scale) return set_error(INTFA_ERR_INVALID_ARG, "q_scale / k_scale is NULL");
  if (!aligned16(p->k_scale) || p->ks_stride[0] % 4 != 0 || p->ks_stride[1] % 4 != 0)
    return set_error(INTFA_ERR_INVALID_ARG, "k_scale must be 16-byte aligned with (B,H) strides that are multiples of 4");
  {
    // the K scales of a KV step are fetched G at a time: every row must have room up to the next multiple of G
    const long long need = ((long long)p->Nk + p->G - 1) / p->G * p->G;
    const int hk = p->H_kv > 0 ? p->H_kv : p->H;
    if ((hk > 1 && p->ks_stride[1] < need) || (p->B > 1 && p->ks_stride[0] < need))
      return set_error(INTFA_ERR_INVALID_ARG, "k_scale rows must be allocated up to the next multiple of G (%lld floats for Nk=%d)", need, p->Nk);
  }
  if (full && !p->v_scale) return set_error(INTFA_ERR_INVALID_ARG, "v_scale is NULL (full-int8)");
  if (p->kv_order != 0 && p->kv_order != 1) return set_error(INTFA_ERR_INVALID_ARG, "kv_order must be 0 (ascending) or 1 (descending)");
  if (p->vs_stride_blk < 0) return set_error(INTFA_ERR_INVALID_ARG, "vs_stride_blk must not be negative");
  if (p->vs_stride_blk != 0 && (p->state_in || p->state_out))
    return set_error(INTFA_ERR_UNSUPPORTED, "carried state with one v_scale row per KV tile is not supported");
  if (p->write_o) {
    if (!p->o) return set_error(INTFA_ERR_INVALID_ARG, "o is NULL");
    if (!aligned16(p->o) || p->o_stride[0] % 8 || p->o_stride[1] % 8 || p->o_stride[2] % 8)
      return set_error(INTFA_ERR_INVALID_ARG, "o must be 16-byte aligned with strides that are multiples of 8 elements");
  }
  if ((p->state_in || p->state_out) && (!p->state_m || !p->state_l || !p->state_acc))
    return set_error(INTFA_ERR_INVALID_ARG, "state_in/state_out set but a state pointer is NULL");
  if ((p->state_in || p->state_out) && !aligned16(p->state_acc))
    return set_error(INTFA_ERR_INVALID_ARG, "state_acc must be 16-byte aligned");
  if (!p->write_o && !p->state_out) return set_error(INTFA_ERR_INVALID_ARG, "nothing to write: write_o and state_out are both 0");
  if (p->dbg_s && (p->dbg_tile < 0 || p->dbg_step < 0)) return set_error(INTFA_ERR_INVALID_ARG, "bad debug tap");
  return fwd_dispatch(p, reinterpret_cast<cudaStream_t>(stream));
}

static int check_quant_args(const void* x, const int64_t* st, const void* x8, const float* scale, int B, int H, int N,
                            int D) {
  if (!x || !st || !x8 || !scale) return set_error(INTFA_ERR_INVALID_ARG, "NULL argument");
  if (B <= 0 || H <= 0 || N <= 0) return set_error(INTFA_ERR_INVALID_ARG, "B, H, N must be positive");
  if (!head_dim_ok(D)) return set_error(INTFA_ERR_UNSUPPORTED, "head_dim %d unsupported: 16, 32, 64, 128 or 256", D);
  if (!aligned16(x) || st[0] % 8 || st[1] % 8 || st[2] % 8)
    return set_error(INTFA_ERR_INVALID_ARG, "input rows must be 16-byte aligned (pointer and strides multiples of 8 elements)");
  if (!aligned16(x8)) return set_error(INTFA_ERR_INVALID_ARG, "int8 output must be 16-byte aligned");
  return INTFA_OK;
}

int intfa_quant_pertoken(const void* x, const int64_t x_stride[3], void* x8, float* scale, int32_t B, int32_t H,
                         int32_t N, int32_t D, void* stream) {
  int rc = check_quant_args(x, x_stride, x8, scale, B, H, N, D);
  if (rc) return rc;
  return quant_pertoken(x, x_stride, x8, scale, B, H, N, D, reinterpret_cast<cudaStream_t>(stream));
}

size_t intfa_quant_v_workspace_bytes(int32_t B, int32_t H, int32_t D) {
  if (B <= 0 || H <= 0 || D <= 0) return 0;
  return (size_t)B * H * D * sizeof(unsigned int);
}

int intfa_quant_v(const void* v, const int64_t v_stride[3], void* v8, float* scale, int32_t mode, int32_t B, int32_t H,
                  int32_t N, int32_t D, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_quant_args(v, v_stride, v8, scale, B, H, N, D);
  if (rc) return rc;
  if (mode != INTFA_VSCALE_PER_TENSOR && mode != INTFA_VSCALE_PER_CHANNEL)
    return set_error(INTFA_ERR_INVALID_ARG, "mode must be INTFA_VSCALE_PER_TENSOR or INTFA_VSCALE_PER_CHANNEL");
  if (!workspace || workspace_bytes < intfa_quant_v_workspace_bytes(B, H, D))
    return set_error(INTFA_ERR_INVALID_ARG, "workspace missing or smaller than intfa_quant_v_workspace_bytes()");
  if ((long long)B * H > 65535) return set_error(INTFA_ERR_TOO_LARGE, "B*H=%lld exceeds 65535", (long long)B * H);
  return quant_v(v, v_stride, v8, scale, mode, B, H, N, D, workspace, reinterpret_cast<cudaStream_t>(stream));
}

size_t intfa_quant_qkv_workspace_bytes(int32_t B, int32_t H_kv, int32_t Nk, int32_t D) {
  if (B <= 0 || H_kv <= 0 || Nk <= 0 || D <= 0) return 0;
  return quant_qkv_workspace_bytes(B, H_kv, Nk, D);
}

int intfa_quant_qkv(const void* q, const void* k, const void* v, const int64_t v_stride[3], void* q8, void* k8, void* v8,
                    float* q_scale, float* k_scale, float* v_scale, int32_t v_mode, int32_t B, int32_t H, int32_t H_kv,
                    int32_t Nq, int32_t Nk, int32_t D, void* workspace, size_t workspace_bytes, void* stream) {
  if (!q || !k || !q8 || !k8 || !q_scale || !k_scale) return set_error(INTFA_ERR_INVALID_ARG, "NULL argument");
  if (B <= 0 || H <= 0 || H_kv <= 0 || Nq <= 0 || Nk <= 0) return set_error(INTFA_ERR_INVALID_ARG, "B, H, H_kv, Nq, Nk must be positive");
  if (!head_dim_ok(D)) return set_error(INTFA_ERR_UNSUPPORTED, "head_dim %d unsupported: 16, 32, 64, 128 or 256", D);
  if (!aligned16(q) || !aligned16(k) || !aligned16(q8) || !aligned16(k8))
    return set_error(INTFA_ERR_INVALID_ARG, "q, k, q8, k8 must be 16-byte aligned (and contiguous)");
  if (v) {
    if (!v_stride || !v8 || !v_scale) return set_error(INTFA_ERR_INVALID_ARG, "v given without v_stride / v8 / v_scale");
    if (!aligned16(v) || !aligned16(v8) || v_stride[0] % 8 || v_stride[1] % 8 || v_stride[2] % 8)
      return set_error(INTFA_ERR_INVALID_ARG, "v rows must be 16-byte aligned (pointer and strides multiples of 8 elements)");
    if (v_mode != INTFA_VSCALE_PER_TENSOR && v_mode != INTFA_VSCALE_PER_CHANNEL)
      return set_error(INTFA_ERR_INVALID_ARG, "v_mode must be INTFA_VSCALE_PER_TENSOR or INTFA_VSCALE_PER_CHANNEL");
    if ((long long)B * H_kv > 65535) return set_error(INTFA_ERR_TOO_LARGE, "B*H_kv=%lld exceeds 65535", (long long)B * H_kv);
    if (!workspace || workspace_bytes < quant_qkv_workspace_bytes(B, H_kv, Nk, D))
      return set_error(INTFA_ERR_INVALID_ARG, "workspace missing or smaller than intfa_quant_qkv_workspace_bytes()");
  }
  return quant_qkv(q, k, v, v_stride, q8, k8, v8, q_scale, k_scale, v_scale, v_mode, B, H, H_kv, Nq, Nk, D, workspace,
                   reinterpret_cast<cudaStream_t>(stream));
}

int intfa_v_colmax(const void* v, const int64_t v_stride[3], void* colmax, int32_t B, int32_t H, int32_t N, int32_t D,
                   void* stream) {
  if (!v || !v_stride || !colmax) return set_error(INTFA_ERR_INVALID_ARG, "NULL argument");
  if (B <= 0 || H <= 0 || N <= 0) return set_error(INTFA_ERR_INVALID_ARG, "B, H, N must be positive");
  if (!head_dim_ok(D)) return set_error(INTFA_ERR_UNSUPPORTED, "head_dim %d unsupported: 16, 32, 64, 128 or 256", D);
  if (!aligned16(v) || v_stride[0] % 8 || v_stride[1] % 8 || v_stride[2] % 8)
    return set_error(INTFA_ERR_INVALID_ARG, "input rows must be 16-byte aligned (pointer and strides multiples of 8 elements)");
  if ((long long)B * H > 65535) return set_error(INTFA_ERR_TOO_LARGE, "B*H=%lld exceeds 65535", (long long)B * H);
  return v_colmax(v, v_stride, colmax, B, H, N, D, reinterpret_cast<cudaStream_t>(stream));
}

int intfa_v_quant_from_colmax(const void* v, const int64_t v_stride[3], const void* colmax, void* v8, float* scale,
                              int32_t mode, int32_t B, int32_t H, int32_t N, int32_t D, void* stream) {
  int rc = check_quant_args(v, v_stride, v8, scale, B, H, N, D);
  if (rc) return rc;
  if (!colmax) return set_error(INTFA_ERR_INVALID_ARG, "colmax is NULL");
  if (mode != INTFA_VSCALE_PER_TENSOR && mode != INTFA_VSCALE_PER_CHANNEL)
    return set_error(INTFA_ERR_INVALID_ARG, "mode must be INTFA_VSCALE_PER_TENSOR or INTFA_VSCALE_PER_CHANNEL");
  if ((long long)B * H > 65535) return set_error(INTFA_ERR_TOO_LARGE, "B*H=%lld exceeds 65535", (long long)B * H);
  return v_quant_from_colmax(v, v_stride, colmax, v8, scale, mode, B, H, N, D, reinterpret_cast<cudaStream_t>(stream));
}

int intfa_quant_v_static(const void* v, const int64_t v_stride[3], void* v8, float* scale, int32_t mode, int32_t B,
                         int32_t H, int32_t N, int32_t D, void* stream) {
  int rc = check_quant_args(v, v_stride, v8, scale, B, H, N, D);
  if (rc) return rc;
  if (mode != INTFA_VSCALE_PER_TENSOR && mode != INTFA_VSCALE_PER_CHANNEL)
    return set_error(INTFA_ERR_INVALID_ARG, "mode must be INTFA_VSCALE_PER_TENSOR or INTFA_VSCALE_PER_CHANNEL");
  if ((long long)B * H > 65535) return set_error(INTFA_ERR_TOO_LARGE, "B*H=%lld exceeds 65535", (long long)B * H);
  return quant_v_static(v, v_stride, v8, scale, mode, B, H, N, D, reinterpret_cast<cudaStream_t>(stream));
}

size_t intfa_quant_v_static_max_words(void) { return (size_t)kStaticColmaxWords; }

int intfa_scales_f16_to_f32(const void* src_f16, float* dst_f32, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!src_f16 || !dst_f32))) return set_error(INTFA_ERR_INVALID_ARG, "bad argument");
  return scales_f16_to_f32(src_f16, dst_f32, n, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
