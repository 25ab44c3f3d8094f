// Fused quantisation prologue (HBM-bound): fp16 -> int8 with absmax scales.
//
// Bit-exact restatement of the reference quantisers, whose arithmetic follows the fp16
// input dtype (benchmark.py:96-107):
//   amax  = max |x|                       (exact in fp16)
//   scale = fp16( fp32(amax) / 127 )      (IEEE fp32 division, then round-to-nearest fp16)
//   q     = int8( rint( fp16( fp32(x) / fp32(scale) ) ) )   (rint = half-to-even, as torch.round)
// The per-element division is evaluated as a correctly rounded quotient from one reciprocal per
// row/channel and two fmas (see quant_pair), so it costs no division instruction per element.
// Scales are written as fp32 holding the fp16-representable value.  amax == 0 gives
// scale 0 and q 0 (the reference computes 0/0 there).
//
// Each row of D fp16 is read by D/8 lanes with one 128-bit load per lane; the row/column
// maxima are reduced with warp shuffles.  Per-token: one pass.  V (per-channel or
// per-(batch,head)): a column-absmax pass, then the quantising pass.  The fused entry (quant_qkv) runs the Q rows,
// the K rows and the V column-absmax pass as ONE launch (partial maxima per chunk, plain stores) and the V
// quantising pass as a second; the stand-alone V entries use atomicMax into a small scratch array instead.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "intfa_internal.h"
#include "intfa_ptx.cuh"

namespace intfa {

__device__ __forceinline__ float scale_from_amax(float amax) {
  return __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
}
// Correctly rounded x / s without a division per element (Markstein): with r = RN(1/s),
// q0 = RN(x*r), e = x - q0*s (exact in one fma), q = RN(q0 + e*r) equals RN(x/s) unless the
// significand of s is all ones -- impossible here because s is an fp16 value held in fp32.
// Then the reference's rounding chain: fp16(q), and rint() done IN fp16 by adding 1536 = 1.5*2^10 (the sum has
// an ulp of 1, so its round-to-nearest-even is rint, and its bit pattern is 0x6600 + n: the two's-complement
// integer is the low byte).  Everything runs two elements per instruction (packed fp32, fp16x2): these kernels
// are as much bound by instruction issue as by HBM.
// A zero scale (an all-zero row or channel; the reference computes 0/0 there) is given the reciprocal 0, which makes
// every quotient 0.
struct Scale2 { uint64_t neg_s, r; };      // (-s, -s') and (1/s, 1/s') of two neighbouring elements
__device__ __forceinline__ float safe_rcp(float s) { return s == 0.f ? 0.f : __frcp_rn(s); }
__device__ __forceinline__ Scale2 make_scale2(float s0, float s1) {
  Scale2 k;
  k.neg_s = f2_pack(-s0, -s1);
  k.r = f2_pack(safe_rcp(s0), safe_rcp(s1));
  return k;
}
// two fp16 inputs -> two int8 in bytes 0 and 2 of the result
__device__ __forceinline__ uint32_t quant_pair(__half2 x, const Scale2& k) {
  const float2 f = __half22float2(x);
  const uint64_t X = f2_pack(f.x, f.y);
  const uint64_t q0 = f2_mul(X, k.r);
  const uint64_t e = f2_fma(q0, k.neg_s, X);
  float qa, qb;
  f2_unpack(f2_fma(e, k.r, q0), qa, qb);
  const __half2 t = __floats2half2_rn(qa, qb);
  const __half2 u = __hadd2(t, __half2(__ushort_as_half(0x6600), __ushort_as_half(0x6600)));
  return *reinterpret_cast<const uint32_t*>(&u);
}
__device__ __forceinline__ float amax8(const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  __half2 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
  return fmaxf(__low2float(m), __high2float(m));
}
// k[i]: the scales of elements 2i, 2i+1 of the 8
__device__ __forceinline__ uint2 quant8(const uint4& v, const Scale2 (&k)[4]) {
  const __half2* h2 = reinterpret_cast<const __half2*>(&v);
  const uint32_t u0 = quant_pair(h2[0], k[0]), u1 = quant_pair(h2[1], k[1]);
  const uint32_t u2 = quant_pair(h2[2], k[2]), u3 = quant_pair(h2[3], k[3]);
  return make_uint2(__byte_perm(u0, u1, 0x6420), __byte_perm(u2, u3, 0x6420));
}

// L2 residency hints.  The first launch of the fused prologue reads V for its column maxima and the second reads it
// again to quantise it: V is loaded "evict last" there and everything that is touched once (Q, K, every int8 store)
// "evict first", and the second launch walks the (batch, head) slabs in the opposite order, so that the slabs read
// last -- as much of V as the L2 holds -- are served from L2 instead of HBM.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ld_hint(const void* p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ void st_hint(void* p, uint2 v, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.v2.u32 [%0], {%1, %2}, %3;" ::"l"(p), "r"(v.x), "r"(v.y), "l"(policy) : "memory");
}

constexpr int kQuantUnroll = 4;    // independent 128-bit loads in flight per lane

// Per-token quantisation of the rows that CTA `cta` of `ncta` owns (a grid-stride loop over groups of rows).
template <int D, bool CONTIG>
__device__ __forceinline__ void pertoken_rows(const __half* __restrict__ x, long long sB, long long sH, long long sN,
                                              int8_t* __restrict__ x8, float* __restrict__ scale, int H, int N,
                                              long long total_rows, int cta, int ncta) {
  constexpr int LPR = D / 8;         // lanes per row
  constexpr int RPW = 32 / LPR;      // rows per warp and load
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR;
  const long long warp_g = (long long)cta * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)ncta * (blockDim.x >> 5);
  const uint64_t once = l2_policy_evict_first();
  for (long long row0 = warp_g * (RPW * kQuantUnroll); row0 < total_rows; row0 += nwarps * (RPW * kQuantUnroll)) {
    uint4 v[kQuantUnroll];
    long long rows[kQuantUnroll];
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      const long long row = row0 + u * RPW + lane / LPR;
      rows[u] = row;
      v[u] = make_uint4(0, 0, 0, 0);
      if (row < total_rows) {
        if (CONTIG) {
          v[u] = ld_hint(x + row * D + sub * 8, once);      // [B,H,N,D] contiguous: the row index is the address
        } else {
          // total_rows < 2^31 (checked by the host): 32-bit divisions
          const unsigned int r32 = (unsigned int)row;
          const unsigned int bh = r32 / (unsigned int)N;
          const unsigned int n = r32 - bh * (unsigned int)N;
          const unsigned int b = bh / (unsigned int)H, h = bh - b * (unsigned int)H;
          v[u] = ld_hint(x + (long long)b * sB + (long long)h * sH + (long long)n * sN + sub * 8, once);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      float a = amax8(v[u]);
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
      const float s = scale_from_amax(a);
      if (rows[u] < total_rows) {
        const Scale2 k1 = make_scale2(s, s);
        const Scale2 k[4] = {k1, k1, k1, k1};
        st_hint(x8 + rows[u] * D + sub * 8, quant8(v[u], k), once);
        if (sub == 0) scale[rows[u]] = s;
      }
    }
  }
}

template <int D, bool CONTIG>
__global__ void __launch_bounds__(256) quant_pertoken_kernel(const __half* __restrict__ x, long long sB, long long sH,
                                                             long long sN, int8_t* __restrict__ x8,
                                                             float* __restrict__ scale, int H, int N,
                                                             long long total_rows) {
  pertoken_rows<D, CONTIG>(x, sB, sH, sN, x8, scale, H, N, total_rows, blockIdx.x, gridDim.x);
}

// Column absmax of chunk `chunk` (rows_per_cta rows) of the (batch, head) slab `bh`.  ATOMIC: atomicMax on the bit
// patterns of non-negative floats into colmax[bh*D + ch] (the caller has zeroed it); otherwise a plain store into
// row `chunk` of a [chunks][B*H][D] array of partial maxima (nothing to clear, nothing to order).
template <int D, bool ATOMIC>
__device__ __forceinline__ void colmax_chunk(const __half* __restrict__ x, long long sB, long long sH, long long sN,
                                             unsigned int* __restrict__ colmax, int H, int N, int rows_per_cta,
                                             int chunk, int bh, int BH) {
  constexpr int LPR = D / 8;
  constexpr int RPW = 32 / LPR;
  __shared__ float red[8][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int sub = lane % LPR;
  const int b = bh / H, h = bh - b * H;
  const __half* base = x + b * sB + h * sH + sub * 8;
  const int r_begin = chunk * rows_per_cta;
  const int r_end = min(N, r_begin + rows_per_cta);
  const uint64_t keep = l2_policy_evict_last();
  __half2 m[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) m[i] = __float2half2_rn(0.f);
  for (int r0 = r_begin + warp * RPW + lane / LPR; r0 < r_end; r0 += nw * RPW * kQuantUnroll) {
    uint4 v[kQuantUnroll];
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      const int r = r0 + u * nw * RPW;
      v[u] = r < r_end ? ld_hint(base + r * sN, keep) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      const __half2* hv = reinterpret_cast<const __half2*>(&v[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) m[i] = __hmax2(m[i], __habs2(hv[i]));
    }
  }
  float f[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(m[i]);
    f[2 * i + 1] = __high2float(m[i]);
  }
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1)
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = fmaxf(f[i], __shfl_xor_sync(0xffffffffu, f[i], o));
  if (lane < LPR)
#pragma unroll
    for (int i = 0; i < 8; ++i) red[warp][sub * 8 + i] = f[i];
  __syncthreads();
  for (int ch = threadIdx.x; ch < D; ch += blockDim.x) {
    float a = 0.f;
    for (int w = 0; w < nw; ++w) a = fmaxf(a, red[w][ch]);
    if (ATOMIC) atomicMax(colmax + (long long)bh * D + ch, __float_as_uint(a));
    else colmax[((long long)chunk * BH + bh) * D + ch] = __float_as_uint(a);
  }
}

template <int D>
__global__ void __launch_bounds__(256) v_colmax_kernel(const __half* __restrict__ x, long long sB, long long sH,
                                                       long long sN, unsigned int* __restrict__ colmax, int H, int N,
                                                       int rows_per_cta) {
  colmax_chunk<D, true>(x, sB, sH, sN, colmax, H, N, rows_per_cta, blockIdx.x, blockIdx.y, gridDim.y);
}

// The first launch of the fused prologue: one grid over three jobs -- CTAs [0, gq) quantise the rows of Q,
// [gq, gq+gk) those of K (both per token, contiguous tensors), the rest take one (chunk, batch*head) piece of V each and
// store its column absmax as a partial result.  Nothing is shared between the jobs, so no ordering is needed.
struct QkvJob {
  const __half* q; int8_t* q8; float* qs; long long q_rows; int gq;
  const __half* k; int8_t* k8; float* ks; long long k_rows; int gk;
  const __half* v; long long vB, vH, vN; unsigned int* partial; int Hkv, Nk, rows_per_cta, chunks, BHkv;
};
template <int D>
__global__ void __launch_bounds__(256) quant_qkv_kernel(const QkvJob j) {
  const int cta = blockIdx.x;
  if (cta < j.gq) {
    pertoken_rows<D, true>(j.q, 0, 0, 0, j.q8, j.qs, 1, 1, j.q_rows, cta, j.gq);
  } else if (cta < j.gq + j.gk) {
    pertoken_rows<D, true>(j.k, 0, 0, 0, j.k8, j.ks, 1, 1, j.k_rows, cta - j.gq, j.gk);
  } else {
    const int i = cta - j.gq - j.gk;
    colmax_chunk<D, false>(j.v, j.vB, j.vH, j.vN, j.partial, j.Hkv, j.Nk, j.rows_per_cta, i % j.chunks, i / j.chunks, j.BHkv);
  }
}

template <int D>
__global__ void __launch_bounds__(256) v_quant_kernel(const __half* __restrict__ x, long long sB, long long sH,
                                                      long long sN, const unsigned int* __restrict__ colmax,
                                                      int8_t* __restrict__ x8, float* __restrict__ scale,
                                                      int per_channel, int H, int N, int rows_per_cta, int nparts) {
  constexpr int LPR = D / 8;
  constexpr int RPW = 32 / LPR;
  __shared__ float s_scale[D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int sub = lane % LPR;
  const int bh = gridDim.y - 1 - blockIdx.y;     // last slab first: the column-absmax pass read it last
  const int b = bh / H, h = bh - b * H;
  const uint64_t once = l2_policy_evict_first();
  if (threadIdx.x < 32) {
    // every channel's absmax; for the per-(batch,head) mode reduce them to one
    constexpr int CPL = (D + 31) / 32;     // channels per lane
    float a[CPL];
    float all = 0.f;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      a[i] = 0.f;      // colmax is [nparts][B*H][D]: one row, or the partial maxima of the fused first launch
      if (lane + 32 * i < D)
        for (int c = 0; c < nparts; ++c) a[i] = fmaxf(a[i], __uint_as_float(colmax[((long long)c * gridDim.y + bh) * D + lane + 32 * i]));
      all = fmaxf(all, a[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) all = fmaxf(all, __shfl_xor_sync(0xffffffffu, all, o));
#pragma unroll
    for (int i = 0; i < CPL; ++i)
      if (lane + 32 * i < D) s_scale[lane + 32 * i] = scale_from_amax(per_channel ? a[i] : all);
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    if (per_channel) {
      for (int ch = threadIdx.x; ch < D; ch += blockDim.x) scale[(long long)bh * D + ch] = s_scale[ch];
    } else if (threadIdx.x == 0) {
      scale[bh] = s_scale[0];
    }
  }
  Scale2 k[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) k[i] = make_scale2(s_scale[sub * 8 + 2 * i], s_scale[sub * 8 + 2 * i + 1]);
  const __half* base = x + b * sB + h * sH + sub * 8;
  int8_t* obase = x8 + (long long)bh * N * D + sub * 8;
  const int r_begin = blockIdx.x * rows_per_cta;
  const int r_end = min(N, r_begin + rows_per_cta);
  for (int r0 = r_begin + warp * RPW + lane / LPR; r0 < r_end; r0 += nw * RPW * kQuantUnroll) {
    uint4 v[kQuantUnroll];
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      const int r = r0 + u * nw * RPW;
      v[u] = r < r_end ? ld_hint(base + r * sN, once) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      const int r = r0 + u * nw * RPW;
      if (r < r_end) st_hint(obase + (long long)r * D, quant8(v[u], k), once);
    }
  }
}

__global__ void scales_f16_to_f32_kernel(const __half* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __half2float(src[i]);
}

// head dims of the reference's ops (flash_atten_full_int8.py:193): one instantiation each
#define INTFA_D_SWITCH(D, CALL)                 \
  switch (D) {                                  \
    case 16: { constexpr int DD = 16; CALL; } break;   \
    case 32: { constexpr int DD = 32; CALL; } break;   \
    case 64: { constexpr int DD = 64; CALL; } break;   \
    case 128: { constexpr int DD = 128; CALL; } break; \
    default: { constexpr int DD = 256; CALL; } break;  \
  }

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return INTFA_OK;
}

int quant_pertoken(const void* x, const int64_t* st, void* x8, float* scale, int B, int H, int N, int D,
                   cudaStream_t stream) {
  const long long rows = (long long)B * H * N;
  const int sms = sm_count_cached();
  if (sms <= 0) return set_error(INTFA_ERR_CUDA, "cannot query SM count");
  const int rpw = 32 / (D / 8) * kQuantUnroll;
  long long want = (rows + 8LL * rpw - 1) / (8LL * rpw);          // CTAs of 8 warps, one row group each
  const int grid = (int)(want < (long long)sms * 8 ? (want < 1 ? 1 : want) : (long long)sms * 8);
  if (rows >= (1LL << 31)) return set_error(INTFA_ERR_TOO_LARGE, "quant_pertoken: B*H*N must be below 2^31");
  const bool contig = st[2] == D && st[1] == (int64_t)N * D && st[0] == (int64_t)H * N * D;
#define INTFA_QPT(CC) \
  quant_pertoken_kernel<DD, CC><<<grid, 256, 0, stream>>>((const __half*)x, st[0], st[1], st[2], (int8_t*)x8, scale, H, N, rows)
  INTFA_D_SWITCH(D, if (contig) INTFA_QPT(true); else INTFA_QPT(false))
#undef INTFA_QPT
  return check_launch("quant_pertoken");
}

static int v_grid(int BH, int N, int sms, int* rows_per_cta) {
  // chunks per (batch, head): enough CTAs to fill the machine a few times over, at least 256 rows each
  int chunks = (sms * 8 + BH - 1) / BH;
  const int max_chunks = (N + 255) / 256;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  *rows_per_cta = (N + chunks - 1) / chunks;
  return chunks;
}

int v_colmax(const void* v, const int64_t* st, void* colmax, int B, int H, int N, int D, cudaStream_t stream) {
  const int sms = sm_count_cached();
  if (sms <= 0) return set_error(INTFA_ERR_CUDA, "cannot query SM count");
  int rows_per_cta;
  dim3 grid(v_grid(B * H, N, sms, &rows_per_cta), B * H);
  INTFA_D_SWITCH(D, (v_colmax_kernel<DD><<<grid, 256, 0, stream>>>((const __half*)v, st[0], st[1], st[2], (unsigned int*)colmax, H, N, rows_per_cta)))
  return check_launch("v_colmax");
}

static int v_quant_launch(const void* v, const int64_t* st, const void* colmax, int nparts, void* v8, float* scale, int mode,
                          int B, int H, int N, int D, cudaStream_t stream) {
  const int sms = sm_count_cached();
  if (sms <= 0) return set_error(INTFA_ERR_CUDA, "cannot query SM count");
  int rows_per_cta;
  dim3 grid(v_grid(B * H, N, sms, &rows_per_cta), B * H);
  const int pc = mode == INTFA_VSCALE_PER_CHANNEL;
  INTFA_D_SWITCH(D, (v_quant_kernel<DD><<<grid, 256, 0, stream>>>((const __half*)v, st[0], st[1], st[2], (const unsigned int*)colmax, (int8_t*)v8, scale, pc, H, N, rows_per_cta, nparts)))
  return check_launch("v_quant");
}

int v_quant_from_colmax(const void* v, const int64_t* st, const void* colmax, void* v8, float* scale, int mode, int B,
                        int H, int N, int D, cudaStream_t stream) {
  return v_quant_launch(v, st, colmax, 1, v8, scale, mode, B, H, N, D, stream);
}

// ---------------------------------------------------------------------------------------------
// fused prologue: Q, K (per token) and V (per channel / per batch-head) in TWO launches, no memset
// ---------------------------------------------------------------------------------------------
size_t quant_qkv_workspace_bytes(int B, int Hkv, int Nk, int D) {
  const int sms = sm_count_cached();
  int rows_per_cta;
  const int chunks = v_grid(B * Hkv, Nk, sms > 0 ? sms : 148, &rows_per_cta);
  return (size_t)chunks * B * Hkv * D * sizeof(unsigned int);
}

int quant_qkv(const void* q, const void* k, const void* v, const int64_t* v_st, void* q8, void* k8, void* v8, float* qs,
              float* ks, float* vs, int mode, int B, int H, int Hkv, int Nq, int Nk, int D, void* workspace,
              cudaStream_t stream) {
  const int sms = sm_count_cached();
  if (sms <= 0) return set_error(INTFA_ERR_CUDA, "cannot query SM count");
  QkvJob j;
  j.q = (const __half*)q; j.q8 = (int8_t*)q8; j.qs = qs; j.q_rows = (long long)B * H * Nq;
  j.k = (const __half*)k; j.k8 = (int8_t*)k8; j.ks = ks; j.k_rows = (long long)B * Hkv * Nk;
  if (j.q_rows >= (1LL << 31) || j.k_rows >= (1LL << 31)) return set_error(INTFA_ERR_TOO_LARGE, "quant_qkv: B*H*N must be below 2^31");
  const int rpw = 32 / (D / 8) * kQuantUnroll;
  auto ctas = [&](long long rows) {
    const long long want = (rows + 8LL * rpw - 1) / (8LL * rpw);
    const long long cap = (long long)sms * 8;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
  };
  j.gq = ctas(j.q_rows);
  j.gk = ctas(j.k_rows);
  j.v = (const __half*)v; j.partial = (unsigned int*)workspace; j.Hkv = Hkv; j.Nk = Nk; j.BHkv = B * Hkv;
  j.chunks = 0; j.rows_per_cta = 0; j.vB = j.vH = j.vN = 0;
  int gv = 0;
  if (v) {
    j.vB = v_st[0]; j.vH = v_st[1]; j.vN = v_st[2];
    j.chunks = v_grid(B * Hkv, Nk, sms, &j.rows_per_cta);
    gv = j.chunks * B * Hkv;
  }
  const int grid = j.gq + j.gk + gv;
  INTFA_D_SWITCH(D, (quant_qkv_kernel<DD><<<grid, 256, 0, stream>>>(j)))
  int rc = check_launch("quant_qkv");
  if (rc || !v) return rc;
  return v_quant_launch(v, v_st, workspace, j.chunks, v8, vs, mode, B, Hkv, Nk, D, stream);
}

int quant_v(const void* v, const int64_t* st, void* v8, float* scale, int mode, int B, int H, int N, int D,
            void* workspace, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(workspace, 0, (size_t)B * H * D * sizeof(unsigned int), stream);
  if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  int rc = v_colmax(v, st, workspace, B, H, N, D, stream);
  if (rc) return rc;
  return v_quant_from_colmax(v, st, workspace, v8, scale, mode, B, H, N, D, stream);
}

// ---------------------------------------------------------------------------------------------
// V quantisation for callers that must not allocate (intfa_quant_v_static)
// ---------------------------------------------------------------------------------------------
// Column-absmax scratch that lives in the library image instead of in a caller-provided buffer.
// Every GPU that loads the library keeps these kStaticColmaxWords*4 bytes until the process exits.
// In host code `g_static_colmax` is only a handle for the symbol, not a device address, so the
// address is looked up once per device with cudaGetSymbolAddress and that pointer is what the
// kernels are given.
__device__ __align__(256) static unsigned int g_static_colmax[kStaticColmaxWords];

static unsigned int* static_colmax_ptr(int* rc) {
  static std::atomic<unsigned int*> ptr[64];     // host threads may race to be first: each stores the same address
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = set_error(INTFA_ERR_CUDA, "cannot query the current device");
    return nullptr;
  }
  unsigned int* q = ptr[dev].load(std::memory_order_acquire);
  if (!q) {
    void* sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_static_colmax);     // with device `dev` current
    if (e != cudaSuccess || sym == nullptr) {
      *rc = set_error(INTFA_ERR_CUDA, "cudaGetSymbolAddress(static colmax scratch): %s", cudaGetErrorString(e));
      return nullptr;
    }
    q = static_cast<unsigned int*>(sym);
    ptr[dev].store(q, std::memory_order_release);
  }
  *rc = INTFA_OK;
  return q;
}

int quant_v_static(const void* v, const int64_t* st, void* v8, float* scale, int mode, int B, int H, int N, int D,
                   cudaStream_t stream) {
  const long long words = (long long)B * H * D;
  if (words > kStaticColmaxWords)
    return set_error(INTFA_ERR_TOO_LARGE, "B*H*D = %lld exceeds the built-in scratch of %d words; use intfa_quant_v",
                     words, kStaticColmaxWords);
  int rc;
  unsigned int* scratch = static_colmax_ptr(&rc);
  if (!scratch) return rc;
  // the scratch keeps the previous call's maxima: clear the part this call uses
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)words * sizeof(unsigned int), stream);
  if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  rc = v_colmax(v, st, scratch, B, H, N, D, stream);
  if (rc) return rc;
  return v_quant_from_colmax(v, st, scratch, v8, scale, mode, B, H, N, D, stream);
}

int scales_f16_to_f32(const void* src, float* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return INTFA_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 4096) blocks = 4096;
  scales_f16_to_f32_kernel<<<(int)blocks, 256, 0, stream>>>((const __half*)src, dst, n);
  return check_launch("scales_f16_to_f32");
}

}  // namespace intfa
