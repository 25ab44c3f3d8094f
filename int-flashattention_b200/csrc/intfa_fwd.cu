// INT8 FlashAttention forward for sm_100a.
//
// Every kernel here gives one CTA one 128-row query tile at a time (work items = (batch*head, query block),
// drawn from a global counter) and walks the KV sequence ASCENDING in tiles of G columns -- G is also the
// granularity at which the running row maximum is updated, which the full-int8 result depends on (the
// reference's BLOCK_N, flash_atten_full_int8.py:30-70).
//
// One kernel family, intfa_fwd_pipe_kernel (intfa_fwd_pipe.cuh), serves full-int8 and half-int8 at head dims
// 16 to 256: one CTA of 512 threads per SM -- TMA producer, two MMA-issuing warps (S = Q K^T with tcgen05.mma
// kind::i8 into int32 TMEM accumulators; O_j = P V with kind::i8, or kind::f16 for half-int8), two softmax groups
// on alternate KV steps, accumulator warps.
//
// Arithmetic contract (what the parity tests pin; reference lines in parentheses):
//   s   = (fp32(S32) * s_q[row]) * s_k[col]                 (flash_atten_full_int8.py:36-38)
//   m'  = max(m, rowmax(s) * c),  x = s*c - m'   (fma)      (:45-46)   c = sm_scale*1.44269504 (:157)
//   on the causal diagonal band:  x0 = s*c + (col<=row ? 0 : -1e6), m' = max(m,rowmax(x0)) (:40-43)
//   p   = exp2(x), l_j = sum p (unquantised), alpha = exp2(m - m')     (:47-48,53-54)
//   full: p8 = trunc(fp16(fp16(fp16(p)*127) + 0.5))          (:49-51)
//         acc = acc*alpha + fp32(P8 V8) * (s_v[ch]/127)      (:56-62)   [evaluated as (s_v/127) * A with A = A*alpha + fp32(P8 V8)]
//   half: acc = acc*alpha + fp16(p) V16 (fp32 accumulate)    (flash_atten_int8.py:54-59)
//   m carried across the off-band/on-band boundary           (flash_atten_int8.py:66,157,166)
//   o   = fp16(acc / l)                                      (:181-182)
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <cstdlib>

#include "intfa_internal.h"
#include "intfa_ptx.cuh"

namespace intfa {

constexpr int kBM = 128;          // query rows per work item

// The int32 accumulators in TMEM are pre-loaded with the bit pattern of the fp32 number 1.5*2^23.
// The tensor core then leaves kMagicI + dot there, which READ AS FP32 is 1.5*2^23 + dot exactly
// (|dot| <= 128*128*128 < 2^22), so one fp32 subtraction replaces an int->float conversion.
constexpr uint32_t kMagicI = 0x4B400000u;
constexpr float kMagicF = 12582912.0f;

// two output values as one 32-bit word: fp16 (the Triton ops' output type) or bf16 (the CUDA path's other one)
__device__ __forceinline__ uint32_t pack_out(float x, float y, int bf16) {
  if (bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(x, y);
  return *reinterpret_cast<const uint32_t*>(&h);
}

struct TileInfo {
  int bh, b, h, hk, mb, work, nsteps;   // hk: the K/V head this query head reads (grouped-query attention)
  int vh;                               // which D-wide slice of the V / output channels this pass covers (head dim 256: 0, 1)
};

template <bool RAGGED = false, int NVH = 1>
__device__ __forceinline__ TileInfo decode_tile(const KParams& p, int tile, int G) {
  TileInfo t;
  t.vh = 0;
  if constexpr (NVH > 1) {
    t.vh = tile % NVH;
    tile /= NVH;
  }
  t.bh = tile / p.MB;
  const int i = tile - t.bh * p.MB;
  t.mb = p.causal ? (p.MB - 1 - i) : i;       // causal: long rows first
  t.b = t.bh / p.H;
  t.h = t.bh - t.b * p.H;
  t.hk = t.h / p.hk_ratio;
  t.work = t.bh * p.MB + t.mb;
  int n = p.Nk / G;
  if constexpr (RAGGED) n = (p.Nk + G - 1) / G;  // the last KV step may be partial
  if (p.causal) {
    // last visible global column for the last row of the block
    const long long last_row = p.q_off + (long long)t.mb * kBM + (kBM - 1);
    const long long rel = last_row - p.kv_off;           // last visible local column
    long long nv = rel < 0 ? 0 : (rel / G + 1);
    if (nv < n) n = (int)nv;
  }
  t.nsteps = n;
  return t;
}

// KV tile visited at step j of a work item with n steps: ascending, or last tile first
__device__ __forceinline__ int kv_tile_of_step(const KParams& p, int j, int n) { return p.kv_desc ? n - 1 - j : j; }

// byte offset of 16-byte chunk `chunk` of row `row` inside a swizzled [rows][ROWB bytes] tile
template <int ROWB>
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
  constexpr int MASK = ROWB / 16 - 1;     // 7 for 128-byte rows, 3 for 64-byte rows
  const uint32_t a = row * ROWB + chunk * 16;
  return a ^ (((a >> 7) & MASK) << 4);
}

#include "intfa_fwd_pipe.cuh"

// ============================================================================
// host side
// ============================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn lookup_encode_fn() {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    return reinterpret_cast<EncodeTiledFn>(ptr);
  return nullptr;
}
static EncodeTiledFn get_encode_fn() {
  static const EncodeTiledFn fn = lookup_encode_fn();     // initialised once, also when threads race to be first
  return fn;
}

// Work-item counters of the launches in flight: a ring of words inside the library image (no allocation at launch
// time); each launch takes the next word and zeroes it on its stream.  A word comes round again after kTileCounters
// launches of the process (all devices and streams share the cursor): a launch that is still queued or running
// by then would have its counter zeroed under it, so at most kTileCounters launches may be in flight at a time.
// The per-device caches below are atomics: host threads may call into the library concurrently.
constexpr int kTileCounters = 4096;
__device__ static unsigned int g_tile_counters[kTileCounters];

static int next_tile_counter(unsigned int** out, cudaStream_t stream) {
  static std::atomic<unsigned int*> base[64];
  static std::atomic<unsigned int> next{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return set_error(INTFA_ERR_CUDA, "cannot query the current device");
  unsigned int* b = base[dev].load(std::memory_order_acquire);
  if (!b) {
    void* sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_tile_counters);
    if (e != cudaSuccess || !sym) return set_error(INTFA_ERR_CUDA, "cudaGetSymbolAddress(tile counters): %s", cudaGetErrorString(e));
    b = static_cast<unsigned int*>(sym);
    base[dev].store(b, std::memory_order_release);       // every thread computes the same address
  }
  unsigned int* c = b + (next.fetch_add(1) % kTileCounters);
  cudaError_t e = cudaMemsetAsync(c, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "cudaMemsetAsync(tile counter): %s", cudaGetErrorString(e));
  *out = c;
  return INTFA_OK;
}

// [B,H,N,D] tensor, element strides for (B,H,N); box = (box_d, box_rows, 1, 1)
static int make_tmap(CUtensorMap* tm, const void* base, int esize, const int64_t* stride, int B, int H, int N, int D,
                     int box_d, int box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(INTFA_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)(stride[2] * esize), (cuuint64_t)(stride[1] * esize),
                           (cuuint64_t)(stride[0] * esize)};
  cuuint32_t box[4] = {(cuuint32_t)box_d, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(INTFA_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
  return INTFA_OK;
}

static inline int kv_heads(const IntfaFwdParams* a) { return a->H_kv > 0 ? a->H_kv : a->H; }

static constexpr CUtensorMapSwizzle swizzle_of_row_bytes(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

// One CTA per SM.  The tensor maps describe the tensors with their own head dim (a->D); the boxes are as wide as the
// kernel's tiles, so at head dim 16 the upper half of every 32-wide box lies outside the tensor and arrives as zeros.
template <int D, int G, bool FULL, bool PRNE, bool RAGGED, int DQ = D, bool F8V = false>
static int launch_pipe(const IntfaFwdParams* a, const KParams& kp, cudaStream_t stream) {
  using C = PipeCfg<D, G, FULL, DQ, F8V>;
  static_assert(C::SMEM_BYTES <= 227 * 1024, "shared memory");
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapSwizzle swzQK = swizzle_of_row_bytes(C::QK_ROWB), swzV = swizzle_of_row_bytes(C::V_ROWB);
  const int hd = a->D;
  int rc;
  if ((rc = make_tmap(&tmQ, a->q, 1, a->q_stride, a->B, a->H, a->Nq, hd, C::QK_ROWB, kBM, swzQK))) return rc;
  if ((rc = make_tmap(&tmK, a->k, 1, a->k_stride, a->B, kv_heads(a), a->Nk, hd, C::QK_ROWB, G, swzQK))) return rc;
  if constexpr (C::BYTE_PV) {
    if ((rc = make_tmap(&tmV, a->v, 1, a->v_stride, a->B, kv_heads(a), a->Nk, hd, D, G, swzV))) return rc;
  } else {
    if ((rc = make_tmap(&tmV, a->v, 2, a->v_stride, a->B, kv_heads(a), a->Nk, hd, D >= 64 ? 64 : D, G, swzV))) return rc;
  }
  auto kern = intfa_fwd_pipe_kernel<D, G, FULL, PRNE, RAGGED, DQ, F8V>;
  static std::atomic<bool> attr_done[64];     // per instantiation and device (the attribute is per device)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return set_error(INTFA_ERR_CUDA, "cannot query the current device");
  if (!attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev].store(true, std::memory_order_release);
  }
  const int sms = sm_count_cached();
  if (sms <= 0) return set_error(INTFA_ERR_CUDA, "cannot query SM count");
  int grid = sms;
  if (grid > kp.num_tiles) grid = kp.num_tiles;
  KParams kpl = kp;
  if ((rc = next_tile_counter(&kpl.tile_counter, stream))) return rc;
  kern<<<grid, kPipeThreads, C::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, kpl);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return INTFA_OK;
}

int fwd_dispatch(const IntfaFwdParams* a, cudaStream_t stream) {
  KParams kp;
  kp.qs = a->q_scale; kp.ks = a->k_scale; kp.vs = a->v_scale;
  kp.o = reinterpret_cast<__half*>(a->o);
  kp.o_sb = a->o_stride[0]; kp.o_sh = a->o_stride[1]; kp.o_sn = a->o_stride[2];
  kp.qs_sb = a->qs_stride[0]; kp.qs_sh = a->qs_stride[1];
  kp.ks_sb = a->ks_stride[0]; kp.ks_sh = a->ks_stride[1];
  kp.vs_sb = a->vs_stride[0]; kp.vs_sh = a->vs_stride[1]; kp.vs_sd = a->vs_stride[2];
  kp.B = a->B; kp.H = a->H; kp.Nq = a->Nq; kp.Nk = a->Nk;
  kp.dh = a->D;
  kp.hk_ratio = a->H / kv_heads(a);
  kp.o_bf16 = a->o_dtype == INTFA_OUT_BF16 ? 1 : 0;
  kp.causal = a->causal ? 1 : 0;
  kp.c = a->sm_scale * 1.44269504f;          // fp32 product, flash_atten_full_int8.py:156-157
  kp.q_off = a->q_offset; kp.kv_off = a->kv_offset;
  kp.lse = a->lse_out; kp.st_m = a->state_m; kp.st_l = a->state_l; kp.st_acc = a->state_acc;
  kp.state_in = a->state_in; kp.state_out = a->state_out; kp.write_o = a->write_o;
  kp.dbg_s = a->dbg_s; kp.dbg_p = a->dbg_p; kp.dbg_tile = a->dbg_tile; kp.dbg_step = a->dbg_step;
  kp.status = a->status;
  kp.wait_limit_kcycles = a->debug_wait_limit_kcycles > 0 ? a->debug_wait_limit_kcycles : (1 << 21);   // default: 2^31 cycles, about a second
  kp.skip_k_load = a->debug_skip_k_load;
  kp.kv_desc = a->kv_order ? 1 : 0;
  kp.vs_sblk = a->vs_stride_blk;
  kp.MB = (a->Nq + kBM - 1) / kBM;            // the last query tile may be partial (pipelined kernel only)
  kp.num_tiles = (int)((long long)a->B * a->H * kp.MB);   // fits: intfa_fwd() has checked it
  const bool full = a->variant == INTFA_VARIANT_FULL;
  const bool f8v = a->variant == INTFA_VARIANT_HALF_FP8;
  const bool rne = full && a->p_round == 1;
  const int D = a->D, G = a->G;
  // Sequence lengths that are not multiples of the tile sizes run the instantiation that masks the last tiles
  // (so do calls with one v_scale row per KV tile: the code for them is compiled into that instantiation only)
  const bool ragged = (a->Nq % kBM) != 0 || (a->Nk % a->G) != 0 || a->vs_stride_blk != 0;
  // HD: head dim of the call; DD, DQ: the kernel's tile width and Q/K width for it; HALF: half-int8 built for this G
#define INTFA_CASE(HD, DD, GG, DQ, HALF)                                                                 \
  if (D == HD && G == GG) {                                                                              \
    if (full && ragged) return rne ? launch_pipe<DD, GG, true, true, true, DQ>(a, kp, stream)            \
                                   : launch_pipe<DD, GG, true, false, true, DQ>(a, kp, stream);          \
    if (full) return rne ? launch_pipe<DD, GG, true, true, false, DQ>(a, kp, stream)                     \
                         : launch_pipe<DD, GG, true, false, false, DQ>(a, kp, stream);                   \
    if constexpr (HALF) {                                                                                \
      if (f8v) return ragged ? launch_pipe<DD, GG, false, false, true, DQ, true>(a, kp, stream)          \
                             : launch_pipe<DD, GG, false, false, false, DQ, true>(a, kp, stream);        \
      return ragged ? launch_pipe<DD, GG, false, false, true, DQ>(a, kp, stream)                         \
                    : launch_pipe<DD, GG, false, false, false, DQ>(a, kp, stream);                       \
    }                                                                                                    \
  }
  INTFA_CASE(128, 128, 128, 128, true)
  INTFA_CASE(128, 128, 64, 128, true)
  INTFA_CASE(64, 64, 64, 64, true)
  INTFA_CASE(64, 64, 128, 64, true)
  INTFA_CASE(32, 32, 32, 32, false)      // G = 32: full-int8 only (fp16 P tiles need 64 columns)
  INTFA_CASE(32, 32, 64, 32, true)
  INTFA_CASE(32, 32, 128, 32, true)
  INTFA_CASE(16, 32, 32, 32, false)      // head dim 16: the 32-wide kernel on zero-filled tiles
  INTFA_CASE(16, 32, 64, 32, true)
  INTFA_CASE(16, 32, 128, 32, true)
  INTFA_CASE(256, 128, 128, 256, false)  // head dim 256: two passes of 128 V channels; fp16 V tiles at G = 128 do not fit
  INTFA_CASE(256, 128, 64, 256, true)
#undef INTFA_CASE
  return set_error(INTFA_ERR_UNSUPPORTED, "unsupported (D=%d, G=%d, %s): G is 64 or 128 (32 too for full-int8 at head dims 16 and 32; half-int8 at head dim 256: 64 only)", D, G, full ? "full-int8" : "half-int8");
}

}  // namespace intfa
