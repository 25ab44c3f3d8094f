// INT8 FlashAttention forward for sm_100a.
//
// Every kernel here gives one CTA one 128-row query tile at a time (work items = (batch*head, query block),
// drawn from a global counter) and walks the KV sequence ASCENDING in tiles of G columns -- G is also the
// granularity at which the running row maximum is updated, which the full-int8 result depends on (the
// reference's BLOCK_N, flash_atten_full_int8.py:30-70).
//
// Two kernels share the helpers, the work-item decoding and the arithmetic contract below:
//   intfa_fwd_pipe_kernel (intfa_fwd_pipe.cuh)  full-int8, and half-int8 at head_dim 128: one CTA of 640
//               threads per SM, two softmax groups on alternate KV steps, separate accumulator warps,
//               double-buffered S in TMEM
//   intfa_fwd_kernel (this file)                half-int8 at head_dim 64 (and everything on request): two
//               CTAs of 384 threads per SM:
//     warp 0      TMA producer: Q tile once per work item; K tile, V tile and the K-scale slice through
//                 an NS-stage shared-memory ring (cp.async.bulk.tensor, no multicast)
//     warp 1      MMA issuer (one thread): S = Q K^T with tcgen05.mma kind::i8 into an int32 TMEM
//                 accumulator; O_j = P V with kind::i8 (full) or kind::f16 (half)
//     warp 2      TMEM allocator; warp 3 watcher (polls the tensor core's mbarriers, releases the
//                 softmax warps through named barriers)
//     warps 4-11  softmax/correction/epilogue, two threads per query row: TMEM -> registers,
//                 dequantise with s_q[row]*s_k[col], online softmax, P -> int8 (or fp16) into
//                 swizzled shared memory for the second MMA, then acc = acc*alpha + O_j*s_v/127
//                 with the fp32 accumulator row in TMEM (the int32 PV tile cannot absorb the fp32
//                 rescale, so PV never accumulates across KV tiles as int32).
//
// Arithmetic contract (what the parity tests pin; reference lines in parentheses):
//   s   = (fp32(S32) * s_q[row]) * s_k[col]                 (flash_atten_full_int8.py:36-38)
//   m'  = max(m, rowmax(s) * c),  x = s*c - m'   (fma)      (:45-46)   c = sm_scale*1.44269504 (:157)
//   on the causal diagonal band:  x0 = s*c + (col<=row ? 0 : -1e6), m' = max(m,rowmax(x0)) (:40-43)
//   p   = exp2(x), l_j = sum p (unquantised), alpha = exp2(m - m')     (:47-48,53-54)
//   full: p8 = trunc(fp16(fp16(fp16(p)*127) + 0.5))          (:49-51)
//         acc = acc*alpha + fp32(P8 V8) * (s_v[ch]/127)      (:56-62)
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
constexpr int kThreads = 384;          // 4 service warps + 8 softmax warps
constexpr int kComputeThreads = 256;
#ifndef INTFA_SLEEP_P
#define INTFA_SLEEP_P 200
#define INTFA_SLEEP_W 40
#define INTFA_SLEEP_M 20
#endif
constexpr int kSleepProducer = INTFA_SLEEP_P, kSleepWatcher = INTFA_SLEEP_W, kSleepMma = INTFA_SLEEP_M;   // ns between polls
constexpr int kBarS = 6, kBarO = 7;   // named barriers the watcher warp releases the softmax warps on
constexpr int kServiceRegs = 40, kComputeRegs = 96;   // setmaxnreg split of the 80 registers/thread at launch

// The int32 accumulators in TMEM are pre-loaded with the bit pattern of the fp32 number 1.5*2^23.
// The tensor core then leaves kMagicI + dot there, which READ AS FP32 is 1.5*2^23 + dot exactly
// (|dot| <= 128*128*128 < 2^22), so one fp32 subtraction replaces an int->float conversion.
constexpr uint32_t kMagicI = 0x4B400000u;
constexpr float kMagicF = 12582912.0f;

// device-side wait codes stored in *status (low byte = which wait, bits 8.. = blockIdx)
enum WaitCode {
  W_Q_EMPTY = 1, W_K_EMPTY, W_V_EMPTY, W_Q_FULL, W_K_FULL, W_V_FULL, W_P_FULL, W_O_EMPTY,
  W_S_FULL, W_O_FULL, W_KS_FULL, W_TILE
};

template <int D, int G, bool FULL>
struct Cfg {
  static constexpr int Q_BYTES = kBM * D;
  static constexpr int K_BYTES = G * D;
  static constexpr int V_BYTES = FULL ? G * D : G * D * 2;
  static constexpr int P_BYTES = FULL ? kBM * G : kBM * G * 2;
  static constexpr int KS_BYTES = G * 4;
  // stages: keep the CTA under ~104 KB so two CTAs share an SM where possible
  static constexpr int BUDGET = 104 * 1024;
  static constexpr int FIXED = Q_BYTES + P_BYTES + 6144;
  static constexpr int PER_STAGE = K_BYTES + V_BYTES + KS_BYTES;
  static constexpr int NS_RAW = (BUDGET - FIXED) / PER_STAGE;
  static constexpr int NS = NS_RAW < 2 ? 2 : (NS_RAW > 4 ? 4 : NS_RAW);
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NS * K_BYTES;
  static constexpr int OFF_P = OFF_V + NS * V_BYTES;
  static constexpr int OFF_KS = OFF_P + P_BYTES;
  static constexpr int OFF_VSD = OFF_KS + NS * KS_BYTES;
  static constexpr int OFF_XCH = OFF_VSD + D * 4;             // half-row maxima / sums exchange: 2 x [2][128] float2 + [2][128] float
  static constexpr int OFF_BAR = OFF_XCH + 5 * 256 * 4;
  static constexpr int NUM_BARS = 6 + 4 * NS + 8;              // + work-item ring: 4 x (published, consumed)
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 32 + 1024;   // misc: tmem slot, abort flag, 4 work-item slots; +1024: alignment slack
  // TMEM columns.  full: one int32 region shared by S = Q K^T (G columns) and O_j = P V (D columns) --
  // S is dead once P is written, O_j is dead once it is folded into the accumulator -- followed by the
  // fp32 accumulator (D columns).  half: S (G columns), then the fp32 accumulator the second MMA adds into.
  static constexpr int COL_S = 0;
  static constexpr int COL_O = 0;
  static constexpr int COL_ACC = FULL ? (G > D ? G : D) : G;
  static constexpr int TMEM_USED = COL_ACC + D;
  static constexpr int TMEM_COLS = TMEM_USED <= 128 ? 128 : 256;
  // swizzle span = bytes of one operand row
  static constexpr uint64_t SWZ_QK = (D == 128) ? kSwz128 : kSwz64;     // Q, K rows are D bytes
  static constexpr uint32_t SBO_QK = 8 * D;
  static constexpr uint64_t SWZ_P = FULL ? ((G == 128) ? kSwz128 : kSwz64) : kSwz128;
  static constexpr uint32_t SBO_P = FULL ? 8 * G : 1024;
  static constexpr uint64_t SWZ_V = FULL ? ((D == 128) ? kSwz128 : kSwz64) : kSwz128;
  static constexpr uint32_t SBO_V = FULL ? 8 * D : 1024;
  static constexpr uint32_t IDESC_QK = make_idesc(2, 1, 1, 0, 0, kBM, G);
  static constexpr uint32_t IDESC_PV = FULL ? make_idesc(2, 1, 1, 0, 1, kBM, D) : make_idesc(1, 0, 0, 0, 1, kBM, D);
};

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
};

template <bool RAGGED = false>
__device__ __forceinline__ TileInfo decode_tile(const KParams& p, int tile, int G) {
  TileInfo t;
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

// byte offset of 16-byte chunk `chunk` of row `row` inside a swizzled [rows][ROWB bytes] tile
template <int ROWB>
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
  constexpr int MASK = ROWB / 16 - 1;     // 7 for 128-byte rows, 3 for 64-byte rows
  const uint32_t a = row * ROWB + chunk * 16;
  return a ^ (((a >> 7) & MASK) << 4);
}

#ifdef INTFA_TRACE
// event trace of 16 consecutive KV steps of CTA 0: dbg_s[((role*16 + step)*8 + event)] = low bits of clock64
#define INTFA_TR(role, step, ev)                                                                              \
  if (p.dbg_s != nullptr && p.dbg_tile == -3 && blockIdx.x == 0 && lane == 0 && (int)(step) >= p.dbg_step &&   \
      (int)(step) < p.dbg_step + 16)                                                                           \
    p.dbg_s[(((role) * 16 + ((int)(step) - p.dbg_step)) * 8 + (ev))] = (int)(clock64() & 0x7fffffff);
#else
#define INTFA_TR(role, step, ev)
#endif
#ifdef INTFA_TIMING
#define INTFA_T0() tq = clock64()
#define INTFA_T(i) { const long long now_ = clock64(); tm[i] += now_ - tq; tq = now_; }
#define INTFA_TDECL() long long tm[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tq = 0
#define INTFA_TDUMP_SOFTMAX()                                                                        \
  if (lane == 0 && p.dbg_s != nullptr && p.dbg_tile == -2 && blockIdx.x < 400 && grp == 0) {         \
    for (int i = 0; i < 6; ++i) p.dbg_s[(blockIdx.x * 4 + quarter) * 8 + i] = (int)(tm[i] >> 4);     \
  }
#define INTFA_TDUMP_MMA()                                                                            \
  if (lane == 0 && p.dbg_s != nullptr && p.dbg_tile == -2 && blockIdx.x < 400) {                     \
    for (int i = 0; i < 8; ++i) if (tm[i]) p.dbg_s[12800 + blockIdx.x * 8 + i] = (int)(tm[i] >> 4);  \
  }
#define INTFA_TDUMP_UPDATE()                                                                         \
  if (lane == 0 && p.dbg_s != nullptr && p.dbg_tile == -2 && blockIdx.x < 400) {                     \
    for (int i = 6; i < 8; ++i) p.dbg_s[(blockIdx.x * 4 + quarter) * 8 + i] = (int)(tm[i] >> 4);     \
  }
#else
#define INTFA_T0()
#define INTFA_T(i)
#define INTFA_TDECL()
#define INTFA_TDUMP_SOFTMAX()
#define INTFA_TDUMP_MMA()
#define INTFA_TDUMP_UPDATE()
#endif

template <int D, int G, bool FULL, bool PRNE>
__global__ void __launch_bounds__(kThreads, 2)
intfa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const KParams p) {
  using C = Cfg<D, G, FULL>;
  constexpr int NS = C::NS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // barrier indices.  B_RFREE: full = the shared S/O region is consumed and re-armed (once per KV step);
  // half = the accumulator has been read out by the epilogue (once per work item).
  // B_OFULL: full = O_j ready (once per KV step); half = last PV of the work item done (once per work item).
  constexpr int B_QFULL = 0, B_QEMPTY = 1, B_SFULL = 2, B_PFULL = 3, B_OFULL = 4, B_RFREE = 5;
  constexpr int B_KFULL = 6, B_KEMPTY = 6 + NS, B_VFULL = 6 + 2 * NS, B_VEMPTY = 6 + 3 * NS;
  constexpr int B_TILE = 6 + 4 * NS;       // work item published in ring slot i (see next_tile)
  constexpr int B_TDONE = B_TILE + 4;      // ... and read by the MMA thread, the watcher and all 8 softmax warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 4);
  volatile int* tile_slot = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 16);

  if (threadIdx.x == 0) {
    mbar_init(BAR(B_QFULL), 1);
    mbar_init(BAR(B_QEMPTY), 1);
    mbar_init(BAR(B_SFULL), 1);
    mbar_init(BAR(B_PFULL), 8);
    mbar_init(BAR(B_OFULL), 1);
    mbar_init(BAR(B_RFREE), 8);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR(B_KFULL + s), 1);
      mbar_init(BAR(B_KEMPTY + s), 1);
      mbar_init(BAR(B_VFULL + s), 1);
      mbar_init(BAR(B_VEMPTY + s), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(BAR(B_TILE + i), 1);
      mbar_init(BAR(B_TDONE + i), 10);
    }
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base + C::COL_S;
  const uint32_t tO = tmem_base + C::COL_O;
  const uint32_t tA = tmem_base + C::COL_ACC;
  const int code_hi = (int)(blockIdx.x << 8);

  // Work items are handed out dynamically: the producer thread draws the next index from a global
  // counter and publishes it in a 4-slot shared-memory ring; every other role reads the same
  // sequence.  (The two CTAs sharing an SM do not run at the same speed, so a static split leaves
  // one of them working alone at the end.)  The producer is never more than two items ahead of the
  // slowest role.  Each reader (MMA thread, watcher, one lane per softmax warp: 10 arrivals) acknowledges
  // a slot once it has read it; the producer waits for those before reusing the slot.  A negative index
  // ends the sequence.
  auto next_tile = [&](uint32_t& seq, bool ack, bool whole_warp) -> int {
    const uint32_t slot = seq & 3u, par = (seq >> 2) & 1u;
    ++seq;
    if (!mbar_wait(BAR(B_TILE + slot), par, abort_flag, p.status, code_hi | W_TILE)) return -1;
    const int t = tile_slot[slot];
    if (whole_warp) __syncwarp();       // every lane has read the slot before lane 0 acknowledges it
    if (ack) mbar_arrive(BAR(B_TDONE + slot));
    return t;
  };

  const uint32_t sQ = smem_u32(smem + C::OFF_Q);
  const uint32_t sK = smem_u32(smem + C::OFF_K);
  const uint32_t sV = smem_u32(smem + C::OFF_V);
  const uint32_t sP = smem_u32(smem + C::OFF_P);
  const uint32_t sKS = smem_u32(smem + C::OFF_KS);

  // arm the int32 region for the first Q K^T (see kMagicI): each softmax thread fills its own TMEM lane
  if (warp >= 4 && warp < 8) {
    const uint32_t lane_sel0 = (uint32_t)((warp & 3) * 32) << 16;
#pragma unroll
    for (int cc = 0; cc < G / 32; ++cc) tmem_fill32(tS + lane_sel0 + cc * 32, kMagicI);
    tmem_st_wait();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();

  if (warp < 4) {
    reg_dealloc<kServiceRegs>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      uint32_t kv_it = 0, tile_it = 0;
      bool ok = true;
      uint32_t tseq = 0;
      while (ok) {
        if (tseq >= 4u) {       // slot reuse: everyone has read the item published four draws ago
          ok = mbar_wait(BAR(B_TDONE + (tseq & 3u)), ((tseq >> 2) - 1u) & 1u, abort_flag, p.status, code_hi | W_TILE);
          if (!ok) break;
        }
        int tile = (int)atomicAdd(p.tile_counter, 1u);
        if (tile >= p.num_tiles) tile = -1;
        tile_slot[tseq & 3u] = tile;
        mbar_arrive(BAR(B_TILE + (tseq & 3u)));        // release: the slot is visible to the waiters
        ++tseq;
        if (tile < 0) break;
        const TileInfo t = decode_tile(p, tile, G);
        if (t.nsteps == 0) continue;
        ok = mbar_wait<kSleepProducer>(BAR(B_QEMPTY), (tile_it & 1) ^ 1, abort_flag, p.status, code_hi | W_Q_EMPTY);
        if (!ok) break;
        mbar_expect_tx(BAR(B_QFULL), C::Q_BYTES);
        tma_load_4d(sQ, &tmQ, BAR(B_QFULL), 0, t.mb * kBM, t.h, t.b);
        const float* ks_row = p.ks + (long long)t.b * p.ks_sb + (long long)t.hk * p.ks_sh;
        for (int j = 0; j < t.nsteps; ++j, ++kv_it) {
          const uint32_t s = kv_it % NS, ph = (kv_it / NS) & 1;
          ok = mbar_wait<kSleepProducer>(BAR(B_KEMPTY + s), ph ^ 1, abort_flag, p.status, code_hi | W_K_EMPTY);
          if (!ok) break;
          mbar_expect_tx(BAR(B_KFULL + s), C::K_BYTES);
          tma_load_4d(sK + s * C::K_BYTES, &tmK, BAR(B_KFULL + s), 0, j * G, t.hk, t.b);
          ok = mbar_wait<kSleepProducer>(BAR(B_VEMPTY + s), ph ^ 1, abort_flag, p.status, code_hi | W_V_EMPTY);
          if (!ok) break;
          mbar_expect_tx(BAR(B_VFULL + s), C::V_BYTES + C::KS_BYTES);
          if constexpr (FULL) {
            tma_load_4d(sV + s * C::V_BYTES, &tmV, BAR(B_VFULL + s), 0, j * G, t.hk, t.b);
          } else {
#pragma unroll
            for (int c = 0; c < D / 64; ++c)
              tma_load_4d(sV + s * C::V_BYTES + c * (G * 128), &tmV, BAR(B_VFULL + s), c * 64, j * G, t.hk, t.b);
          }
          bulk_load_1d(sKS + s * C::KS_BYTES, ks_row + j * G, C::KS_BYTES, BAR(B_VFULL + s));
        }
        ++tile_it;
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      uint32_t kv_it = 0;      // KV steps issued so far (all work items)
      uint32_t tile_it = 0;    // work items with at least one KV step
      bool ok = true;
      auto issue_qk = [&](uint32_t it) -> bool {
        const uint32_t s = it % NS, ph = (it / NS) & 1;
        if (!mbar_wait(BAR(B_KFULL + s), ph, abort_flag, p.status, code_hi | W_K_FULL)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk) {
          const uint64_t ad = make_smem_desc(sQ + kk * 32, 16, C::SBO_QK, C::SWZ_QK);
          const uint64_t bd = make_smem_desc(sK + s * C::K_BYTES + kk * 32, 16, C::SBO_QK, C::SWZ_QK);
          umma_i8(tS, ad, bd, C::IDESC_QK, 1);      // onto the pre-loaded magic
        }
        umma_commit(BAR(B_SFULL));
        umma_commit(BAR(B_KEMPTY + s));
        return true;
      };
      uint32_t tseq = 0;
      while (ok) {
        const int tile = next_tile(tseq, true, false);
        if (tile < 0) break;
        const TileInfo t = decode_tile(p, tile, G);
        if (t.nsteps == 0) continue;
        ok = mbar_wait(BAR(B_QFULL), tile_it & 1, abort_flag, p.status, code_hi | W_Q_FULL);
        if (!ok) break;
        if constexpr (FULL) {
          for (int j = 0; j < t.nsteps; ++j, ++kv_it) {
            const uint32_t s = kv_it % NS, ph = (kv_it / NS) & 1;
            // the shared S/O region must have been folded into the accumulator and re-armed
            ok = mbar_wait<kSleepMma>(BAR(B_RFREE), (kv_it & 1) ^ 1, abort_flag, p.status, code_hi | W_O_EMPTY);
            if (!ok) break;
            ok = issue_qk(kv_it);
            if (!ok) break;
            if (j + 1 == t.nsteps) umma_commit(BAR(B_QEMPTY));
            ok = mbar_wait<kSleepMma>(BAR(B_PFULL), kv_it & 1, abort_flag, p.status, code_hi | W_P_FULL);
            if (!ok) break;
            ok = mbar_wait(BAR(B_VFULL + s), ph, abort_flag, p.status, code_hi | W_V_FULL);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < G / 32; ++kk) {
              const uint64_t ad = make_smem_desc(sP + kk * 32, 16, C::SBO_P, C::SWZ_P);
              const uint64_t bd = make_smem_desc(sV + s * C::V_BYTES + kk * (32 * D), 16, C::SBO_V, C::SWZ_V);
              umma_i8(tO, ad, bd, C::IDESC_PV, 1);      // onto the re-armed magic
            }
            umma_commit(BAR(B_OFULL));
            umma_commit(BAR(B_VEMPTY + s));
          }
        } else {
          // the previous work item's accumulator must have been read out before PV overwrites it
          ok = mbar_wait<kSleepMma>(BAR(B_RFREE), (tile_it & 1) ^ 1, abort_flag, p.status, code_hi | W_O_EMPTY);
          if (!ok) break;
          ok = issue_qk(kv_it);
          if (!ok) break;
          if (t.nsteps == 1) umma_commit(BAR(B_QEMPTY));
          for (int j = 0; j < t.nsteps; ++j, ++kv_it) {
            const uint32_t s = kv_it % NS, ph = (kv_it / NS) & 1;
            ok = mbar_wait<kSleepMma>(BAR(B_PFULL), kv_it & 1, abort_flag, p.status, code_hi | W_P_FULL);
            if (!ok) break;
            ok = mbar_wait(BAR(B_VFULL + s), ph, abort_flag, p.status, code_hi | W_V_FULL);
            if (!ok) break;
            tc_fence_after();
            const uint32_t keep = (j > 0 || p.state_in) ? 1u : 0u;     // first PV of a fresh work item overwrites
#pragma unroll
            for (int kk = 0; kk < G / 16; ++kk) {
              const uint64_t ad =
                  make_smem_desc(sP + (kk >> 2) * (kBM * 128) + (kk & 3) * 32, 16, C::SBO_P, C::SWZ_P);
              const uint64_t bd = make_smem_desc(sV + s * C::V_BYTES + kk * 2048, G * 128, C::SBO_V, C::SWZ_V);
              umma_f16(tA, ad, bd, C::IDESC_PV, kk > 0 ? 1u : keep);
            }
            umma_commit(BAR(B_VEMPTY + s));
            if (j + 1 < t.nsteps) {
              ok = issue_qk(kv_it + 1);
              if (!ok) break;
              if (j + 2 == t.nsteps) umma_commit(BAR(B_QEMPTY));
            } else {
              umma_commit(BAR(B_OFULL));
            }
          }
        }
        ++tile_it;
      }
    } else if (warp == 3) {
      // ------------------------------------------------------------------ watcher
      // Turns the tensor core's mbarrier completions into named-barrier releases: the eight softmax
      // warps block in bar.sync (no issue slots) instead of polling; this one warp polls for them.
      uint32_t kv_it = 0, tile_it = 0;
      bool ok = true;
      uint32_t tseq = 0;
      while (ok) {
        const int tile = next_tile(tseq, lane == 0, true);
        if (tile < 0) break;
        const TileInfo t = decode_tile(p, tile, G);
        if (t.nsteps == 0) continue;
        for (int j = 0; ok && j < t.nsteps; ++j, ++kv_it) {
          ok = mbar_wait<kSleepWatcher>(BAR(B_SFULL), kv_it & 1, abort_flag, p.status, code_hi | W_S_FULL);
          named_bar_arrive(kBarS, kComputeThreads + 32);
          if constexpr (FULL) {
            if (ok) ok = mbar_wait<kSleepWatcher>(BAR(B_OFULL), kv_it & 1, abort_flag, p.status, code_hi | W_O_FULL);
            named_bar_arrive(kBarO, kComputeThreads + 32);
          }
        }
        if constexpr (!FULL) {
          if (ok) ok = mbar_wait<kSleepWatcher>(BAR(B_OFULL), tile_it & 1, abort_flag, p.status, code_hi | W_O_FULL);
          named_bar_arrive(kBarO, kComputeThreads + 32);
        }
        ++tile_it;
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------------- softmax / correction / epilogue
    // Eight warps, TWO threads per query row: warps cw and cw+4 own the same 32 TMEM lanes (rows) and
    // split every row in halves -- `half` takes KV columns [half*G/2, ..) of S / P and output
    // channels [half*D/2, ..) of O_j and the accumulator.  Per KV step the two threads of a row
    // exchange one number (their partial row maximum) through shared memory; the row sum is kept
    // as two partial sums and joined in the epilogue.
    reg_alloc<kComputeRegs>();
    const int cw = warp - 4;                                 // 0..7
    const int quarter = cw & 3;                              // TMEM lane quarter this warp may access
    const int half = cw >> 2;
    const int row = quarter * 32 + lane;                     // row of the query tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    constexpr int GH = G / 2, DH = D / 2;                    // columns / channels per thread
    const int col0 = half * GH, ch0 = half * DH;
    float* vsd_s = reinterpret_cast<float*>(smem + C::OFF_VSD);
    float* xch_s = reinterpret_cast<float*>(smem + C::OFF_XCH);      // [2 parities][2 halves][128 rows] float2, then the epilogue's floats
    uint8_t* sP_gen = smem + C::OFF_P;
    const uint64_t NEG_MAGIC2 = f2_pack(-kMagicF, -kMagicF);
    const int pair_bar = 2 + quarter;                        // named barrier of the two warps sharing these rows
    uint32_t step_it = 0, tile_it = 0;
    bool ok = true;
#ifdef INTFA_TIMING
    long long tm[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tq;
    const long long life0 = clock64();
    unsigned long long gt0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt0));
#endif
    uint32_t tseq = 0;
    while (true) {
      const int tile = next_tile(tseq, lane == 0, true);
      if (tile < 0) break;
      const TileInfo t = decode_tile(p, tile, G);
      const long long rowg = (long long)t.bh * p.Nq + (long long)t.mb * kBM + row;   // row in [B*H*Nq)
      const long long grow = p.q_off + (long long)t.mb * kBM + row;                  // global position
      const float qs_r = p.qs[(long long)t.b * p.qs_sb + (long long)t.h * p.qs_sh + t.mb * kBM + row];
      // (magic + S)*s_q - magic*s_q is S*s_q exactly, so when magic*s_q is representable (always for a
      // scale that came from fp16) one fma yields the same rounded fp32(S)*s_q as subtract-then-multiply.
      // Warps holding a row where it is not take the general path below.
      const float mq = kMagicF * qs_r;
      const bool fold = __all_sync(0xffffffffu, fmaf(kMagicF, qs_r, -mq) == 0.0f);
      float m_i = -INFINITY;
      float l_i = 1.0f;                                      // full row sum, kept identical in both threads of the row
      float ls_pend = 0.f, alpha_pend = 1.f;                 // this thread's half-row sum of the latest KV step, not yet
      bool have_pend = false;                                // folded into l_i (it travels with the next exchange)
      // fp32 accumulator row lives in TMEM (columns COL_ACC..): start from zero or from the carried state.
      // (half-int8, fresh start: nothing to do -- the first P V of the work item overwrites it)
      if (p.state_in) {
        m_i = p.st_m[rowg];
        l_i = p.st_l[rowg];
#pragma unroll
        for (int cc = 0; cc < DH / 32; ++cc) {
          uint32_t r[32];
          const uint4* a4 = reinterpret_cast<const uint4*>(p.st_acc + rowg * D + ch0 + cc * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 v = a4[i];
            r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
          }
          tmem_st32(tA + lane_sel + ch0 + cc * 32, r);
        }
        tmem_st_wait();
      } else if (FULL || t.nsteps == 0) {
#pragma unroll
        for (int cc = 0; cc < DH / 32; ++cc) tmem_fill32(tA + lane_sel + ch0 + cc * 32, 0u);
        tmem_st_wait();
      }
      if constexpr (FULL) {
        named_bar_sync(1, kComputeThreads);       // previous work item done with vsd_s
        const int ch = threadIdx.x - 128;
        if (ch < D)
          vsd_s[ch] = p.vs[(long long)t.b * p.vs_sb + (long long)t.hk * p.vs_sh + (long long)ch * p.vs_sd] / 127.0f;
        named_bar_sync(1, kComputeThreads);
      }

      for (int j = 0; ok && j < t.nsteps; ++j, ++step_it) {
        const uint32_t s = step_it % NS, ph = (step_it / NS) & 1;
        const float* ks_s = reinterpret_cast<const float*>(smem + C::OFF_KS + s * C::KS_BYTES) + col0;
        INTFA_T0();
        ok = mbar_wait(BAR(B_VFULL + s), ph, abort_flag, p.status, code_hi | W_KS_FULL);
        if (!ok) break;
        INTFA_T(0);
        named_bar_sync(kBarS, kComputeThreads + 32);          // S = Q K^T is in TMEM (released by the watcher warp)
        ok = (*abort_flag == 0);
        if (!ok) break;
        tc_fence_after();
        INTFA_T(1);
        const long long gcol0 = p.kv_off + (long long)j * G;
        const bool masked = p.causal && (gcol0 + G - 1 > p.q_off + (long long)t.mb * kBM);
        const bool dbg_here = (p.dbg_s != nullptr) && t.work == p.dbg_tile && j == p.dbg_step;
        const float c = p.c;
        const uint32_t tSh = tS + lane_sel + col0;           // this thread's S columns

        // ---- pass A: TMEM holds kMagicI + S32, i.e. the fp32 number 1.5*2^23 + S32.  Subtracting the
        // magic gives fp32(S32) exactly; s = (fp32(S32)*s_q)*s_k goes back into the same TMEM columns
        // (on the causal band: x0 = s*c + bias) and the row maximum is taken on the way.  The chunk
        // loops are deliberately NOT unrolled: the whole KV step has to stay resident in the
        // instruction cache while the CTAs of an SM run different phases of it.
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
        for (int cc = 0; cc < GH / 32; ++cc) {
          uint32_t r[32];
          tmem_ld32(tSh + cc * 32, r);
          tmem_ld_wait(r);
          if (dbg_here) {
#pragma unroll
            for (int i = 0; i < 32; ++i) p.dbg_s[row * G + col0 + cc * 32 + i] = (int)(r[i] - kMagicI);
          }
          const float4* k4 = reinterpret_cast<const float4*>(ks_s + cc * 32);
          if (!masked && fold) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 kk = k4[i];
              const float s0 = fmaf(__uint_as_float(r[4 * i + 0]), qs_r, -mq) * kk.x;
              const float s1 = fmaf(__uint_as_float(r[4 * i + 1]), qs_r, -mq) * kk.y;
              const float s2 = fmaf(__uint_as_float(r[4 * i + 2]), qs_r, -mq) * kk.z;
              const float s3 = fmaf(__uint_as_float(r[4 * i + 3]), qs_r, -mq) * kk.w;
              if (i & 1) {
                mx2 = max3(mx2, s0, s1);
                mx3 = max3(mx3, s2, s3);
              } else {
                mx0 = max3(mx0, s0, s1);
                mx1 = max3(mx1, s2, s3);
              }
              r[4 * i + 0] = __float_as_uint(s0);
              r[4 * i + 1] = __float_as_uint(s1);
              r[4 * i + 2] = __float_as_uint(s2);
              r[4 * i + 3] = __float_as_uint(s3);
            }
          } else {
            const long long gc0 = gcol0 + col0 + cc * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float sraw = ((__uint_as_float(r[i]) - kMagicF) * qs_r) * ks_s[cc * 32 + i];
              const float x0 = masked ? fmaf(sraw, c, (gc0 + i <= grow) ? 0.f : -1.0e6f) : sraw;
              mx0 = fmaxf(mx0, x0);
              r[i] = __float_as_uint(x0);
            }
          }
          tmem_st32(tSh + cc * 32, r);
        }
        // join the two half-row maxima; the previous step's half-row sums ride along, so that the row
        // sum is formed as l = l*alpha + (sum_half0 + sum_half1) in both threads, step by step
        float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        {
          float2* x = reinterpret_cast<float2*>(xch_s) + (step_it & 1) * 256;
          x[half * 128 + row] = make_float2(mx, ls_pend);
          named_bar_sync(pair_bar, 64);
          const float2 e0 = x[row], e1 = x[128 + row];
          mx = fmaxf(e0.x, e1.x);
          if (have_pend) l_i = l_i * alpha_pend + (e0.y + e1.y);
        }
        tmem_st_wait();
        INTFA_T(2);
        const float m_new = masked ? fmaxf(m_i, mx) : fmaxf(m_i, mx * c);
        const float alpha = ex2_approx(m_i - m_new);
        // x = u*cm - m_new with one rounding: u = s, cm = c off the band; u = x0, cm = 1 on it
        const float cm = masked ? 1.0f : c;
        const float neg_m = -m_new;

        // half-int8: bring the accumulator to the new maximum before P V adds into it
        if constexpr (!FULL) {
          const bool have_acc = (j > 0) || p.state_in;
          if (have_acc && !__all_sync(0xffffffffu, alpha == 1.0f)) {
            const uint64_t ALPHA2 = f2_pack(alpha, alpha);
#pragma unroll 1
            for (int cc = 0; cc < DH / 32; ++cc) {
              uint32_t r[32];
              tmem_ld32(tA + lane_sel + ch0 + cc * 32, r);
              tmem_ld_wait(r);
#pragma unroll
              for (int i = 0; i < 16; ++i) f2_unpacku(f2_mul(f2_packu(r[2 * i], r[2 * i + 1]), ALPHA2), r[2 * i], r[2 * i + 1]);
              tmem_st32(tA + lane_sel + ch0 + cc * 32, r);
            }
          }
        }

        // ---- pass B: p = exp2(x), row sum of the un-quantised p, P -> shared memory; each chunk of the
        // region is re-armed with the magic as soon as it has been read (full-int8: for O_j = P V;
        // half-int8: for the next Q K^T)
        float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
#pragma unroll 1
        for (int cc = 0; cc < GH / 32; ++cc) {
          uint32_t r[32];
          tmem_ld32(tSh + cc * 32, r);
          tmem_ld_wait(r);
          tmem_fill32(tSh + cc * 32, kMagicI);
          uint32_t pk[FULL ? 8 : 16];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(r[4 * i + 0]), cm, neg_m));
            const float p1 = ex2_approx(fmaf(__uint_as_float(r[4 * i + 1]), cm, neg_m));
            const float p2 = ex2_approx(fmaf(__uint_as_float(r[4 * i + 2]), cm, neg_m));
            const float p3 = ex2_approx(fmaf(__uint_as_float(r[4 * i + 3]), cm, neg_m));
            ls0 += p0;
            ls1 += p1;
            ls2 += p2;
            ls3 += p3;
            if constexpr (FULL) {
              if constexpr (PRNE) {
                // fp32 p*127 rounded to nearest-even integer: adding 1.5*2^23 leaves it in the low mantissa bits
                const uint32_t u0 = __float_as_uint(__fadd_rn(__fmul_rn(p0, 127.f), kMagicF));
                const uint32_t u1 = __float_as_uint(__fadd_rn(__fmul_rn(p1, 127.f), kMagicF));
                const uint32_t u2 = __float_as_uint(__fadd_rn(__fmul_rn(p2, 127.f), kMagicF));
                const uint32_t u3 = __float_as_uint(__fadd_rn(__fmul_rn(p3, 127.f), kMagicF));
                pk[i] = __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
              } else {
                // fp16(p)*127 and +0.5 as two separately rounded fp16 operations, then truncation.
                // floor(y) without a conversion instruction: t = y + 1024 is 1024 + round(y) exactly
                // (fp16 spacing is 1 there); where round(y) > y one is taken off; the integer then sits
                // in the low byte of each half of t.
                const __half2 k127 = __float2half2_rn(127.f), khalf = __float2half2_rn(0.5f);
                const __half2 k1024 = __float2half2_rn(1024.f);
                const __half2 y01 = __hadd2_rn(__hmul2_rn(__floats2half2_rn(p0, p1), k127), khalf);
                const __half2 y23 = __hadd2_rn(__hmul2_rn(__floats2half2_rn(p2, p3), k127), khalf);
                const __half2 t01 = __hadd2_rn(y01, k1024), t23 = __hadd2_rn(y23, k1024);
                const __half2 f01 = __hsub2(t01, __hgt2(__hsub2(t01, k1024), y01));
                const __half2 f23 = __hsub2(t23, __hgt2(__hsub2(t23, k1024), y23));
                pk[i] = __byte_perm(*reinterpret_cast<const uint32_t*>(&f01), *reinterpret_cast<const uint32_t*>(&f23), 0x6420);
              }
            } else {
              const __half2 h01 = __floats2half2_rn(p0, p1);
              const __half2 h23 = __floats2half2_rn(p2, p3);
              pk[2 * i] = *reinterpret_cast<const uint32_t*>(&h01);
              pk[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&h23);
            }
          }
          const int colb = col0 + cc * 32;                   // first column of this chunk within the KV tile
          if constexpr (FULL) {
            // 32 int8 = two 16-byte chunks of this row
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t off = swz_off<G>(row, (colb >> 4) + h);
              *reinterpret_cast<uint4*>(sP_gen + off) = make_uint4(pk[4 * h], pk[4 * h + 1], pk[4 * h + 2], pk[4 * h + 3]);
            }
            if (dbg_here && p.dbg_p) {
              uint32_t* dp = reinterpret_cast<uint32_t*>(reinterpret_cast<int8_t*>(p.dbg_p) + row * G + colb);
#pragma unroll
              for (int i = 0; i < 8; ++i) dp[i] = pk[i];
            }
          } else {
            // 32 fp16 = four 16-byte chunks; columns [64*blk, 64*blk+64) live in block blk of 128 rows x 128 B
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const int col = colb + h * 8;
              const uint32_t off = (col >> 6) * (kBM * 128) + swz_off<128>(row, (col & 63) >> 3);
              *reinterpret_cast<uint4*>(sP_gen + off) = make_uint4(pk[4 * h], pk[4 * h + 1], pk[4 * h + 2], pk[4 * h + 3]);
            }
            if (dbg_here && p.dbg_p) {
              uint32_t* dp = reinterpret_cast<uint32_t*>(reinterpret_cast<__half*>(p.dbg_p) + row * G + colb);
#pragma unroll
              for (int i = 0; i < 16; ++i) dp[i] = pk[i];
            }
          }
        }
        if constexpr (FULL && (D > G)) {
          // O_j is wider than S: arm the columns S did not cover (split between the two threads of the row)
#pragma unroll
          for (int cc = 0; cc < (D - G) / 64; ++cc) tmem_fill32(tS + lane_sel + G + half * ((D - G) / 2) + cc * 32, kMagicI);
        }
        tmem_st_wait();
        // P visible to the tensor core's shared-memory reads; TMEM region re-armed / accumulator rescaled
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(B_PFULL));
        INTFA_T(3);
        ls_pend = (ls0 + ls1) + (ls2 + ls3);
        alpha_pend = alpha;
        have_pend = true;
        m_i = m_new;

        if constexpr (FULL) {
          // ---- correction: acc = acc*alpha + fp32(O_j) * s_v/127, accumulator row in TMEM
          named_bar_sync(kBarO, kComputeThreads + 32);        // O_j = P V is in TMEM
          ok = (*abort_flag == 0);
          if (!ok) break;
          tc_fence_after();
          INTFA_T(4);
          const uint64_t ALPHA2 = f2_pack(alpha, alpha);
#pragma unroll 1
          for (int cc = 0; cc < DH / 16; ++cc) {
            uint32_t r[16], a[16];
            const int chb = ch0 + cc * 16;
            tmem_ld16(tO + lane_sel + chb, r);
            tmem_ld16(tA + lane_sel + chb, a);
            tmem_ld_wait16(r);
            tmem_ld_wait16(a);
            const ulonglong2* v2 = reinterpret_cast<const ulonglong2*>(vsd_s + chb);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const ulonglong2 vv = v2[i];
              const uint64_t a01 = f2_fma(f2_add(f2_packu(r[4 * i + 0], r[4 * i + 1]), NEG_MAGIC2), vv.x,
                                          f2_mul(f2_packu(a[4 * i + 0], a[4 * i + 1]), ALPHA2));
              const uint64_t a23 = f2_fma(f2_add(f2_packu(r[4 * i + 2], r[4 * i + 3]), NEG_MAGIC2), vv.y,
                                          f2_mul(f2_packu(a[4 * i + 2], a[4 * i + 3]), ALPHA2));
              f2_unpacku(a01, a[4 * i + 0], a[4 * i + 1]);
              f2_unpacku(a23, a[4 * i + 2], a[4 * i + 3]);
            }
            tmem_st16(tA + lane_sel + chb, a);
          }
          // O_j is folded in: re-arm the columns this thread has just read that the next Q K^T will
          // accumulate into (the first G of the region)
#pragma unroll
          for (int cc = 0; cc < DH / 32; ++cc)
            if (ch0 + cc * 32 < G) tmem_fill32(tS + lane_sel + ch0 + cc * 32, kMagicI);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR(B_RFREE));
          INTFA_T(5);
        }
      }
      if (!ok) break;

      // ---- epilogue
      if constexpr (!FULL) {
        if (t.nsteps > 0) {
          named_bar_sync(kBarO, kComputeThreads + 32);        // last P V of the work item is in the accumulator
          ok = (*abort_flag == 0);
          if (!ok) break;
          tc_fence_after();
        }
      }
      // fold in the last KV step's half-row sums
      float l_row = l_i;
      if (have_pend) {
        float* x = xch_s + 1024;                             // [2 halves][128 rows], epilogue only
        named_bar_sync(pair_bar, 64);                        // partner done reading the previous work item's sums
        x[half * 128 + row] = ls_pend;
        named_bar_sync(pair_bar, 64);
        l_row = l_i * alpha_pend + (x[row] + x[128 + row]);
      }
      __half* orow = p.o + (long long)t.b * p.o_sb + (long long)t.h * p.o_sh + (long long)(t.mb * kBM + row) * p.o_sn + ch0;
#pragma unroll
      for (int cc = 0; cc < DH / 32; ++cc) {
        uint32_t a[32];
        tmem_ld32(tA + lane_sel + ch0 + cc * 32, a);
        tmem_ld_wait(a);
        if (p.state_out) {
          uint4* a4 = reinterpret_cast<uint4*>(p.st_acc + rowg * D + ch0 + cc * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) a4[i] = make_uint4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
        }
        if (p.write_o) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              w[e] = pack_out(__uint_as_float(a[8 * i + 2 * e]) / l_row, __uint_as_float(a[8 * i + 2 * e + 1]) / l_row,
                              p.o_bf16);
            }
            *reinterpret_cast<uint4*>(orow + cc * 32 + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (half == 0) {
        if (p.state_out) {
          p.st_m[rowg] = m_i;
          p.st_l[rowg] = l_row;
        }
        if (p.write_o && p.lse) p.lse[rowg] = m_i + log2f(l_row);
      }
      if constexpr (!FULL) {
        if (t.nsteps > 0) {
          // accumulator read out: the next work item's first P V may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR(B_RFREE));
          ++tile_it;
        }
      }
    }
#ifdef INTFA_TIMING
    if (lane == 0 && p.dbg_s != nullptr && p.dbg_tile == -2 && blockIdx.x < 400 && half == 0) {
      for (int i = 0; i < 8; ++i) p.dbg_s[(blockIdx.x * 4 + quarter) * 8 + i] = (int)(tm[i] >> 4);
    }
#endif
  }

  // -------------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

#include "intfa_fwd_pipe.cuh"

// ============================================================================
// host side
// ============================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Work-item counters of the launches in flight: a small ring of words inside the library image (no
// allocation at launch time); each launch takes the next word and zeroes it on its stream.
constexpr int kTileCounters = 4096;
__device__ static unsigned int g_tile_counters[kTileCounters];

static int next_tile_counter(unsigned int** out, cudaStream_t stream) {
  static unsigned int* base[64];
  static bool have[64];
  static std::atomic<unsigned int> next{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return set_error(INTFA_ERR_CUDA, "cannot query the current device");
  if (!have[dev]) {
    void* sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_tile_counters);
    if (e != cudaSuccess || !sym) return set_error(INTFA_ERR_CUDA, "cudaGetSymbolAddress(tile counters): %s", cudaGetErrorString(e));
    base[dev] = static_cast<unsigned int*>(sym);
    have[dev] = true;
  }
  unsigned int* c = base[dev] + (next.fetch_add(1) % kTileCounters);
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

template <int D, int G, bool FULL, bool PRNE>
static int launch(const IntfaFwdParams* a, const KParams& kp, cudaStream_t stream) {
  using C = Cfg<D, G, FULL>;
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapSwizzle swzD = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  int rc;
  if ((rc = make_tmap(&tmQ, a->q, 1, a->q_stride, a->B, a->H, a->Nq, D, D, kBM, swzD))) return rc;
  if ((rc = make_tmap(&tmK, a->k, 1, a->k_stride, a->B, kv_heads(a), a->Nk, D, D, G, swzD))) return rc;
  if constexpr (FULL) {
    if ((rc = make_tmap(&tmV, a->v, 1, a->v_stride, a->B, kv_heads(a), a->Nk, D, D, G, swzD))) return rc;
  } else {
    if ((rc = make_tmap(&tmV, a->v, 2, a->v_stride, a->B, kv_heads(a), a->Nk, D, 64, G, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }
  auto kern = intfa_fwd_kernel<D, G, FULL, PRNE>;
  static bool attr_done = false;     // per instantiation; the attribute is per device, so set it every time a device changes
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done || attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done = true;
    attr_dev = dev;
  }
  const int sms = sm_count_cached();
  if (sms <= 0) return set_error(INTFA_ERR_CUDA, "cannot query SM count");
  const int ctas_per_sm = (C::SMEM_BYTES + 1024) * 2 <= 227 * 1024 ? 2 : 1;
  int grid = sms * ctas_per_sm;
#ifdef INTFA_TIMING
  if (getenv("INTFA_ONE_CTA_PER_SM")) grid = sms;
#endif
  if (grid > kp.num_tiles) grid = kp.num_tiles;
  KParams kpl = kp;
  if ((rc = next_tile_counter(&kpl.tile_counter, stream))) return rc;
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, kpl);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return INTFA_OK;
}

// Pipelined full-int8 kernel: one CTA per SM.
template <int D, int G, bool FULL, bool PRNE, bool RAGGED>
static int launch_pipe(const IntfaFwdParams* a, const KParams& kp, cudaStream_t stream) {
  using C = PipeCfg<D, G, FULL>;
  static_assert(C::SMEM_BYTES <= 227 * 1024, "shared memory");
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapSwizzle swzD = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : (D == 64) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  int rc;
  if ((rc = make_tmap(&tmQ, a->q, 1, a->q_stride, a->B, a->H, a->Nq, D, D, kBM, swzD))) return rc;
  if ((rc = make_tmap(&tmK, a->k, 1, a->k_stride, a->B, kv_heads(a), a->Nk, D, D, G, swzD))) return rc;
  if constexpr (FULL) {
    if ((rc = make_tmap(&tmV, a->v, 1, a->v_stride, a->B, kv_heads(a), a->Nk, D, D, G, swzD))) return rc;
  } else {
    if ((rc = make_tmap(&tmV, a->v, 2, a->v_stride, a->B, kv_heads(a), a->Nk, D, D >= 64 ? 64 : D, G,
                        D >= 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
  }
  auto kern = intfa_fwd_pipe_kernel<D, G, FULL, PRNE, RAGGED>;
  static bool attr_done = false;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done || attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return set_error(INTFA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done = true;
    attr_dev = dev;
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
  kp.hk_ratio = a->H / kv_heads(a);
  kp.o_bf16 = a->o_dtype == INTFA_OUT_BF16 ? 1 : 0;
  kp.causal = a->causal ? 1 : 0;
  kp.c = a->sm_scale * 1.44269504f;          // fp32 product, flash_atten_full_int8.py:156-157
  kp.q_off = a->q_offset; kp.kv_off = a->kv_offset;
  kp.lse = a->lse_out; kp.st_m = a->state_m; kp.st_l = a->state_l; kp.st_acc = a->state_acc;
  kp.state_in = a->state_in; kp.state_out = a->state_out; kp.write_o = a->write_o;
  kp.dbg_s = a->dbg_s; kp.dbg_p = a->dbg_p; kp.dbg_tile = a->dbg_tile; kp.dbg_step = a->dbg_step;
  kp.status = a->status;
  kp.MB = (a->Nq + kBM - 1) / kBM;            // the last query tile may be partial (pipelined kernel only)
  kp.num_tiles = a->B * a->H * kp.MB;
  const bool full = a->variant == INTFA_VARIANT_FULL;
  const bool rne = full && a->p_round == 1;
  const int D = a->D, G = a->G;
  // The one-CTA pipelined kernel serves full-int8 and half-int8 at head_dim 128; half-int8 at head_dim 64 is
  // faster on the two-CTA kernel (measured), which INTFA_LEGACY_KERNEL in the environment selects for everything.
  static const bool use_pipe = getenv("INTFA_LEGACY_KERNEL") == nullptr;
  // Sequence lengths that are not multiples of the tile sizes: only the pipelined kernel masks them
  const bool ragged = (a->Nq % kBM) != 0 || (a->Nk % a->G) != 0;
  if (ragged && !use_pipe)
    return set_error(INTFA_ERR_UNSUPPORTED, "Nq=%d / Nk=%d not multiples of 128 / G=%d: not supported by the kernel INTFA_LEGACY_KERNEL selects", a->Nq, a->Nk, a->G);
#define INTFA_CASE(DD, GG)                                                       \
  if (D == DD && G == GG) {                                                      \
    if (full && use_pipe && ragged) return rne ? launch_pipe<DD, GG, true, true, true>(a, kp, stream)   \
                                               : launch_pipe<DD, GG, true, false, true>(a, kp, stream); \
    if (full && use_pipe) return rne ? launch_pipe<DD, GG, true, true, false>(a, kp, stream)            \
                                     : launch_pipe<DD, GG, true, false, false>(a, kp, stream);          \
    if (use_pipe && ragged) return launch_pipe<DD, GG, false, false, true>(a, kp, stream);              \
    if (use_pipe && DD == 128) return launch_pipe<DD, GG, false, false, false>(a, kp, stream);          \
    if (full) return rne ? launch<DD, GG, true, true>(a, kp, stream)             \
                         : launch<DD, GG, true, false>(a, kp, stream);           \
    return launch<DD, GG, false, false>(a, kp, stream);                          \
  }
  INTFA_CASE(128, 128)
  INTFA_CASE(128, 64)
  INTFA_CASE(64, 64)
  INTFA_CASE(64, 128)
#undef INTFA_CASE
  // head_dim 32: the pipelined kernel only (G = 32 for full-int8 only: fp16 P tiles need 64 columns)
#define INTFA_CASE32(GG)                                                                                          \
  if (D == 32 && G == GG && use_pipe) {                                                                           \
    if (full && ragged) return rne ? launch_pipe<32, GG, true, true, true>(a, kp, stream)                         \
                                   : launch_pipe<32, GG, true, false, true>(a, kp, stream);                       \
    if (full) return rne ? launch_pipe<32, GG, true, true, false>(a, kp, stream)                                  \
                         : launch_pipe<32, GG, true, false, false>(a, kp, stream);                                \
    if constexpr (GG >= 64) {                                                                                     \
      return ragged ? launch_pipe<32, GG, false, false, true>(a, kp, stream)                                      \
                    : launch_pipe<32, GG, false, false, false>(a, kp, stream);                                    \
    }                                                                                                             \
  }
  INTFA_CASE32(32)
  INTFA_CASE32(64)
  INTFA_CASE32(128)
#undef INTFA_CASE32
  return set_error(INTFA_ERR_UNSUPPORTED, "unsupported (D=%d, G=%d, %s): supported are D in {64,128} with G in {64,128}, and D=32 with G in {32,64,128} (G=32: full-int8 only; not with INTFA_LEGACY_KERNEL)", D, G, full ? "full-int8" : "half-int8");
}

}  // namespace intfa
