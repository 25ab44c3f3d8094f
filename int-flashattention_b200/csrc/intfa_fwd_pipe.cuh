// INT8 attention forward (full-int8 and half-int8): ONE CTA per SM, one 128-row query tile at a time.
// (Included by intfa_fwd.cu inside namespace intfa, after the shared helpers.)
//
// 512 threads:
//   warp 0        TMA producer (Q once per work item; K and V through rings of shared-memory stages, the K-scale
//                 slices through a ring of their own); it also draws the work items from the global counter
//   warp 1        MMA issuer for S = Q K^T (whole warp runs the loop, one elected lane issues): up to three KV steps
//                 ahead of the softmax groups, into S buffer (step mod 3)
//   warp 2        TMEM allocator
//   warp 3        MMA issuer for O_j = P V
//   warps 4-7     softmax group 0, warps 8-11 softmax group 1: one thread per query row.  The groups take
//                 ALTERNATE KV steps (group g owns the steps whose running index is g mod 2), each with its own
//                 P buffer in shared memory, so that on every scheduler one warp is in pass A (dequantise, row
//                 max: FMA pipe) while the other is in pass B (exp2, P: exp2 unit).  The running max m of a row
//                 travels between the two threads that own it through shared memory, once per step.
//   warps 12-15   accumulator update and epilogue, one thread per query row:
//                 full-int8: A = A*alpha + fp32(O_j) with the fp32 row A in REGISTERS and O_j (int32) in TMEM;
//                 half-int8: P V (fp16 MMA) accumulates straight into an fp32 accumulator in TMEM, these warps
//                 multiply the row by alpha beforehand when some alpha of the warp's 32 rows is not 1.
//                 They also carry the row sum l = l*alpha + rowsum(P) (see PipeCfg::L_IN_ACC).
// TMEM columns: S0 [0,G) | S1 [G,2G) | S2 [2G,3G) | O_j, or the half-int8 accumulator [3G, 3G+D)  (<= 512).
// S and O_j are int32 accumulators that start each KV step from the bit pattern of 1.5*2^23, written by a
// small fp16 MMA ahead of the int8 MMAs, so that the threads read fp32(S32) + 1.5*2^23 without a conversion.
// The arithmetic contract is at the top of intfa_fwd.cu.
#pragma once

constexpr int kPipeThreads = 512;
constexpr int kPipeSoftmaxThreads = 256;
constexpr int kPipeCorrThreads = 128;
// Registers: the CTA is launched with kPipeLaunchRegs per thread and setmaxnreg only moves registers around
// INSIDE that allocation -- an increase beyond it would block for ever, hence the static_assert in PipeCfg.
constexpr int kPipeLaunchRegs = (65536 / kPipeThreads) / 8 * 8;
constexpr int kPipeServiceRegs = 40;

// D: channels of V and of the accumulator that one pass covers (and the width the tensor-core tiles are built for);
// DQ: head dim of Q and K.  DQ == D except at head dim 256, which runs as DQ = 256, D = 128: every query tile is
// taken twice in a row by the same CTA, once per half of the V channels (the accumulator row of one thread and the
// TMEM columns hold 128 channels); S, the running max and P are the same in both passes.
// F8V: the half-int8 op with V (and therefore P) in float8_e5m2 (flash_atten_int8.py:55-56): one-byte P and V tiles laid
// out like the int8 ones, P V with kind::f8f6f4 accumulating in fp32 like the fp16 form.
template <int D, int G, bool FULL, int DQ = D, bool F8V = false>
struct PipeCfg {
  static_assert(!(FULL && F8V), "fp8 V belongs to the half-int8 op");
  static constexpr bool BYTE_PV = FULL || F8V;                     // P and V elements are one byte
  static_assert(DQ == D || (DQ == 256 && D == 128), "head dims");
  static constexpr int NVH = DQ / D;                               // passes per query tile
  static constexpr int QK_ROWB = DQ < 128 ? DQ : 128;              // Q and K sit in shared memory as panels of [rows][QK_ROWB bytes]
  static constexpr int QK_PANELS = DQ / QK_ROWB;
  static constexpr int Q_BYTES = kBM * DQ;
  static constexpr int K_BYTES = G * DQ;
  static constexpr int V_BYTES = BYTE_PV ? G * D : G * D * 2;         // int8, or fp16 as D/64 boxes of [G keys][64 channels]
  static constexpr int P_BYTES = BYTE_PV ? kBM * G : kBM * G * 2;     // int8, or fp16 as G/64 blocks of [128 rows][64 columns]
  static constexpr int KS_BYTES = G * 4;
  static constexpr bool BIG = DQ > 128 && G == 128;                // 32 KB K tiles: three stages are what fits
  static constexpr int NSK = BIG ? 3 : 4;                          // K stages
  static constexpr int NSV = BIG ? 3 : (BYTE_PV || G == 64) ? 4 : 2;  // V stages (fp16 V tiles are twice the size)
  static constexpr int NKS = 8;                                    // K-scale slots: a slot is rewritten 8 steps later, when
                                                                   // the three S buffers have long forced its step out
  static constexpr int NSB = 3;                                    // S buffers in TMEM
  // Who carries the row sum l = l*alpha + rowsum(P)?  Where a KV step is as wide as the head (G >= D) the accumulator
  // warps do, next to the accumulator row: the softmax groups then meet once per step (running max) instead of
  // twice.  Where the head is wider than the step (head_dim 128 at G = 64) the accumulator warps are the busier
  // side and the softmax groups keep l, handing it over like the running max (measured: 582 against 474 TOPS).
  static constexpr bool L_IN_ACC = G >= D;
  // setmaxnreg split between the softmax and the accumulator warps.  The accumulator row of 128 channels fits either
  // way; with 128-column KV steps, and for half-int8 (no accumulator row in registers), the softmax passes gain more
  // from 16 further registers than the update loses (measured +2..3 %); full-int8 at G = 64 is the other way round.
  // A vectorised pass A for the causal diagonal band (otherwise those steps take the general, scalar path): compiled in
  // for 128-column KV steps, where it measured +2..5 % on causal workloads; with 64-column steps its code costs the
  // non-causal case more (instruction cache) than it gives.
  static constexpr bool BAND_FAST = G == 128;
  // instructions of never-executed filler between the softmax passes (see intfa_fwd_pipe_softmax.inc): 4 KB with the
  // band path compiled in, else 2 KB, and none for full-int8 at head dim 64 -- each the best of a sweep
  static constexpr int CODE_FILLER = BAND_FAST ? 256 : (FULL && D == 64) ? 0 : 128;
  static constexpr bool MORE_SOFTMAX_REGS = !FULL || G == 128;
  static constexpr int SOFTMAX_REGS = MORE_SOFTMAX_REGS ? 152 : 136;
  static constexpr int CORR_REGS = MORE_SOFTMAX_REGS ? 168 : 184;
  static_assert(128 * kPipeServiceRegs + kPipeSoftmaxThreads * SOFTMAX_REGS + kPipeCorrThreads * CORR_REGS <=
                    kPipeThreads * kPipeLaunchRegs, "setmaxnreg budget exceeds the registers the CTA is launched with");
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NSK * K_BYTES;
  static constexpr int OFF_P = OFF_V + NSV * V_BYTES;             // two P buffers
  static constexpr int OFF_KS = OFF_P + 2 * P_BYTES;
  static constexpr int OFF_VSD = OFF_KS + NKS * KS_BYTES;         // s_v/127 per channel
  static constexpr int OFF_HM = OFF_VSD + D * 4;                  // [2 groups][128] float: running max after the group's latest step
  static constexpr int OFF_RS = OFF_HM + 2 * 128 * 4;             // [4][128] float: row sum of P of step j, for the accumulator warps
                                                                   //   (!L_IN_ACC: [2 groups][128] float, l after the group's latest step)
  static constexpr int OFF_ALPHA = OFF_RS + 4 * 128 * 4;          // [4][128] float: alpha of step j, for the accumulator warps
  static constexpr int OFF_FIN = OFF_ALPHA + 4 * 128 * 4;         // [2][128] float2: final running max of a work item (.x)
  static constexpr int OFF_MAGIC = OFF_FIN + 2 * 128 * 8;          // 4 KB constant fp16 operand of the "arm" MMA
  static constexpr int MAGIC_BYTES = 4096;
  static constexpr int OFF_BAR = OFF_MAGIC + MAGIC_BYTES;
  static constexpr int NUM_BARS = 18 + 2 * NSK + 2 * NSV + 8 + 4 + 2 * NSB;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 32 + 1024;
  // S buffer b at COL_S + b*G; then O_j (full-int8: the accumulator itself lives in registers) or the fp32
  // accumulator the second MMA adds into (half-int8)
  static constexpr int COL_S = 0, COL_O = NSB * G, COL_ACC = NSB * G;
  static_assert(NSB * G + D <= 512, "TMEM columns");
  static constexpr int TMEM_COLS = 512;
  static_assert(FULL || G >= 64, "half-int8: fp16 P tiles are built from 64-column blocks");
  static constexpr uint64_t SWZ_QK = (QK_ROWB == 128) ? kSwz128 : (QK_ROWB == 64) ? kSwz64 : kSwz32;
  static constexpr uint32_t SBO_QK = 8 * QK_ROWB;
  // start-address offset (16-byte units) of the kk-th 32-byte K slice of a [ROWS][DQ] operand
  __host__ __device__ static constexpr uint32_t qk_slice(int kk, int rows) { return (uint32_t)((kk / 4) * ((rows * QK_ROWB) >> 4) + 2 * (kk % 4)); }
  static constexpr uint64_t SWZ_P = BYTE_PV ? ((G == 128) ? kSwz128 : (G == 64) ? kSwz64 : kSwz32) : kSwz128;
  static constexpr uint32_t SBO_P = BYTE_PV ? 8 * G : 1024;
  // V rows: D bytes (int8), or boxes of min(D, 64) fp16 channels = 128 / 64 bytes
  static constexpr int V_BOXES = BYTE_PV ? 1 : (D >= 64 ? D / 64 : 1);
  static constexpr int V_ROWB = BYTE_PV ? D : (D >= 64 ? 128 : 2 * D);
  static constexpr uint64_t SWZ_V = (V_ROWB == 128) ? kSwz128 : (V_ROWB == 64) ? kSwz64 : kSwz32;
  static constexpr uint32_t SBO_V = 8 * V_ROWB;
  static constexpr uint32_t IDESC_QK = make_idesc(2, 1, 1, 0, 0, kBM, G);
  // (kind::f8f6f4: A / B format 1 = e5m2, D format 1 = f32)
  static constexpr uint32_t IDESC_PV = FULL ? make_idesc(2, 1, 1, 0, 1, kBM, D)
                                       : F8V ? make_idesc(1, 1, 1, 0, 1, kBM, D) : make_idesc(1, 0, 0, 0, 1, kBM, D);
  // fp16 x fp16 -> fp32, K = 16: writes the fp32 constant 1.5*2^23 into a whole accumulator tile
  static constexpr uint32_t IDESC_ARM_S = make_idesc(1, 0, 0, 0, 0, kBM, G);
  static constexpr uint32_t IDESC_ARM_O = make_idesc(1, 0, 0, 0, 0, kBM, D);
};

enum PipeWait { PW_TILE = 32, PW_QE, PW_KE, PW_VE, PW_QF, PW_KF, PW_VF, PW_SFREE, PW_PFULL, PW_OFREE, PW_SFULL,
                PW_PFREE, PW_HM, PW_OFULL, PW_FIN, PW_FINFREE, PW_HL, PW_AFULL };

// RAGGED: Nq / Nk are not multiples of 128 / G -- the last query tile and the last KV step are partial.  A separate
// instantiation, so that the code of the common case stays as small as it was (instruction cache).
template <int D, int G, bool FULL, bool PRNE, bool RAGGED, int DQ = D, bool F8V = false>
__global__ void __launch_bounds__(kPipeThreads, 1)
intfa_fwd_pipe_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const KParams p) {
  using C = PipeCfg<D, G, FULL, DQ, F8V>;
  constexpr int NSK = C::NSK, NSV = C::NSV, NSB = C::NSB, NVH = C::NVH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t bar0 = smem_u32(smem + C::OFF_BAR);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // mbarriers.  "commit" = arrived on by tcgen05.commit, i.e. when the MMAs issued so far are done.
  constexpr int B_QFULL = 0;      // TMA: Q tile landed
  constexpr int B_QEMPTY = 1;     // commit: last Q K^T of the work item done
  constexpr int B_PFULL = 4;      // [2] softmax group b (4 warps): P in shared-memory buffer b, and S buffer b read out
  constexpr int B_PFREE = 6;      // [2] commit: the P V that read P buffer b is done
  constexpr int B_OFULL = 8;      // commit: O_j = P V in TMEM
  constexpr int B_OFREE = 9;      // accumulator warps (4): O_j read out
  constexpr int B_HL = 16;        // [2] !L_IN_ACC: softmax group g (4 warps): row sum after its step published
  constexpr int B_FIN = 10;       // [2] softmax (4 warps of one group): final (m, l) of the work item published; one
                                  //     barrier per slot, so that a short next work item cannot complete it twice
                                  //     before a slow accumulator warp has waited for the first completion
  constexpr int B_FINFREE = 12;   // [2] accumulator warps (4): they have read them
  constexpr int B_HM = 14;        // [2] softmax group g (4 warps): running max after its step published
  constexpr int B_KFULL = 18, B_KEMPTY = 18 + NSK, B_VFULL = 18 + 2 * NSK, B_VEMPTY = 18 + 2 * NSK + NSV;
  constexpr int B_TILE = 18 + 2 * NSK + 2 * NSV, B_TDONE = B_TILE + 4;
  constexpr int B_AFULL = B_TDONE + 4;   // [4] half-int8: alpha of step j (slot j mod 4) published, for the accumulator warps
  constexpr int B_SFULL = B_AFULL + 4;   // [3] commit: S = Q K^T in TMEM buffer b
  constexpr int B_SFREE = B_SFULL + NSB; // [3] softmax group of the step (4 warps): S buffer b read out for good
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 4);
  volatile int* tile_slot = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 16);

  if (threadIdx.x == 0) {
    mbar_init(BAR(B_QFULL), 1);
    mbar_init(BAR(B_QEMPTY), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(BAR(B_PFULL + b), 4);
      mbar_init(BAR(B_PFREE + b), 1);
      mbar_init(BAR(B_FINFREE + b), 4);
      mbar_init(BAR(B_HM + b), 4);
      mbar_init(BAR(B_HL + b), 4);
      mbar_init(BAR(B_FIN + b), 4);
    }
    mbar_init(BAR(B_OFULL), 1);
    mbar_init(BAR(B_OFREE), 4);
    for (int s = 0; s < NSK; ++s) {
      mbar_init(BAR(B_KFULL + s), 1);
      mbar_init(BAR(B_KEMPTY + s), 1);
    }
    for (int s = 0; s < NSV; ++s) {
      mbar_init(BAR(B_VFULL + s), 1);
      mbar_init(BAR(B_VEMPTY + s), 1);
    }
    for (int b = 0; b < NSB; ++b) {
      mbar_init(BAR(B_SFULL + b), 1);
      mbar_init(BAR(B_SFREE + b), 4);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(BAR(B_TILE + i), 1);
      mbar_init(BAR(B_TDONE + i), 14);       // 2 MMA warps + 8 softmax warps + 4 accumulator warps
      mbar_init(BAR(B_AFULL + i), 4);
    }
    abort_flag[0] = 0;
    abort_flag[1] = p.wait_limit_kcycles;
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
  const uint32_t sQ = smem_u32(smem + C::OFF_Q);
  const uint32_t sK = smem_u32(smem + C::OFF_K);
  const uint32_t sV = smem_u32(smem + C::OFF_V);
  const uint32_t sP = smem_u32(smem + C::OFF_P);
  const uint32_t sKS = smem_u32(smem + C::OFF_KS);

  // The int32 accumulator tiles start every KV step from the bit pattern of 1.5*2^23 (see kMagicI).  It is
  // written by the tensor core itself: an fp16 MMA (K = 16, no accumulate) of a constant operand with
  // itself.  Every 16-byte chunk of the operand holds (1024, 1024, 2048, 0, 0, 0, 0, 0), so whatever the
  // layout each row's 16 values are two such chunks and the dot product of any two rows is
  // 2*(2^20 + 2^20 + 2^22) = 12582912 = 1.5*2^23, exactly, in fp32.
  if (threadIdx.x < C::MAGIC_BYTES / 16) {
    reinterpret_cast<uint4*>(smem + C::OFF_MAGIC)[threadIdx.x] = make_uint4(0x64006400u, 0x00006800u, 0u, 0u);
    fence_proxy_async_smem();
  }
  __syncthreads();
  const uint64_t descArm = make_smem_desc(smem_u32(smem + C::OFF_MAGIC), 128, 256, 0);

  // work items: drawn from a global counter by the producer, published in a 4-slot ring
  auto next_tile = [&](uint32_t& seq, bool ack, bool whole_warp) -> int {
    const uint32_t slot = seq & 3u, par = (seq >> 2) & 1u;
    ++seq;
    bool got = mbar_wait(BAR(B_TILE + slot), par, abort_flag, p.status, code_hi | PW_TILE);
    if (whole_warp) got = __all_sync(0xffffffffu, got);
    if (!got) return -1;
    const int t = tile_slot[slot];
    if (whole_warp) __syncwarp();
    if (ack) mbar_arrive(BAR(B_TDONE + slot));
    return t;
  };

  // registers: 512 x 128 at launch; the service warps and the accumulator warps give theirs to the softmax warps
  if (warp < 4) reg_dealloc<kPipeServiceRegs>();

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      uint32_t kv_it = 0, tile_it = 0, tseq = 0;
      int drawn = 0, passes_left = 0;      // NVH > 1: the query tile in hand and how many of its passes are still to publish
      bool ok = true;
      while (ok) {
        if (tseq >= 4u) {
          ok = mbar_wait(BAR(B_TDONE + (tseq & 3u)), ((tseq >> 2) - 1u) & 1u, abort_flag, p.status, code_hi | PW_TILE);
          if (!ok) break;
        }
        int tile;
        if (NVH > 1 && passes_left > 0) {
          tile = drawn * NVH + (NVH - passes_left);      // the next pass over the same query tile, on this CTA
          --passes_left;
        } else {
          tile = (int)atomicAdd(p.tile_counter, 1u);
          if (tile >= p.num_tiles) {
            tile = -1;
          } else if (NVH > 1) {
            drawn = tile;
            tile *= NVH;
            passes_left = NVH - 1;
          }
        }
        tile_slot[tseq & 3u] = tile;
        mbar_arrive(BAR(B_TILE + (tseq & 3u)));
        ++tseq;
        if (tile < 0) break;
        const TileInfo t = decode_tile<RAGGED, NVH>(p, tile, G);
        if (t.nsteps == 0) continue;
        ok = mbar_wait(BAR(B_QEMPTY), (tile_it & 1) ^ 1, abort_flag, p.status, code_hi | PW_QE);
        if (!ok) break;
        mbar_expect_tx(BAR(B_QFULL), C::Q_BYTES);
#pragma unroll
        for (int pn = 0; pn < C::QK_PANELS; ++pn)
          tma_load_4d(sQ + pn * (kBM * C::QK_ROWB), &tmQ, BAR(B_QFULL), pn * C::QK_ROWB, t.mb * kBM, t.h, t.b);
        const float* ks_row = p.ks + (long long)t.b * p.ks_sb + (long long)t.hk * p.ks_sh;
        for (int j = 0; j < t.nsteps; ++j, ++kv_it) {
          const uint32_t s = kv_it % NSK, ph = (kv_it / NSK) & 1;
          ok = mbar_wait(BAR(B_KEMPTY + s), ph ^ 1, abort_flag, p.status, code_hi | PW_KE);
          if (!ok) break;
          const int jb = kv_tile_of_step(p, j, t.nsteps);
          if (p.skip_k_load == 0 || kv_it + 1 != (uint32_t)p.skip_k_load) {      // (test hook: a K tile that never arrives)
            mbar_expect_tx(BAR(B_KFULL + s), C::K_BYTES + C::KS_BYTES);
#pragma unroll
            for (int pn = 0; pn < C::QK_PANELS; ++pn)
              tma_load_4d(sK + s * C::K_BYTES + pn * (G * C::QK_ROWB), &tmK, BAR(B_KFULL + s), pn * C::QK_ROWB, jb * G, t.hk, t.b);
            bulk_load_1d(sKS + (kv_it % C::NKS) * C::KS_BYTES, ks_row + jb * G, C::KS_BYTES, BAR(B_KFULL + s));
          }
          const uint32_t sv = kv_it % NSV, phv = (kv_it / NSV) & 1;
          ok = mbar_wait(BAR(B_VEMPTY + sv), phv ^ 1, abort_flag, p.status, code_hi | PW_VE);
          if (!ok) break;
          mbar_expect_tx(BAR(B_VFULL + sv), C::V_BYTES);
          if constexpr (C::BYTE_PV) {
            tma_load_4d(sV + sv * C::V_BYTES, &tmV, BAR(B_VFULL + sv), t.vh * D, jb * G, t.hk, t.b);
          } else {
#pragma unroll
            for (int c = 0; c < C::V_BOXES; ++c)
              tma_load_4d(sV + sv * C::V_BYTES + c * (G * 128), &tmV, BAR(B_VFULL + sv), t.vh * D + c * 64, jb * G, t.hk, t.b);
          }
        }
        ++tile_it;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    {
      // ------------------------------------------------------------------ MMA issuer for S = Q K^T
      // The whole warp runs the loop and the waits (warp-uniform control flow keeps the descriptor arithmetic
      // off the per-thread path); one elected lane issues the tensor-core instructions.
      // Step it goes into S buffer it mod 3 as soon as the step three back has been read out of it and K has landed --
      // up to three steps ahead of the softmax groups.  The K stage is handed back by the tensor core itself (the
      // K scales sit in a ring of their own).
      uint32_t kv_it = 0, tile_it = 0, tseq = 0, sfree_seen = 0;
      bool ok = true;
      // operand descriptors of stage 0 / K step 0; the start-address field (16-byte units) takes the offsets
      const uint64_t descQ0 = make_smem_desc(sQ, 16, C::SBO_QK, C::SWZ_QK);
      const uint64_t descK0 = make_smem_desc(sK, 16, C::SBO_QK, C::SWZ_QK);
      while (ok) {
        const int tile = next_tile(tseq, lane == 0, true);
        if (tile < 0) break;
        const TileInfo t = decode_tile<RAGGED, NVH>(p, tile, G);
        if (t.nsteps == 0) continue;
        ok = mbar_wait_warp(BAR(B_QFULL), tile_it & 1, abort_flag, p.status, code_hi | PW_QF);
        if (!ok) break;
        for (int j = 0; j < t.nsteps; ++j, ++kv_it) {
          const uint32_t s = kv_it % NSK, ph = (kv_it / NSK) & 1;
          const uint32_t sb = kv_it % NSB;
          // every S_FREE is waited for exactly once, in step order, so the phases of the barriers stay in step
          while (ok && sfree_seen + NSB <= kv_it) {
            ok = mbar_wait_warp(BAR(B_SFREE + sfree_seen % NSB), (sfree_seen / NSB) & 1, abort_flag, p.status, code_hi | PW_SFREE);
            ++sfree_seen;
          }
          if (!ok) break;
          ok = mbar_wait_warp(BAR(B_KFULL + s), ph, abort_flag, p.status, code_hi | PW_KF);
          if (!ok) break;
          tc_fence_after();
          const uint64_t bd0 = descK0 + (uint64_t)(s * (C::K_BYTES >> 4));
          const uint32_t tSb = tS + sb * G;
          if (elect_one()) {
            umma_f16(tSb, descArm, descArm, C::IDESC_ARM_S, 0);
#pragma unroll
            for (int kk = 0; kk < DQ / 32; ++kk) umma_i8(tSb, descQ0 + C::qk_slice(kk, kBM), bd0 + C::qk_slice(kk, G), C::IDESC_QK, 1);
            umma_commit(BAR(B_SFULL + sb));
            umma_commit(BAR(B_KEMPTY + s));
            if (j + 1 == t.nsteps) umma_commit(BAR(B_QEMPTY));
          }
          __syncwarp();
        }
        ++tile_it;
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    {
      // ------------------------------------------------------------------ MMA issuer for O_j = P V
      // A warp of its own, so that a Q K^T whose S buffer is free never queues behind the wait for a P tile.
      // Per step j: [P(j) written] [V(j) landed] [O_j of step j-1 read out] PV(j).
      uint32_t kv_it = 0, tseq = 0;
      bool ok = true;
      const uint64_t descP0 = make_smem_desc(sP, 16, C::SBO_P, C::SWZ_P);
      const uint64_t descV0 = make_smem_desc(sV, C::BYTE_PV ? 16 : G * 128, C::SBO_V, C::SWZ_V);
      while (ok) {
        const int tile = next_tile(tseq, lane == 0, true);
        if (tile < 0) break;
        const TileInfo t = decode_tile<RAGGED, NVH>(p, tile, G);
        for (int j = 0; j < t.nsteps; ++j, ++kv_it) {
          const uint32_t s = kv_it % NSV, ph = (kv_it / NSV) & 1;
          const uint32_t b = kv_it & 1;
          // P(j) written; V(j) landed; full-int8: O_j of the previous step has been read out, half-int8: the
          // accumulator has been brought to this step's running max (and the previous P V has landed in it).
          // (One copy of the wait code for the three.)
#pragma unroll 1
          for (int w = 0; w < 3; ++w) {
            const uint32_t wb = w == 0 ? BAR(B_PFULL + b) : w == 1 ? BAR(B_VFULL + s) : BAR(B_OFREE);
            const uint32_t wp = w == 0 ? ((kv_it >> 1) & 1) : w == 1 ? ph : (FULL ? ((kv_it & 1) ^ 1) : (kv_it & 1));
            ok = mbar_wait_warp(wb, wp, abort_flag, p.status, code_hi | (w == 0 ? PW_PFULL : w == 1 ? PW_VF : PW_OFREE));
            if (!ok) break;
          }
          if (!ok) break;
          tc_fence_after();
          const uint64_t ad0 = descP0 + (uint64_t)(b * (C::P_BYTES >> 4));
          const uint64_t vd0 = descV0 + (uint64_t)(s * (C::V_BYTES >> 4));
          if (elect_one()) {
            if constexpr (FULL) {
              umma_f16(tO, descArm, descArm, C::IDESC_ARM_O, 0);
#pragma unroll
              for (int kk = 0; kk < G / 32; ++kk) umma_i8(tO, ad0 + 2 * kk, vd0 + kk * ((32 * D) >> 4), C::IDESC_PV, 1);
            } else if constexpr (F8V) {
              // e5m2 P x e5m2 V (both one byte, laid out like the int8 tiles), fp32 accumulate straight into the accumulator
              const uint32_t keep = (j > 0 || p.state_in) ? 1u : 0u;
#pragma unroll
              for (int kk = 0; kk < G / 32; ++kk) umma_f8(tA, ad0 + 2 * kk, vd0 + kk * ((32 * D) >> 4), C::IDESC_PV, kk > 0 ? 1u : keep);
            } else {
              // fp16 P (K-major, 64-column blocks of 128-byte rows) x fp16 V (MN-major), fp32 accumulate straight
              // into the accumulator; the first P V of a fresh work item overwrites it
              const uint32_t keep = (j > 0 || p.state_in) ? 1u : 0u;
#pragma unroll
              for (int kk = 0; kk < G / 16; ++kk)
                umma_f16(tA, ad0 + (uint64_t)((kk >> 2) * ((kBM * 128) >> 4) + (kk & 3) * 2), vd0 + (uint64_t)(kk * ((16 * C::V_ROWB) >> 4)),
                         C::IDESC_PV, kk > 0 ? 1u : keep);
            }
            umma_commit(BAR(B_OFULL));
            umma_commit(BAR(B_VEMPTY + s));
            umma_commit(BAR(B_PFREE + b));
          }
          __syncwarp();
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 12) {
    reg_alloc<C::SOFTMAX_REGS>();
#include "intfa_fwd_pipe_softmax.inc"
  } else if (warp >= 12) {
    if constexpr (C::CORR_REGS > kPipeLaunchRegs) reg_alloc<C::CORR_REGS>(); else reg_dealloc<C::CORR_REGS>();
#include "intfa_fwd_pipe_update.inc"
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

