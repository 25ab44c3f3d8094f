/*
 * intfa.h -- C ABI of the B200 (sm_100a) INT8 FlashAttention forward library (libintfa.so).
 *
 * Plain C types only: device pointers, sizes, element strides.  Every function
 * returns an int status (0 = ok, negative = error, see INTFA_ERR_*) and never
 * throws or aborts; intfa_last_error() gives the message of the calling thread's
 * last failure.  All launches are asynchronous on the CUDA stream passed in
 * (`stream` is a cudaStream_t cast to void*, NULL = the default stream) on the
 * CURRENT device; the caller owns every buffer.
 *
 * Each entry point names the reference interface it stands in for
 * (paths relative to the reference project root).
 */
#ifndef INTFA_H_
#define INTFA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INTFA_OK                 0
#define INTFA_ERR_INVALID_ARG   -1   /* null pointer, bad enum, misaligned pointer or stride */
#define INTFA_ERR_UNSUPPORTED   -2   /* shape the sm_100a kernels do not cover (there is no fallback) */
#define INTFA_ERR_CUDA          -3   /* a CUDA runtime/driver call failed */
#define INTFA_ERR_DEVICE_WAIT   -4   /* a bounded device-side wait ran out (read back from `status`) */
#define INTFA_ERR_TOO_LARGE     -5   /* size beyond a fixed built-in limit */

#define INTFA_VARIANT_FULL 0         /* int8 Q/K/V, int8 P  (flash_atten_full_int8.py) */
#define INTFA_VARIANT_HALF 1         /* int8 Q/K, fp16 V, fp16 P (flash_atten_int8.py)  */
#define INTFA_VARIANT_HALF_FP8 2     /* int8 Q/K, float8_e5m2 V and P (flash_atten_int8.py:55-56); v is one byte per element */

#define INTFA_OUT_FP16 0             /* o as fp16: the Triton ops (flash_atten_full_int8.py:194-195) */
#define INTFA_OUT_BF16 1             /* o as bf16: csrc/flash_fwd_hdim128_bf16_sm80_{full,half}_qi8.cu */

#define INTFA_VSCALE_PER_TENSOR  0   /* one V scale per (batch, head): benchmark.py:102-107 */
#define INTFA_VSCALE_PER_CHANNEL 1   /* one V scale per (batch, head, channel)              */

/* Library version (major*10000 + minor*100 + patch). */
int intfa_version(void);

/* Copies the calling thread's last error message (NUL terminated) into buf. */
int intfa_last_error(char* buf, size_t len);

/*
 * Arguments of one attention forward launch.
 * Replaces: the positional arguments + stride list the reference passes to its
 * Triton kernels (flash_atten_full_int8.py:204-216, flash_atten_int8.py:199-210)
 * and the Qkv_params/Flash_fwd_params block of its CUDA path (csrc/flash.h:24-159).
 *
 * Tensors are [B, H, N, D]; strides are in ELEMENTS for dims (B, H, N); the last
 * dim must be contiguous.  q,k: int8.  v: int8 (FULL) or fp16 (HALF).  o: fp16.
 * Byte strides of q/k/v and their base pointers must be multiples of 16 (TMA).
 * q_scale [B,H,Nq], k_scale [B,H,Nk]: fp32, contiguous over N, strides for (B,H).
 * v_scale (FULL only): fp32, element strides for (B,H,D); stride 0 over D
 * broadcasts a per-(batch,head) scale.
 */
typedef struct IntfaFwdParams {
  const void*  q;  const void* k;  const void* v;  void* o;
  const float* q_scale;  const float* k_scale;  const float* v_scale;
  int64_t q_stride[3];  int64_t k_stride[3];  int64_t v_stride[3];  int64_t o_stride[3];
  int64_t qs_stride[2]; int64_t ks_stride[2]; int64_t vs_stride[3];
  int32_t B, H, Nq, Nk, D;      /* D in {16,32,64,128,256} (flash_atten_full_int8.py:193).  Nq, Nk need not be multiples of the tile sizes (128 rows, G
                                   columns): the last tiles are masked (csrc/mask.h:277-285); but every row of
                                   k_scale must be ALLOCATED up to the next multiple of G floats (the values past
                                   Nk are ignored) -- the scales of a KV step are fetched G at a time */
  int32_t variant;              /* INTFA_VARIANT_* */
  int32_t causal;               /* 0/1; mask is (kv_offset + col) <= (q_offset + row) */
  float   sm_scale;             /* natural-log softmax scale; kernel multiplies by 1.44269504 */
  int32_t G;                    /* running-max column granularity = KV tile width: 64 or 128 (32 as well for
                                   full-int8 at D<=32; half-int8 at D=256: 64 only)
                                   (the reference's BLOCK_N; full-int8 results depend on it).  The
                                   reference only allows BLOCK_N <= HEAD_DIM (flash_atten_full_int8.py:88);
                                   G=128 with D=64 is accepted here as a faster granularity of its own. */
  int32_t p_round;              /* 0: fp16(p)*127+0.5 truncated (Triton op); 1: fp32 p*127 RNE (CUDA path) */
  int64_t q_offset, kv_offset;  /* global position of row 0 / column 0 (ring attention); 0 otherwise */
  /* optional outputs / carried state, all fp32 and contiguous: m,l,lse [B,H,Nq]; acc [B,H,Nq,D].
     full-int8 with one v_scale row per (batch, head): the carried acc is in units of v_scale[ch]/127 (the
     channel factor is applied when o is written); it is only meaningful to a later call with the same v_scale. */
  float*  lse_out;              /* log2-domain LSE  m + log2(l)  (flash_atten_int8.py:172), or NULL */
  float*  state_m; float* state_l; float* state_acc;
  int32_t state_in;             /* 1: start from (m,l,acc) in state_* instead of (-inf,1,0) */
  int32_t state_out;            /* 1: write (m,l,acc) back to state_* after the last KV tile */
  int32_t write_o;              /* 1: write o = fp16(acc/l) (and lse_out if set) */
  /* debug taps for bit-exact checks of one tile: raw int32 QK^T and int8/fp16 P of KV step
     dbg_step of work item dbg_tile (= (b*H+h)*(Nq/128) + m_block); both [128, G]; NULL = off */
  int32_t* dbg_s; void* dbg_p; int32_t dbg_tile; int32_t dbg_step;
  int32_t* status;              /* device int32, zeroed by the caller; a device-side wait that runs
                                   out stores a non-zero code here.  May be NULL. */
  int32_t H_kv;                 /* grouped-query / multi-query attention: number of K/V heads; k, v and
                                   their scales are [B,H_kv,...], query head h reads K/V head h / (H/H_kv)
                                   (h_h_k_ratio, csrc/flash.h:60-63, csrc/flash_fwd_kernel_full_qi8.h:141-160).
                                   0 means H.  H must be a multiple of H_kv. */
  int32_t o_dtype;              /* INTFA_OUT_*: element type of o (2 bytes either way) */
  int32_t kv_order;             /* 0: KV tiles visited ascending (the Triton ops, flash_atten_full_int8.py:30);
                                   1: descending, last tile first (the CUDA path's loop,
                                   csrc/flash_fwd_kernel_full_qi8.h:331-469).  The full-int8 result depends on it. */
  int64_t vs_stride_blk;        /* 0: v_scale is [B,H_kv,D] (or [B,H_kv] via stride 0).  Otherwise v_scale is
                                   [B,H_kv,ceil(Nk/G),D]: one scale row per KV tile of G keys and channel, the CUDA
                                   path's layout (csrc/flash_fwd_kernel_full_qi8.h:156-160,348,399,
                                   csrc/mask.h:313-340); this is the element stride of the tile axis. */
  /* Test hooks for the bounded device-side waits (both 0 in normal use).  debug_wait_limit_kcycles: give up a wait
     after this many thousand SM cycles instead of about a second.  debug_skip_k_load = n > 0: the producer leaves
     out the K tile of the n-th KV step the CTA runs, so the wait for it runs out, the CTA drains and `status`
     receives the wait's code -- the path a lost transfer would take. */
  int32_t debug_wait_limit_kcycles; int32_t debug_skip_k_load;
} IntfaFwdParams;

/*
 * One INT8 attention forward.
 * Replaces: _attention_full_int8.forward / _attention_int8.forward
 * (flash_atten_full_int8.py:184-221, flash_atten_int8.py:178-215) and
 * run_mha_fwd_{full,half}_qi8_<T,128> (csrc/flash.h:206-207,
 * csrc/flash_fwd_launch_template.h:116-191,469-523).
 */
int intfa_fwd(const IntfaFwdParams* p, void* stream);

/*
 * Fused quantisation prologue: fp16 -> int8 with absmax scales.
 * Replaces: quant_pertoken (benchmark.py:96-100) for q and k, and quant_pertensor
 * (benchmark.py:102-107) / its per-channel generalisation for v, bit-exactly
 * (fp16 scale = fp16(absmax/127), value = rint(fp16(x / scale))); scales are
 * stored as fp32 holding the fp16-representable value.  An all-zero row/column
 * yields value 0 and scale 0 (the reference divides 0/0 there).
 *
 * x: fp16 [B,H,N,D] with element strides for (B,H,N), last dim contiguous and
 * 16-byte aligned rows.  Outputs are contiguous.
 */
int intfa_quant_pertoken(const void* x, const int64_t x_stride[3],
                         void* x8, float* scale,
                         int32_t B, int32_t H, int32_t N, int32_t D, void* stream);

/* Bytes of zero-initialisable scratch intfa_quant_v needs (any mode). */
size_t intfa_quant_v_workspace_bytes(int32_t B, int32_t H, int32_t D);

/*
 * v: fp16 [B,H,N,D] -> v8 int8 + scale.  mode PER_TENSOR writes scale [B,H],
 * PER_CHANNEL writes scale [B,H,D].  `workspace` is caller-provided device
 * scratch of intfa_quant_v_workspace_bytes(); the call clears it itself.
 * Replaces: quant_pertensor (benchmark.py:102-107).
 */
int intfa_quant_v(const void* v, const int64_t v_stride[3],
                  void* v8, float* scale, int32_t mode,
                  int32_t B, int32_t H, int32_t N, int32_t D,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * The two halves of intfa_quant_v, for a V tensor whose token axis is sharded over devices:
 * intfa_v_colmax accumulates (atomic max) the column absmax of the local shard into
 * `colmax` (B*H*D words holding fp32 bit patterns, which the CALLER zeroes first and may
 * max-reduce across devices as int32); intfa_v_quant_from_colmax then quantises with it.
 * Replaces: quant_pertensor (benchmark.py:102-107) applied to the unsharded tensor.
 */
int intfa_v_colmax(const void* v, const int64_t v_stride[3], void* colmax,
                   int32_t B, int32_t H, int32_t N, int32_t D, void* stream);
int intfa_v_quant_from_colmax(const void* v, const int64_t v_stride[3], const void* colmax,
                              void* v8, float* scale, int32_t mode,
                              int32_t B, int32_t H, int32_t N, int32_t D, void* stream);

/*
 * The whole quantisation prologue of one attention call in TWO launches and no memset: the first quantises the rows
 * of q and of k per token (as intfa_quant_pertoken) and, in the same grid, takes the column absmax of v chunk by
 * chunk into `workspace` (partial maxima, plain stores -- nothing to clear); the second quantises v (as
 * intfa_quant_v).  Results are bit-identical to the separate entry points.
 * Replaces: quant_pertoken(q), quant_pertoken(k), quant_pertensor(v) as benchmark.py:158-160 calls them in a row.
 * q [B,H,Nq,D] and k [B,H_kv,Nk,D]: fp16, CONTIGUOUS; v [B,H_kv,Nk,D]: fp16 with element strides for (B,H,N), or
 * NULL (half-int8: V stays fp16) -- then v8, v_scale, workspace are not used.  `workspace`: device scratch of
 * intfa_quant_qkv_workspace_bytes() bytes, contents irrelevant.
 */
size_t intfa_quant_qkv_workspace_bytes(int32_t B, int32_t H_kv, int32_t Nk, int32_t D);
int intfa_quant_qkv(const void* q, const void* k, const void* v, const int64_t v_stride[3],
                    void* q8, void* k8, void* v8, float* q_scale, float* k_scale, float* v_scale, int32_t v_mode,
                    int32_t B, int32_t H, int32_t H_kv, int32_t Nq, int32_t Nk, int32_t D,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * intfa_quant_v for callers that cannot allocate device memory.
 * No counterpart in the reference (its quantisers are PyTorch expressions that allocate freely).
 *
 * Some hosts of this library -- a plug-in running inside another runtime's memory pool, a callback
 * on a serving thread that may not call cudaMalloc, code between the capture points of a larger
 * pipeline -- have nowhere to get the B*H*D-word scratch that intfa_quant_v asks for.  This variant
 * takes the same inputs and outputs and no workspace: the column-absmax scratch is a fixed array
 * inside the library image (256 KiB on every GPU that loads the library, held until the process
 * exits).  It calls no cudaMalloc/cudaFree and no allocating library routine.
 *
 *  - Limit: B*H*D <= intfa_quant_v_static_max_words() (65536); larger shapes get INTFA_ERR_TOO_LARGE
 *    and should use intfa_quant_v.
 *  - The first call on each device looks the array's device address up (cudaGetSymbolAddress with
 *    that device current) and remembers it; make that first call before any stream capture begins.
 *  - All calls on a device share the one array.  Each call clears the part it uses (the array keeps
 *    the previous call's maxima), so calls issued one after another on a stream are fine, but two
 *    calls that can overlap on the GPU (different streams, no dependency) race on it and must be
 *    serialised by the caller.
 * Results are bit-identical to intfa_quant_v.
 */
int intfa_quant_v_static(const void* v, const int64_t v_stride[3],
                         void* v8, float* scale, int32_t mode,
                         int32_t B, int32_t H, int32_t N, int32_t D, void* stream);
size_t intfa_quant_v_static_max_words(void);

/* Widens fp16 scales (as benchmark.py produces them) to the fp32 the kernel reads
 * (promotion done in-kernel by the reference, flash_atten_full_int8.py:37-38). n elements. */
int intfa_scales_f16_to_f32(const void* src_f16, float* dst_f32, int64_t n, void* stream);

/* Number of SMs of the current device (persistent-grid sizing); <0 on error. */
int intfa_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif  /* INTFA_H_ */
