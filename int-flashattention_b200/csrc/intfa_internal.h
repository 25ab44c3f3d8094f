// Internal declarations shared by the translation units of libintfa.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/intfa.h"

namespace intfa {

// Arguments of the attention kernel (plain data, passed by value).
struct KParams {
  const float* qs; const float* ks; const float* vs;
  __half* o;
  long long o_sb, o_sh, o_sn;
  long long qs_sb, qs_sh, ks_sb, ks_sh, vs_sb, vs_sh, vs_sd;
  int B, H, Nq, Nk;
  int dh;                        // head dim of the tensors in memory (16 runs the 32-wide kernel on zero-filled tiles,
                                 // 256 the 128-wide one twice per query tile, once per half of the V channels)
  int hk_ratio;                  // query heads per K/V head (1 unless grouped-query attention)
  int o_bf16;                    // output element type: 0 fp16, 1 bf16
  int causal;
  float c;                       // sm_scale * 1.44269504 (fp32)
  long long q_off, kv_off;
  float* lse; float* st_m; float* st_l; float* st_acc;
  int state_in, state_out, write_o;
  int* dbg_s; void* dbg_p; int dbg_tile, dbg_step;
  int* status;
  int MB, num_tiles;
  int wait_limit_kcycles;        // bounded waits give up after this many thousand SM cycles
  int skip_k_load;               // test hook: 1-based KV step whose K tile the producer leaves out; 0: none
  int kv_desc;                   // 1: KV tiles visited last-to-first
  long long vs_sblk;             // element stride of the KV-tile axis of v_scale; 0: one scale row per (batch, head)
  unsigned int* tile_counter;    // zeroed word the CTAs draw work-item indices from
};

// Records the calling thread's last error (printf-style) and returns `code`.
int set_error(int code, const char* fmt, ...);
// SM count of the current device, cached per device; <=0 on failure.
int sm_count_cached();

int fwd_dispatch(const IntfaFwdParams* a, cudaStream_t stream);
int quant_pertoken(const void* x, const int64_t* st, void* x8, float* scale, int B, int H, int N, int D,
                   cudaStream_t stream);
int quant_v(const void* v, const int64_t* st, void* v8, float* scale, int mode, int B, int H, int N, int D,
            void* workspace, cudaStream_t stream);
int v_colmax(const void* v, const int64_t* st, void* colmax, int B, int H, int N, int D, cudaStream_t stream);
int v_quant_from_colmax(const void* v, const int64_t* st, const void* colmax, void* v8, float* scale, int mode, int B,
                        int H, int N, int D, cudaStream_t stream);
constexpr int kStaticColmaxWords = 65536;   // 256 KiB: built-in scratch of intfa_quant_v_static (B*H*D limit)
int quant_v_static(const void* v, const int64_t* st, void* v8, float* scale, int mode, int B, int H, int N, int D,
                   cudaStream_t stream);
size_t quant_qkv_workspace_bytes(int B, int Hkv, int Nk, int D);
int quant_qkv(const void* q, const void* k, const void* v, const int64_t* v_st, void* q8, void* k8, void* v8, float* qs,
              float* ks, float* vs, int mode, int B, int H, int Hkv, int Nq, int Nk, int D, void* workspace,
              cudaStream_t stream);
int scales_f16_to_f32(const void* src, float* dst, long long n, cudaStream_t stream);

}  // namespace intfa
