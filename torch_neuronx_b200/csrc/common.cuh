// Shared device-side declarations for the sm_100a SDPA kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/b200_sdpa.h"

namespace b200 {

// Problem description handed to kernels by value (a trimmed copy of
// B200SdpaParams with derived fields).
struct Problem {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  int64_t qs[4], ks[4], vs[4], os[4];
  int64_t ls[3];
  int B, Hq, Hkv, L, S, E, Dv;
  int group;            // Hq / Hkv
  float scale;
  int causal;
  int64_t causal_shift; // q_offset - k_offset: key j visible iff j <= i + causal_shift
  const int* kv_lens;
  const void* bias;
  int bias_dtype;
  int64_t bs[4];
  int* status;
  // Paged key/value cache (decode only): when block_table is set, k and v point at page
  // pools, ks/vs hold (page, head, row-in-page, element) strides and key s of batch b lives
  // in page block_table[b * table_stride + (s >> page_shift)] at row s & (page_size - 1).
  const int* block_table;
  int table_stride;
  int page_shift;
  // Decode with append: the key/value row of the token being decoded arrives separately
  // ((B, Hkv, D), unit inner stride); it is attended to as key kv_lens[b] and written into the
  // cache at that position by the CTA that reads it.  lens_out (if set, not aliasing kv_lens)
  // receives the new lengths.
  const void* k_new;
  const void* v_new;
  int64_t kns[2], vns[2];
  int* lens_out;
  // Rotary position embedding fused into the append step: q and k_new are rotated by the angles of
  // position kv_lens[b] before use (and k_new is stored rotated); cos/sin are fp32 (positions, D/2).
  const float* rope_cos;
  const float* rope_sin;
  int rope_stride;       // floats between positions
  int rope_interleaved;  // 0: pairs (i, i + D/2); 1: pairs (2i, 2i + 1)
  int rope_positions;    // rows in the cos/sin tables (positions beyond use the last row)
  // Accumulating form (persistent prefill kernel only): fold the result into a running fp32 (acc, acc_lse)
  // instead of writing out / lse.  0 = off, 1 = first block, 2 = merge.
  int acc_mode;
  float* acc;
  float* acc_lse;
  int64_t as[3], als[3];
};

// Backward: the forward's description (out and lse are inputs here) plus the upstream
// gradient and the four gradient outputs.
struct BwdProblem {
  Problem f;
  const void* dout;
  int64_t dos[4];
  void* dq;
  void* dk;
  void* dv;
  void* dbias;  // optional: gradient of the logits, (B, Hq, L, S)
  int64_t dqs[4], dks[4], dvs[4], dbs[4];
};

enum KernelId {
  KID_GENERIC = 0,
  KID_PREFILL = 1,
  KID_DECODE = 2,
  KID_COMBINE = 3,
  KID_MERGE = 4,
  KID_BWD_DQ = 5,
  KID_BWD_DKV = 6,
  KID_BWD_PREP = 7,
  KID_COUNT = 8
};

// Host launchers implemented in the per-kernel translation units.  Each returns
// a b200_sdpa_status and never synchronises.
int launch_generic(const Problem& p, int dtype, cudaStream_t stream);
int plan_generic(const Problem& p, int dtype, B200SdpaPlan* plan);

int launch_decode(const Problem& p, int dtype, int kv_chunk, void* workspace, uint64_t workspace_bytes,
                  cudaStream_t stream);
int plan_decode(const Problem& p, int dtype, int kv_chunk, B200SdpaPlan* plan);
bool decode_eligible(const Problem& p, int dtype);
bool decode_mma_eligible(const Problem& p, int dtype);
int launch_decode_partial_mma(const Problem& p, int dtype, int chunk, int nsplit, float* part_o, float* part_ml,
                              cudaStream_t stream);
int launch_decode_static(const Problem& p, int dtype, int kv_chunk, cudaStream_t stream);

// `workspace` (optional, >= 4 bytes): the counter from which the persistent CTAs draw their work items
int launch_prefill(const Problem& p, int dtype, void* workspace, uint64_t workspace_bytes, cudaStream_t stream);
int plan_prefill(const Problem& p, int dtype, B200SdpaPlan* plan);
bool prefill_eligible(const Problem& p, int dtype, bool* alignment_only_failure);
// persistent form of the prefill kernel (prefill_persistent_sm100.cu): head dimension 128, large problems
bool prefill_persistent_wanted(const Problem& p);
bool prefill_accumulate_eligible(const Problem& p);   // accumulating form: layout rules of (acc, acc_lse)
void plan_prefill_persistent(const Problem& p, B200SdpaPlan* plan);
int launch_prefill_persistent(const Problem& p, int dtype, void* workspace, uint64_t workspace_bytes, cudaStream_t stream);
// unequal head dimensions (E = 192, Dv = 128): prefill_wide_sm100.cu
bool prefill_wide_eligible(const Problem& p, int dtype, bool* alignment_only_failure);
int plan_prefill_wide(const Problem& p, int dtype, B200SdpaPlan* plan);
int launch_prefill_wide(const Problem& p, int dtype, cudaStream_t stream);

int launch_merge(const B200SdpaMergeParams& m, cudaStream_t stream);

int launch_bwd_generic(const BwdProblem& bp, int dtype, cudaStream_t stream);
int plan_bwd_generic(const BwdProblem& bp, int dtype, B200SdpaPlan* plan);
bool bwd_tc_eligible(const BwdProblem& bp, int dtype, bool* alignment_only_failure);
uint64_t bwd_tc_workspace_bytes(const BwdProblem& bp);
int plan_bwd_tc(const BwdProblem& bp, int dtype, B200SdpaPlan* plan);
int launch_bwd_tc(const BwdProblem& bp, int dtype, void* workspace, uint64_t workspace_bytes, cudaStream_t stream);

void count_launch(int kernel_id);

// ---- small device helpers -------------------------------------------------

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float load_as_f32(const void* base, int64_t idx, int dtype) {
  if (dtype == B200_SDPA_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == B200_SDPA_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

// Number of keys batch b may look at (right padding / ragged cache).
__device__ __forceinline__ int valid_keys(const Problem& p, int b) {
  int n = p.S;
  if (p.kv_lens != nullptr) {
    int len = p.kv_lens[b];
    len = len < 0 ? 0 : len;
    if (p.k_new != nullptr) ++len;   // the appended row counts
    n = len < n ? len : n;
  }
  return n;
}

}  // namespace b200
