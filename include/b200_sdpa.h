/*
 * b200_sdpa.h -- C ABI of the B200 (sm_100a) fused scaled-dot-product-attention
 * forward (and its backward).
 *
 * This is the drop-in boundary for the one path this library accelerates.  The
 * upstream project reaches its device kernel through a Python/C++ kernel
 * registration layer; the entry points below are what a binding for that path
 * would call instead.  Each declaration names the upstream interface it
 * replaces (path inside the upstream repository : line).
 *
 * Conventions
 *   - plain C types only; every pointer in the parameter blocks is a DEVICE
 *     pointer unless its name says host;
 *   - the library allocates nothing and keeps nothing: the caller owns inputs,
 *     outputs and scratch ("workspace") and must keep them alive until the work
 *     queued on `stream` has finished;
 *   - every call is asynchronous with respect to the host and ordered on the
 *     CUDA stream passed in (a `cudaStream_t` cast to `void*`; NULL = default);
 *   - every function returns a `b200_sdpa_status`; nothing throws, aborts or
 *     traps the GPU.  Device-side waits are bounded; a wait that gave up is
 *     reported through the optional `status` word;
 *   - tensors are 4-D `(B, H, S, D)` described by a base pointer and four
 *     strides counted in ELEMENTS, so transposed views of `(B, S, H, D)` storage
 *     are passed as they are.
 */
#ifndef B200_SDPA_H_
#define B200_SDPA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_SDPA_ABI_VERSION 6

typedef enum b200_sdpa_status {
  B200_SDPA_OK = 0,
  B200_SDPA_ERR_NULL = 1,         /* a required pointer is NULL                     */
  B200_SDPA_ERR_STRUCT = 2,       /* struct_size does not match this library        */
  B200_SDPA_ERR_DTYPE = 3,        /* dtype not one of f32 / f16 / bf16              */
  B200_SDPA_ERR_SHAPE = 4,        /* negative/zero extent, Hq % Hkv != 0, ...       */
  B200_SDPA_ERR_UNSUPPORTED = 5,  /* valid request this build has no kernel for     */
  B200_SDPA_ERR_WORKSPACE = 6,    /* workspace missing or too small                 */
  B200_SDPA_ERR_ALIGNMENT = 7,    /* forced tensor-core path but pointers/strides
                                     do not meet its 16-byte rules                   */
  B200_SDPA_ERR_CUDA = 8,         /* a CUDA runtime/driver call failed              */
  B200_SDPA_ERR_DEVICE = 9,       /* not an sm_100 device                           */
  B200_SDPA_ERR_TIMEOUT = 10,     /* (status word only) a device-side wait gave up  */
  B200_SDPA_ERR_TOO_LARGE = 11,   /* exceeds a fixed-capacity entry point's limit   */
  B200_SDPA_ERR_CACHE_FULL = 12,  /* (status word only) decode with append met a
                                     sequence whose cache is full: its new row was
                                     not stored and not attended to; [1] = batch    */
  B200_SDPA_ERR_BOUNDS = 13       /* (status word only, checked build of the library)
                                     an index left its tensor, a scratch slot its
                                     buffer or a tensor-memory access its columns;
                                     the access was skipped; [1] = site, [2] = index,
                                     [3] = limit                                    */
} b200_sdpa_status;

typedef enum b200_sdpa_dtype {
  B200_SDPA_F32 = 0,
  B200_SDPA_F16 = 1,
  B200_SDPA_BF16 = 2
} b200_sdpa_dtype;

/* Which kernel family served (or must serve) a request. */
typedef enum b200_sdpa_path {
  B200_SDPA_PATH_AUTO = 0,
  B200_SDPA_PATH_GENERIC = 1,  /* CUDA-core fp32-accumulate flash kernel: any dtype,
                                  any strides, additive bias, head dim <= 512        */
  B200_SDPA_PATH_PREFILL = 2,  /* TMA + tcgen05/TMEM warp-specialised kernels:
                                  f16/bf16, E == Dv in {64,128,256} or E = 192
                                  with Dv = 128, unit inner stride; also with an
                                  additive bias of the same dtype that has unit
                                  stride along the keys, S % 8 == 0 and 16-byte
                                  aligned rows                                       */
  B200_SDPA_PATH_DECODE = 3    /* split-KV flash-decoding kernel + combine, L == 1  */
} b200_sdpa_path;

/*
 * One attention problem.
 *
 *   out[b,h,i,:] = softmax_j( scale * q[b,h,i,:].k[b,h/g,j,:] + bias[b,h,i,j] ) . v[b,h/g,j,:]
 *   lse[b,h,i]   = log sum_j exp( ... )                       (natural log, fp32)
 *
 * with g = Hq / Hkv (grouped-query heads: query head h reads kv head h / g).
 * Key j is visible to query row i of batch b iff
 *     j < kv_lens[b]                    (when kv_lens != NULL), and
 *     k_offset + j <= q_offset + i      (when is_causal != 0).
 * A row that sees no key gets out = 0 and lse = -inf.
 *
 * Field semantics follow
 *   torch_neuronx/_sdpa_math.py:51-95          (arithmetic, mask order, dead rows)
 *   torch_neuronx/neuron_dynamo_backend/decompositions.py:2083-2128
 *                                               (GQA head mapping, default scale,
 *                                                bool mask -> additive bias).
 */
typedef struct B200SdpaParams {
  uint32_t struct_size;   /* = sizeof(B200SdpaParams)                                  */
  int32_t dtype;          /* b200_sdpa_dtype of q, k, v and out                        */
  int32_t device;         /* CUDA device ordinal, or -1 to use the current device      */
  int32_t force_path;     /* b200_sdpa_path; AUTO picks the fastest eligible kernel    */

  const void* q;          /* (B, Hq,  L, E)                                            */
  const void* k;          /* (B, Hkv, S, E)                                            */
  const void* v;          /* (B, Hkv, S, Dv)                                           */
  void* out;              /* (B, Hq,  L, Dv), same dtype as q                          */
  float* lse;             /* (B, Hq,  L) fp32, or NULL when not wanted                 */

  int64_t q_stride[4];    /* element strides in (B, H, S, D) order                     */
  int64_t k_stride[4];
  int64_t v_stride[4];
  int64_t out_stride[4];
  int64_t lse_stride[3];  /* (B, H, L)                                                 */

  int32_t B, Hq, Hkv, L, S, E, Dv;
  float scale;            /* multiplies q.k; the caller resolves None -> 1/sqrt(E)     */
  int32_t is_causal;
  int64_t q_offset;       /* global position of query row 0 (blocks of a ring)         */
  int64_t k_offset;       /* global position of key 0                                  */

  const int32_t* kv_lens; /* (B) valid key count per batch (right padding / ragged
                             cache), or NULL = all S keys                              */

  const void* bias;       /* optional additive bias broadcastable to (B,Hq,L,S), or
                             NULL.  The tensor-core kernels read it when it has the
                             query's dtype, unit stride along the keys, S % 8 == 0 and
                             16-byte aligned rows; any other bias runs the generic path */
  int32_t bias_dtype;     /* b200_sdpa_dtype of bias                                   */
  int32_t kv_chunk;       /* decode: keys per split, 0 = library default               */
  int64_t bias_stride[4]; /* 0 for broadcast dimensions                                */

  void* workspace;        /* scratch, b200_sdpa_query_plan() says how much             */
  uint64_t workspace_bytes;
  int32_t* status;        /* optional device int32[4]: [0] = first error code seen by
                             a kernel (0 = none), [1..3] = where; caller zeroes it     */

  /* Paged key/value cache (decode, L == 1, f16/bf16 only); NULL = dense cache.
   * With a block table, k and v point at page pools, k_stride / v_stride are the
   * (page, head, row-in-page, element) strides of a pool, S is the largest context
   * (<= block_table_stride * page_size), kv_lens is required, and key s of batch b
   * is row s % page_size of page block_table[b * block_table_stride + s / page_size].
   * Upstream keeps a dense cache only; this is the layout of the serving engines
   * that would call the decode kernel.                                               */
  const int32_t* block_table;   /* (B, block_table_stride) page numbers               */
  int32_t block_table_stride;
  int32_t page_size;            /* rows per page, a power of two                      */

  /* Decode with append (L == 1, f16/bf16): the key/value row of the token being decoded,
   * (B, Hkv, D) with unit inner stride and (batch, head) element strides that are
   * multiples of 8.  Batch b attends keys [0, kv_lens[b]] -- the new row is key
   * kv_lens[b] -- and the kernel that reads the row also writes it into the cache
   * (dense or paged) at that position, so no separate append pass is needed.  A
   * sequence whose cache is full (kv_lens[b] >= S) appends nothing and reports
   * B200_SDPA_ERR_CACHE_FULL through the status word.  kv_lens is
   * required; kv_lens_out, if given, receives min(kv_lens[b] + 1, S) and must not alias
   * kv_lens.  Both NULL = plain decode.  Upstream appends to the cache with separate
   * ops before calling the attention op.                                              */
  const void* k_new;
  const void* v_new;
  int64_t k_new_stride[2];
  int64_t v_new_stride[2];
  int32_t* kv_lens_out;

  /* Rotary position embedding fused into the append step (needs k_new): q and k_new are
   * rotated by the angles of position kv_lens[b] -- in fp32, rounded to the storage dtype
   * once -- before they are used, and k_new is written to the cache rotated.  rope_cos /
   * rope_sin are fp32 (rope_positions, >= E/2 columns) with rope_stride floats between
   * positions; rope_interleaved = 0 pairs element i with i + E/2 (the "rotate half"
   * convention), 1 pairs 2i with 2i + 1.  NULL = no rotation.  rope_positions (>= 1) is
   * the number of rows in the tables; a length beyond the last row uses the last row's
   * angles rather than reading past the tables, so give tables that cover the cache
   * capacity S.  Upstream applies the embedding with separate ops before the attention
   * op.                                                                               */
  const float* rope_cos;
  const float* rope_sin;
  int32_t rope_stride;
  int32_t rope_interleaved;
  int32_t rope_positions;

  /* Accumulating form (one step of a ring over key/value blocks): instead of writing `out` and
   * `lse`, the kernel folds this call's result into a running fp32 result over earlier key
   * blocks for the same query rows,
   *     lse' = logaddexp(acc_lse, lse)
   *     acc' = acc * exp(acc_lse - lse') + result * exp(lse - lse')
   * in its epilogue, without the partial ever leaving the chip in the storage dtype.
   * acc_mode 0 = off (acc, acc_lse ignored); 1 = first block (acc, acc_lse are overwritten);
   * 2 = fold into acc, acc_lse.  acc is (B, Hq, L, Dv) fp32 with unit inner stride and
   * 16-byte aligned rows, acc_lse (B, Hq, L) fp32; strides in elements.  `out` and `lse` may be
   * NULL then.  Served by the tensor-core prefill kernels (f16/bf16, E = Dv = 128, no
   * bias); b200_sdpa_query_plan() answers B200_SDPA_ERR_UNSUPPORTED otherwise and the caller
   * merges with b200_sdpa_merge() instead.  Replaces the (out, lse) merge upstream's ring does
   * between per-block calls (torch_neuronx/distributed/tensor/cp_ring_handler.py:308-318).  */
  int32_t acc_mode;
  float* acc;
  float* acc_lse;
  int64_t acc_stride[3];      /* (B, H, L)                                             */
  int64_t acc_lse_stride[3];
} B200SdpaParams;

/* What the library would do (or did) for a parameter block. */
typedef struct B200SdpaPlan {
  uint32_t struct_size;   /* = sizeof(B200SdpaPlan)                                    */
  int32_t path;           /* b200_sdpa_path chosen                                     */
  int32_t block_m;        /* query rows per CTA                                        */
  int32_t block_n;        /* keys per inner tile                                       */
  int32_t grid_x, grid_y, grid_z;
  int32_t threads;
  int32_t smem_bytes;     /* dynamic shared memory per CTA                             */
  int32_t kv_splits;      /* decode: splits along the key axis                         */
  int32_t launches;       /* kernels one call enqueues                                 */
  uint64_t workspace_bytes; /* scratch the call needs (0 = none)                       */
} B200SdpaPlan;

/*
 * Merge of two partial attention results over disjoint key sets for the same
 * queries (one ring step):
 *     lse' = logaddexp(acc_lse, part_lse)
 *     acc' = acc * exp(acc_lse - lse') + part * exp(part_lse - lse')
 * `acc` (fp32, (B, Hq, L, Dv) with unit inner stride) and `acc_lse` (fp32, (B, Hq, L)) are
 * updated in place -- they may be views of larger accumulators, hence the strides; when
 * `final_out` is non-NULL the merged rows are also written there in `dtype` with the given
 * strides.
 *
 * Replaces the (out, lse) merge that upstream's templated ring attention does in
 * Python between per-block calls of the op
 * (torch_neuronx/distributed/tensor/cp_ring_handler.py:308-318).
 */
typedef struct B200SdpaMergeParams {
  uint32_t struct_size;
  int32_t dtype;           /* dtype of part and final_out                              */
  int32_t device;
  int32_t first;           /* != 0: acc is uninitialised, just take the partial        */
  float* acc;              /* (B, Hq, L, Dv) fp32, unit inner stride                    */
  float* acc_lse;          /* (B, Hq, L) fp32                                           */
  const void* part;        /* (B, Hq, L, Dv) in dtype                                   */
  const float* part_lse;   /* (B, Hq, L) fp32                                           */
  void* final_out;         /* optional (B, Hq, L, Dv) in dtype                          */
  int64_t part_stride[4];
  int64_t part_lse_stride[3];
  int64_t final_stride[4];
  int32_t B, Hq, L, Dv;
  int64_t acc_stride[3];      /* (B, H, L) element strides of acc                      */
  int64_t acc_lse_stride[3];
} B200SdpaMergeParams;

/*
 * Backward of one attention problem: given the upstream gradient `grad_out` and
 * the forward's inputs, output and log-sum-exp,
 *     P      = exp(scale * q.k^T + bias - lse)      (masked entries and rows with
 *                                                    lse = -inf give 0)
 *     grad_v = P^T grad_out                          summed over the heads of a group
 *     dS     = P * (grad_out v^T - rowsum(grad_out * out))
 *     grad_q = scale * dS k        grad_k = scale * dS^T q   (summed over the group)
 *     grad_bias = dS               (optional, full (B,Hq,L,S), no broadcast reduction)
 * Shapes, masks, offsets and `kv_lens` mean what they mean in B200SdpaParams; the
 * gradients are written with the strides given, so they can take the layout of the
 * tensors they belong to.  Arithmetic is fp32 whatever the storage dtype.
 *
 * Field semantics follow
 *   torch_neuronx/_sdpa_math.py:98-176   (compute_attention_backward)
 *   torch_neuronx/neuron_dynamo_backend/decompositions.py:2535-2598
 *                                         (group expansion and gradient reduction)
 *   torch_neuronx/csrc/core/dispatch/NeuronDispatcher.cpp:2523-2582
 *                                         (gradients laid out like their inputs).
 */
typedef struct B200SdpaBwdParams {
  uint32_t struct_size;    /* = sizeof(B200SdpaBwdParams)                              */
  int32_t dtype;           /* dtype of q, k, v, out, grad_out and all gradients        */
  int32_t device;
  int32_t force_path;      /* AUTO, GENERIC (CUDA-core kernels) or PREFILL (tcgen05 kernels) */

  const void* grad_out;    /* (B, Hq,  L, Dv)                                           */
  const void* q;           /* (B, Hq,  L, E)                                            */
  const void* k;           /* (B, Hkv, S, E)                                            */
  const void* v;           /* (B, Hkv, S, Dv)                                           */
  const void* out;         /* (B, Hq,  L, Dv) forward output                            */
  const float* lse;        /* (B, Hq,  L) fp32 forward log-sum-exp                      */
  void* grad_q;            /* (B, Hq,  L, E)                                            */
  void* grad_k;            /* (B, Hkv, S, E)                                            */
  void* grad_v;            /* (B, Hkv, S, Dv)                                           */
  void* grad_bias;         /* optional (B, Hq, L, S) in dtype, or NULL                  */

  int64_t grad_out_stride[4];
  int64_t q_stride[4];
  int64_t k_stride[4];
  int64_t v_stride[4];
  int64_t out_stride[4];
  int64_t lse_stride[3];
  int64_t grad_q_stride[4];
  int64_t grad_k_stride[4];
  int64_t grad_v_stride[4];
  int64_t grad_bias_stride[4];

  int32_t B, Hq, Hkv, L, S, E, Dv;
  float scale;
  int32_t is_causal;
  int32_t bias_dtype;
  int64_t q_offset;
  int64_t k_offset;
  const int32_t* kv_lens;
  const void* bias;        /* the forward's additive bias, or NULL                      */
  int64_t bias_stride[4];

  void* workspace;         /* scratch of the tensor-core kernels (16-byte aligned);
                              b200_sdpa_bwd_query_plan() says how much.  Without it
                              an AUTO request runs the CUDA-core kernels              */
  uint64_t workspace_bytes;
  int32_t* status;
} B200SdpaBwdParams;

/* ABI version of the loaded library (compare with B200_SDPA_ABI_VERSION). */
int b200_sdpa_abi_version(void);

/* Human-readable text for a status code; never NULL. */
const char* b200_sdpa_strerror(int status);

/*
 * Validate a parameter block and report the kernel, launch geometry and scratch
 * size without launching.  Host-only, no CUDA calls, usable without a GPU.
 * Upstream counterpart: the eligibility gate + kernel configuration lookup
 *   torch_neuronx/neuron_dynamo_backend/decompositions.py:2161-2207
 *   torch_neuronx/nki_hop.py:426-466 (get_kernel_config).
 */
int b200_sdpa_query_plan(const B200SdpaParams* params, B200SdpaPlan* plan);

/*
 * Enqueue the attention forward on `stream`.  Dispatches to the tcgen05 prefill
 * kernel, the split-KV decode kernel or the generic kernel (see b200_sdpa_path).
 * Upstream counterpart: the eager kernel launch
 *   torch_neuronx/csrc/core/NeuronBindings.cpp:900 (_nki_dispatch_eager)
 *   torch_neuronx/nki_hop.py:980-987
 *   torch_neuronx/neuron_dynamo_backend/decompositions.py:2210-2264
 *     (_compute_attention_nki: the kernel call and its LSE post-processing).
 */
int b200_sdpa_fwd(const B200SdpaParams* params, void* stream);

/*
 * Enqueue split-KV flash decoding (L == 1) explicitly: one partial kernel over
 * (batch x kv head x key split) and one combine kernel.  Needs `workspace`.
 * Upstream has no decode-specific kernel; the same op runs with S_q = 1
 *   torch_neuronx/python_ops/torch_mlir/ops/scaled_dot_product_attention.py:64-68.
 */
int b200_sdpa_decode(const B200SdpaParams* params, void* stream);

/*
 * Split-KV flash decoding for callers that cannot supply a workspace.  Same
 * contract and results as b200_sdpa_decode(), except that `workspace` and
 * `workspace_bytes` are ignored: the partial results go to a fixed scratch array
 * that lives inside the library (B200_SDPA_STATIC_SCRATCH_BYTES on every GPU that
 * loads it, until the process ends).  Meant for hosts that gave all device
 * memory to their own pool at start-up, or that run where allocator calls are not
 * allowed; the call itself performs no allocation of any kind.
 *   - a request whose partials need more than the capacity (see `workspace_bytes`
 *     of b200_sdpa_query_plan) returns B200_SDPA_ERR_TOO_LARGE and launches nothing;
 *   - the first call on each device resolves the array's device address; make that
 *     first call outside any stream capture;
 *   - all calls share the one array, which keeps the previous call's contents; the
 *     kernels overwrite every slot they read, but calls that overlap on the GPU
 *     (different streams) race on it -- serialise them.
 * This entry point has no counterpart in the upstream project.
 */
#define B200_SDPA_STATIC_SCRATCH_BYTES (16u << 20)
int b200_sdpa_decode_static(const B200SdpaParams* params, void* stream);

/*
 * Kernel family, launch geometry (grid_x: grad_q kernel, grid_y: grad_k/grad_v kernel)
 * and scratch size of a backward request, without launching.  Host-only.
 * `path` is B200_SDPA_PATH_PREFILL for the tcgen05 kernels (f16/bf16, E == Dv in
 * {64,128}, no grad_bias, a bias only under the forward's rules for that path, unit
 * inner strides, 16-byte aligned bases and outer strides of q, k, v, grad_out and the
 * three gradients) and B200_SDPA_PATH_GENERIC otherwise.
 */
int b200_sdpa_bwd_query_plan(const B200SdpaBwdParams* params, B200SdpaPlan* plan);

/*
 * Enqueue the attention backward on `stream`: a grad_q kernel (which also writes
 * grad_bias) and a grad_k / grad_v kernel, preceded on the tensor-core path by a small
 * row-statistics kernel.  Head dims up to 256 on the CUDA-core path.
 * Upstream counterpart: the backward op's eager launch and CPU definition
 *   torch_neuronx/python_ops/scaled_dot_product_fused_attention.py:511-781
 *   torch_neuronx/csrc/core/dispatch/NeuronDispatcher.cpp:2523-2582 (DispatchSdpaBwdImpl)
 *   torch_neuronx/_sdpa_math.py:98-176.
 */
int b200_sdpa_bwd(const B200SdpaBwdParams* params, void* stream);

/* Enqueue one ring-step merge (see B200SdpaMergeParams). */
int b200_sdpa_merge(const B200SdpaMergeParams* params, void* stream);

/*
 * Launch counters, one per kernel family, so a caller can prove which kernel ran.
 * Upstream counterpart: executed-op tracking
 *   torch_neuronx/__init__.py:528-546, tests/utils/neuron_test_utils.py:18-135.
 * kernel ids: 0 generic, 1 prefill, 2 decode partial, 3 decode combine, 4 merge,
 * 5 backward grad_q, 6 backward grad_k/grad_v, 7 backward row statistics.
 */
uint64_t b200_sdpa_launch_count(int kernel_id);
void b200_sdpa_reset_launch_counts(void);

/*
 * The checked build (the same sources compiled with -DB200_SDPA_DEBUG into
 * libb200_sdpa_checked.so): every global store whose address a kernel computes from
 * decoded indices, every scratch slot and every tensor-memory column range is verified
 * first; a violation puts B200_SDPA_ERR_BOUNDS into the status word and skips the
 * access -- the device never traps.  Upstream counterpart: the debug / bounds-checking
 * runs of its kernels under the simulator; here it is a second library with the same ABI.
 *   b200_sdpa_checked_build()   1 in the checked build, 0 otherwise
 *   b200_sdpa_debug_selftest()  checked build only (B200_SDPA_ERR_UNSUPPORTED otherwise):
 *                               launches one thread that offers the checker an index
 *                               past its limit, so a caller can see the report arrive in
 *                               `status` (device int32[4], zeroed) without any real
 *                               access being wrong.
 */
int b200_sdpa_checked_build(void);
int b200_sdpa_debug_selftest(int device, int32_t* status, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_SDPA_H_ */
