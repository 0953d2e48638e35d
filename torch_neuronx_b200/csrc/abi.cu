// C ABI of the library: validation, kernel selection and launch bookkeeping.
// See include/b200_sdpa.h for the contract of every entry point.
#include "common.cuh"
#include "debug.cuh"

#include <atomic>

namespace b200 {

namespace {

std::atomic<uint64_t> g_launches[KID_COUNT];

int validate(const B200SdpaParams* a, Problem* p) {
  if (a == nullptr) return B200_SDPA_ERR_NULL;
  if (a->struct_size != sizeof(B200SdpaParams)) return B200_SDPA_ERR_STRUCT;
  if (a->dtype != B200_SDPA_F32 && a->dtype != B200_SDPA_F16 && a->dtype != B200_SDPA_BF16) return B200_SDPA_ERR_DTYPE;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->L <= 0 || a->S < 0 || a->E <= 0 || a->Dv <= 0)
    return B200_SDPA_ERR_SHAPE;
  if (a->Hq % a->Hkv != 0) return B200_SDPA_ERR_SHAPE;
  if (a->acc_mode < 0 || a->acc_mode > 2) return B200_SDPA_ERR_UNSUPPORTED;
  if (a->q == nullptr || (a->out == nullptr && a->acc_mode == 0)) return B200_SDPA_ERR_NULL;
  if (a->acc_mode != 0 && (a->acc == nullptr || a->acc_lse == nullptr)) return B200_SDPA_ERR_NULL;
  if (a->S > 0 && (a->k == nullptr || a->v == nullptr)) return B200_SDPA_ERR_NULL;
  if (a->bias != nullptr && a->bias_dtype != B200_SDPA_F32 && a->bias_dtype != B200_SDPA_F16 &&
      a->bias_dtype != B200_SDPA_BF16)
    return B200_SDPA_ERR_DTYPE;
  p->q = a->q;
  p->k = a->k;
  p->v = a->v;
  p->out = a->out;
  p->lse = a->lse;
  for (int i = 0; i < 4; ++i) {
    p->qs[i] = a->q_stride[i];
    p->ks[i] = a->k_stride[i];
    p->vs[i] = a->v_stride[i];
    p->os[i] = a->out_stride[i];
    p->bs[i] = a->bias_stride[i];
  }
  for (int i = 0; i < 3; ++i) p->ls[i] = a->lse_stride[i];
  p->B = a->B;
  p->Hq = a->Hq;
  p->Hkv = a->Hkv;
  p->L = a->L;
  p->S = a->S;
  p->E = a->E;
  p->Dv = a->Dv;
  p->group = a->Hq / a->Hkv;
  p->scale = a->scale;
  p->causal = a->is_causal != 0;
  p->causal_shift = a->q_offset - a->k_offset;
  p->kv_lens = a->kv_lens;
  p->bias = a->bias;
  p->bias_dtype = a->bias_dtype;
  p->status = a->status;
  p->block_table = a->block_table;
  p->table_stride = a->block_table_stride;
  p->page_shift = 0;
  p->k_new = a->k_new;
  p->v_new = a->v_new;
  p->lens_out = a->kv_lens_out;
  for (int i = 0; i < 2; ++i) {
    p->kns[i] = a->k_new_stride[i];
    p->vns[i] = a->v_new_stride[i];
  }
  p->rope_cos = a->rope_cos;
  p->rope_sin = a->rope_sin;
  p->rope_stride = a->rope_stride;
  p->rope_interleaved = a->rope_interleaved != 0;
  p->rope_positions = a->rope_positions;
  if (a->rope_cos != nullptr && a->rope_positions < 1) return B200_SDPA_ERR_SHAPE;
  p->acc_mode = a->acc_mode;
  p->acc = a->acc;
  p->acc_lse = a->acc_lse;
  for (int i = 0; i < 3; ++i) {
    p->as[i] = a->acc_stride[i];
    p->als[i] = a->acc_lse_stride[i];
  }
  if ((a->rope_cos == nullptr) != (a->rope_sin == nullptr)) return B200_SDPA_ERR_NULL;
  if (a->rope_cos != nullptr && (a->k_new == nullptr || a->rope_stride < a->E / 2)) return B200_SDPA_ERR_UNSUPPORTED;
  if ((a->k_new == nullptr) != (a->v_new == nullptr)) return B200_SDPA_ERR_NULL;
  if (a->k_new != nullptr) {
    if (a->kv_lens == nullptr) return B200_SDPA_ERR_NULL;
    if (a->kv_lens_out != nullptr && a->kv_lens_out == a->kv_lens) return B200_SDPA_ERR_UNSUPPORTED;
  }
  if (a->block_table != nullptr) {
    const int ps = a->page_size;
    if (ps < 1 || (ps & (ps - 1)) != 0 || a->block_table_stride < 1) return B200_SDPA_ERR_SHAPE;
    if (a->kv_lens == nullptr) return B200_SDPA_ERR_NULL;
    if (static_cast<int64_t>(a->S) > static_cast<int64_t>(a->block_table_stride) * ps) return B200_SDPA_ERR_SHAPE;
    while ((1 << p->page_shift) < ps) ++p->page_shift;
  }
  return B200_SDPA_OK;
}

// Kernel selection.  `have_workspace` is false when only planning.
int choose(const B200SdpaParams* a, const Problem& p, int* path) {
  const int want = a->force_path;
  if (want != B200_SDPA_PATH_AUTO && want != B200_SDPA_PATH_GENERIC && want != B200_SDPA_PATH_PREFILL &&
      want != B200_SDPA_PATH_DECODE)
    return B200_SDPA_ERR_UNSUPPORTED;
  if (p.acc_mode != 0) {
    // the accumulating form exists in the persistent tensor-core prefill kernel only
    bool unused = false;
    if ((want != B200_SDPA_PATH_AUTO && want != B200_SDPA_PATH_PREFILL) || p.block_table != nullptr ||
        p.k_new != nullptr || p.S < 1 || !prefill_eligible(p, a->dtype, &unused) || !prefill_accumulate_eligible(p))
      return B200_SDPA_ERR_UNSUPPORTED;
    *path = B200_SDPA_PATH_PREFILL;
    return B200_SDPA_OK;
  }
  if (p.block_table != nullptr || p.k_new != nullptr) {
    // a paged cache and the append of a new row are only understood by the split-KV decode kernel
    if ((want != B200_SDPA_PATH_AUTO && want != B200_SDPA_PATH_DECODE) || !decode_eligible(p, a->dtype))
      return B200_SDPA_ERR_UNSUPPORTED;
    *path = B200_SDPA_PATH_DECODE;
    return B200_SDPA_OK;
  }
  if (want == B200_SDPA_PATH_GENERIC) {
    *path = want;
    return B200_SDPA_OK;
  }
  if (want == B200_SDPA_PATH_DECODE) {
    if (!decode_eligible(p, a->dtype)) return B200_SDPA_ERR_UNSUPPORTED;
    *path = want;
    return B200_SDPA_OK;
  }
  bool align_only = false;
  const bool pre = prefill_eligible(p, a->dtype, &align_only);
  if (want == B200_SDPA_PATH_PREFILL) {
    if (!pre) return align_only ? B200_SDPA_ERR_ALIGNMENT : B200_SDPA_ERR_UNSUPPORTED;
    *path = want;
    return B200_SDPA_OK;
  }
  if (decode_eligible(p, a->dtype)) {
    *path = B200_SDPA_PATH_DECODE;
  } else if (pre) {
    *path = B200_SDPA_PATH_PREFILL;
  } else {
    *path = B200_SDPA_PATH_GENERIC;
  }
  return B200_SDPA_OK;
}

// Makes the requested device current for the duration of one entry point and puts the caller's
// device back afterwards (a library call must not change which device the host thread is on).
// Also the one place that checks the compute capability: every kernel here is sm_100a code.
class DeviceScope {
 public:
  explicit DeviceScope(int device) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) {
      cudaGetLastError();
      rc_ = B200_SDPA_ERR_CUDA;
      return;
    }
    int want = device < 0 ? cur : device;
    if (want != cur) {
      if (cudaSetDevice(want) != cudaSuccess) {
        cudaGetLastError();
        rc_ = B200_SDPA_ERR_CUDA;
        return;
      }
      restore_ = cur;
    }
    rc_ = is_sm100(want) ? B200_SDPA_OK : B200_SDPA_ERR_DEVICE;
  }
  ~DeviceScope() {
    if (restore_ >= 0 && cudaSetDevice(restore_) != cudaSuccess) cudaGetLastError();
  }
  DeviceScope(const DeviceScope&) = delete;
  DeviceScope& operator=(const DeviceScope&) = delete;
  int status() const { return rc_; }

 private:
  static bool is_sm100(int dev) {
    constexpr int kMax = 64;
    static std::atomic<int> known[kMax];   // 0 = not asked yet, 1 = sm_100, 2 = something else
    if (dev >= 0 && dev < kMax) {
      const int k = known[dev].load(std::memory_order_relaxed);
      if (k != 0) return k == 1;
    }
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (dev >= 0 && dev < kMax) known[dev].store(major == 10 ? 1 : 2, std::memory_order_relaxed);
    return major == 10;
  }
  int restore_ = -1;
  int rc_ = B200_SDPA_OK;
};

int validate_bwd(const B200SdpaBwdParams* a, BwdProblem& bp) {
  if (a == nullptr) return B200_SDPA_ERR_NULL;
  if (a->struct_size != sizeof(B200SdpaBwdParams)) return B200_SDPA_ERR_STRUCT;
  if (a->dtype != B200_SDPA_F32 && a->dtype != B200_SDPA_F16 && a->dtype != B200_SDPA_BF16) return B200_SDPA_ERR_DTYPE;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->L <= 0 || a->S < 0 || a->E <= 0 || a->Dv <= 0)
    return B200_SDPA_ERR_SHAPE;
  if (a->Hq % a->Hkv != 0) return B200_SDPA_ERR_SHAPE;
  if (a->grad_out == nullptr || a->q == nullptr || a->out == nullptr || a->lse == nullptr || a->grad_q == nullptr)
    return B200_SDPA_ERR_NULL;
  if (a->S > 0 && (a->k == nullptr || a->v == nullptr || a->grad_k == nullptr || a->grad_v == nullptr))
    return B200_SDPA_ERR_NULL;
  if (a->bias != nullptr && a->bias_dtype != B200_SDPA_F32 && a->bias_dtype != B200_SDPA_F16 &&
      a->bias_dtype != B200_SDPA_BF16)
    return B200_SDPA_ERR_DTYPE;
  Problem& p = bp.f;
  p.q = a->q;
  p.k = a->k;
  p.v = a->v;
  p.out = const_cast<void*>(a->out);
  p.lse = const_cast<float*>(a->lse);
  bp.dout = a->grad_out;
  bp.dq = a->grad_q;
  bp.dk = a->grad_k;
  bp.dv = a->grad_v;
  bp.dbias = a->grad_bias;
  for (int i = 0; i < 4; ++i) {
    p.qs[i] = a->q_stride[i];
    p.ks[i] = a->k_stride[i];
    p.vs[i] = a->v_stride[i];
    p.os[i] = a->out_stride[i];
    p.bs[i] = a->bias_stride[i];
    bp.dos[i] = a->grad_out_stride[i];
    bp.dqs[i] = a->grad_q_stride[i];
    bp.dks[i] = a->grad_k_stride[i];
    bp.dvs[i] = a->grad_v_stride[i];
    bp.dbs[i] = a->grad_bias_stride[i];
  }
  for (int i = 0; i < 3; ++i) p.ls[i] = a->lse_stride[i];
  p.B = a->B;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.L = a->L;
  p.S = a->S;
  p.E = a->E;
  p.Dv = a->Dv;
  p.group = a->Hq / a->Hkv;
  p.scale = a->scale;
  p.causal = a->is_causal != 0;
  p.causal_shift = a->q_offset - a->k_offset;
  p.kv_lens = a->kv_lens;
  p.bias = a->bias;
  p.bias_dtype = a->bias_dtype;
  p.status = a->status;
  p.block_table = nullptr;
  p.table_stride = 0;
  p.page_shift = 0;
  p.k_new = nullptr;
  p.v_new = nullptr;
  p.lens_out = nullptr;
  p.rope_cos = nullptr;
  p.rope_sin = nullptr;
  p.rope_positions = 0;
  p.acc_mode = 0;
  p.acc = nullptr;
  p.acc_lse = nullptr;
  if (a->force_path != B200_SDPA_PATH_AUTO && a->force_path != B200_SDPA_PATH_GENERIC &&
      a->force_path != B200_SDPA_PATH_PREFILL)
    return B200_SDPA_ERR_UNSUPPORTED;
  return B200_SDPA_OK;
}

// Backward kernel family: tensor-core kernels when eligible (and, for a launch, when the
// scratch is there), otherwise the CUDA-core kernels.
int choose_bwd(const B200SdpaBwdParams* a, const BwdProblem& bp, int* path) {
  bool align_only = false;
  const bool tc_ok = bwd_tc_eligible(bp, a->dtype, &align_only);
  if (a->force_path == B200_SDPA_PATH_PREFILL && !tc_ok)
    return align_only ? B200_SDPA_ERR_ALIGNMENT : B200_SDPA_ERR_UNSUPPORTED;
  *path = (a->force_path != B200_SDPA_PATH_GENERIC && tc_ok) ? B200_SDPA_PATH_PREFILL : B200_SDPA_PATH_GENERIC;
  return B200_SDPA_OK;
}

}  // namespace

void count_launch(int kernel_id) {
  if (kernel_id >= 0 && kernel_id < KID_COUNT) g_launches[kernel_id].fetch_add(1, std::memory_order_relaxed);
}

}  // namespace b200

namespace b200 {
// One thread offers the checker an index in range (accepted, nothing recorded) and one past its limit
// (refused and recorded); nothing is accessed either way.
__global__ void debug_selftest_kernel(int* status) {
  if (!dbg_range(status, 9901, 5, 1, 8)) return;
  if (dbg_range(status, 9902, 8, 1, 8)) status[1] = -1;   // must not happen in the checked build
}
}  // namespace b200

using namespace b200;

extern "C" {

int b200_sdpa_abi_version(void) { return B200_SDPA_ABI_VERSION; }

const char* b200_sdpa_strerror(int status) {
  switch (status) {
    case B200_SDPA_OK: return "ok";
    case B200_SDPA_ERR_NULL: return "a required pointer is NULL";
    case B200_SDPA_ERR_STRUCT: return "parameter block size does not match this library (ABI mismatch)";
    case B200_SDPA_ERR_DTYPE: return "dtype must be float32, float16 or bfloat16";
    case B200_SDPA_ERR_SHAPE: return "invalid shape (extents must be positive and Hq divisible by Hkv)";
    case B200_SDPA_ERR_UNSUPPORTED: return "no kernel in this build serves the request on the requested path";
    case B200_SDPA_ERR_WORKSPACE: return "workspace missing or smaller than b200_sdpa_query_plan() reports";
    case B200_SDPA_ERR_ALIGNMENT: return "tensor-core path needs unit inner stride and 16-byte aligned bases/strides";
    case B200_SDPA_ERR_CUDA: return "a CUDA call failed";
    case B200_SDPA_ERR_DEVICE: return "device is not sm_100";
    case B200_SDPA_ERR_BOUNDS: return "checked build: an index, scratch slot or tensor-memory column left its range (access skipped)";
    case B200_SDPA_ERR_TIMEOUT: return "a device-side wait gave up (kernel drained and returned)";
    case B200_SDPA_ERR_TOO_LARGE: return "request exceeds the fixed capacity of this entry point";
    case B200_SDPA_ERR_CACHE_FULL: return "decode with append: a sequence's cache is full, its new row was dropped";
    default: return "unknown status";
  }
}

int b200_sdpa_query_plan(const B200SdpaParams* params, B200SdpaPlan* plan) {
  if (plan == nullptr) return B200_SDPA_ERR_NULL;
  if (plan->struct_size != sizeof(B200SdpaPlan)) return B200_SDPA_ERR_STRUCT;
  Problem p;
  int rc = validate(params, &p);
  if (rc != B200_SDPA_OK) return rc;
  int path = 0;
  rc = choose(params, p, &path);
  if (rc != B200_SDPA_OK) return rc;
  if (p.S == 0) path = B200_SDPA_PATH_GENERIC;
  switch (path) {
    case B200_SDPA_PATH_DECODE: return plan_decode(p, params->dtype, params->kv_chunk, plan);
    case B200_SDPA_PATH_PREFILL: return plan_prefill(p, params->dtype, plan);
    default: return plan_generic(p, params->dtype, plan);
  }
}

int b200_sdpa_fwd(const B200SdpaParams* params, void* stream) {
  Problem p;
  int rc = validate(params, &p);
  if (rc != B200_SDPA_OK) return rc;
  int path = 0;
  rc = choose(params, p, &path);
  if (rc != B200_SDPA_OK) return rc;
  if (p.S == 0) path = B200_SDPA_PATH_GENERIC;  // nothing to attend to: zeros and -inf
  DeviceScope scope(params->device);
  if (scope.status() != B200_SDPA_OK) return scope.status();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (path == B200_SDPA_PATH_DECODE) {
    rc = launch_decode(p, params->dtype, params->kv_chunk, params->workspace, params->workspace_bytes, st);
    // Without scratch an automatic choice falls through to a kernel that needs none
    // (there is none for a paged cache).
    if (rc != B200_SDPA_ERR_WORKSPACE || params->force_path == B200_SDPA_PATH_DECODE || p.block_table != nullptr ||
        p.k_new != nullptr)
      return rc;
    bool unused = false;
    path = prefill_eligible(p, params->dtype, &unused) ? B200_SDPA_PATH_PREFILL : B200_SDPA_PATH_GENERIC;
  }
  if (path == B200_SDPA_PATH_PREFILL) return launch_prefill(p, params->dtype, params->workspace, params->workspace_bytes, st);
  return launch_generic(p, params->dtype, st);
}

int b200_sdpa_decode(const B200SdpaParams* params, void* stream) {
  Problem p;
  int rc = validate(params, &p);
  if (rc != B200_SDPA_OK) return rc;
  if (!decode_eligible(p, params->dtype)) return B200_SDPA_ERR_UNSUPPORTED;
  DeviceScope scope(params->device);
  if (scope.status() != B200_SDPA_OK) return scope.status();
  return launch_decode(p, params->dtype, params->kv_chunk, params->workspace, params->workspace_bytes,
                       reinterpret_cast<cudaStream_t>(stream));
}

int b200_sdpa_decode_static(const B200SdpaParams* params, void* stream) {
  Problem p;
  int rc = validate(params, &p);
  if (rc != B200_SDPA_OK) return rc;
  if (!decode_eligible(p, params->dtype)) return B200_SDPA_ERR_UNSUPPORTED;
  DeviceScope scope(params->device);
  if (scope.status() != B200_SDPA_OK) return scope.status();
  return launch_decode_static(p, params->dtype, params->kv_chunk, reinterpret_cast<cudaStream_t>(stream));
}

int b200_sdpa_bwd_query_plan(const B200SdpaBwdParams* a, B200SdpaPlan* plan) {
  if (plan == nullptr) return B200_SDPA_ERR_NULL;
  if (plan->struct_size != sizeof(B200SdpaPlan)) return B200_SDPA_ERR_STRUCT;
  BwdProblem bp;
  int rc = validate_bwd(a, bp);
  if (rc != B200_SDPA_OK) return rc;
  int path = 0;
  rc = choose_bwd(a, bp, &path);
  if (rc != B200_SDPA_OK) return rc;
  return path == B200_SDPA_PATH_PREFILL ? plan_bwd_tc(bp, a->dtype, plan) : plan_bwd_generic(bp, a->dtype, plan);
}

int b200_sdpa_bwd(const B200SdpaBwdParams* a, void* stream) {
  BwdProblem bp;
  int rc = validate_bwd(a, bp);
  if (rc != B200_SDPA_OK) return rc;
  int path = 0;
  rc = choose_bwd(a, bp, &path);
  if (rc != B200_SDPA_OK) return rc;
  DeviceScope scope(a->device);
  if (scope.status() != B200_SDPA_OK) return scope.status();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (path == B200_SDPA_PATH_PREFILL) {
    rc = launch_bwd_tc(bp, a->dtype, a->workspace, a->workspace_bytes, st);
    // without scratch an automatic choice falls through to the kernels that need none
    if (rc != B200_SDPA_ERR_WORKSPACE || a->force_path == B200_SDPA_PATH_PREFILL) return rc;
  }
  return launch_bwd_generic(bp, a->dtype, st);
}

int b200_sdpa_merge(const B200SdpaMergeParams* m, void* stream) {
  if (m == nullptr) return B200_SDPA_ERR_NULL;
  if (m->struct_size != sizeof(B200SdpaMergeParams)) return B200_SDPA_ERR_STRUCT;
  if (m->acc == nullptr || m->acc_lse == nullptr || m->part == nullptr || m->part_lse == nullptr)
    return B200_SDPA_ERR_NULL;
  if (m->B < 0 || m->Hq < 0 || m->L < 0 || m->Dv < 0) return B200_SDPA_ERR_SHAPE;
  DeviceScope scope(m->device);
  if (scope.status() != B200_SDPA_OK) return scope.status();
  return launch_merge(*m, reinterpret_cast<cudaStream_t>(stream));
}

uint64_t b200_sdpa_launch_count(int kernel_id) {
  if (kernel_id < 0 || kernel_id >= KID_COUNT) return 0;
  return g_launches[kernel_id].load(std::memory_order_relaxed);
}

void b200_sdpa_reset_launch_counts(void) {
  for (int i = 0; i < KID_COUNT; ++i) g_launches[i].store(0, std::memory_order_relaxed);
}

int b200_sdpa_checked_build(void) { return kChecked ? 1 : 0; }

int b200_sdpa_debug_selftest(int device, int32_t* status, void* stream) {
  if (!kChecked) return B200_SDPA_ERR_UNSUPPORTED;
  if (status == nullptr) return B200_SDPA_ERR_NULL;
  DeviceScope scope(device);
  if (scope.status() != B200_SDPA_OK) return scope.status();
  debug_selftest_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status);
  return cudaGetLastError() == cudaSuccess ? B200_SDPA_OK : B200_SDPA_ERR_CUDA;
}

}  // extern "C"
