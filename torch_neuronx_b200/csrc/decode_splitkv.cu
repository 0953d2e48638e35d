// Split-KV flash decoding (one query row per sequence) for sm_100a.
//
// The key/value cache is the only large operand, so the kernel is organised
// around reading it exactly once at full HBM rate:
//   * grid = (key split, kv head, batch): every CTA streams one contiguous
//     chunk of one kv head's cache and serves ALL query heads of that group,
//     so grouped-query heads never re-read K/V;
//   * every lane issues 128-bit loads; a warp-wide load covers whole cache rows
//     back to back (fully coalesced), several rows in flight per lane;
//   * per-lane online softmax state in the exp2 domain; lanes, warps and finally
//     splits are merged with the usual (max, sum, weighted accumulator) rule --
//     across splits by a second small kernel that reads the fp32 partials.
// Sequences are ragged: split s of batch b covers keys [s*chunk, min((s+1)*chunk,
// kv_lens[b])) and CTAs past the end exit at once.
//
// Arithmetic restates torch_neuronx/_sdpa_math.py:79-95 for a single query row
// with a key-length mask; dead rows (no visible key) give out = 0, lse = -inf.
#include "common.cuh"
#include "debug.cuh"

#include <cstdlib>
#include <mutex>

namespace b200 {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kUnroll = 4;  // cache rows in flight per lane (x2 for K and V)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float (&f)[Vec<T>::N]);
template <>
__device__ __forceinline__ void unpack<float>(const uint4& raw, float (&f)[4]) {
  f[0] = __uint_as_float(raw.x);
  f[1] = __uint_as_float(raw.y);
  f[2] = __uint_as_float(raw.z);
  f[3] = __uint_as_float(raw.w);
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack<__half>(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 ld_stream_16B(const void* ptr) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(ptr));
  return r;
}

// Workspace layout (fp32): part_o[B][Hq][nsplit][D] then part_ml[B][Hq][nsplit][2]
// with ml = (running max in the exp2 domain, running sum).
template <typename T, int D, int G>
__global__ void __launch_bounds__(kThreads) decode_partial_kernel(const Problem p, const int chunk, const int nsplit,
                                                                   float* __restrict__ part_o,
                                                                   float* __restrict__ part_ml) {
  constexpr int V = Vec<T>::N;
  constexpr int LPR = D / V;       // lanes that share one cache row
  constexpr int RPW = 32 / LPR;    // rows covered by one warp-wide load
  constexpr int NSTATE = kWarps * RPW;
  static_assert(LPR <= 32 && LPR >= 1, "head dim not supported by this mapping");
  __shared__ float sm_acc[NSTATE][G][D];
  __shared__ float sm_ml[NSTATE][G][2];

  const int split = blockIdx.z;          // slowest: the launch ends on the last (short or empty) chunks
  const int hk = blockIdx.x % p.Hkv;
  const int gsub = blockIdx.x / p.Hkv;   // sub-block of the query-head group when group > G
  const int b = blockIdx.y;
  const int n_keys = valid_keys(p, b);
  const int s0 = split * chunk;
  if (s0 >= n_keys && !(split == 0)) return;  // split 0 still writes an empty partial
  const int s1 = (s0 + chunk < n_keys) ? s0 + chunk : n_keys;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, col = (lane % LPR) * V;
  const int h0 = hk * p.group + gsub * G;                      // first query head served here
  const int n_heads = (p.group - gsub * G) < G ? (p.group - gsub * G) : G;

  const T* __restrict__ q = reinterpret_cast<const T*>(p.q);
  const char* __restrict__ kbase = reinterpret_cast<const char*>(p.k) +
                                   (b * p.ks[0] + hk * p.ks[1] + col) * static_cast<int64_t>(sizeof(T));
  const char* __restrict__ vbase = reinterpret_cast<const char*>(p.v) +
                                   (b * p.vs[0] + hk * p.vs[1] + col) * static_cast<int64_t>(sizeof(T));
  const int64_t k_row_bytes = p.ks[2] * static_cast<int64_t>(sizeof(T));
  const int64_t v_row_bytes = p.vs[2] * static_cast<int64_t>(sizeof(T));

  const float qscale = p.scale * kLog2e;
  float qr[G][V];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < V; ++e)
      qr[g][e] = g < n_heads ? to_f32<T>(q[b * p.qs[0] + (h0 + g) * p.qs[1] + (col + e) * p.qs[3]]) * qscale : 0.f;

  float m[G], l[G], acc[G][V];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < V; ++e) acc[g][e] = 0.f;
  }

  constexpr int kStep = RPW * kUnroll;  // rows per warp iteration
  for (int base = s0 + warp * kStep; base < s1; base += kWarps * kStep) {
    uint4 kraw[kUnroll], vraw[kUnroll];
    bool ok[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int row = base + u * RPW + sub;
      ok[u] = row < s1;
      const int srow = ok[u] ? row : s0;  // always a readable row of this sequence
      kraw[u] = ld_stream_16B(kbase + srow * k_row_bytes);
      vraw[u] = ld_stream_16B(vbase + srow * v_row_bytes);
    }
    float s[kUnroll][G];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float kf[V];
      unpack<T>(kraw[u], kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < V; ++e) d = fmaf(qr[g][e], kf[e], d);
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        s[u][g] = ok[u] ? d : -CUDART_INF_F;
      }
    }
    float pw[kUnroll][G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = m[g];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) mx = fmaxf(mx, s[u][g]);
      const float ms = (mx == -CUDART_INF_F) ? 0.f : mx;
      const float alpha = exp2f(m[g] - ms);  // m = -inf -> 0
      m[g] = mx;
      float sum = 0.f;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        pw[u][g] = exp2f(s[u][g] - ms);
        sum += pw[u][g];
      }
      l[g] = l[g] * alpha + sum;
#pragma unroll
      for (int e = 0; e < V; ++e) acc[g][e] *= alpha;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float vf[V];
      unpack<T>(vraw[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < V; ++e) acc[g][e] = fmaf(pw[u][g], vf[e], acc[g][e]);
    }
  }

  // lane states -> shared memory, then one merged partial per query head
  const int st = warp * RPW + sub;
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int e = 0; e < V; ++e) sm_acc[st][g][col + e] = acc[g][e];
    if ((lane % LPR) == 0) {
      sm_ml[st][g][0] = m[g];
      sm_ml[st][g][1] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kThreads) {
    const int g = idx / D, d = idx - g * D;
    if (g >= n_heads) continue;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int s_ = 0; s_ < NSTATE; ++s_) mx = fmaxf(mx, sm_ml[s_][g][0]);
    const float ms = (mx == -CUDART_INF_F) ? 0.f : mx;
    float o = 0.f, lsum = 0.f;
#pragma unroll
    for (int s_ = 0; s_ < NSTATE; ++s_) {
      const float w = exp2f(sm_ml[s_][g][0] - ms);
      o = fmaf(sm_acc[s_][g][d], w, o);
      lsum = fmaf(sm_ml[s_][g][1], w, lsum);
    }
    const int64_t slot = (static_cast<int64_t>(b) * p.Hq + (h0 + g)) * nsplit + split;
    if (!dbg_range(p.status, DBG_DECODE_SIMT * 100 + 1, slot, 1, static_cast<int64_t>(p.B) * p.Hq * nsplit) ||
        !dbg_range(p.status, DBG_DECODE_SIMT * 100 + 2, h0 + g, 1, p.Hq))
      continue;
    part_o[slot * D + d] = o;
    if (d == 0) {
      part_ml[slot * 2] = mx;
      part_ml[slot * 2 + 1] = lsum;
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const Problem p, const int chunk, const int nsplit,
                                                           const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml) {
  const int h = blockIdx.x % p.Hq;
  const int b = blockIdx.x / p.Hq;
  const int d = threadIdx.x;
  const int n_keys = valid_keys(p, b);
  // launched as a programmatic dependent of the partial kernel: nothing that kernel wrote may be read
  // before it has completed
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (p.lens_out != nullptr && h == 0 && d == 0) p.lens_out[b] = n_keys;   // lengths after the append
  int used = (n_keys + chunk - 1) / chunk;
  used = used < 1 ? 1 : (used > nsplit ? nsplit : used);
  const int64_t slot0 = (static_cast<int64_t>(b) * p.Hq + h) * nsplit;
  if (!dbg_range(p.status, DBG_DECODE_SIMT * 100 + 3, slot0, used, static_cast<int64_t>(p.B) * p.Hq * nsplit) ||
      !dbg_bhrc(p.status, DBG_DECODE_SIMT * 100 + 4, b, p.B, h, p.Hq, 0, 1, d, 1, p.Dv))
    return;
  float mx = -CUDART_INF_F;
  for (int s = 0; s < used; ++s) mx = fmaxf(mx, part_ml[(slot0 + s) * 2]);
  const float ms = (mx == -CUDART_INF_F) ? 0.f : mx;
  float o = 0.f, lsum = 0.f;
  for (int s = 0; s < used; ++s) {
    const float w = exp2f(part_ml[(slot0 + s) * 2] - ms);
    lsum = fmaf(part_ml[(slot0 + s) * 2 + 1], w, lsum);
    o = fmaf(part_o[(slot0 + s) * D + d], w, o);
  }
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  T* out = reinterpret_cast<T*>(p.out);
  out[b * p.os[0] + h * p.os[1] + d * p.os[3]] = from_f32<T>(o * inv);
  if (p.lse != nullptr && d == 0)
    p.lse[b * p.ls[0] + h * p.ls[1]] = (mx == -CUDART_INF_F) ? -CUDART_INF_F : fmaf(mx, kLn2, logf(lsum));
}

int pick_group(int group) { return group >= 8 ? 8 : group > 2 ? 4 : group; }

int default_chunk(const Problem& p) {
  // Enough CTAs to fill 148 SMs several times over even when half the splits of
  // a ragged batch are empty, but never chunks so small that the per-CTA
  // epilogue shows.
  const int64_t units = static_cast<int64_t>(p.B) * p.Hkv;
  int64_t want = (148LL * 16 + units - 1) / units;   // splits per (batch, kv head)
  int64_t chunk = (p.S + want - 1) / want;
  chunk = (chunk + 127) / 128 * 128;
  if (chunk < 256) chunk = 256;
  if (chunk > 2048) chunk = 2048;
  return static_cast<int>(chunk);
}

struct DecodeGeom {
  int chunk, nsplit, g, nsub;
  uint64_t ws_bytes;
};

DecodeGeom geometry(const Problem& p, int kv_chunk) {
  DecodeGeom gm;
  gm.chunk = kv_chunk > 0 ? (kv_chunk + 31) / 32 * 32 : default_chunk(p);
  gm.nsplit = (p.S + gm.chunk - 1) / gm.chunk;
  if (gm.nsplit < 1) gm.nsplit = 1;
  gm.g = pick_group(p.group);
  gm.nsub = (p.group + gm.g - 1) / gm.g;
  gm.ws_bytes = static_cast<uint64_t>(p.B) * p.Hq * gm.nsplit * (p.Dv + 2) * sizeof(float);
  return gm;
}

template <typename T, int D>
int launch_combine(const Problem& p, const DecodeGeom& gm, float* po, float* pml, cudaStream_t stream) {
  // Programmatic dependent launch: the combine grid may be placed while the partial kernel's last CTAs
  // are finishing; its threads wait (griddepcontrol.wait) until that grid has completed and its stores
  // are visible before they read a partial.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.B * p.Hq);
  cfg.blockDim = dim3(D);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* cpo = po;
  const float* cpml = pml;
  if (cudaLaunchKernelEx(&cfg, decode_combine_kernel<T, D>, p, gm.chunk, gm.nsplit, cpo, cpml) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  count_launch(KID_COMBINE);
  return B200_SDPA_OK;
}

template <typename T, int D, int G>
int launch_pg(const Problem& p, const DecodeGeom& gm, float* po, float* pml, cudaStream_t stream) {
  dim3 grid(p.Hkv * gm.nsub, p.B, gm.nsplit);
  decode_partial_kernel<T, D, G><<<grid, kThreads, 0, stream>>>(p, gm.chunk, gm.nsplit, po, pml);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_DECODE);
  return launch_combine<T, D>(p, gm, po, pml, stream);
}

// 16-bit caches go to the tensor-core partial kernel (decode_mma.cu); the CUDA-core
// kernel above keeps fp32 caches and can be forced with B200_SDPA_DECODE_SIMT=1.
bool use_mma_partial(const Problem& p, int dtype) {
  static const bool forced_simt = [] {
    const char* e = getenv("B200_SDPA_DECODE_SIMT");
    return e != nullptr && e[0] == '1';
  }();
  if (p.block_table != nullptr || p.k_new != nullptr) return true;   // only the tensor-core kernel serves these
  return !forced_simt && decode_mma_eligible(p, dtype);
}

template <typename T, int D>
int launch_g(const Problem& p, const DecodeGeom& gm, float* po, float* pml, cudaStream_t stream) {
  switch (gm.g) {
    case 1: return launch_pg<T, D, 1>(p, gm, po, pml, stream);
    case 2: return launch_pg<T, D, 2>(p, gm, po, pml, stream);
    case 4: return launch_pg<T, D, 4>(p, gm, po, pml, stream);
    default: return launch_pg<T, D, 8>(p, gm, po, pml, stream);
  }
}

}  // namespace

bool decode_eligible(const Problem& p, int dtype) {
  if (p.L != 1 || p.bias != nullptr || p.E != p.Dv) return false;
  // a paged cache or an appended row: 16-bit caches only (the tensor-core partial kernel)
  if ((p.block_table != nullptr || p.k_new != nullptr) && !decode_mma_eligible(p, dtype)) return false;
  if (p.k_new != nullptr) {
    if (p.kns[0] % 8 || p.kns[1] % 8 || p.vns[0] % 8 || p.vns[1] % 8) return false;
    if (reinterpret_cast<uintptr_t>(p.k_new) % 16 || reinterpret_cast<uintptr_t>(p.v_new) % 16) return false;
  }
  if (p.E != 64 && p.E != 128) return false;
  if (p.B > 65535 || static_cast<int64_t>(p.Hkv) * ((p.group + 7) / 8) > 65535) return false;
  // is_causal with one query row only limits keys to j <= causal_shift; the host
  // layer folds that into kv_lens, so here causal rows are left to other paths.
  if (p.causal) return false;
  const int64_t es = dtype == B200_SDPA_F32 ? 4 : 2;
  // 128-bit loads: unit inner stride, 16-byte aligned rows and bases
  if (p.ks[3] != 1 || p.vs[3] != 1) return false;
  if ((p.ks[0] * es) % 16 || (p.ks[1] * es) % 16 || (p.ks[2] * es) % 16) return false;
  if ((p.vs[0] * es) % 16 || (p.vs[1] * es) % 16 || (p.vs[2] * es) % 16) return false;
  if (reinterpret_cast<uintptr_t>(p.k) % 16 || reinterpret_cast<uintptr_t>(p.v) % 16) return false;
  return true;
}

int plan_decode(const Problem& p, int dtype, int kv_chunk, B200SdpaPlan* plan) {
  if (!decode_eligible(p, dtype)) return B200_SDPA_ERR_UNSUPPORTED;
  const DecodeGeom gm = geometry(p, kv_chunk);
  if (gm.nsplit > 65535) return B200_SDPA_ERR_UNSUPPORTED;   // grid.z
  plan->path = B200_SDPA_PATH_DECODE;
  plan->block_m = 1;
  plan->block_n = gm.chunk;
  plan->grid_x = p.Hkv * gm.nsub;
  plan->grid_y = p.B;
  plan->grid_z = gm.nsplit;
  plan->threads = kThreads;
  plan->smem_bytes = 0;
  plan->kv_splits = gm.nsplit;
  plan->launches = 2;
  plan->workspace_bytes = gm.ws_bytes;
  return B200_SDPA_OK;
}

int launch_decode(const Problem& p, int dtype, int kv_chunk, void* workspace, uint64_t workspace_bytes,
                  cudaStream_t stream) {
  if (!decode_eligible(p, dtype)) return B200_SDPA_ERR_UNSUPPORTED;
  const DecodeGeom gm = geometry(p, kv_chunk);
  if (gm.nsplit > 65535) return B200_SDPA_ERR_UNSUPPORTED;   // grid.z
  if (workspace == nullptr || workspace_bytes < gm.ws_bytes) return B200_SDPA_ERR_WORKSPACE;
  float* po = reinterpret_cast<float*>(workspace);
  float* pml = po + static_cast<uint64_t>(p.B) * p.Hq * gm.nsplit * p.Dv;
  const bool d128 = p.E == 128;
  if (use_mma_partial(p, dtype)) {
    const int rc = launch_decode_partial_mma(p, dtype, gm.chunk, gm.nsplit, po, pml, stream);
    if (rc != B200_SDPA_OK) return rc;
    if (dtype == B200_SDPA_BF16)
      return d128 ? launch_combine<__nv_bfloat16, 128>(p, gm, po, pml, stream)
                  : launch_combine<__nv_bfloat16, 64>(p, gm, po, pml, stream);
    return d128 ? launch_combine<__half, 128>(p, gm, po, pml, stream) : launch_combine<__half, 64>(p, gm, po, pml, stream);
  }
  switch (dtype) {
    case B200_SDPA_F32:
      return d128 ? launch_g<float, 128>(p, gm, po, pml, stream) : launch_g<float, 64>(p, gm, po, pml, stream);
    case B200_SDPA_F16:
      return d128 ? launch_g<__half, 128>(p, gm, po, pml, stream) : launch_g<__half, 64>(p, gm, po, pml, stream);
    case B200_SDPA_BF16:
      return d128 ? launch_g<__nv_bfloat16, 128>(p, gm, po, pml, stream)
                  : launch_g<__nv_bfloat16, 64>(p, gm, po, pml, stream);
    default: return B200_SDPA_ERR_DTYPE;
  }
}

// ---------------------------------------------------------------------------
// Decode with built-in scratch.
//
// Some hosts cannot give this library a workspace at call time: a serving
// process that handed all device memory to its own pool when it started (so a
// later cudaMalloc fails or is forbidden), or code on a path where allocator
// calls are not permitted at all.  For them the partials of the split-KV
// kernel live in the fixed array below instead of caller-provided memory.
// Every GPU that loads the library carries the array until the process exits,
// which is why it is kept modest; requests whose partials do not fit are
// rejected, never truncated.
//
// The array's name is only a host-side handle.  Its device address is looked
// up once per device with cudaGetSymbolAddress(), with that device current, the
// first time the entry point is used on the device -- so the first call per
// device should be made outside any stream capture.  All calls share the array
// and it keeps whatever the previous call left: the kernels write every slot
// they later read, so nothing has to be cleared, but two calls that overlap on
// the GPU (different streams) would race on it.
// ---------------------------------------------------------------------------
constexpr unsigned long long kStaticScratchBytes = B200_SDPA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices] = {};
}  // namespace

int launch_decode_static(const Problem& p, int dtype, int kv_chunk, cudaStream_t stream) {
  if (!decode_eligible(p, dtype)) return B200_SDPA_ERR_UNSUPPORTED;
  const DecodeGeom gm = geometry(p, kv_chunk);
  if (gm.ws_bytes > kStaticScratchBytes) return B200_SDPA_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
      void* found = nullptr;
      if (cudaGetSymbolAddress(&found, g_decode_scratch) != cudaSuccess || found == nullptr) {
        cudaGetLastError();
        return B200_SDPA_ERR_CUDA;
      }
      g_scratch_ptr[dev] = found;
    }
    ptr = g_scratch_ptr[dev];
  }
  return launch_decode(p, dtype, kv_chunk, ptr, kStaticScratchBytes, stream);
}


}  // namespace b200
