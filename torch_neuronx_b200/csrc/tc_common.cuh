// Helpers shared by the tcgen05 kernels (forward prefill and backward): fast math,
// packed conversions, bounded barrier waits with a CTA-wide abort flag, the device
// status word, and host-side TMA tensor-map construction.
#pragma once

#include "common.cuh"
#include "ptx_sm100.cuh"

#include <mutex>

namespace b200 {
namespace tc {

using namespace ptx;

constexpr int kTileRows = 128;                    // rows of every operand tile (= TMEM lanes)
constexpr int kBoxBytes = kTileRows * 128;        // one TMA box: 128 rows x 64 16-bit elements
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// packed fp32 pairs (one instruction for two lanes of arithmetic)
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if (BF16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

// Limits below this many cycles are taken literally: the barrier is polled without suspending and
// the clock is read after every poll, so a wait that is not satisfied within the limit gives up
// after about that long.  (Used to exercise the give-up path; production limits are seconds.)
constexpr long long kLiteralLimit = 1LL << 16;
// How long an aborting CTA waits for work it already issued (copies, MMAs) before it lets go of
// shared and tensor memory; independent of the wait limit.
constexpr long long kDrainCycles = 1LL << 26;

__device__ __forceinline__ bool wait_clocked(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             long long limit_cycles) {
  // production limits: suspending polls, the clock read every 16th; literal limits: non-suspending polls,
  // the clock read after every one (one loop for both, to keep the many wait sites small)
  const bool literal = limit_cycles < kLiteralLimit;
  if (literal ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (literal ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if (literal || (++spins & 15u) == 0u) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// The same bounded wait for roles that are in no hurry (an epilogue waiting for a whole work item to
// finish): between polls the thread sleeps, so that it does not take issue slots from the warps that
// are on the critical path.
#ifndef B200_RELAXED_SLEEP_NS
#define B200_RELAXED_SLEEP_NS 256
#endif
__device__ __forceinline__ bool wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             long long limit_cycles) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (B200_RELAXED_SLEEP_NS > 0) __nanosleep(B200_RELAXED_SLEEP_NS);
    if (mbar_test_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > limit_cycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Wait (bounded by kDrainCycles, whatever the wait limit) for something this CTA issued itself.
__device__ __forceinline__ bool wait_drain(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kDrainCycles) return false;
  }
  return true;
}

__device__ __forceinline__ void report(int* status, int role, int step, int extra) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, B200_SDPA_ERR_TIMEOUT) == 0) {
    status[1] = role;
    status[2] = step;
    status[3] = extra;
  }
}


// ------------------------------------------------------------------ host side --

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    } else {
      cudaGetLastError();
    }
  });
  return fn;
}

// (D, rows, heads, batch) view of a (B, H, S, D) tensor with unit inner stride.
inline bool make_map(CUtensorMap* map, const void* base, bool bf16, int d, int rows, int heads, int batch,
              const int64_t* stride /* elements, (B,H,S,D) order */) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  auto fix = [&](int64_t s, int n) -> cuuint64_t {
    // a dimension of extent 1 is never stepped; give it any legal stride
    return static_cast<cuuint64_t>((n == 1 ? static_cast<int64_t>(d) : s) * 2);
  };
  const cuuint64_t strides[3] = {fix(stride[2], rows), fix(stride[1], heads), fix(stride[0], batch)};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(kTileRows), 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                         const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

inline bool strides_ok(const void* base, const int64_t* s, int rows, int heads, int batch) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return false;
  if (s[3] != 1) return false;
  const int n[3] = {batch, heads, rows};
  for (int i = 0; i < 3; ++i) {
    if (n[i] == 1) continue;
    if (s[i] <= 0 || (s[i] * 2) % 16 != 0 || s[i] * 2 >= (1LL << 40)) return false;
  }
  return true;
}

// One thread's 8 N bias elements (16-bit) of a key tile: N 16-byte pieces, fetched as N / 2
// 32-byte loads when the row allows it (`wide`: the row start and the key offset on a 32-byte
// boundary) -- every thread reads its own row, so the number of load instructions is what the
// load/store unit feels.  Pieces at or beyond `n_cols` (a multiple of 8) read as zero.  The loads bypass L1
// (every byte is read once): the softmax loop's spilled registers live there and must not be evicted.
template <int N>
__device__ __forceinline__ void load_bias_row(uint4 (&bv)[N], const uint4* row, const int col0, const int n_cols,
                                              const bool wide) {
  if (row == nullptr) {
#pragma unroll
    for (int i = 0; i < N; ++i) bv[i] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  if (wide && col0 + 8 * N <= n_cols) {
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(bv[2 * i].x), "=r"(bv[2 * i].y), "=r"(bv[2 * i].z), "=r"(bv[2 * i].w), "=r"(bv[2 * i + 1].x),
                     "=r"(bv[2 * i + 1].y), "=r"(bv[2 * i + 1].z), "=r"(bv[2 * i + 1].w)
                   : "l"(row + (col0 >> 3) + 2 * i));
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const int c = col0 + 8 * i;
    bv[i] = make_uint4(0u, 0u, 0u, 0u);
    if (c < n_cols)
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(bv[i].x), "=r"(bv[i].y), "=r"(bv[i].z), "=r"(bv[i].w)
                   : "l"(row + (c >> 3)));
  }
}

// Whether every row of the bias starts on a 32-byte boundary.
__host__ __device__ inline bool bias_rows_32b(const Problem& p) {
  return reinterpret_cast<uintptr_t>(p.bias) % 32 == 0 && p.bs[0] % 16 == 0 && p.bs[1] % 16 == 0 && p.bs[2] % 16 == 0;
}

// Eight logits s * scale + bias (natural units), the bias as eight 16-bit elements of the query's
// dtype; one packed fma per pair of elements.
template <bool BF16>
__device__ __forceinline__ void add_bias8(uint32_t* sv, const uint4 bias, const float scale) {
  const uint32_t w[4] = {bias.x, bias.y, bias.z, bias.w};
  const uint64_t scale2 = f2_pack(scale, scale);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float lo, hi;
    if (BF16) {
      lo = __uint_as_float(w[i] << 16);
      hi = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      lo = f.x;
      hi = f.y;
    }
    const uint64_t t = f2_fma(f2_pack(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), scale2, f2_pack(lo, hi));
    float t0, t1;
    f2_unpack(t, t0, t1);
    sv[2 * i] = __float_as_uint(t0);
    sv[2 * i + 1] = __float_as_uint(t1);
  }
}

// An additive bias the tensor-core kernels can read as 16-byte pieces of a row: the query's dtype,
// unit stride along the keys, a key count that is a multiple of 8, every row start on a 16-byte
// boundary (broadcast dimensions have stride 0).
inline bool bias_readable(const Problem& p, int dtype, bool* alignment_only_failure) {
  if (p.bias_dtype != dtype || p.bs[3] != 1 || p.S % 8 != 0) return false;
  if (reinterpret_cast<uintptr_t>(p.bias) % 16 != 0 || p.bs[0] % 8 != 0 || p.bs[1] % 8 != 0 || p.bs[2] % 8 != 0) {
    if (alignment_only_failure) *alignment_only_failure = true;
    return false;
  }
  return true;
}

// Key/value bytes that the CTAs of one wave of (batch, kv head) streams read together: about a quarter
// of the 126 MB L2, so that a wave's streams stay resident while its query blocks sweep over them.
#ifndef B200_WAVE_BYTES
#define B200_WAVE_BYTES (32LL << 20)
#endif
inline int kv_streams_per_wave(long long stream_bytes, long long n_streams) {
  long long per_wave = B200_WAVE_BYTES / (stream_bytes > 0 ? stream_bytes : 1);
  per_wave = per_wave < 1 ? 1 : (per_wave > n_streams ? n_streams : per_wave);
  return static_cast<int>(per_wave);
}

inline long long wait_limit_cycles() {
  // about two seconds at 2 GHz; B200_SDPA_WAIT_LIMIT overrides (cycles)
  static long long v = [] {
    const char* e = getenv("B200_SDPA_WAIT_LIMIT");
    long long x = e ? atoll(e) : 0;
    return x > 0 ? x : (1LL << 32);
  }();
  return v;
}


}  // namespace tc
}  // namespace b200
