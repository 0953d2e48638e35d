// Checked build of the library (-DB200_SDPA_DEBUG; `python -m torch_neuronx_b200.build --checked`
// writes libb200_sdpa_checked.so beside the normal library).
//
// In the checked build every global store whose address a kernel computes from decoded indices, every
// scratch slot and every tensor-memory column range is verified first.  A violation is recorded once in
// the status word -- B200_SDPA_ERR_BOUNDS, the number of the site, the offending index and its limit --
// and the access is skipped; nothing traps and the kernel runs on to its end, so the context stays
// usable and the caller reads the verdict after synchronising.  In the normal build every function here
// folds to `true` at compile time.
#pragma once

#include "common.cuh"

namespace b200 {

#ifdef B200_SDPA_DEBUG
constexpr bool kChecked = true;
#else
constexpr bool kChecked = false;
#endif

// Site numbers: 100 x file + position in the file (the table of sites is the grep of `dbg_` calls).
enum DebugFile {
  DBG_GENERIC_FWD = 1,
  DBG_GENERIC_BWD = 2,
  DBG_DECODE_SIMT = 3,
  DBG_DECODE_MMA = 4,
  DBG_PREFILL = 5,
  DBG_PREFILL_PERSISTENT = 6,
  DBG_PREFILL_WIDE = 7,
  DBG_BWD_TC = 8
};

__device__ __forceinline__ bool dbg_fail(int* status, int site, long long index, long long limit) {
  if (status != nullptr && atomicCAS(status, 0, B200_SDPA_ERR_BOUNDS) == 0) {
    status[1] = site;
    status[2] = static_cast<int>(index > 0x7fffffffLL ? 0x7fffffffLL : (index < -0x7fffffffLL ? -0x7fffffffLL : index));
    status[3] = static_cast<int>(limit > 0x7fffffffLL ? 0x7fffffffLL : limit);
  }
  return false;
}

// 0 <= index and index + count <= limit
__device__ __forceinline__ bool dbg_range(int* status, int site, long long index, long long count, long long limit) {
  if (!kChecked) return true;
  if (index >= 0 && index + count <= limit) return true;
  return dbg_fail(status, site, index, limit);
}

// (b, h, row, col .. col + n) inside a (B, H, R, C) tensor
__device__ __forceinline__ bool dbg_bhrc(int* status, int site, long long b, int B, long long h, int H, long long r,
                                         long long R, long long c, int n, int C) {
  if (!kChecked) return true;
  return dbg_range(status, site, b, 1, B) && dbg_range(status, site, h, 1, H) && dbg_range(status, site, r, 1, R) &&
         dbg_range(status, site, c, n, C);
}

// A tensor-memory access of `ncols` columns at address `taddr` stays inside the `allocated` columns that
// start at `tmem_base`, and names one of the 128 lanes.
__device__ __forceinline__ bool dbg_tmem(int* status, int site, uint32_t taddr, uint32_t tmem_base, int ncols,
                                         int allocated) {
  if (!kChecked) return true;
  const long long col = static_cast<long long>(taddr & 0xffffu) - static_cast<long long>(tmem_base & 0xffffu);
  const long long lane = (taddr >> 16) - (tmem_base >> 16);
  return dbg_range(status, site, col, ncols, allocated) && dbg_range(status, site, lane, 1, 128);
}

}  // namespace b200
