// Split-KV flash decoding, 16-bit cache, products on tensor cores (mma.sync).
//
// Same decomposition and workspace format as decode_splitkv.cu -- grid
// (key split, kv head, batch), fp32 partials (o, m, l) per (batch, query head,
// split) -- but the two products run as m16n8k16 MMAs with the query heads of the
// group in the M dimension, so one cache row costs a handful of instructions
// instead of ~70 and the kernel can keep enough loads in flight to stream the
// cache at HBM rate:
//   * the CTA walks its chunk in blocks of 64 keys; K and V blocks go global ->
//     shared memory with 16-byte cp.async through a 2-stage ring (rows padded by
//     16 bytes so ldmatrix is conflict free); rows past the end are zero-filled;
//     68 KB per CTA, so three CTAs share an SM and one CTA's start and end overlap
//     the others' streaming (measured against 3 stages x 2 CTAs: 6080 against 5941
//     GB/s on a uniform 8192-key cache, equal on ragged lengths);
//   * warp w owns keys 16w..16w+15 of every block: S = Q K^T (heads x 16 keys),
//     online softmax on the accumulator fragments (row max across the four lanes
//     of a quad, row sums kept per lane until the end), P repacked in registers
//     as the A operand of O += P V (V fragments by transposing ldmatrix);
//   * the four warps' (O, m, l) are merged in shared memory and written as one
//     partial; decode_combine_kernel merges the splits.
// A paged cache (page pools + block table, the layout serving engines keep) is read by the
// same kernel: only the row address of a copy changes -- one table lookup per row.
// The group of Hq/Hkv query heads is padded to 16 rows; groups above 16 are cut
// into blocks of 16 (grid.y).  Softmax in the exp2 domain on raw scores, fp32
// statistics, the running maximum raised lazily (threshold 2^8) so O is rarely
// rescaled; P rounded to the cache dtype once (torch_neuronx/_sdpa_math.py:94).
#include "common.cuh"
#include "debug.cuh"

namespace b200 {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kBlockKeys = 64;
constexpr int kStages = 2;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

template <int D> struct Geo {
  static constexpr int kRowBytes = D * 2 + 16;                 // padded row
  static constexpr int kTileBytes = kBlockKeys * kRowBytes;    // one K or V block
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes;
  static constexpr int kChunksPerRow = D * 2 / 16;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool BF16> __device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  uint32_t r;
  if (BF16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

template <bool BF16> __device__ __forceinline__ float half_to_f32(uint16_t x) {
  if (BF16) return __uint_as_float(static_cast<uint32_t>(x) << 16);
  return __half2float(__ushort_as_half(x));
}
template <bool BF16> __device__ __forceinline__ uint16_t f32_to_half(float x) {
  if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(x));
  return __half_as_ushort(__float2half_rn(x));
}
// Rotary embedding of element `col` of a row: the partner element and the angle index.
template <int D> __device__ __forceinline__ void rope_partner(int col, bool interleaved, int* partner, int* angle, float* sign) {
  if (interleaved) {
    *partner = col ^ 1;
    *angle = col >> 1;
    *sign = (col & 1) ? 1.f : -1.f;
  } else {
    *partner = col < D / 2 ? col + D / 2 : col - D / 2;
    *angle = col < D / 2 ? col : col - D / 2;
    *sign = col < D / 2 ? -1.f : 1.f;
  }
}

// Row of the cos/sin tables for the token being decoded: its position is the sequence's old length;
// a length beyond the tables uses their last row (never a read past the end).
__device__ __forceinline__ int rope_row(const Problem& p, int b) {
  int len = p.kv_lens[b];
  len = len < 0 ? 0 : len;
  return len < p.rope_positions ? len : p.rope_positions - 1;
}

template <int D, bool BF16, bool PAGED, bool APPEND, bool ROPE>
__global__ void __launch_bounds__(kThreads, 3) decode_mma_kernel(const Problem p, const int chunk, const int nsplit,
                                                                 float* __restrict__ part_o,
                                                                 float* __restrict__ part_ml) {
  using G = Geo<D>;
  constexpr int KS = D / 16;   // k-steps of the first product
  constexpr int NB = D / 8;    // n-blocks of the second product
  extern __shared__ __align__(16) uint8_t smem[];

  // the split index is the slowest grid dimension: the CTAs that run last are the last chunks of the
  // longest sequences (partial, or empty for shorter ones), which keeps the tail of the launch short
  const int split = blockIdx.z;
  const int hk = blockIdx.x % p.Hkv;
  const int gsub = blockIdx.x / p.Hkv;
  const int b = blockIdx.y;
  const int n_keys = valid_keys(p, b);
  const int s0 = split * chunk;
  if (s0 >= n_keys && split != 0) return;  // split 0 still writes an (empty) partial
  const int s1 = (s0 + chunk < n_keys) ? s0 + chunk : n_keys;
  const int n_blocks = s1 > s0 ? (s1 - s0 + kBlockKeys - 1) / kBlockKeys : 0;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;          // fragment row / column pair
  const int h0 = hk * p.group + gsub * 16;          // first query head of this CTA
  const int n_heads = (p.group - gsub * 16) < 16 ? (p.group - gsub * 16) : 16;
  const bool row_lo = g < n_heads, row_hi = g + 8 < n_heads;

  // ---- Q fragments (A operand), rows = query heads, zero for padding rows
  uint32_t qf[KS][4];
  {
    const uint16_t* q16 = reinterpret_cast<const uint16_t*>(p.q);
    const int64_t base = b * p.qs[0];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = g + (r & 1) * 8;
        const int col = ks * 16 + tq * 2 + (r >> 1) * 8;
        uint32_t v = 0;
        if (row < n_heads) {
          const int64_t o = base + (h0 + row) * p.qs[1] + col * p.qs[3];
          if (ROPE) {
            // out[c] = x[c] cos + sign x[partner] sin at this step's position, in fp32, rounded once
            const int at = rope_row(p, b);
            const float* cs = p.rope_cos + static_cast<int64_t>(at) * p.rope_stride;
            const float* sn = p.rope_sin + static_cast<int64_t>(at) * p.rope_stride;
            uint16_t outv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              int partner, angle;
              float sign;
              rope_partner<D>(col + e, p.rope_interleaved != 0, &partner, &angle, &sign);
              const float x = half_to_f32<BF16>(q16[o + e * p.qs[3]]);
              const float y = half_to_f32<BF16>(q16[o + (partner - col) * p.qs[3]]);
              outv[e] = f32_to_half<BF16>(fmaf(sign * y, sn[angle], x * cs[angle]));
            }
            v = static_cast<uint32_t>(outv[0]) | (static_cast<uint32_t>(outv[1]) << 16);
          } else {
            v = static_cast<uint32_t>(q16[o]) | (static_cast<uint32_t>(q16[o + p.qs[3]]) << 16);
          }
        }
        qf[ks][r] = v;
      }
    }
  }

  // ---- cache block loader: 64 keys of K and of V -> one ring stage
  // dense cache: (batch, head, row, element) strides; paged cache: (page, head, row-in-page, element)
  // strides and one block-table lookup per row
  const char* kbase = reinterpret_cast<const char*>(p.k) + ((PAGED ? 0 : b * p.ks[0]) + hk * p.ks[1]) * 2;
  const char* vbase = reinterpret_cast<const char*>(p.v) + ((PAGED ? 0 : b * p.vs[0]) + hk * p.vs[1]) * 2;
  const int64_t k_row = p.ks[2] * 2, v_row = p.vs[2] * 2;
  const int* table = PAGED ? p.block_table + static_cast<int64_t>(b) * p.table_stride : nullptr;
  const int page_mask = (1 << p.page_shift) - 1;
  // append: the row at position `pos` (the sequence's old length) comes from k_new / v_new and is
  // written into the cache by the thread that copies it (a full cache appends nothing)
  int pos = -1;
  const char* knew = nullptr;
  const char* vnew = nullptr;
  if (APPEND) {
    int len = p.kv_lens[b];
    len = len < 0 ? 0 : len;
    pos = len < p.S ? len : -1;
    // a full cache drops the new row: say so once per sequence through the status word
    if (pos < 0 && split == 0 && blockIdx.x == 0 && tid == 0 && p.status != nullptr &&
        atomicCAS(p.status, 0, B200_SDPA_ERR_CACHE_FULL) == 0) {
      p.status[1] = b;
      p.status[2] = len;
      p.status[3] = p.S;
    }
    knew = reinterpret_cast<const char*>(p.k_new) + (b * p.kns[0] + hk * p.kns[1]) * 2;
    vnew = reinterpret_cast<const char*>(p.v_new) + (b * p.vns[0] + hk * p.vns[1]) * 2;
  }
  const uint32_t smem_base = smem_addr(smem);
  auto load_block = [&](int blk) {
    const uint32_t stage = smem_base + (blk % kStages) * G::kStageBytes;
    const int key0 = s0 + blk * kBlockKeys;
#pragma unroll
    for (int i = 0; i < kBlockKeys * G::kChunksPerRow / kThreads; ++i) {
      const int c = tid + i * kThreads;
      const int row = c / G::kChunksPerRow, ch = c % G::kChunksPerRow;
      const bool ok = key0 + row < s1;
      const int srow = ok ? key0 + row : s0;
      int64_t k_off, v_off;
      if (PAGED) {
        // (checked build: the block-table slot of this row exists; page numbers themselves are the caller's)
        const int64_t page = dbg_range(p.status, DBG_DECODE_MMA * 100 + 1, srow >> p.page_shift, 1, p.table_stride)
                                 ? table[srow >> p.page_shift]
                                 : 0;
        const int in_page = srow & page_mask;
        k_off = (page * p.ks[0]) * 2 + in_page * k_row;
        v_off = (page * p.vs[0]) * 2 + in_page * v_row;
      } else {
        k_off = srow * k_row;
        v_off = srow * v_row;
      }
      const char* ksrc = kbase + k_off + ch * 16;
      const char* vsrc = vbase + v_off + ch * 16;
      bool k_by_copy = true;
      if (APPEND && ok && srow == pos) {
        uint4 kq = *reinterpret_cast<const uint4*>(knew + ch * 16);
        const uint4 vq = *reinterpret_cast<const uint4*>(vnew + ch * 16);
        if (ROPE) {
          // rotate the eight elements of this chunk (their partners sit in this chunk or in one other)
          const int at = rope_row(p, b);
          const float* cs = p.rope_cos + static_cast<int64_t>(at) * p.rope_stride;
          const float* sn = p.rope_sin + static_cast<int64_t>(at) * p.rope_stride;
          const uint16_t* row16 = reinterpret_cast<const uint16_t*>(knew);
          uint16_t* kv16 = reinterpret_cast<uint16_t*>(&kq);
          uint16_t rot[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            int partner, angle;
            float sign;
            rope_partner<D>(ch * 8 + e, p.rope_interleaved != 0, &partner, &angle, &sign);
            const float x = half_to_f32<BF16>(kv16[e]);
            const float y = half_to_f32<BF16>(row16[partner]);
            rot[e] = f32_to_half<BF16>(fmaf(sign * y, sn[angle], x * cs[angle]));
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) kv16[e] = rot[e];
          // the rotated chunk goes to shared memory by a plain store (visible after the block barrier
          // that follows the copy wait) instead of an asynchronous copy from k_new
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + row * G::kRowBytes + ch * 16), "r"(kq.x),
                       "r"(kq.y), "r"(kq.z), "r"(kq.w)
                       : "memory");
          k_by_copy = false;
        }
        // the append: this thread's 16 bytes of the new row go into the cache at position `pos`
        if (dbg_bhrc(p.status, DBG_DECODE_MMA * 100 + 2, b, p.B, hk, p.Hkv, srow, p.S, ch * 8, 8, D)) {
          *reinterpret_cast<uint4*>(const_cast<char*>(ksrc)) = kq;
          *reinterpret_cast<uint4*>(const_cast<char*>(vsrc)) = vq;
        }
        ksrc = knew + ch * 16;
        vsrc = vnew + ch * 16;
      }
      if (k_by_copy) cp_async_16(stage + row * G::kRowBytes + ch * 16, ksrc, ok);
      cp_async_16(stage + G::kTileBytes + row * G::kRowBytes + ch * 16, vsrc, ok);
    }
  };

  float o_acc[NB][4];
#pragma unroll
  for (int n = 0; n < NB; ++n)
#pragma unroll
    for (int r = 0; r < 4; ++r) o_acc[n][r] = 0.f;
  float m_lo = -CUDART_INF_F, m_hi = -CUDART_INF_F;   // running maxima (raw scores) of rows g, g+8
  float l_lo = 0.f, l_hi = 0.f;                       // this lane's share of the row sums
  const float sl2 = p.scale * kLog2e;

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_blocks) load_block(s);
    cp_async_commit();
  }

  for (int blk = 0; blk < n_blocks; ++blk) {
    if (blk + kStages - 1 < n_blocks) load_block(blk + kStages - 1);
    cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncthreads();

    const uint32_t kt = smem_base + (blk % kStages) * G::kStageBytes;
    const uint32_t vt = kt + G::kTileBytes;
    const int key_w = s0 + blk * kBlockKeys + warp * 16;   // first key of this warp's 16
    if (key_w < s1) {
      // ---- S = Q K^T for 16 keys: two n-blocks of 8 keys
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        // lane l addresses row (l % 8) of matrix (l / 8): matrices = (keys 0-7, d lo), (keys 0-7, d hi),
        // (keys 8-15, d lo), (keys 8-15, d hi)
        const uint32_t a0 = kt + (warp * 16 + (lane >> 4) * 8 + (lane & 7)) * G::kRowBytes + ((lane >> 3) & 1) * 16;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t kf[4];
          ldsm_x4(a0 + ks * 32, kf);
          mma16816<BF16>(sc[0], qf[ks], kf[0], kf[1]);
          mma16816<BF16>(sc[1], qf[ks], kf[2], kf[3]);
        }
      }
      // ---- mask the tail, row maxima over the quad
      if (key_w + 16 > s1) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int r = 0; r < 4; ++r)
            if (key_w + n * 8 + tq * 2 + (r & 1) >= s1) sc[n][r] = -CUDART_INF_F;
      }
      float mx_lo = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      float mx_hi = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const bool grow = ((mn_lo - m_lo) * sl2 > kRescaleThreshold) || ((mn_hi - m_hi) * sl2 > kRescaleThreshold);
      if (__any_sync(0xffffffffu, grow)) {
        // raise the reference maxima (uniformly over the quad: all four lanes saw the same maxima)
        const float a_lo = (mn_lo == m_lo) ? 1.f : ex2f((m_lo - mn_lo) * sl2);   // -inf -> 0
        const float a_hi = (mn_hi == m_hi) ? 1.f : ex2f((m_hi - mn_hi) * sl2);
        m_lo = mn_lo;
        m_hi = mn_hi;
        l_lo *= a_lo;
        l_hi *= a_hi;
#pragma unroll
        for (int n = 0; n < NB; ++n) {
          o_acc[n][0] *= a_lo;
          o_acc[n][1] *= a_lo;
          o_acc[n][2] *= a_hi;
          o_acc[n][3] *= a_hi;
        }
      }
      // ---- probabilities (padding rows stay exactly zero)
      const float nm_lo = (m_lo == -CUDART_INF_F) ? 0.f : -m_lo * sl2;
      const float nm_hi = (m_hi == -CUDART_INF_F) ? 0.f : -m_hi * sl2;
      float pr[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        pr[n][0] = row_lo ? ex2f(fmaf(sc[n][0], sl2, nm_lo)) : 0.f;
        pr[n][1] = row_lo ? ex2f(fmaf(sc[n][1], sl2, nm_lo)) : 0.f;
        pr[n][2] = row_hi ? ex2f(fmaf(sc[n][2], sl2, nm_hi)) : 0.f;
        pr[n][3] = row_hi ? ex2f(fmaf(sc[n][3], sl2, nm_hi)) : 0.f;
      }
      l_lo += (pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]);
      l_hi += (pr[0][2] + pr[0][3]) + (pr[1][2] + pr[1][3]);
      uint32_t pf[4];   // A operand of the second product: rows g / g+8, keys 2t,2t+1 / 8+2t,8+2t+1
      pf[0] = pack16<BF16>(pr[0][0], pr[0][1]);
      pf[1] = pack16<BF16>(pr[0][2], pr[0][3]);
      pf[2] = pack16<BF16>(pr[1][0], pr[1][1]);
      pf[3] = pack16<BF16>(pr[1][2], pr[1][3]);
      // ---- O += P V: V fragments by transposing ldmatrix, two n-blocks (16 columns) per load
      {
        // matrices = (keys 0-7, cols n..n+7), (keys 8-15, cols n..n+7), (keys 0-7, cols n+8..), (keys 8-15, cols n+8..)
        const uint32_t v0 = vt + (warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * G::kRowBytes + (lane >> 4) * 16;
#pragma unroll
        for (int n2 = 0; n2 < NB / 2; ++n2) {
          uint32_t vf[4];
          ldsm_x4_trans(v0 + n2 * 32, vf);
          mma16816<BF16>(o_acc[2 * n2], pf, vf[0], vf[1]);
          mma16816<BF16>(o_acc[2 * n2 + 1], pf, vf[2], vf[3]);
        }
      }
    }
    __syncthreads();   // the stage may be refilled from here on
  }
  cp_async_wait<0>();
  // the cache has been streamed: the combine kernel (a programmatic dependent launch) may be placed now;
  // it still waits for this grid to complete before it reads a partial
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- quad-reduce the row sums, then merge the four warps through shared memory
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float* sm_o = reinterpret_cast<float*>(smem);               // [warp][16][D]
  float* sm_ml = sm_o + kWarps * 16 * D;                      // [warp][16][2] (max in log2 units, sum)
  __syncthreads();
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    const int col = n * 8 + tq * 2;
    *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g) * D + col]) = make_float2(o_acc[n][0], o_acc[n][1]);
    *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g + 8) * D + col]) = make_float2(o_acc[n][2], o_acc[n][3]);
  }
  if (tq == 0) {
    sm_ml[(warp * 16 + g) * 2] = m_lo * sl2;        // -inf stays -inf (sl2 > 0)
    sm_ml[(warp * 16 + g) * 2 + 1] = l_lo;
    sm_ml[(warp * 16 + g + 8) * 2] = m_hi * sl2;
    sm_ml[(warp * 16 + g + 8) * 2 + 1] = l_hi;
  }
  __syncthreads();
  for (int idx = tid; idx < n_heads * D; idx += kThreads) {
    const int row = idx / D, d = idx - row * D;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, sm_ml[(w * 16 + row) * 2]);
    const float ms = (mx == -CUDART_INF_F) ? 0.f : mx;
    float o = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float wgt = ex2f(sm_ml[(w * 16 + row) * 2] - ms);
      o = fmaf(sm_o[(w * 16 + row) * D + d], wgt, o);
      lsum = fmaf(sm_ml[(w * 16 + row) * 2 + 1], wgt, lsum);
    }
    const int64_t slot = (static_cast<int64_t>(b) * p.Hq + (h0 + row)) * nsplit + split;
    if (!dbg_range(p.status, DBG_DECODE_MMA * 100 + 3, slot, 1, static_cast<int64_t>(p.B) * p.Hq * nsplit) ||
        !dbg_range(p.status, DBG_DECODE_MMA * 100 + 4, h0 + row, 1, p.Hq))
      continue;
    part_o[slot * D + d] = o;
    if (d == 0) {
      part_ml[slot * 2] = mx;
      part_ml[slot * 2 + 1] = lsum;
    }
  }
}

template <int D, bool BF16, bool PAGED, bool APPEND, bool ROPE>
int launch_one(const Problem& p, int chunk, int nsplit, float* po, float* pml, cudaStream_t stream) {
  using G = Geo<D>;
  static_assert(kWarps * 16 * D * 4 + kWarps * 16 * 2 * 4 <= G::kSmemBytes, "merge buffer must fit in the ring");
  auto kern = decode_mma_kernel<D, BF16, PAGED, APPEND, ROPE>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  const int nsub = (p.group + 15) / 16;
  dim3 grid(p.Hkv * nsub, p.B, nsplit);
  kern<<<grid, kThreads, G::kSmemBytes, stream>>>(p, chunk, nsplit, po, pml);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_DECODE);
  return B200_SDPA_OK;
}

}  // namespace

bool decode_mma_eligible(const Problem& p, int dtype) {
  if (dtype != B200_SDPA_F16 && dtype != B200_SDPA_BF16) return false;
  if (!(p.scale > 0.f) || !(p.scale < 1e30f)) return false;   // raw-score maxima assume a positive scale
  if (static_cast<int64_t>(p.Hkv) * ((p.group + 15) / 16) > 65535) return false;
  return p.E == p.Dv && (p.E == 64 || p.E == 128);
}

int launch_decode_partial_mma(const Problem& p, int dtype, int chunk, int nsplit, float* po, float* pml,
                              cudaStream_t stream) {
  const bool bf16 = dtype == B200_SDPA_BF16;
  const bool d128 = p.E == 128, paged = p.block_table != nullptr, append = p.k_new != nullptr;
  const bool rope = p.rope_cos != nullptr;
  if (rope) {
#define B200_DECODE_ROPE_CASE(DD, BB, PP)                                                              \
  if (d128 == (DD == 128) && bf16 == BB && paged == PP) return launch_one<DD, BB, PP, true, true>(p, chunk, nsplit, po, pml, stream);
    B200_DECODE_ROPE_CASE(128, true, false)
    B200_DECODE_ROPE_CASE(128, false, false)
    B200_DECODE_ROPE_CASE(64, true, false)
    B200_DECODE_ROPE_CASE(64, false, false)
    B200_DECODE_ROPE_CASE(128, true, true)
    B200_DECODE_ROPE_CASE(128, false, true)
    B200_DECODE_ROPE_CASE(64, true, true)
    B200_DECODE_ROPE_CASE(64, false, true)
#undef B200_DECODE_ROPE_CASE
    return B200_SDPA_ERR_UNSUPPORTED;
  }
#define B200_DECODE_CASE(DD, BB, PP, AA)                                                               \
  if (d128 == (DD == 128) && bf16 == BB && paged == PP && append == AA)                                \
    return launch_one<DD, BB, PP, AA, false>(p, chunk, nsplit, po, pml, stream);
  B200_DECODE_CASE(128, true, false, false)
  B200_DECODE_CASE(128, false, false, false)
  B200_DECODE_CASE(64, true, false, false)
  B200_DECODE_CASE(64, false, false, false)
  B200_DECODE_CASE(128, true, true, false)
  B200_DECODE_CASE(128, false, true, false)
  B200_DECODE_CASE(64, true, true, false)
  B200_DECODE_CASE(64, false, true, false)
  B200_DECODE_CASE(128, true, false, true)
  B200_DECODE_CASE(128, false, false, true)
  B200_DECODE_CASE(64, true, false, true)
  B200_DECODE_CASE(64, false, false, true)
  B200_DECODE_CASE(128, true, true, true)
  B200_DECODE_CASE(128, false, true, true)
  B200_DECODE_CASE(64, true, true, true)
  B200_DECODE_CASE(64, false, true, true)
#undef B200_DECODE_CASE
  return B200_SDPA_ERR_UNSUPPORTED;
}

}  // namespace b200
