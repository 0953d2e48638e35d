// Tensor-core backward for sm_100a: TMA -> shared memory -> tcgen05 with every
// accumulator and every 16-bit intermediate (P, dS) in tensor memory.
//
// Three launches, no atomics, no [L,S] matrix in HBM:
//   bwd_prep_kernel     delta[b,h,i] = sum_d dO*out and the forward's log-sum-exp in log2
//                       units (rows without a visible key, and pad rows, get +inf so that
//                       their rebuilt probabilities are exactly 0)
//   bwd_dq_tc_kernel    one CTA per 128 query rows of one head; walks the key tiles:
//                         S = Q K^T, dP = dO V^T            (SS MMAs, accumulators in TMEM)
//                         dS = exp2(S*c - lse2) * (dP - delta)   -> 16-bit, over dP in TMEM
//                         dQ += dS K                         (TS MMA: A operand from TMEM)
//   bwd_dkv_tc_kernel   one CTA per 128 keys of one kv head; walks the group's query heads
//                       and their row tiles in the transposed orientation (TMEM lane = key):
//                         S^T = K Q^T, dP^T = V dO^T
//                         P^T -> over S^T, dS^T -> over dP^T (16-bit, in TMEM)
//                         dV += P^T dO, dK += dS^T Q         (TS MMAs)
//                       so the grouped-query sum is part of the accumulation.
// The two main kernels recompute S and dP independently (7 tile products instead of 5);
// in exchange dQ needs neither atomics nor an fp32 scratch tensor, and results are
// deterministic.  Arithmetic: torch_neuronx/_sdpa_math.py:133-176 with P and dS rounded
// to the input dtype before their second product (upstream rounds P the same way in the
// forward, :94).  Roles per CTA (320 threads): warps 0-7 elementwise (two threads per TMEM
// lane), warp 8 TMA producer, warp 9 MMA issuer.
//
// The dK/dV kernel works in units of 64 score columns (half an operand tile) with the two
// score-shaped accumulators double-buffered in tensor memory, so the elementwise role works
// on unit u+1 while the tensor cores run the accumulating products of unit u and the score
// products of unit u+2 (the MMA pipe executes in issue order, which makes "scores of u+2
// after the accumulating products of u" safe on the shared buffer):
//   TMEM columns  [0,64) [64,128)  S^T buffers 0/1   [128,192) [192,256)  dP^T buffers 0/1
//                 [256, 256+2D)    dV and dK (fp32)
// Its tensor memory is full with that; the dQ kernel has one accumulator less and works on
// whole 128-column tiles instead (layout and pipeline described at the kernel).
// Every wait is bounded (see tc_common.cuh).
#include "tc_common.cuh"
#include "debug.cuh"

namespace b200 {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kT = 128;                 // tile edge: query rows, keys, TMEM lanes
constexpr int kThreads = 320;
constexpr int kEThreads = 256;            // elementwise role: two column halves x 128 lanes
constexpr int kU = 64;                    // score columns per unit
constexpr uint32_t kColS = 0, kColDP = 128, kColAcc = 256;   // TMEM layout (buffer b at + 64 b)
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxStages = 4;

template <int D> struct BCfg {
  static constexpr int kBoxes = D / 64;
  static constexpr int kTileBytes = kT * D * 2;
  static constexpr int kStages = (D == 128) ? 2 : 4;           // ring slots of two tiles each
  static constexpr int kSmemTiles = (2 + 2 * kStages) * kTileBytes;
  static constexpr int kStatBytes = kStages * 2 * kT * 4;       // (lse2, delta) of a query tile per slot
  static constexpr int kSmemBytes = kSmemTiles + kStatBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct BSync {
  uint64_t fixed_full;
  uint64_t ring_full[kMaxStages];
  uint64_t ring_empty[kMaxStages];
  uint64_t sp_full[2];  // both score-shaped accumulators of a unit are complete (per buffer)
  uint64_t e_ready[2];  // the elementwise role has written the unit's 16-bit operands
  uint64_t acc_done;    // last accumulating MMA has retired
  uint64_t staged;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

static_assert(sizeof(BSync) <= 272, "barrier block must fit its reserve (272 bytes + up to 1008 of alignment <= 1280)");

// ------------------------------------------------------------------ prep --

// Eight lanes per row (four rows per warp) when rows can be read 16 bytes at a time,
// otherwise one warp per row with scalar loads.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) bwd_prep_kernel(const BwdProblem bp, float* __restrict__ lse2,
                                                        float* __restrict__ delta, const int l_pad) {
  const Problem& p = bp.f;
  constexpr int kLanes = VEC ? 8 : 32;             // lanes cooperating on one row
  constexpr int kRowsPerWarp = 32 / kLanes;
  const long long gwarp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanes;
  const long long row_id = gwarp * kRowsPerWarp + lane / kLanes;
  const long long total = static_cast<long long>(p.B) * p.Hq * l_pad;
  const bool in_range = row_id < total;
  const int i = in_range ? static_cast<int>(row_id % l_pad) : 0;
  const long long bh = in_range ? row_id / l_pad : 0;
  const int h = static_cast<int>(bh % p.Hq);
  const int b = static_cast<int>(bh / p.Hq);
  float d = 0.f, l2 = CUDART_INF_F;
  const bool live = in_range && i < p.L;
  if (live) {
    const T* __restrict__ go = reinterpret_cast<const T*>(bp.dout) + b * bp.dos[0] + h * bp.dos[1] + i * bp.dos[2];
    const T* __restrict__ o = reinterpret_cast<const T*>(p.out) + b * p.os[0] + h * p.os[1] + i * p.os[2];
    if (VEC) {
      for (int e = sub * 8; e < p.Dv; e += 64) {
        const uint4 a = *reinterpret_cast<const uint4*>(go + e);
        const uint4 c = *reinterpret_cast<const uint4*>(o + e);
        const T* av = reinterpret_cast<const T*>(&a);
        const T* cv = reinterpret_cast<const T*>(&c);
#pragma unroll
        for (int u = 0; u < 8; ++u) d = fmaf(to_f32<T>(av[u]), to_f32<T>(cv[u]), d);
      }
    } else {
      for (int e = sub; e < p.Dv; e += 32) d = fmaf(to_f32<T>(go[e * bp.dos[3]]), to_f32<T>(o[e * p.os[3]]), d);
    }
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
  if (live && sub == 0) {
    const float l = p.lse[b * p.ls[0] + h * p.ls[1] + i * p.ls[2]];
    l2 = (l == -CUDART_INF_F) ? CUDART_INF_F : l * kLog2e;
  }
  if (in_range && sub == 0 && dbg_range(p.status, DBG_BWD_TC * 100 + 1, row_id, 1, total)) {
    lse2[row_id] = l2;
    delta[row_id] = live ? d : 0.f;
  }
}

// --------------------------------------------------------------- shared bits --

// K-major operand descriptor of a 128-row tile; k-step kk covers 16 elements of D.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile) { return smem_desc_sw128(tile, 16, 1024); }
__device__ __forceinline__ uint64_t kmajor_step(int kk) {
  return static_cast<uint64_t>(((kk >> 2) * kBoxBytes + (kk & 3) * 32) >> 4);
}
// MN-major B operand descriptor of the same tile (rows are the contraction axis);
// k-step kk covers 16 rows.
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t tile) { return smem_desc_sw128(tile, kBoxBytes, 1024); }
__device__ __forceinline__ uint64_t mnmajor_step(int kk) { return static_cast<uint64_t>(kk * (2048 >> 4)); }

// acc[tmem d, 128 x 64] = A[smem tile, K-major] * B[rows 64 hh .. 64 hh + 63 of a smem tile, K-major]^T over D
template <int D>
__device__ __forceinline__ void issue_ss(uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile, int hh, uint32_t idesc) {
  const uint64_t ad = kmajor_desc(a_tile), bd = kmajor_desc(b_tile + static_cast<uint32_t>(hh) * (kU * 128));
  if (elect_one()) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) mma_ss(d_tmem, ad + kmajor_step(kk), bd + kmajor_step(kk), idesc, kk > 0 ? 1u : 0u);
  }
}
// acc[tmem d] (+)= A[tmem] * B[rows 64 hh .. 64 hh + 63 of a smem tile, MN-major].  The 16-bit A
// operand sits where the two column halves of the elementwise role left it: contraction
// indices 0-31 packed into columns [0,16) of the unit's buffer, 32-63 into columns [32,48).
__device__ __forceinline__ void issue_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_tile, int hh, uint32_t idesc,
                                         bool accumulate) {
  const uint64_t bd = mnmajor_desc(b_tile) + mnmajor_step(4 * hh);
  if (elect_one()) {
#pragma unroll
    for (int kk = 0; kk < kU / 16; ++kk)
      mma_ts(d_tmem, a_tmem + static_cast<uint32_t>((kk >> 1) * 32 + (kk & 1) * 8), bd + mnmajor_step(kk), idesc,
             (kk > 0 || accumulate) ? 1u : 0u);
  }
}

// One thread's accumulator row (TMEM lane) -> 16-bit -> the 128-byte-swizzled staging
// tile a TMA store expects.
template <int D, bool BF16>
__device__ __forceinline__ void stage_row(uint32_t acc_addr, bool have_acc, float mul, uint8_t* stage, int r,
                                          int half) {
  // the two threads of a lane share the row: D/64 chunks of 32 columns each
#pragma unroll
  for (int cc = 0; cc < D / 64; ++cc) {
    const int c = half * (D / 64) + cc;
    uint32_t v[32];
    if (have_acc) {
      tmem_ld_32x32(acc_addr + c * 32, v);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0u;
    }
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2)
      pk[i >> 1] = pack2<BF16>(__uint_as_float(v[i]) * mul, __uint_as_float(v[i + 1]) * mul);
    uint8_t* box = stage + (c >> 1) * kBoxBytes + r * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int unit = ((c & 1) * 4 + u) ^ (r & 7);
      *reinterpret_cast<uint4*>(box + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
    }
  }
}

__device__ __forceinline__ void init_common_barriers(BSync* sync) {
  for (int i = 0; i < 2; ++i) {
    mbar_init(smem_u32(&sync->sp_full[i]), 1);
    mbar_init(smem_u32(&sync->e_ready[i]), kEThreads);
  }
  mbar_init(smem_u32(&sync->acc_done), 1);
  mbar_init(smem_u32(&sync->staged), kEThreads);
  mbar_init(smem_u32(&sync->drain), 1);
  sync->abort_flag = 0;
  mbar_fence_init();
}

__device__ __forceinline__ void drain_after_abort(BSync* sync, long long wait_limit) {
  // let whatever was issued retire before tensor memory is released
  if (elect_one()) mma_commit(smem_u32(&sync->drain));
  const long long t0 = clock64();
  while (!mbar_try_wait(smem_u32(&sync->drain), 0) && clock64() - t0 < kDrainCycles) {
  }
}

// ------------------------------------------------------------------ dQ kernel --
//
// Whole 128-key tiles per step (a 128-column score product costs the tensor pipe the same
// as a 64-column one).  The elementwise role copies S and dP of a tile into registers and
// releases the two accumulators at once, so the score products of tile j+1 run while it
// computes dS of tile j; dS goes to one of two operand buffers, so dQ += dS K of tile j runs
// while tile j+1 is being computed.  K tiles live until their dQ product, V tiles only until
// their dP product, hence separate rings (3 and 2 slots).
//   TMEM columns: [0,128) S, [128,256) dP, [256,320) [320,384) dS operand buffers, [384, 384+D) dQ

template <int D> struct ACfg {
  static constexpr int kBoxes = D / 64;
  static constexpr int kTileBytes = kT * D * 2;
  static constexpr int kKSlots = 3, kVSlots = 2;
  static constexpr int kSmemTiles = (2 + kKSlots + kVSlots) * kTileBytes;
  static constexpr int kSmemBytes = kSmemTiles + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct ASync {
  uint64_t fixed_full;
  uint64_t k_full[3], k_empty[3];
  uint64_t v_full[2], v_empty[2];
  uint64_t sp_full;      // S and dP of a tile are complete
  uint64_t f_free;       // the elementwise role holds them in registers
  uint64_t e_ready[2];   // dS of a tile is in its operand buffer
  uint64_t op_empty[2];  // the product reading an operand buffer has retired
  uint64_t acc_done;
  uint64_t staged;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

// One 16-bit bias element (the query's dtype) as fp32.
template <bool BF16>
__device__ __forceinline__ float bias_to_f32(const uint32_t bits16) {
  if (BF16) return __uint_as_float(bits16 << 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

static_assert(sizeof(ASync) <= 272, "barrier block must fit its reserve (272 bytes + up to 1008 of alignment <= 1280)");

template <int D, bool BF16, bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_dq, const Problem p, const float* __restrict__ lse2,
                 const float* __restrict__ delta, const int l_pad, const int n_qblk, const int streams_per_wave,
                 const long long wait_limit) {
  using C = ACfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles = (raw_addr + 1023u) & ~1023u;
  ASync* sync = reinterpret_cast<ASync*>(smem_raw + (tiles - raw_addr) + C::kSmemTiles);
  volatile int* abort_flag = &sync->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // Latest query blocks (most key tiles under a causal mask) first, within waves of
  // `streams_per_wave` (batch, kv head) key/value streams that fit in L2 together.
  const int n_streams = p.Hkv * p.B;
  const int full_wave_ctas = n_qblk * streams_per_wave * p.group;
  const int wave = static_cast<int>(blockIdx.x / full_wave_ctas);
  const int in_wave = static_cast<int>(blockIdx.x - static_cast<unsigned>(wave) * full_wave_ctas);
  const int first_stream = wave * streams_per_wave;
  const int wave_streams = (n_streams - first_stream) < streams_per_wave ? (n_streams - first_stream) : streams_per_wave;
  const int per_blk = wave_streams * p.group;
  const int qblk = n_qblk - 1 - in_wave / per_blk;
  const int rem = in_wave % per_blk;
  const int kv_stream = first_stream + rem / p.group;
  const int hk = kv_stream % p.Hkv;
  const int b = kv_stream / p.Hkv;
  const int h = hk * p.group + rem % p.group;
  const int row0 = qblk * kT;
  const int kv_limit = valid_keys(p, b);
  long long end = kv_limit, first = kv_limit;
  if (p.causal) {
    const int last_row = (row0 + kT < p.L ? row0 + kT : p.L) - 1;
    const long long e = static_cast<long long>(last_row) + p.causal_shift + 1;
    const long long f = static_cast<long long>(row0) + p.causal_shift + 1;
    end = e < end ? e : end;
    first = f < first ? f : first;
  }
  if (end < 0) end = 0;
  if (first < -1) first = -1;
  const int n_tiles = static_cast<int>((end + kT - 1) / kT);
  const int min_lim = static_cast<int>(first);

  const uint32_t q_tile = tiles, do_tile = tiles + C::kTileBytes;
  const uint32_t k_ring = tiles + 2 * C::kTileBytes;
  const uint32_t v_ring = k_ring + C::kKSlots * C::kTileBytes;

  if (warp == kProducerWarp && lane == 0) {
    mbar_init(smem_u32(&sync->fixed_full), 1);
    for (int s = 0; s < C::kKSlots; ++s) {
      mbar_init(smem_u32(&sync->k_full[s]), 1);
      mbar_init(smem_u32(&sync->k_empty[s]), 1);
    }
    for (int s = 0; s < C::kVSlots; ++s) {
      mbar_init(smem_u32(&sync->v_full[s]), 1);
      mbar_init(smem_u32(&sync->v_empty[s]), 1);
    }
    mbar_fence_init();
    if (n_tiles > 0) {
      const uint32_t bar = smem_u32(&sync->fixed_full);
      mbar_arrive_expect_tx(bar, 2 * C::kTileBytes);
      for (int bx = 0; bx < C::kBoxes; ++bx) {
        tma_load_4d(q_tile + bx * kBoxBytes, &tm_q, bar, bx * 64, row0, h, b);
        tma_load_4d(do_tile + bx * kBoxBytes, &tm_do, bar, bx * 64, row0, h, b);
      }
    }
    prefetch_tmap(&tm_dq);
  }
  if (tid == 0) {
    mbar_init(smem_u32(&sync->sp_full), 1);
    mbar_init(smem_u32(&sync->f_free), kEThreads);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sync->e_ready[i]), kEThreads);
      mbar_init(smem_u32(&sync->op_empty[i]), 1);
    }
    mbar_init(smem_u32(&sync->acc_done), 1);
    mbar_init(smem_u32(&sync->staged), kEThreads);
    mbar_init(smem_u32(&sync->drain), 1);
    sync->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sync->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sync->tmem_base;
  constexpr uint32_t kColS = 0, kColDP = 128, kColOp = 256, kColDQ = 384;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int ks = j % C::kKSlots, vs = j % C::kVSlots;
        if (j >= C::kKSlots &&
            !wait_clocked(smem_u32(&sync->k_empty[ks]), (j / C::kKSlots - 1) & 1u, abort_flag, wait_limit)) {
          report(p.status, 11, j, ks);
          break;
        }
        {
          const uint32_t bar = smem_u32(&sync->k_full[ks]);
          mbar_arrive_expect_tx(bar, C::kTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(k_ring + ks * C::kTileBytes + bx * kBoxBytes, &tm_k, bar, bx * 64, j * kT, hk, b);
        }
        if (j >= C::kVSlots &&
            !wait_clocked(smem_u32(&sync->v_empty[vs]), (j / C::kVSlots - 1) & 1u, abort_flag, wait_limit)) {
          report(p.status, 11, j, 8 + vs);
          break;
        }
        {
          const uint32_t bar = smem_u32(&sync->v_full[vs]);
          mbar_arrive_expect_tx(bar, C::kTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(v_ring + vs * C::kTileBytes + bx * kBoxBytes, &tm_v, bar, bx * 64, j * kT, hk, b);
        }
      }
      if (*abort_flag != 0) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);   // copies in flight must land before exit
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    constexpr uint32_t idesc_score = make_idesc(BF16, false, kT, kT);
    constexpr uint32_t idesc_acc = make_idesc(BF16, true, kT, D);
    bool alive = n_tiles > 0;
    if (alive) {
      alive = wait_clocked(smem_u32(&sync->fixed_full), 0, abort_flag, wait_limit);
      if (!alive && lane == 0) report(p.status, 12, -1, 0);
    }
    // S_j = Q K_j^T, dP_j = dO V_j^T over whole tiles
    auto issue_scores = [&](int j) -> bool {
      const int ks = j % C::kKSlots, vs = j % C::kVSlots;
      if (!wait_clocked(smem_u32(&sync->k_full[ks]), (j / C::kKSlots) & 1u, abort_flag, wait_limit) ||
          !wait_clocked(smem_u32(&sync->v_full[vs]), (j / C::kVSlots) & 1u, abort_flag, wait_limit)) {
        if (lane == 0) report(p.status, 12, j, ks);
        return false;
      }
      tc_fence_after_sync();
      const uint64_t qd = kmajor_desc(q_tile), kd = kmajor_desc(k_ring + ks * C::kTileBytes);
      const uint64_t od = kmajor_desc(do_tile), vd = kmajor_desc(v_ring + vs * C::kTileBytes);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem_base + kColS, qd + kmajor_step(kk), kd + kmajor_step(kk), idesc_score, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem_base + kColDP, od + kmajor_step(kk), vd + kmajor_step(kk), idesc_score, kk > 0 ? 1u : 0u);
        mma_commit(smem_u32(&sync->sp_full));
        mma_commit(smem_u32(&sync->v_empty[vs]));   // V_j has no reader after dP_j
      }
      return true;
    };
    if (alive) alive = issue_scores(0);
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int buf = j & 1, ks = j % C::kKSlots;
      // S_j and dP_j are in registers: the next tile's score products may overwrite them
      alive = wait_clocked(smem_u32(&sync->f_free), j & 1, abort_flag, wait_limit);
      if (!alive) {
        if (lane == 0) report(p.status, 13, j, 1);
        break;
      }
      tc_fence_after_sync();
      if (j + 1 < n_tiles) {
        alive = issue_scores(j + 1);
        if (!alive) break;
      }
      alive = wait_clocked(smem_u32(&sync->e_ready[buf]), (j >> 1) & 1, abort_flag, wait_limit);
      if (!alive) {
        if (lane == 0) report(p.status, 13, j, 0);
        break;
      }
      tc_fence_after_sync();
      const uint64_t bd = mnmajor_desc(k_ring + ks * C::kTileBytes);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < kT / 16; ++kk)   // dQ += dS_j K_j
          mma_ts(tmem_base + kColDQ, tmem_base + kColOp + buf * 64 + static_cast<uint32_t>(kk * 8), bd + mnmajor_step(kk),
                 idesc_acc, (kk > 0 || j > 0) ? 1u : 0u);
        mma_commit(smem_u32(&sync->op_empty[buf]));
        mma_commit(smem_u32(&sync->k_empty[ks]));
        if (j + 1 == n_tiles) mma_commit(smem_u32(&sync->acc_done));
      }
    }
    if (*abort_flag != 0) {
      if (elect_one()) mma_commit(smem_u32(&sync->drain));
      const long long t0 = clock64();
      while (!mbar_try_wait(smem_u32(&sync->drain), 0) && clock64() - t0 < kDrainCycles) {
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------- elementwise role
    const int r = tid & (kT - 1);              // query row inside the tile = TMEM lane
    const int half = tid >> 7;                 // which 64 of the tile's 128 score columns
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + kColS + half * 64;
    const uint32_t dp_addr = tmem_base + lane_off + kColDP + half * 64;
    const uint32_t op_addr = tmem_base + lane_off + kColOp + half * 32;
    const uint32_t dq_addr = tmem_base + lane_off + kColDQ;
    // checked build: the column ranges of this thread's tensor-memory traffic; a violation drains the CTA
    if (!dbg_tmem(p.status, DBG_BWD_TC * 100 + 2, s_addr, tmem_base, 64, kTmemCols) || !dbg_tmem(p.status, DBG_BWD_TC * 100 + 3, dp_addr, tmem_base, 64, kTmemCols) ||
        !dbg_tmem(p.status, DBG_BWD_TC * 100 + 4, op_addr, tmem_base, 32, kTmemCols) || !dbg_tmem(p.status, DBG_BWD_TC * 100 + 5, dq_addr, tmem_base, D, kTmemCols))
      *abort_flag = 1;
    const int row_g = row0 + r;
    int lim = kv_limit;
    if (p.causal) {
      const long long c = static_cast<long long>(row_g) + p.causal_shift + 1;
      lim = c < lim ? static_cast<int>(c < 0 ? 0 : c) : lim;
    }
    const long long stat_idx = (static_cast<long long>(b) * p.Hq + h) * l_pad + row_g;
    const bool stat_ok = dbg_range(p.status, DBG_BWD_TC * 100 + 6, stat_idx, 1, static_cast<long long>(p.B) * p.Hq * l_pad);
    const float neg_l2 = stat_ok ? -lse2[stat_idx] : -CUDART_INF_F;      // -inf for rows without a visible key
    const float dl = stat_ok ? delta[stat_idx] : 0.f;
    const float sl2 = p.scale * kLog2e;
    bool alive = true;
    // this row of the forward's additive bias (the query's dtype, unit stride along the keys)
    const uint4* bias_row = nullptr;
    if constexpr (BIAS) {
      if (row_g < p.L)
        bias_row = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + b * p.bs[0] +
                                                  static_cast<long long>(h) * p.bs[1] +
                                                  static_cast<long long>(row_g) * p.bs[2]);
    }
    const bool bias_wide = BIAS && bias_rows_32b(p);
    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      uint4 bv[BIAS ? 8 : 1];   // this thread's 64 bias elements of the tile, fetched under the wait
      if constexpr (BIAS) load_bias_row(bv, bias_row, j * kT + half * 64, p.S, bias_wide);
      const uint32_t* bw = reinterpret_cast<const uint32_t*>(bv);
      bool ok = wait_clocked(smem_u32(&sync->sp_full), j & 1, abort_flag, wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 14, j, warp);
        alive = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t sv[64], dv[64];
      tmem_ld_32x32(s_addr, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
      tmem_ld_32x32(s_addr + 32, reinterpret_cast<uint32_t(&)[32]>(sv[32]));
      tmem_ld_32x32(dp_addr, reinterpret_cast<uint32_t(&)[32]>(dv[0]));
      tmem_ld_32x32(dp_addr + 32, reinterpret_cast<uint32_t(&)[32]>(dv[32]));
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sync->f_free));
      const int col0 = j * kT + half * 64;
      const bool need_mask = j * kT + kT > min_lim;
      uint32_t pk[32];
      // two columns per instruction (packed fp32 pairs) wherever the arithmetic allows: the loop is bound by
      // what the eight warps can issue beside their 64 exponentials each
      const uint64_t sl2_2 = f2_pack(sl2, sl2), neg_dl2 = f2_pack(-dl, -dl);
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        float off0 = neg_l2, off1 = neg_l2;
        if constexpr (BIAS) {
          off0 = fmaf(bias_to_f32<BF16>(bw[i >> 1] & 0xffffu), kLog2e, neg_l2);
          off1 = fmaf(bias_to_f32<BF16>(bw[i >> 1] >> 16), kLog2e, neg_l2);
        }
        float a0, a1;
        f2_unpack(f2_fma(f2_pack(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sl2_2, f2_pack(off0, off1)), a0, a1);
        float p0 = ex2(a0);
        float p1 = ex2(a1);
        if (need_mask) {
          p0 = (col0 + i < lim) ? p0 : 0.f;
          p1 = (col0 + i + 1 < lim) ? p1 : 0.f;
        }
        float d0, d1;
        f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack(__uint_as_float(dv[i]), __uint_as_float(dv[i + 1])), neg_dl2)), d0, d1);
        pk[i >> 1] = pack2<BF16>(d0, d1);
      }
      if (j >= 2) {   // the product that read this operand buffer two tiles ago must have retired
        ok = wait_clocked(smem_u32(&sync->op_empty[buf]), ((j >> 1) - 1) & 1, abort_flag, wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 16, j, warp);
          alive = false;
          break;
        }
        tc_fence_after_sync();
      }
      tmem_st_32x16(op_addr + buf * 64, reinterpret_cast<uint32_t(&)[16]>(pk[0]));
      tmem_st_32x16(op_addr + buf * 64 + 16, reinterpret_cast<uint32_t(&)[16]>(pk[16]));
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sync->e_ready[buf]));
    }
    if (alive && n_tiles > 0) {
      bool ok = wait_clocked(smem_u32(&sync->acc_done), 0, abort_flag, wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 15, 0, warp);
        alive = false;
      }
      tc_fence_after_sync();
    }
    if (alive) {
      uint8_t* stage = smem_raw + (q_tile - raw_addr);   // Q is no longer needed
      stage_row<D, BF16>(dq_addr, n_tiles > 0, p.scale, stage, r, half);
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sync->staged));
      if (tid == 0 && wait_clocked(smem_u32(&sync->staged), 0, abort_flag, wait_limit)) {
        for (int bx = 0; bx < C::kBoxes; ++bx) tma_store_4d(&tm_dq, q_tile + bx * kBoxBytes, bx * 64, row0, h, b);
        tma_store_commit();
        tma_store_wait_read();
      }
    }
  }

  // Launched as a programmatic dependent of the dK/dV kernel, of which it reads nothing.  One CTA -- the last
  // of the grid, which is also the last to be placed -- waits for that grid before it exits, so that this grid
  // cannot complete before it and work queued behind finds both done; the others must not wait (a finished CTA
  // parked on its SM would keep the next one from starting).
  if (blockIdx.x == gridDim.x - 1) asm volatile("griddepcontrol.wait;" ::: "memory");
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------- dK/dV kernel --

template <int D, bool BF16, bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                  const Problem p, const float* __restrict__ lse2, const float* __restrict__ delta, const int l_pad,
                  const int n_kblk, const int streams_per_wave, const long long wait_limit) {
  using C = BCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles = (raw_addr + 1023u) & ~1023u;
  float* stats = reinterpret_cast<float*>(smem_raw + (tiles - raw_addr) + C::kSmemTiles);
  BSync* sync = reinterpret_cast<BSync*>(smem_raw + (tiles - raw_addr) + C::kSmemTiles + C::kStatBytes);
  volatile int* abort_flag = &sync->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // the dQ kernel (a programmatic dependent launch that does not read anything this kernel writes) may be
  // placed on SMs as soon as every CTA of this grid is resident
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Earliest key blocks (seen by the most query tiles under a causal mask) first, within waves of
  // `streams_per_wave` (batch, kv head) groups whose query-side operands fit in L2 together.
  const int n_streams = p.Hkv * p.B;
  const int full_wave_ctas = n_kblk * streams_per_wave;
  const int wave = static_cast<int>(blockIdx.x / full_wave_ctas);
  const int in_wave = static_cast<int>(blockIdx.x - static_cast<unsigned>(wave) * full_wave_ctas);
  const int first_stream = wave * streams_per_wave;
  const int wave_streams = (n_streams - first_stream) < streams_per_wave ? (n_streams - first_stream) : streams_per_wave;
  const int kblk = in_wave / wave_streams;
  const int kv_stream = first_stream + in_wave % wave_streams;
  const int hk = kv_stream % p.Hkv;
  const int b = kv_stream / p.Hkv;
  const int j0 = kblk * kT;
  const int n_keys = valid_keys(p, b);
  const int n_qt = (p.L + kT - 1) / kT;
  int i_first = 0;
  if (p.causal) {
    const long long f = static_cast<long long>(j0) - p.causal_shift;   // first row that sees key j0
    i_first = f <= 0 ? 0 : (f >= p.L ? n_qt : static_cast<int>(f / kT));
  }
  const int per_head = (j0 < n_keys && n_qt > i_first) ? n_qt - i_first : 0;
  const int n_items = per_head * p.group;

  const uint32_t k_tile = tiles, v_tile = tiles + C::kTileBytes;
  const uint32_t ring = tiles + 2 * C::kTileBytes;   // slot s: Q at ring + 2 s tile, dO right after

  if (warp == kProducerWarp && lane == 0) {
    mbar_init(smem_u32(&sync->fixed_full), 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sync->ring_full[s]), 1);
      mbar_init(smem_u32(&sync->ring_empty[s]), 1);
    }
    mbar_fence_init();
    if (n_items > 0) {
      const uint32_t bar = smem_u32(&sync->fixed_full);
      mbar_arrive_expect_tx(bar, 2 * C::kTileBytes);
      for (int bx = 0; bx < C::kBoxes; ++bx) {
        tma_load_4d(k_tile + bx * kBoxBytes, &tm_k, bar, bx * 64, j0, hk, b);
        tma_load_4d(v_tile + bx * kBoxBytes, &tm_v, bar, bx * 64, j0, hk, b);
      }
    }
    prefetch_tmap(&tm_dk);
    prefetch_tmap(&tm_dv);
  }
  if (tid == 0) init_common_barriers(sync);
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sync->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sync->tmem_base;
  constexpr uint32_t kColDV = kColAcc, kColDK = kColAcc + D;
  const int n_units = 2 * n_items;

  if (warp == kProducerWarp) {
    // the whole warp runs the loop: the lanes copy the query tile's row statistics into
    // the slot, lane 0 then arms the barrier (its release makes the copies visible) and
    // starts the tile copies
    bool alive = true;
    // The row statistics of an item are fetched one item ahead, so that their global-memory latency
    // passes during the wait for the slot instead of between the slot's release and the tile copies
    // (measured: 1.2-2.0 k cycles per item on the path that feeds the MMA warp).
    float4 st_l = make_float4(0.f, 0.f, 0.f, 0.f), st_d = st_l;
    auto fetch_stats = [&](int item) {
      const int h_ = hk * p.group + item / per_head;
      const int qrow_ = (i_first + item % per_head) * kT;
      const long long src = (static_cast<long long>(b) * p.Hq + h_) * l_pad + qrow_;
      if (dbg_range(p.status, DBG_BWD_TC * 100 + 10, src, kT, static_cast<long long>(p.B) * p.Hq * l_pad)) {
        st_l = reinterpret_cast<const float4*>(lse2 + src)[lane];
        st_d = reinterpret_cast<const float4*>(delta + src)[lane];
      }
    };
    if (n_items > 0) fetch_stats(0);
    for (int it = 0; it < n_items && alive; ++it) {
      const int stage = it % C::kStages;
      const uint32_t round = static_cast<uint32_t>(it / C::kStages);
      if (round > 0) {
        alive = wait_clocked(smem_u32(&sync->ring_empty[stage]), (round - 1) & 1u, abort_flag, wait_limit);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) {
          if (lane == 0) report(p.status, 21, it, stage);
          break;
        }
      }
      const int h = hk * p.group + it / per_head;
      const int qrow0 = (i_first + it % per_head) * kT;
      float4* dst = reinterpret_cast<float4*>(stats + stage * 2 * kT);
      dst[lane] = st_l;
      dst[32 + lane] = st_d;
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = smem_u32(&sync->ring_full[stage]);
        const uint32_t q_dst = ring + stage * 2 * C::kTileBytes;
        mbar_arrive_expect_tx(bar, 2 * C::kTileBytes);
        for (int bx = 0; bx < C::kBoxes; ++bx) {
          tma_load_4d(q_dst + bx * kBoxBytes, &tm_q, bar, bx * 64, qrow0, h, b);
          tma_load_4d(q_dst + C::kTileBytes + bx * kBoxBytes, &tm_do, bar, bx * 64, qrow0, h, b);
        }
      }
      if (it + 1 < n_items) fetch_stats(it + 1);
    }
    if (*abort_flag != 0 && lane == 0) {
      for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    constexpr uint32_t idesc_score = make_idesc(BF16, false, kT, kU);
    constexpr uint32_t idesc_acc = make_idesc(BF16, true, kT, D);
    bool alive = n_items > 0;
    if (alive) {
      alive = wait_clocked(smem_u32(&sync->fixed_full), 0, abort_flag, wait_limit);
      if (!alive && lane == 0) report(p.status, 22, -1, 0);
    }
    // S^T_u = K Q_u^T and dP^T_u = V dO_u^T into buffer u & 1 (waits for the query tile when the unit opens it)
    auto issue_scores = [&](int u) -> bool {
      const int it = u >> 1, hh = u & 1, buf = u & 1;
      const int stage = it % C::kStages;
      if (hh == 0) {
        const uint32_t round = static_cast<uint32_t>(it / C::kStages);
        if (!wait_clocked(smem_u32(&sync->ring_full[stage]), round & 1u, abort_flag, wait_limit)) {
          if (lane == 0) report(p.status, 22, it, stage);
          return false;
        }
        tc_fence_after_sync();
      }
      const uint32_t q_tile = ring + stage * 2 * C::kTileBytes, do_tile = q_tile + C::kTileBytes;
      issue_ss<D>(tmem_base + kColS + buf * kU, k_tile, q_tile, hh, idesc_score);
      issue_ss<D>(tmem_base + kColDP + buf * kU, v_tile, do_tile, hh, idesc_score);
      if (elect_one()) mma_commit(smem_u32(&sync->sp_full[buf]));
      return true;
    };
    if (alive) alive = issue_scores(0);
    if (alive) alive = issue_scores(1);
    for (int u = 0; u < n_units && alive; ++u) {
      const int it = u >> 1, hh = u & 1, buf = u & 1;
      const int stage = it % C::kStages;
      alive = wait_clocked(smem_u32(&sync->e_ready[buf]), (u >> 1) & 1, abort_flag, wait_limit);
      if (!alive) {
        if (lane == 0) report(p.status, 23, u, 0);
        break;
      }
      tc_fence_after_sync();
      const uint32_t q_tile = ring + stage * 2 * C::kTileBytes, do_tile = q_tile + C::kTileBytes;
      issue_ts(tmem_base + kColDV, tmem_base + kColS + buf * kU, do_tile, hh, idesc_acc, u > 0);   // dV += P^T_u dO_u
      issue_ts(tmem_base + kColDK, tmem_base + kColDP + buf * kU, q_tile, hh, idesc_acc, u > 0);   // dK += dS^T_u Q_u
      if (elect_one()) {
        if (hh == 1) mma_commit(smem_u32(&sync->ring_empty[stage]));
        if (u + 1 == n_units) mma_commit(smem_u32(&sync->acc_done));
      }
      if (u + 2 < n_units) alive = issue_scores(u + 2);
    }
    if (*abort_flag != 0) drain_after_abort(sync, wait_limit);
    __syncwarp();
  } else {
    // -------------------------------------------------------- elementwise role
    const int r = tid & (kT - 1);              // key inside the tile = TMEM lane
    const int half = tid >> 7;                 // which 32 of the unit's 64 query columns
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + kColS + half * 32;
    const uint32_t dp_addr = tmem_base + lane_off + kColDP + half * 32;
    // checked build: both buffers of the score-shaped units and the two accumulators
    if (!dbg_tmem(p.status, DBG_BWD_TC * 100 + 7, s_addr, tmem_base, kU + 32, kTmemCols) ||
        !dbg_tmem(p.status, DBG_BWD_TC * 100 + 8, dp_addr, tmem_base, kU + 32, kTmemCols) ||
        !dbg_tmem(p.status, DBG_BWD_TC * 100 + 9, tmem_base + lane_off + kColDK, tmem_base, D, kTmemCols))
      *abort_flag = 1;
    const int key_g = j0 + r;
    // query rows i >= i_min see this key; a padded key is seen by nobody
    int i_min = 0;
    if (p.causal) {
      const long long v = static_cast<long long>(key_g) - p.causal_shift;
      i_min = v < 0 ? 0 : (v > (1 << 30) ? (1 << 30) : static_cast<int>(v));
    }
    if (key_g >= n_keys) i_min = 1 << 30;
    const bool tile_has_padding = j0 + kT > n_keys;
    const float sl2 = p.scale * kLog2e;
    const uint64_t sl2_2 = f2_pack(sl2, sl2);
    bool alive = true;
    for (int u = 0; u < n_units; ++u) {
      const int it = u >> 1, hh = u & 1, buf = u & 1;
      const int unit_row0 = (i_first + it % per_head) * kT + hh * kU;   // first query row of the unit
      const int qrow0 = unit_row0 + half * 32;                          // ... and of this thread's columns
      uint32_t bq[BIAS ? 32 : 1];   // bias of this key under the thread's 32 query rows, fetched under the wait
      if constexpr (BIAS) {
        // neighbouring lanes are neighbouring keys: each of the 32 loads is one 64-byte piece per warp
        const uint16_t* col = static_cast<const uint16_t*>(p.bias) + b * p.bs[0] +
                              static_cast<long long>(hk * p.group + it / per_head) * p.bs[1] + key_g;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          bq[i] = (key_g < p.S && qrow0 + i < p.L) ? __ldg(col + static_cast<long long>(qrow0 + i) * p.bs[2]) : 0u;
      }
      bool ok = wait_clocked(smem_u32(&sync->sp_full[buf]), (u >> 1) & 1, abort_flag, wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 24, u, warp);
        alive = false;
        break;
      }
      tc_fence_after_sync();
      const int stage = it % C::kStages;
      const float4* st4 = reinterpret_cast<const float4*>(stats + stage * 2 * kT) + hh * 16 + half * 8;
      // some key of this tile hides some row of this unit
      const bool need_mask = tile_has_padding ||
                             (p.causal && static_cast<long long>(unit_row0) < static_cast<long long>(j0) + kT - 1 - p.causal_shift);
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(s_addr + buf * kU, sv);
      tmem_ld_32x32(dp_addr + buf * kU, dv);
      tmem_ld_wait();
      uint32_t pkp[16], pkd[16];
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4) {
        const float4 l4 = st4[q4];
        const float4 d4 = st4[32 + q4];
        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
        const float ds_[4] = {d4.x, d4.y, d4.z, d4.w};
        float pr[4], dsv[4];
#pragma unroll
        for (int e = 0; e < 4; e += 2) {   // two query columns per instruction (packed fp32 pairs)
          const int i = q4 * 4 + e;
          float off0 = -ls[e], off1 = -ls[e + 1];
          if constexpr (BIAS) {
            off0 = fmaf(bias_to_f32<BF16>(bq[i]), kLog2e, off0);
            off1 = fmaf(bias_to_f32<BF16>(bq[i + 1]), kLog2e, off1);
          }
          float a0, a1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sl2_2, f2_pack(off0, off1)), a0, a1);
          float p0 = ex2(a0), p1 = ex2(a1);
          if (need_mask) {
            p0 = (qrow0 + i >= i_min) ? p0 : 0.f;
            p1 = (qrow0 + i + 1 >= i_min) ? p1 : 0.f;
          }
          pr[e] = p0;
          pr[e + 1] = p1;
          f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack(__uint_as_float(dv[i]), __uint_as_float(dv[i + 1])),
                                                    f2_pack(-ds_[e], -ds_[e + 1]))),
                    dsv[e], dsv[e + 1]);
        }
        pkp[q4 * 2] = pack2<BF16>(pr[0], pr[1]);
        pkp[q4 * 2 + 1] = pack2<BF16>(pr[2], pr[3]);
        pkd[q4 * 2] = pack2<BF16>(dsv[0], dsv[1]);
        pkd[q4 * 2 + 1] = pack2<BF16>(dsv[2], dsv[3]);
      }
      tmem_st_32x16(s_addr + buf * kU, pkp);
      tmem_st_32x16(dp_addr + buf * kU, pkd);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sync->e_ready[buf]));
    }
    if (alive && n_items > 0) {
      bool ok = wait_clocked(smem_u32(&sync->acc_done), 0, abort_flag, wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 25, 0, warp);
        alive = false;
      }
      tc_fence_after_sync();
    }
    if (alive) {
      // ring slot 0 is idle by now: its two tiles stage dK and dV
      uint8_t* stage_k = smem_raw + (ring - raw_addr);
      uint8_t* stage_v = stage_k + C::kTileBytes;
      stage_row<D, BF16>(tmem_base + lane_off + kColDK, n_items > 0, p.scale, stage_k, r, half);
      stage_row<D, BF16>(tmem_base + lane_off + kColDV, n_items > 0, 1.f, stage_v, r, half);
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sync->staged));
      if (tid == 0 && wait_clocked(smem_u32(&sync->staged), 0, abort_flag, wait_limit)) {
        for (int bx = 0; bx < C::kBoxes; ++bx) {
          tma_store_4d(&tm_dk, ring + bx * kBoxBytes, bx * 64, j0, hk, b);
          tma_store_4d(&tm_dv, ring + C::kTileBytes + bx * kBoxBytes, bx * 64, j0, hk, b);
        }
        tma_store_commit();
        tma_store_wait_read();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side --

int padded_rows(const Problem& p) { return (p.L + kT - 1) / kT * kT; }

template <int D, bool BF16, bool BIAS>
int launch_tc(const BwdProblem& bp, float* lse2, float* delta, cudaStream_t stream) {
  using C = BCfg<D>;
  const Problem& p = bp.f;
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (!make_map(&tq, p.q, BF16, D, p.L, p.Hq, p.B, p.qs) || !make_map(&tk, p.k, BF16, D, p.S, p.Hkv, p.B, p.ks) ||
      !make_map(&tv, p.v, BF16, D, p.S, p.Hkv, p.B, p.vs) || !make_map(&tdo, bp.dout, BF16, D, p.L, p.Hq, p.B, bp.dos) ||
      !make_map(&tdq, bp.dq, BF16, D, p.L, p.Hq, p.B, bp.dqs) ||
      !make_map(&tdk, bp.dk, BF16, D, p.S, p.Hkv, p.B, bp.dks) ||
      !make_map(&tdv, bp.dv, BF16, D, p.S, p.Hkv, p.B, bp.dvs))
    return B200_SDPA_ERR_CUDA;
  auto kq = bwd_dq_tc_kernel<D, BF16, BIAS>;
  auto kkv = bwd_dkv_tc_kernel<D, BF16, BIAS>;
  if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, ACfg<D>::kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  const int l_pad = padded_rows(p);
  {
    const long long rows = static_cast<long long>(p.B) * p.Hq * l_pad;
    auto rows_aligned = [](const void* base, const int64_t* st) {
      return st[3] == 1 && reinterpret_cast<uintptr_t>(base) % 16 == 0 && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
    };
    const bool vec = p.Dv % 8 == 0 && rows_aligned(bp.dout, bp.dos) && rows_aligned(p.out, p.os);
    const long long warps = vec ? (rows + 3) / 4 : rows;
    const long long blocks = (warps * 32 + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
    const unsigned grid = static_cast<unsigned>(blocks);
    if (BF16) {
      if (vec) bwd_prep_kernel<__nv_bfloat16, true><<<grid, 256, 0, stream>>>(bp, lse2, delta, l_pad);
      else bwd_prep_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>(bp, lse2, delta, l_pad);
    } else {
      if (vec) bwd_prep_kernel<__half, true><<<grid, 256, 0, stream>>>(bp, lse2, delta, l_pad);
      else bwd_prep_kernel<__half, false><<<grid, 256, 0, stream>>>(bp, lse2, delta, l_pad);
    }
    if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
    count_launch(KID_BWD_PREP);
  }
  const int n_qblk = (p.L + kT - 1) / kT, n_kblk = (p.S + kT - 1) / kT;
  const long long grid_q = static_cast<long long>(n_qblk) * p.Hq * p.B;
  const long long grid_kv = static_cast<long long>(n_kblk) * p.Hkv * p.B;
  if (grid_q > 0x7fffffffLL || grid_kv > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  const long long limit = wait_limit_cycles();
  const long long n_streams = static_cast<long long>(p.Hkv) * p.B;
  // the dQ kernel streams keys and values; the dK/dV kernel the queries, dO and row statistics of a group
  const int wave_q = kv_streams_per_wave(static_cast<long long>(p.S) * 2 * D * 2, n_streams);
  const int wave_kv = kv_streams_per_wave(static_cast<long long>(p.L) * p.group * (2 * D * 2 + 8), n_streams);
  // The two kernels are independent of each other (both read the row statistics of the kernel before them).
  // The dK/dV kernel, whose CTAs are long, goes first and releases its dependents as soon as its last CTA is
  // resident; the dQ kernel is a programmatic dependent launch, so its CTAs take the SMs the first kernel's
  // tail leaves idle.  It waits for the first kernel's completion only before it exits (stream order for
  // whatever follows).
  kkv<<<static_cast<unsigned>(grid_kv), kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, tdk, tdv, p, lse2, delta,
                                                                          l_pad, n_kblk, wave_kv, limit);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_BWD_DKV);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid_q));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = ACfg<D>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* c_lse2 = lse2;
  const float* c_delta = delta;
  if (cudaLaunchKernelEx(&cfg, kq, tq, tk, tv, tdo, tdq, p, c_lse2, c_delta, l_pad, n_qblk, wave_q, limit) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  count_launch(KID_BWD_DQ);
  return B200_SDPA_OK;
}

}  // namespace


bool bwd_tc_eligible(const BwdProblem& bp, int dtype, bool* alignment_only_failure) {
  const Problem& p = bp.f;
  if (alignment_only_failure) *alignment_only_failure = false;
  if (dtype != B200_SDPA_F16 && dtype != B200_SDPA_BF16) return false;
  if (p.E != p.Dv || (p.E != 64 && p.E != 128)) return false;
  if (bp.dbias != nullptr) return false;   // the logit gradient is written by the CUDA-core kernels only
  if (!(p.scale > 0.f) || !(p.scale < 1e30f)) return false;
  if (p.L < 1 || p.S < 1) return false;
  if (p.bias != nullptr) {
    if (!bias_readable(p, dtype, alignment_only_failure)) return false;   // as in the forward
  }
  const bool ok = strides_ok(p.q, p.qs, p.L, p.Hq, p.B) && strides_ok(p.k, p.ks, p.S, p.Hkv, p.B) &&
                  strides_ok(p.v, p.vs, p.S, p.Hkv, p.B) && strides_ok(bp.dout, bp.dos, p.L, p.Hq, p.B) &&
                  strides_ok(bp.dq, bp.dqs, p.L, p.Hq, p.B) && strides_ok(bp.dk, bp.dks, p.S, p.Hkv, p.B) &&
                  strides_ok(bp.dv, bp.dvs, p.S, p.Hkv, p.B);
  if (!ok && alignment_only_failure) *alignment_only_failure = true;
  return ok;
}

uint64_t bwd_tc_workspace_bytes(const BwdProblem& bp) {
  return 2ull * sizeof(float) * static_cast<uint64_t>(bp.f.B) * bp.f.Hq * padded_rows(bp.f);
}

int plan_bwd_tc(const BwdProblem& bp, int dtype, B200SdpaPlan* plan) {
  const Problem& p = bp.f;
  (void)dtype;
  plan->path = B200_SDPA_PATH_PREFILL;
  plan->block_m = kT;
  plan->block_n = kT;
  plan->grid_x = static_cast<int32_t>(static_cast<long long>((p.L + kT - 1) / kT) * p.Hq * p.B);
  plan->grid_y = static_cast<int32_t>(static_cast<long long>((p.S + kT - 1) / kT) * p.Hkv * p.B);
  plan->grid_z = 1;
  plan->threads = kThreads;
  plan->smem_bytes = p.E == 128 ? BCfg<128>::kSmemBytes : BCfg<64>::kSmemBytes;
  plan->kv_splits = 1;
  plan->launches = 3;
  plan->workspace_bytes = bwd_tc_workspace_bytes(bp);
  return B200_SDPA_OK;
}

int launch_bwd_tc(const BwdProblem& bp, int dtype, void* workspace, uint64_t workspace_bytes, cudaStream_t stream) {
  if (!bwd_tc_eligible(bp, dtype, nullptr)) return B200_SDPA_ERR_UNSUPPORTED;
  const uint64_t need = bwd_tc_workspace_bytes(bp);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 16)
    return B200_SDPA_ERR_WORKSPACE;
  float* lse2 = reinterpret_cast<float*>(workspace);
  float* delta = lse2 + need / (2 * sizeof(float));
  const bool bf16 = dtype == B200_SDPA_BF16;
  if (bp.f.bias != nullptr) {
    if (bp.f.E == 128)
      return bf16 ? launch_tc<128, true, true>(bp, lse2, delta, stream) : launch_tc<128, false, true>(bp, lse2, delta, stream);
    return bf16 ? launch_tc<64, true, true>(bp, lse2, delta, stream) : launch_tc<64, false, true>(bp, lse2, delta, stream);
  }
  if (bp.f.E == 128)
    return bf16 ? launch_tc<128, true, false>(bp, lse2, delta, stream) : launch_tc<128, false, false>(bp, lse2, delta, stream);
  return bf16 ? launch_tc<64, true, false>(bp, lse2, delta, stream) : launch_tc<64, false, false>(bp, lse2, delta, stream);
}

}  // namespace b200
