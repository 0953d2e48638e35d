// Prefill kernel for head dimensions beyond 128: query/key dimension E = 192 with value
// dimension Dv = 128 (the shape of multi-head-latent-attention models, which upstream tests as
// tests/python_ops/test_scaled_dot_product_attention.py:46-97,117-180), and E = Dv = 256.
//
// Same arithmetic, operand layouts and barrier discipline as prefill_sm100.cu.  The 48 KB Q
// and K tiles leave no room for two query tiles per CTA, so one CTA owns one 128-row tile:
// Q (48 KB) + two K slots (48 KB each) + two V slots (32 KB each) = 208 KB of shared memory
// (at 256: Q, one K slot and one V slot of 64 KB each).
// Roles (192 threads): warps 0-3 softmax (one thread per query row = TMEM lane), warp 4 TMA
// producer, warp 5 MMA issuer.  TMEM columns: [0,128) and [128,256) scores of even and odd key
// tiles (P overwrites the first 64 columns of its buffer as 16-bit pairs), [256,256+Dv) O.  With
// two score buffers Q K^T of the next key tile runs under the softmax of this one.
#include "tc_common.cuh"
#include "debug.cuh"

namespace b200 {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kM = 128;   // rows per query tile (= TMEM lanes)
constexpr int kN = 128;   // keys per tile
constexpr int kThreads = 192;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr float kRescaleThreshold = 8.0f;   // in units of log2

template <int E, int DV> struct CfgW {
  static constexpr int kBoxesQK = E / 64;
  static constexpr int kBoxesV = DV / 64;
  static constexpr int kTileQK = kN * E * 2;
  static constexpr int kTileV = kN * DV * 2;
  static constexpr int kSlots = (E <= 192) ? 2 : 1;      // K slots and V slots that fit beside Q
  static constexpr int kSmemTiles = (1 + kSlots) * kTileQK + kSlots * kTileV;
  static constexpr int kSmemBytes = kSmemTiles + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr uint32_t kTmemCols = 512;   // two score buffers + O (2 * 128 + DV), a power of two
};

struct SyncW {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2];       // per score buffer
  uint64_t p_ready[2][2];   // per score buffer, halves of P
  uint64_t pv_done;         // P V of a key tile has retired: O may be rescaled
  uint64_t o_done;
  uint64_t o_staged;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

static_assert(sizeof(SyncW) <= 272, "barrier block must fit its reserve (272 bytes + up to 1008 of alignment <= 1280)");

template <int E, int DV, bool BF16, bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
prefill_wide_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const Problem p,
                const int n_qblk, const int streams_per_wave, const long long wait_limit) {
  using C = CfgW<E, DV>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles = (raw_addr + 1023u) & ~1023u;
  SyncW* sync = reinterpret_cast<SyncW*>(smem_raw + (tiles - raw_addr) + C::kSmemTiles);
  volatile int* abort_flag = &sync->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // Work order.  The (batch, kv head) key/value streams are taken `streams_per_wave` at a time, so that
  // the keys and values the CTAs in flight read together fit in L2; inside such a wave: latest query
  // blocks (most key tiles under a causal mask) first, the query heads of a kv head adjacent.
  const int n_streams = p.Hkv * p.B;
  const int full_wave_ctas = n_qblk * streams_per_wave * p.group;
  const int wave = static_cast<int>(blockIdx.x / full_wave_ctas);
  const int in_wave = static_cast<int>(blockIdx.x - static_cast<unsigned>(wave) * full_wave_ctas);
  const int first_stream = wave * streams_per_wave;
  const int wave_streams = (n_streams - first_stream) < streams_per_wave ? (n_streams - first_stream) : streams_per_wave;
  const int per_blk = wave_streams * p.group;
  const int qblk = n_qblk - 1 - in_wave / per_blk;
  const int rem = in_wave % per_blk;
  const int stream = first_stream + rem / p.group;
  const int hk = stream % p.Hkv;
  const int b = stream / p.Hkv;
  const int h = hk * p.group + rem % p.group;
  const int row0 = qblk * kM;
  const int kv_limit = valid_keys(p, b);
  long long end = kv_limit, first = kv_limit;
  if (p.causal) {
    const int last_row = (row0 + kM < p.L ? row0 + kM : p.L) - 1;
    const long long e = static_cast<long long>(last_row) + p.causal_shift + 1;
    const long long f = static_cast<long long>(row0) + p.causal_shift + 1;
    end = e < end ? e : end;
    first = f < first ? f : first;
  }
  if (end < 0) end = 0;
  if (first < -1) first = -1;
  const int n_tiles = static_cast<int>((end + kN - 1) / kN);
  const int min_lim = static_cast<int>(first);

  const uint32_t q_smem = tiles;
  const uint32_t k_smem = tiles + C::kTileQK;                       // slot s at + s * kTileQK
  const uint32_t v_smem = k_smem + C::kSlots * C::kTileQK;          // slot s at + s * kTileV
  auto load_k = [&](int j) {
    const uint32_t bar = smem_u32(&sync->k_full[j % C::kSlots]);
    mbar_arrive_expect_tx(bar, C::kTileQK);
    for (int bx = 0; bx < C::kBoxesQK; ++bx)
      tma_load_4d(k_smem + (j % C::kSlots) * C::kTileQK + bx * kBoxBytes, &tm_k, bar, bx * 64, j * kN, hk, b);
  };
  auto load_v = [&](int j) {
    const uint32_t bar = smem_u32(&sync->v_full[j % C::kSlots]);
    mbar_arrive_expect_tx(bar, C::kTileV);
    for (int bx = 0; bx < C::kBoxesV; ++bx)
      tma_load_4d(v_smem + (j % C::kSlots) * C::kTileV + bx * kBoxBytes, &tm_v, bar, bx * 64, j * kN, hk, b);
  };

  int tiles_issued = 0;   // (producer lane) key tiles whose K and V were issued before the set-up barrier
  if (warp == kProducerWarp && lane == 0) {
    mbar_init(smem_u32(&sync->q_full), 1);
    for (int s = 0; s < C::kSlots; ++s) {
      mbar_init(smem_u32(&sync->k_full[s]), 1);
      mbar_init(smem_u32(&sync->k_empty[s]), 1);
      mbar_init(smem_u32(&sync->v_full[s]), 1);
      mbar_init(smem_u32(&sync->v_empty[s]), 1);
    }
    mbar_fence_init();
    if (n_tiles > 0) {
      // a tile without visible keys never reads Q: its slot stages the all-zero output at once
      const uint32_t qbar = smem_u32(&sync->q_full);
      mbar_arrive_expect_tx(qbar, C::kTileQK);
      for (int bx = 0; bx < C::kBoxesQK; ++bx) tma_load_4d(q_smem + bx * kBoxBytes, &tm_q, qbar, bx * 64, row0, h, b);
    }
    for (; tiles_issued < n_tiles && tiles_issued < C::kSlots; ++tiles_issued) {
      load_k(tiles_issued);
      load_v(tiles_issued);
    }
    prefetch_tmap(&tm_o);
  }
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sync->s_full[i]), 1);
      mbar_init(smem_u32(&sync->p_ready[i][0]), kM);
      mbar_init(smem_u32(&sync->p_ready[i][1]), kM);
    }
    mbar_init(smem_u32(&sync->pv_done), 1);
    mbar_init(smem_u32(&sync->o_done), 1);
    mbar_init(smem_u32(&sync->o_staged), kM);
    mbar_init(smem_u32(&sync->drain), 1);
    sync->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sync->tmem_base), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sync->tmem_base;
  // Scores of key tile j live in buffer j & 1, so that Q K^T of the next tile runs under the softmax
  // of this one and P V of this one under the softmax of the next.
  constexpr uint32_t kColS = 0, kColO = 256;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = tiles_issued; j < n_tiles; ++j) {
        const int slot = j % C::kSlots;
        const uint32_t parity = static_cast<uint32_t>(j / C::kSlots - 1) & 1u;
        if (!wait_clocked(smem_u32(&sync->k_empty[slot]), parity, abort_flag, wait_limit)) {
          report(p.status, 1, j, slot);
          break;
        }
        load_k(j);
        if (!wait_clocked(smem_u32(&sync->v_empty[slot]), parity, abort_flag, wait_limit)) {
          report(p.status, 1, j, 8 + slot);
          break;
        }
        load_v(j);
      }
      if (*abort_flag != 0) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);   // copies in flight must land before exit
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = make_idesc(BF16, false, kM, kN);
    constexpr uint32_t idesc_pv = make_idesc(BF16, true, kM, DV);
    bool alive = n_tiles > 0;
    const uint64_t q_desc = smem_desc_sw128(q_smem, 16, 1024);
    auto issue_qk = [&](int j) -> bool {
      const int slot = j % C::kSlots;
      if (!wait_clocked(smem_u32(&sync->k_full[slot]), static_cast<uint32_t>(j / C::kSlots) & 1u, abort_flag, wait_limit)) {
        if (lane == 0) report(p.status, 2, j, slot);
        return false;
      }
      tc_fence_after_sync();
      const uint64_t kd = smem_desc_sw128(k_smem + slot * C::kTileQK, 16, 1024);   // K tile as K-major B operand
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < E / 16; ++kk) {
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * kBoxBytes + (kk & 3) * 32) >> 4);
          mma_ss(tmem_base + kColS + static_cast<uint32_t>((j & 1) * kN), q_desc + off, kd + off, idesc_qk, kk > 0 ? 1u : 0u);
        }
        mma_commit(smem_u32(&sync->s_full[j & 1]));
        mma_commit(smem_u32(&sync->k_empty[slot]));
      }
      return true;
    };
    if (alive) {
      alive = wait_clocked(smem_u32(&sync->q_full), 0, abort_flag, wait_limit);
      if (!alive && lane == 0) report(p.status, 2, -1, 0);
    }
    if (alive) alive = issue_qk(0);
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int slot = j % C::kSlots;
      // The buffer of tile j + 1 held P of tile j - 1, whose P V was issued before (MMAs run in order).
      // With a single K slot the next key tile lands late, and waiting for it here would hold back
      // P V (j): then the score product follows P V instead.
      if (C::kSlots > 1 && j + 1 < n_tiles) {
        alive = issue_qk(j + 1);
        if (!alive) break;
      }
      alive = wait_clocked(smem_u32(&sync->v_full[slot]), static_cast<uint32_t>(j / C::kSlots) & 1u, abort_flag, wait_limit);
      if (!alive) {
        if (lane == 0) report(p.status, 2, j, 8 + slot);
        break;
      }
      const uint64_t vd0 = smem_desc_sw128(v_smem + slot * C::kTileV, kBoxBytes, 1024);   // V tile as MN-major B operand
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        alive = wait_clocked(smem_u32(&sync->p_ready[j & 1][half]), static_cast<uint32_t>(j >> 1) & 1u, abort_flag, wait_limit);
        if (!alive) {
          if (lane == 0) report(p.status, 3, j, half);
          break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ts(tmem_base + kColO, tmem_base + kColS + static_cast<uint32_t>((j & 1) * kN + half * 32 + kk * 8),
                   vd0 + static_cast<uint64_t>((half * 4 + kk) * (2048 >> 4)), idesc_pv, (j > 0 || half > 0 || kk > 0) ? 1u : 0u);
        }
      }
      if (!alive) break;
      if (elect_one()) {
        mma_commit(smem_u32(&sync->v_empty[slot]));
        mma_commit(smem_u32(&sync->pv_done));
        if (j + 1 == n_tiles) mma_commit(smem_u32(&sync->o_done));
      }
      if (C::kSlots == 1 && j + 1 < n_tiles) alive = issue_qk(j + 1);
    }
    if (*abort_flag != 0) {
      if (elect_one()) mma_commit(smem_u32(&sync->drain));
      const long long t0 = clock64();
      while (!mbar_try_wait(smem_u32(&sync->drain), 0) && clock64() - t0 < kDrainCycles) {
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax role
    const int r = tid;                       // row inside the tile = TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t s_base = tmem_base + lane_off + kColS;
    const uint32_t o_addr = tmem_base + lane_off + kColO;
    // checked build: both score buffers and the accumulator stay inside the allocation
    if (!dbg_tmem(p.status, DBG_PREFILL_WIDE * 100 + 1, s_base, tmem_base, 2 * kN, C::kTmemCols) ||
        !dbg_tmem(p.status, DBG_PREFILL_WIDE * 100 + 2, o_addr, tmem_base, DV, C::kTmemCols))
      *abort_flag = 1;
    const int row_g = row0 + r;
    int lim = kv_limit;                      // keys [0, lim) are visible to this row
    if (p.causal) {
      const long long c = static_cast<long long>(row_g) + p.causal_shift + 1;
      lim = c < lim ? static_cast<int>(c < 0 ? 0 : c) : lim;
    }
    // with an additive bias the logits s * scale + bias are formed as the scores are read (see prefill_sm100.cu)
    const float sl2_in = BIAS ? p.scale : p.scale * kLog2e;
    const float sl2 = BIAS ? kLog2e : sl2_in;
    float m_run = -CUDART_INF_F, l_run = 0.f;
    bool alive = true;
    const uint4* bias_row = nullptr;
    if constexpr (BIAS) {
      if (row_g < p.L)
        bias_row = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + b * p.bs[0] +
                                                  static_cast<long long>(h) * p.bs[1] +
                                                  static_cast<long long>(row_g) * p.bs[2]);
    }

    const bool bias_wide = BIAS && bias_rows_32b(p);

    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t s_addr = s_base + static_cast<uint32_t>((j & 1) * kN);
      uint4 bv[BIAS ? kN / 8 : 1];
      if constexpr (BIAS) {
        load_bias_row(bv, bias_row, j * kN, p.S, bias_wide);
      }
      bool ok = wait_clocked(smem_u32(&sync->s_full[j & 1]), static_cast<uint32_t>(j >> 1) & 1u, abort_flag, wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 4, j, warp);
        alive = false;
        break;
      }
      tc_fence_after_sync();
      const int col0 = j * kN;
      const bool need_mask = col0 + kN > min_lim;

      uint32_t sv[kN];
      tmem_ld_32x32(s_addr, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
      tmem_ld_32x32(s_addr + 32, reinterpret_cast<uint32_t(&)[32]>(sv[32]));
      tmem_ld_wait();
      tmem_ld_32x32(s_addr + 64, reinterpret_cast<uint32_t(&)[32]>(sv[64]));
      tmem_ld_32x32(s_addr + 96, reinterpret_cast<uint32_t(&)[32]>(sv[96]));
      float mxa = -CUDART_INF_F, mxb = -CUDART_INF_F;
      if constexpr (BIAS) {
#pragma unroll
        for (int i = 0; i < 8; ++i) add_bias8<BF16>(&sv[8 * i], bv[i], sl2_in);
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i) sv[i] = (col0 + i < lim) ? sv[i] : 0xff800000u;   // -inf
      }
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        mxa = max3(mxa, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
        mxb = max3(mxb, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
      }
      tmem_ld_wait();
      if constexpr (BIAS) {
#pragma unroll
        for (int i = 8; i < 16; ++i) add_bias8<BF16>(&sv[8 * i], bv[i], sl2_in);
      }
      if (need_mask) {
#pragma unroll
        for (int i = 64; i < kN; ++i) sv[i] = (col0 + i < lim) ? sv[i] : 0xff800000u;
      }
#pragma unroll
      for (int i = 64; i < kN; i += 4) {
        mxa = max3(mxa, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
        mxb = max3(mxb, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
      }
      const float mx = fmaxf(mxa, mxb);
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new - m_run) * sl2 > kRescaleThreshold;   // false for NaN (-inf - -inf)
      float alpha = 1.f;
      if (grow) {
        alpha = ex2((m_run - m_new) * sl2);   // m_run = -inf -> 0
        l_run *= alpha;
        m_run = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // raise the reference maximum: O *= alpha, once P V of the previous tile has retired
        ok = wait_clocked(smem_u32(&sync->pv_done), static_cast<uint32_t>(j - 1) & 1u, abort_flag, wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 5, j, warp);
          alive = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DV / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x16(o_addr + c * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x16(o_addr + c * 16, v);
        }
        tmem_st_wait();
      }
      const float nms = (m_run == -CUDART_INF_F) ? 0.f : -m_run * sl2;

      const uint64_t sl2_2 = f2_pack(sl2, sl2), nms_2 = f2_pack(nms, nms);
      uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
      for (int c = 0; c < kN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a0, a1;   // both exponents with one packed fma
          f2_unpack(f2_fma(f2_pack(__uint_as_float(sv[c * 32 + i]), __uint_as_float(sv[c * 32 + i + 1])), sl2_2, nms_2), a0, a1);
          const float p0 = ex2(a0);
          const float p1 = ex2(a1);
          sum2[(i >> 1) & 1] = f2_add(sum2[(i >> 1) & 1], f2_pack(p0, p1));
          pk[i >> 1] = pack2<BF16>(p0, p1);
        }
        tmem_st_32x16(s_addr + c * 16, pk);
        if (c == 1) {
          // first 64 keys of P are in TMEM: let P V start on them while the rest is computed
          tmem_st_wait();
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&sync->p_ready[j & 1][0]));
        }
      }
      float sum4[4];
      f2_unpack(sum2[0], sum4[0], sum4[1]);
      f2_unpack(sum2[1], sum4[2], sum4[3]);
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sync->p_ready[j & 1][1]));
    }

    // ------------------------------------------------------------- epilogue
    if (alive && n_tiles > 0) {
      bool ok = wait_clocked(smem_u32(&sync->o_done), 0, abort_flag, wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 6, 0, warp);
        alive = false;
      }
      tc_fence_after_sync();
    }
    if (alive) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint8_t* o_stage = smem_raw + (q_smem - raw_addr);   // the Q tile is no longer needed
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(o_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          pk[i >> 1] = pack2<BF16>(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
        uint8_t* box = o_stage + (c >> 1) * kBoxBytes + r * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int unit = ((c & 1) * 4 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(box + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sync->o_staged));
      if (r == 0 && wait_clocked(smem_u32(&sync->o_staged), 0, abort_flag, wait_limit)) {
        for (int bx = 0; bx < C::kBoxesV; ++bx) tma_store_4d(&tm_o, q_smem + bx * kBoxBytes, bx * 64, row0, h, b);
        tma_store_commit();
        tma_store_wait_read();
      }
      if (p.lse != nullptr && row_g < p.L) {
        const float lse = l_run > 0.f ? fmaf(m_run, BIAS ? 1.f : p.scale, lg2(l_run) * kLn2) : -CUDART_INF_F;
        if (dbg_bhrc(p.status, DBG_PREFILL_WIDE * 100 + 3, b, p.B, h, p.Hq, row_g, p.L, 0, 0, 1))
          p.lse[b * p.ls[0] + h * p.ls[1] + row_g * p.ls[2]] = lse;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int E, int DV, bool BF16, bool BIAS>
int launch_wide(const Problem& p, cudaStream_t stream) {
  using C = CfgW<E, DV>;
  CUtensorMap tq, tk, tv, to;
  if (!make_map(&tq, p.q, BF16, E, p.L, p.Hq, p.B, p.qs) || !make_map(&tk, p.k, BF16, E, p.S, p.Hkv, p.B, p.ks) ||
      !make_map(&tv, p.v, BF16, DV, p.S, p.Hkv, p.B, p.vs) || !make_map(&to, p.out, BF16, DV, p.L, p.Hq, p.B, p.os))
    return B200_SDPA_ERR_CUDA;
  auto kern = prefill_wide_kernel<E, DV, BF16, BIAS>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  const int n_qblk = (p.L + kM - 1) / kM;
  const long long grid = static_cast<long long>(n_qblk) * p.Hq * p.B;
  if (grid <= 0 || grid > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  const int per_wave = kv_streams_per_wave(static_cast<long long>(p.S) * (E + DV) * 2, static_cast<long long>(p.Hkv) * p.B);
  kern<<<static_cast<unsigned>(grid), kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, to, p, n_qblk,
                                                                         per_wave, wait_limit_cycles());
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_PREFILL);
  return B200_SDPA_OK;
}

}  // namespace

bool prefill_wide_eligible(const Problem& p, int dtype, bool* alignment_only_failure) {
  if (alignment_only_failure) *alignment_only_failure = false;
  if (dtype != B200_SDPA_F16 && dtype != B200_SDPA_BF16) return false;
  if (!((p.E == 192 && p.Dv == 128) || (p.E == 256 && p.Dv == 256))) return false;
  if (p.block_table != nullptr || p.k_new != nullptr) return false;
  if (p.bias != nullptr && !bias_readable(p, dtype, alignment_only_failure)) return false;
  if (!(p.scale > 0.f) || !(p.scale < 1e30f)) return false;
  if (p.L < 1 || p.S < 1) return false;
  const bool ok = strides_ok(p.q, p.qs, p.L, p.Hq, p.B) && strides_ok(p.k, p.ks, p.S, p.Hkv, p.B) &&
                  strides_ok(p.v, p.vs, p.S, p.Hkv, p.B) && strides_ok(p.out, p.os, p.L, p.Hq, p.B);
  if (!ok && alignment_only_failure) *alignment_only_failure = true;
  return ok;
}

int plan_prefill_wide(const Problem& p, int dtype, B200SdpaPlan* plan) {
  if (!prefill_wide_eligible(p, dtype, nullptr)) return B200_SDPA_ERR_UNSUPPORTED;
  const long long grid = static_cast<long long>((p.L + kM - 1) / kM) * p.Hq * p.B;
  if (grid > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  plan->path = B200_SDPA_PATH_PREFILL;
  plan->block_m = kM;
  plan->block_n = kN;
  plan->grid_x = static_cast<int32_t>(grid);
  plan->grid_y = plan->grid_z = 1;
  plan->threads = kThreads;
  plan->smem_bytes = p.E == 192 ? CfgW<192, 128>::kSmemBytes : CfgW<256, 256>::kSmemBytes;
  plan->kv_splits = 1;
  plan->launches = 1;
  plan->workspace_bytes = 0;
  return B200_SDPA_OK;
}

int launch_prefill_wide(const Problem& p, int dtype, cudaStream_t stream) {
  if (!prefill_wide_eligible(p, dtype, nullptr)) return B200_SDPA_ERR_UNSUPPORTED;
  const bool bf16 = dtype == B200_SDPA_BF16;
  if (p.bias != nullptr) {
    if (p.E == 192) return bf16 ? launch_wide<192, 128, true, true>(p, stream) : launch_wide<192, 128, false, true>(p, stream);
    return bf16 ? launch_wide<256, 256, true, true>(p, stream) : launch_wide<256, 256, false, true>(p, stream);
  }
  if (p.E == 192) return bf16 ? launch_wide<192, 128, true, false>(p, stream) : launch_wide<192, 128, false, false>(p, stream);
  return bf16 ? launch_wide<256, 256, true, false>(p, stream) : launch_wide<256, 256, false, false>(p, stream);
}

}  // namespace b200
