// FlashAttention-style prefill kernel for sm_100a: TMA -> shared memory ->
// tcgen05 tensor cores with accumulators in tensor memory (TMEM).  One work item per CTA; large
// problems at head dimension 128 run the persistent form of the same kernel
// (prefill_persistent_sm100.cu), which produces the same bits.
//
// One CTA owns 256 query rows of one (batch, query head): two 128-row tiles
// that take turns on the tensor cores while the other one is in its softmax.
// Roles (320 threads):
//   warps 0-3   softmax of tile 0: one thread per query row (= one TMEM lane)
//   warps 4-7   softmax of tile 1
//   warp  8     TMA producer: Q once, then K(j), V(j) tiles through a ring
//   warp  9     MMA issuer: S_t = Q_t K(j)^T and O_t += P_t V(j), one thread
// TMEM columns: [0,128) S0, [128,256) S1, [256,256+D) O0, [256+D,256+2D) O1;
// the probabilities P_t (16-bit, two per column) overwrite the first 64 columns
// of S_t and are fed to the second product straight from TMEM.  With D = 64 there
// are 128 columns to spare: P_t then has columns of its own and the next score
// product does not wait for P V (Cfg::kSplitP).
//
// Online softmax in the exp2 domain on raw scores: p = 2^(s*c - m*c) with
// c = scale*log2(e); the running maximum m is only raised when it grows by more
// than 2^8, so O is rarely rescaled.  All statistics and O stay fp32; P is
// rounded to the input dtype exactly once, as upstream rounds its
// probabilities (torch_neuronx/_sdpa_math.py:94).  Rows without a visible key
// give out = 0, lse = -inf (:85-91).  The causal rule is j <= i + shift with
// shift = q_offset - k_offset (0 reproduces the top-left aligned triangle of
// :20-28); kv_lens masks right padding; key tiles that no row of the CTA can
// see are never loaded.
//
// Every wait is bounded: on expiry the role raises a CTA-wide abort flag, every
// other role drains, tensor memory is freed and the status word reports
// B200_SDPA_ERR_TIMEOUT.
#include "tc_common.cuh"
#include "debug.cuh"

#include <type_traits>

namespace b200 {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kBlockM = 128;   // rows per query tile (= TMEM lanes)
constexpr int kBlockN = 128;   // keys per tile
constexpr int kTilesPerCta = 2;
constexpr int kRowsPerCta = kBlockM * kTilesPerCta;
constexpr int kThreads = 320;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;         // in units of log2

template <int D> struct Cfg {
  static constexpr int kBoxes = D / 64;                      // TMA boxes per tile
  static constexpr int kTileBytes = kBlockN * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 8;         // K/V ring slots
  static constexpr int kSmemTiles = (kTilesPerCta + kStages) * kTileBytes;
  static constexpr int kSmemBytes = kSmemTiles + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // With D = 64 the two O accumulators leave 128 tensor-memory columns free: P_t gets columns of its
  // own ([384,448) / [448,512)) instead of overwriting S_t, so Q_t K(j+1)^T no longer has to wait for
  // P_t(j) V(j) -- it is issued as soon as the softmax warps have copied S_t(j) into registers.
  static constexpr bool kSplitP = (D == 64);
};

struct Sync {
  uint64_t q_full;
  uint64_t kv_full[8];
  uint64_t kv_empty[8];
  uint64_t s_full[2];
  uint64_t p_ready[2][2];  // [tile][half of P]
  uint64_t s_free[2];      // (D = 64) the softmax warps hold S_t(j) in registers
  uint64_t pv_done[2];     // (D = 64) P_t(j) V(j) has retired
  uint64_t o_done[2];
  uint64_t o_staged[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

static_assert(sizeof(Sync) <= 272, "barrier block must fit its reserve (272 bytes + up to 1008 of alignment <= 1280)");

// Visible-key geometry of one 128-row tile.
struct TileGeom {
  int row0;       // first query row
  int n_tiles;    // key tiles to process (0: nothing visible, or tile beyond L)
  int min_lim;    // visible-key count of the tile's first row (may be <= 0)
  bool in_range;  // row0 < L
};

__device__ __forceinline__ TileGeom tile_geometry(const Problem& p, int row0, int kv_limit) {
  TileGeom g;
  g.row0 = row0;
  g.in_range = row0 < p.L;
  long long end = kv_limit, first = kv_limit;
  if (p.causal) {
    const int last_row = (row0 + kBlockM < p.L ? row0 + kBlockM : p.L) - 1;
    const long long e = static_cast<long long>(last_row) + p.causal_shift + 1;
    const long long f = static_cast<long long>(row0) + p.causal_shift + 1;
    end = e < end ? e : end;
    first = f < first ? f : first;
  }
  if (end < 0) end = 0;
  if (first < -1) first = -1;
  g.n_tiles = g.in_range ? static_cast<int>((end + kBlockN - 1) / kBlockN) : 0;
  g.min_lim = static_cast<int>(first);
  return g;
}

template <int D, bool BF16, bool BIAS, bool ACC>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const Problem p,
               const int n_qblk, const int pair_heads, const int streams_per_wave, const long long wait_limit) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles = (raw_addr + 1023u) & ~1023u;            // 1024-byte aligned tile area
  Sync* sync = reinterpret_cast<Sync*>(smem_raw + (tiles - raw_addr) + C::kSmemTiles);
  volatile int* abort_flag = &sync->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // Work item: longest (latest) query blocks first, heads of one kv group adjacent.
  // Two layouts of the CTA's two 128-row tiles:
  //   pair_heads == 0: rows [256 q, +128) and [256 q + 128, +128) of one query head;
  //   pair_heads == 1: the same 128 rows of two query heads that share a kv head
  //     (even group size) -- both tiles then see exactly the same keys, so under a
  //     causal mask neither waits for the other's extra diagonal tile.
  // The (batch, kv head) key/value streams are taken `streams_per_wave` at a time, so that what the
  // CTAs in flight read together fits in L2 (all streams at once when they do).
  const int heads_per_cta = pair_heads ? 2 : 1;
  const int ctas_per_stream = p.group / heads_per_cta;            // per query block
  const int n_streams = p.Hkv * p.B;
  const int full_wave_ctas = n_qblk * streams_per_wave * ctas_per_stream;
  const int wave = static_cast<int>(blockIdx.x / full_wave_ctas);
  const int in_wave = static_cast<int>(blockIdx.x - static_cast<unsigned>(wave) * full_wave_ctas);
  const int first_stream = wave * streams_per_wave;
  const int wave_streams = (n_streams - first_stream) < streams_per_wave ? (n_streams - first_stream) : streams_per_wave;
  const int per_blk = wave_streams * ctas_per_stream;
  const int qblk = n_qblk - 1 - in_wave / per_blk;
  const int rem = in_wave % per_blk;
  const int stream = first_stream + rem / ctas_per_stream;
  const int hk = stream % p.Hkv;
  const int b = stream / p.Hkv;
  const int hq0 = hk * p.group + (rem % ctas_per_stream) * heads_per_cta;
  const int head_of_tile[2] = {hq0, pair_heads ? hq0 + 1 : hq0};
  const int kv_limit = valid_keys(p, b);
  const int rows_per_cta = pair_heads ? kBlockM : kRowsPerCta;
  const TileGeom tg0 = tile_geometry(p, qblk * rows_per_cta, kv_limit);
  const TileGeom tg1 = tile_geometry(p, qblk * rows_per_cta + (pair_heads ? 0 : kBlockM), kv_limit);
  const int n_iter = tg0.n_tiles > tg1.n_tiles ? tg0.n_tiles : tg1.n_tiles;


  const uint32_t q_smem[2] = {tiles, tiles + C::kTileBytes};
  const uint32_t kv_smem = tiles + kTilesPerCta * C::kTileBytes;

  // Set-up is spread over the roles so that the first copies are in flight while
  // barriers are initialised and tensor memory is allocated: the producer lane owns
  // the barriers of its own copies and starts Q and the first ring slots at once.
  int items_issued = 0;   // (producer lane) ring items already issued
  bool q_armed = false;   // (producer lane) a copy into the Q slots is in flight or has landed
  if (warp == kProducerWarp && lane == 0) {
    mbar_init(smem_u32(&sync->q_full), 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sync->kv_full[s]), 1);
      mbar_init(smem_u32(&sync->kv_empty[s]), 1);
    }
    mbar_fence_init();
    // A tile without visible keys never reads its Q: its shared-memory slot is used
    // straight away to stage the all-zero output, so nothing may be in flight into it.
    uint32_t q_bytes = 0;
    if (tg0.n_tiles > 0) q_bytes += C::kTileBytes;
    if (tg1.n_tiles > 0) q_bytes += C::kTileBytes;
    const uint32_t qbar = smem_u32(&sync->q_full);
    if (q_bytes > 0) mbar_arrive_expect_tx(qbar, q_bytes);
    q_armed = q_bytes > 0;
    for (int t = 0; t < 2; ++t) {
      const TileGeom& tg = t == 0 ? tg0 : tg1;
      if (tg.n_tiles == 0) continue;
      for (int bx = 0; bx < C::kBoxes; ++bx)
        tma_load_4d(q_smem[t] + bx * kBoxBytes, &tm_q, qbar, bx * 64, tg.row0, head_of_tile[t], b);
    }
    for (; items_issued < 2 * n_iter && items_issued < C::kStages; ++items_issued) {
      const uint32_t bar = smem_u32(&sync->kv_full[items_issued]);
      mbar_arrive_expect_tx(bar, C::kTileBytes);
      const CUtensorMap* map = (items_issued & 1) ? &tm_v : &tm_k;
      for (int bx = 0; bx < C::kBoxes; ++bx)
        tma_load_4d(kv_smem + items_issued * C::kTileBytes + bx * kBoxBytes, map, bar, bx * 64,
                    (items_issued >> 1) * kBlockN, hk, b);
    }
    prefetch_tmap(&tm_o);
  }
  if (tid < 2) {
    const int t = tid;
    mbar_init(smem_u32(&sync->s_full[t]), 1);
    mbar_init(smem_u32(&sync->p_ready[t][0]), kBlockM);
    mbar_init(smem_u32(&sync->p_ready[t][1]), kBlockM);
    mbar_init(smem_u32(&sync->o_done[t]), 1);
    mbar_init(smem_u32(&sync->o_staged[t]), kBlockM);
    mbar_init(smem_u32(&sync->s_free[t]), kBlockM);
    mbar_init(smem_u32(&sync->pv_done[t]), 1);
    if (t == 0) {
      mbar_init(smem_u32(&sync->drain), 1);
      sync->abort_flag = 0;
    }
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

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool alive = true;
      for (int item = items_issued; item < 2 * n_iter && alive; ++item) {
        const int j = item >> 1;
        const int stage = item % C::kStages;
        const uint32_t round = static_cast<uint32_t>(item / C::kStages);
        if (round > 0) {
          alive = wait_clocked(smem_u32(&sync->kv_empty[stage]), (round - 1) & 1u, abort_flag, wait_limit);
          if (!alive) {
            report(p.status, 1, item, stage);
            break;
          }
        }
        const uint32_t bar = smem_u32(&sync->kv_full[stage]);
        const uint32_t dst = kv_smem + stage * C::kTileBytes;
        mbar_arrive_expect_tx(bar, C::kTileBytes);
        const CUtensorMap* map = (item & 1) ? &tm_v : &tm_k;
        for (int bx = 0; bx < C::kBoxes; ++bx) tma_load_4d(dst + bx * kBoxBytes, map, bar, bx * 64, j * kBlockN, hk, b);
        items_issued = item + 1;
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    // The whole warp runs the control flow (waits included) so that addresses and
    // descriptors stay in the uniform datapath; one elected lane issues.  The tile
    // index is a compile-time constant everywhere for the same reason.
    {
      constexpr uint32_t idesc_qk = make_idesc(BF16, false, kBlockM, kBlockN);
      constexpr uint32_t idesc_pv = make_idesc(BF16, true, kBlockM, D);
      bool alive = n_iter > 0;

      // descriptors: fixed fields once, then only the 16-byte-unit start address moves
      const uint64_t q_desc0 = smem_desc_sw128(q_smem[0], 16, 1024), q_desc1 = smem_desc_sw128(q_smem[1], 16, 1024);
      const uint64_t kv_desc_k = smem_desc_sw128(kv_smem, 16, 1024);          // K tile as K-major B operand
      const uint64_t kv_desc_v = smem_desc_sw128(kv_smem, kBoxBytes, 1024);   // V tile as MN-major B operand
      auto issue_qk = [&](auto tile_const, uint32_t stage) {
        constexpr int t = decltype(tile_const)::value;
        const uint64_t qd = t == 0 ? q_desc0 : q_desc1;
        const uint64_t kd = kv_desc_k + static_cast<uint64_t>(stage * (C::kTileBytes >> 4));
        const uint32_t d_addr = tmem_base + static_cast<uint32_t>(t * 128);
        if (elect_one() && dbg_tmem(p.status, DBG_PREFILL * 100 + 1, d_addr, tmem_base, 128, 512)) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * kBoxBytes + (kk & 3) * 32) >> 4);
            mma_ss(d_addr, qd + off, kd + off, idesc_qk, kk > 0 ? 1u : 0u);
          }
        }
      };
      // O_t (+)= P_t[:, half*64 .. half*64+63] . V[half*64 .. , :]   (four K-steps of 16 keys)
      auto issue_pv_half = [&](auto tile_const, uint32_t stage, int half, bool accumulate) {
        constexpr int t = decltype(tile_const)::value;
        const uint64_t vd = kv_desc_v + static_cast<uint64_t>(stage * (C::kTileBytes >> 4) + half * 4 * (2048 >> 4));
        const uint32_t d_addr = tmem_base + static_cast<uint32_t>(256 + t * D);
        const uint32_t a_addr = tmem_base + static_cast<uint32_t>(C::kSplitP ? 384 + t * 64 + half * 32 : t * 128 + half * 32);
        const uint32_t acc0 = (accumulate || half > 0) ? 1u : 0u;
        if (elect_one() && dbg_tmem(p.status, DBG_PREFILL * 100 + 2, d_addr, tmem_base, D, 512) &&
            dbg_tmem(p.status, DBG_PREFILL * 100 + 3, a_addr, tmem_base, 32, 512)) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            mma_ts(d_addr, a_addr + static_cast<uint32_t>(kk * 8), vd + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv,
                   kk > 0 ? 1u : acc0);
          }
        }
      };
      auto commit = [&](uint32_t bar) {
        if (elect_one()) mma_commit(bar);
      };
      auto wait_full = [&](int item) -> bool {
        const int stage = item % C::kStages;
        const uint32_t round = static_cast<uint32_t>(item / C::kStages);
        const bool ok = wait_clocked(smem_u32(&sync->kv_full[stage]), round & 1u, abort_flag, wait_limit);
        if (!ok && lane == 0) report(p.status, 2, item, stage);
        return ok;
      };
      auto stage_addr = [&](int item) { return static_cast<uint32_t>(item % C::kStages); };
      auto empty_bar = [&](int item) { return smem_u32(&sync->kv_empty[item % C::kStages]); };
      const std::integral_constant<int, 0> T0{};
      const std::integral_constant<int, 1> T1{};

      if (alive) {
        alive = wait_clocked(smem_u32(&sync->q_full), 0, abort_flag, wait_limit);
        if (!alive && lane == 0) report(p.status, 2, -1, 0);
      }
      if (alive) alive = wait_full(0);
      if (alive) {
        tc_fence_after_sync();
        if (tg0.n_tiles > 0) {
          issue_qk(T0, stage_addr(0));
          commit(smem_u32(&sync->s_full[0]));
        }
        if (tg1.n_tiles > 0) {
          issue_qk(T1, stage_addr(0));
          commit(smem_u32(&sync->s_full[1]));
        }
        commit(empty_bar(0));
      }
      for (int j = 0; j < n_iter && alive; ++j) {
        const int item_v = 2 * j + 1, item_kn = 2 * j + 2;
        const bool has_next = j + 1 < n_iter;
        alive = wait_full(item_v);
        if (!alive) break;
        // one tile: P_t(j) V(j) in two halves as the halves of P arrive, then Q_t K(j+1)^T
        auto serve = [&](auto tile_const) {
          constexpr int t = decltype(tile_const)::value;
          const int nt = t == 0 ? tg0.n_tiles : tg1.n_tiles;
          if (C::kSplitP) {
            // next scores first: S_t(j) only has to be out of tensor memory, not consumed
            if (t == 0 && has_next) {
              alive = wait_full(item_kn);
              if (!alive) return;
            }
            if (j + 1 < nt) {
              alive = wait_clocked(smem_u32(&sync->s_free[t]), j & 1, abort_flag, wait_limit);
              if (!alive) {
                if (lane == 0) report(p.status, 9, j, t);
                return;
              }
              tc_fence_after_sync();
              issue_qk(tile_const, stage_addr(item_kn));
              commit(smem_u32(&sync->s_full[t]));
            }
          }
          if (j < nt) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              alive = wait_clocked(smem_u32(&sync->p_ready[t][half]), j & 1, abort_flag, wait_limit);
              if (!alive) {
                if (lane == 0) report(p.status, 3, j, t);
                return;
              }
              tc_fence_after_sync();
              issue_pv_half(tile_const, stage_addr(item_v), half, j > 0);
            }
          }
          if (C::kSplitP) {
            if (j < nt) {
              commit(smem_u32(&sync->pv_done[t]));
              if (j + 1 >= nt) commit(smem_u32(&sync->o_done[t]));
            }
          } else {
            if (t == 0 && has_next) {
              alive = wait_full(item_kn);
              if (!alive) return;
              tc_fence_after_sync();
            }
            if (j + 1 < nt) {
              issue_qk(tile_const, stage_addr(item_kn));
              commit(smem_u32(&sync->s_full[t]));
            } else if (j < nt) {
              commit(smem_u32(&sync->o_done[t]));
            }
          }
        };
        serve(T0);
        if (!alive) break;
        serve(T1);
        if (!alive) break;
        commit(empty_bar(item_v));
        if (has_next) commit(empty_bar(item_kn));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax roles
    const int t = warp >> 2;                 // which 128-row tile
    const int quad = warp & 3;               // TMEM lane quadrant this warp may touch
    const int r = tid & 127;                 // row inside the tile
    const TileGeom& tg = t == 0 ? tg0 : tg1;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + static_cast<uint32_t>(t) * 128u;
    const uint32_t o_addr = tmem_base + lane_off + 256u + static_cast<uint32_t>(t) * D;
    const uint32_t p_addr = C::kSplitP ? tmem_base + lane_off + 384u + static_cast<uint32_t>(t) * 64u : s_addr;
    // checked build: the three column ranges this thread reads and writes; a violation drains the CTA
    if (!dbg_tmem(p.status, DBG_PREFILL * 100 + 4, s_addr, tmem_base, 128, 512) ||
        !dbg_tmem(p.status, DBG_PREFILL * 100 + 5, o_addr, tmem_base, D, 512) ||
        !dbg_tmem(p.status, DBG_PREFILL * 100 + 6, p_addr, tmem_base, 64, 512))
      *abort_flag = 1;
    const int row_g = tg.row0 + r;
    int lim = kv_limit;                      // keys [0, lim) are visible to this row
    if (p.causal) {
      const long long c = static_cast<long long>(row_g) + p.causal_shift + 1;
      lim = c < lim ? static_cast<int>(c < 0 ? 0 : c) : lim;
    }
    // With an additive bias the logits s * scale + bias are formed when the scores are read;
    // everything after that then works on them with scale 1 (log2 e in the exponent).
    const float sl2_in = BIAS ? p.scale : p.scale * kLog2e;
    const float sl2 = BIAS ? kLog2e : sl2_in;
    float m_run = -CUDART_INF_F, l_run = 0.f;
    bool alive = true;
    // accumulating form: the row's running lse is fetched now and used in the epilogue
    float old_lse = -CUDART_INF_F;
    if constexpr (ACC) {
      if (row_g < p.L && p.acc_mode == 2)
        old_lse = p.acc_lse[b * p.als[0] + head_of_tile[t] * p.als[1] + row_g * p.als[2]];
    }
    // this row of the bias, 16-bit elements in the query's dtype, unit stride along the keys
    const uint4* bias_row = nullptr;
    if constexpr (BIAS) {
      if (row_g < p.L)
        bias_row = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + b * p.bs[0] +
                                                  static_cast<long long>(head_of_tile[t]) * p.bs[1] +
                                                  static_cast<long long>(row_g) * p.bs[2]);
    }

    const bool bias_wide = BIAS && bias_rows_32b(p);

    if (tg.in_range) {
      for (int j = 0; j < tg.n_tiles; ++j) {
        uint4 bv[BIAS ? kBlockN / 8 : 1];
        if constexpr (BIAS) {
          // the bias of this key tile travels while the scores are awaited
          load_bias_row(bv, bias_row, j * kBlockN, p.S, bias_wide);
        }
        bool ok = wait_clocked(smem_u32(&sync->s_full[t]), j & 1, abort_flag, wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 4 + t, j, quad);
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const int col0 = j * kBlockN;
        const bool need_mask = col0 + kBlockN > tg.min_lim;

        // S row -> registers in two halves; the second half is in flight while the
        // maximum of the first is taken
        uint32_t sv[kBlockN];
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
          for (int i = 0; i < 64; ++i) sv[i] = (col0 + i < lim) ? sv[i] : 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          mxa = max3(mxa, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
          mxb = max3(mxb, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
        }
        tmem_ld_wait();
        if (C::kSplitP) {
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&sync->s_free[t]));
        }
        if constexpr (BIAS) {
#pragma unroll
          for (int i = 8; i < 16; ++i) add_bias8<BF16>(&sv[8 * i], bv[i], sl2_in);
        }
        if (need_mask) {
#pragma unroll
          for (int i = 64; i < kBlockN; ++i) sv[i] = (col0 + i < lim) ? sv[i] : 0xff800000u;
        }
#pragma unroll
        for (int i = 64; i < kBlockN; i += 4) {
          mxa = max3(mxa, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
          mxb = max3(mxb, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
        }
        const float mx = fmaxf(mxa, mxb);
        const float m_new = fmaxf(m_run, mx);
        const bool grow = (m_new - m_run) * sl2 > kRescaleThreshold;  // false for NaN (-inf - -inf)
        float alpha = 1.f;
        if (grow) {
          alpha = ex2((m_run - m_new) * sl2);   // m_run = -inf -> 0
          l_run *= alpha;
          m_run = m_new;
        }
        if (C::kSplitP && j > 0) {
          // here S(j) can be ready before P V of the previous tile has retired, and that product
          // still reads the P columns and writes O_t: wait for it before touching either
          bool pv_ok = wait_clocked(smem_u32(&sync->pv_done[t]), (j - 1) & 1, abort_flag, wait_limit);
          pv_ok = __all_sync(0xffffffffu, pv_ok);
          if (!pv_ok) {
            if (lane == 0) report(p.status, 10, j, t);
            alive = false;
            break;
          }
          tc_fence_after_sync();
        }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // raise the reference maximum: O_t *= alpha (PV(j-1) has retired: without the split its
          // completion is ordered before s_full(j))
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
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

        // probabilities, row sum (two packed accumulators), P -> TMEM over the first 64
        // columns of S.  (Measured alternatives that lost: a polynomial exp2 on the FMA
        // pipe for part of the row, and ex2 on packed 16-bit pairs.)
        uint64_t sum2[2] = {0ull, 0ull};           // two packed accumulators = four chains
#pragma unroll
        for (int c = 0; c < kBlockN / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(sv[c * 32 + i]), sl2, nms));
            const float p1 = ex2(fmaf(__uint_as_float(sv[c * 32 + i + 1]), sl2, nms));
            sum2[(i >> 1) & 1] = f2_add(sum2[(i >> 1) & 1], f2_pack(p0, p1));
            pk[i >> 1] = pack2<BF16>(p0, p1);
          }
          tmem_st_32x16(p_addr + c * 16, pk);
          if (c == 1) {
            // first 64 keys of P are in TMEM: let P V start on them while the rest is computed
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&sync->p_ready[t][0]));
          }
        }
        float sum4[4];
        f2_unpack(sum2[0], sum4[0], sum4[1]);
        f2_unpack(sum2[1], sum4[2], sum4[3]);
        const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        l_run += sum;
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&sync->p_ready[t][1]));
      }

      // ------------------------------------------------------------- epilogue
      if (alive && tg.n_tiles > 0) {
        bool ok = wait_clocked(smem_u32(&sync->o_done[t]), 0, abort_flag, wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 6 + t, 0, quad);
          alive = false;
        }
        tc_fence_after_sync();
      }
      if constexpr (ACC) {
        // Accumulating form (a ring step): fold this block's result into the row's running fp32 pair
        // (acc, acc_lse) in place -- acc = acc * w_acc + O * w_o -- instead of writing out / lse.  Same
        // arithmetic as the persistent kernel's accumulating epilogue.  A tile without a visible key
        // leaves a started accumulator alone.
        if (alive && !(tg.n_tiles == 0 && p.acc_mode == 2)) {
          const bool row_ok = row_g < p.L &&
                              dbg_bhrc(p.status, DBG_PREFILL * 100 + 8, b, p.B, head_of_tile[t], p.Hq, row_g, p.L, 0, D, p.Dv);
          const float lse = l_run > 0.f ? fmaf(m_run, p.scale, lg2(l_run) * kLn2) : -CUDART_INF_F;
          float w_acc = 0.f, w_o = l_run > 0.f ? 1.f / l_run : 0.f;
          const float hi = fmaxf(old_lse, lse);
          float merged = -CUDART_INF_F;
          if (hi != -CUDART_INF_F) {
            const float e_old = ex2((old_lse - hi) * kLog2e), e_new = ex2((lse - hi) * kLog2e);   // -inf -> 0
            merged = hi + lg2(e_old + e_new) * kLn2;
            w_acc = ex2((old_lse - merged) * kLog2e);
            w_o *= ex2((lse - merged) * kLog2e);
          } else {
            w_o = 0.f;
          }
          float* arow = p.acc + b * p.as[0] + static_cast<long long>(head_of_tile[t]) * p.as[1] +
                        static_cast<long long>(row_g) * p.as[2];
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            if (tg.n_tiles > 0) {   // (uniform over the warp: tensor-memory loads stay outside per-lane conditions)
              tmem_ld_32x32(o_addr + c * 32, v);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
            if (row_ok) {
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                float4* dst = reinterpret_cast<float4*>(arow + c * 32 + u * 4);
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                if (p.acc_mode == 2) a = *dst;
                a.x = fmaf(a.x, w_acc, __uint_as_float(v[4 * u]) * w_o);
                a.y = fmaf(a.y, w_acc, __uint_as_float(v[4 * u + 1]) * w_o);
                a.z = fmaf(a.z, w_acc, __uint_as_float(v[4 * u + 2]) * w_o);
                a.w = fmaf(a.w, w_acc, __uint_as_float(v[4 * u + 3]) * w_o);
                *dst = a;
              }
            }
          }
          if (row_ok) p.acc_lse[b * p.als[0] + head_of_tile[t] * p.als[1] + row_g * p.als[2]] = merged;
        }
      } else if (alive) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint8_t* o_stage = smem_raw + (q_smem[t] - raw_addr);   // the Q tile is no longer needed
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          if (tg.n_tiles > 0) {
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
          // 32 columns = 64 bytes = four 16-byte units of the 128-byte swizzled row
          uint8_t* box = o_stage + (c >> 1) * kBoxBytes + r * 128;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int unit = ((c & 1) * 4 + u) ^ (r & 7);
            *reinterpret_cast<uint4*>(box + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
          }
        }
        // Every writer publishes its rows to the async proxy and arrives; only the
        // storing thread waits (bounded), so a role that gave up cannot strand the
        // others at a barrier.
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&sync->o_staged[t]));
        if (r == 0 && wait_clocked(smem_u32(&sync->o_staged[t]), 0, abort_flag, wait_limit)) {
          for (int bx = 0; bx < C::kBoxes; ++bx) tma_store_4d(&tm_o, q_smem[t] + bx * kBoxBytes, bx * 64, tg.row0, head_of_tile[t], b);
          tma_store_commit();
          tma_store_wait_read();
        }
        if (p.lse != nullptr && row_g < p.L) {
          // one rounding at the magnitude of the maximum: m*scale + ln(l)
          const float lse = l_run > 0.f ? fmaf(m_run, BIAS ? 1.f : p.scale, lg2(l_run) * kLn2) : -CUDART_INF_F;
          if (dbg_bhrc(p.status, DBG_PREFILL * 100 + 7, b, p.B, head_of_tile[t], p.Hq, row_g, p.L, 0, 0, 1))
            p.lse[b * p.ls[0] + head_of_tile[t] * p.ls[1] + row_g * p.ls[2]] = lse;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (sync->abort_flag != 0) {
    // A role gave up.  Before shared and tensor memory are handed back, whatever this CTA already
    // issued must have finished: the copies into the Q slots and the ring (their barriers complete
    // when the bytes have landed) and every MMA (one more commit, which arrives when all earlier ones
    // have retired).  These waits have their own generous bound, whatever the wait limit.
    if (warp == kProducerWarp && lane == 0) {
      if (q_armed) wait_drain(smem_u32(&sync->q_full), 0);
      for (int s = 0; s < C::kStages && s < items_issued; ++s) {
        const uint32_t last_round = static_cast<uint32_t>((items_issued - 1 - s) / C::kStages);
        wait_drain(smem_u32(&sync->kv_full[s]), last_round & 1u);
      }
    }
    if (warp == kMmaWarp) {
      if (elect_one()) mma_commit(smem_u32(&sync->drain));
      wait_drain(smem_u32(&sync->drain), 0);
    }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side --

// Pair two query heads of one kv head per CTA when the group size allows it and the
// mask is causal (that is where the row-block layout leaves one tile idle at the end).
int pair_heads_mode(const Problem& p) { return (p.causal && p.group % 2 == 0) ? 1 : 0; }

template <int D, bool BF16, bool BIAS, bool ACC = false>
int launch_variant(const Problem& p, cudaStream_t stream) {
  using C = Cfg<D>;
  CUtensorMap tq, tk, tv, to;
  if (!make_map(&tq, p.q, BF16, D, p.L, p.Hq, p.B, p.qs) || !make_map(&tk, p.k, BF16, D, p.S, p.Hkv, p.B, p.ks) ||
      !make_map(&tv, p.v, BF16, D, p.S, p.Hkv, p.B, p.vs))
    return B200_SDPA_ERR_CUDA;
  if (ACC) {
    to = tq;   // the accumulating form stores through plain pointers; the map is never used
  } else if (!make_map(&to, p.out, BF16, D, p.L, p.Hq, p.B, p.os)) {
    return B200_SDPA_ERR_CUDA;
  }
  auto kern = prefill_kernel<D, BF16, BIAS, ACC>;
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute: set on every
  // launch (a cheap host-side call), so a process that drives several GPUs gets it on each of them
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  const int pair_heads = pair_heads_mode(p);
  const int rows = pair_heads ? kBlockM : kRowsPerCta;
  const int n_qblk = (p.L + rows - 1) / rows;
  const long long grid = static_cast<long long>(n_qblk) * (p.Hq / (pair_heads ? 2 : 1)) * p.B;
  if (grid <= 0 || grid > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  const int per_wave = kv_streams_per_wave(static_cast<long long>(p.S) * 2 * D * 2, static_cast<long long>(p.Hkv) * p.B);
  kern<<<static_cast<unsigned>(grid), kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, to, p, n_qblk, pair_heads,
                                                                         per_wave, wait_limit_cycles());
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_PREFILL);
  return B200_SDPA_OK;
}

}  // namespace

bool prefill_eligible(const Problem& p, int dtype, bool* alignment_only_failure) {
  if (p.E > 128) return prefill_wide_eligible(p, dtype, alignment_only_failure);
  if (alignment_only_failure) *alignment_only_failure = false;
  if (dtype != B200_SDPA_F16 && dtype != B200_SDPA_BF16) return false;
  if (p.E != p.Dv || (p.E != 64 && p.E != 128)) return false;
  if (!(p.scale > 0.f) || !(p.scale < 1e30f)) return false;
  if (p.L < 1 || p.S < 1) return false;
  if (p.bias != nullptr) {
    if (!bias_readable(p, dtype, alignment_only_failure)) return false;
  }
  const bool ok = strides_ok(p.q, p.qs, p.L, p.Hq, p.B) && strides_ok(p.k, p.ks, p.S, p.Hkv, p.B) &&
                  strides_ok(p.v, p.vs, p.S, p.Hkv, p.B) && strides_ok(p.out, p.os, p.L, p.Hq, p.B);
  if (!ok && alignment_only_failure) *alignment_only_failure = true;
  return ok;
}

int plan_prefill(const Problem& p, int dtype, B200SdpaPlan* plan) {
  if (p.E > 128) return plan_prefill_wide(p, dtype, plan);
  if (!prefill_eligible(p, dtype, nullptr)) return B200_SDPA_ERR_UNSUPPORTED;
  if (prefill_persistent_wanted(p)) {
    plan_prefill_persistent(p, plan);
    return B200_SDPA_OK;
  }
  const int pair_heads = pair_heads_mode(p);
  const int rows = pair_heads ? kBlockM : kRowsPerCta;
  const int n_qblk = (p.L + rows - 1) / rows;
  const long long grid = static_cast<long long>(n_qblk) * (p.Hq / (pair_heads ? 2 : 1)) * p.B;
  if (grid > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  plan->path = B200_SDPA_PATH_PREFILL;
  plan->block_m = rows;
  plan->block_n = kBlockN;
  plan->grid_x = static_cast<int32_t>(grid);
  plan->grid_y = plan->grid_z = 1;
  plan->threads = kThreads;
  plan->smem_bytes = p.E == 128 ? Cfg<128>::kSmemBytes : Cfg<64>::kSmemBytes;
  plan->kv_splits = 1;
  plan->launches = 1;
  plan->workspace_bytes = 0;
  return B200_SDPA_OK;
}

int launch_prefill(const Problem& p, int dtype, void* workspace, uint64_t workspace_bytes, cudaStream_t stream) {
  if (p.E > 128) return launch_prefill_wide(p, dtype, stream);
  if (!prefill_eligible(p, dtype, nullptr)) return B200_SDPA_ERR_UNSUPPORTED;
  if (prefill_persistent_wanted(p)) return launch_prefill_persistent(p, dtype, workspace, workspace_bytes, stream);
  const bool bf16 = dtype == B200_SDPA_BF16;
  if (p.acc_mode != 0) {
    if (!prefill_accumulate_eligible(p)) return B200_SDPA_ERR_UNSUPPORTED;
    return bf16 ? launch_variant<128, true, false, true>(p, stream) : launch_variant<128, false, false, true>(p, stream);
  }
  if (p.bias != nullptr) {
    if (p.E == 128) return bf16 ? launch_variant<128, true, true>(p, stream) : launch_variant<128, false, true>(p, stream);
    return bf16 ? launch_variant<64, true, true>(p, stream) : launch_variant<64, false, true>(p, stream);
  }
  if (p.E == 128) return bf16 ? launch_variant<128, true, false>(p, stream) : launch_variant<128, false, false>(p, stream);
  return bf16 ? launch_variant<64, true, false>(p, stream) : launch_variant<64, false, false>(p, stream);
}

}  // namespace b200
