// Persistent form of the prefill kernel (prefill_sm100.cu) for large problems with head dimension 128:
// TMA -> shared memory -> tcgen05 tensor cores with accumulators in tensor memory (TMEM).
//
// One CTA per SM walks a list of work items (longest first, handed out one at a time through an
// atomic counter, or in a fixed interleaved order when the caller gave no scratch for the counter).
// An item is two 128-row query tiles that take turns on the tensor cores while the other one is in
// its softmax: 256 consecutive rows of one (batch, query head), or -- causal mask, even group --
// the same 128 rows of two query heads that share a kv head.
// Roles (512 threads = four warpgroups, registers redistributed with setmaxnreg):
//   warps 0-3    softmax of tile 0: one thread per query row (= one TMEM lane)
//   warps 4-7    softmax of tile 1
//   warps 8-11   epilogue: drains O of a finished item from TMEM, normalises, stores out and lse
//                while the other roles are already on the next item
//   warp  12     TMA producer + scheduler: Q of the next item as soon as the last Q K^T of this
//                one has been issued, then K(j), V(j) tiles through a ring that never drains
//                between items
//   warp  13     MMA issuer: S_t = Q_t K(j)^T and O_t += P_t V(j), one elected thread
//   warps 14-15  idle (they only complete the warpgroup)
// TMEM columns: [0,128) S0, [128,256) S1, [256,256+D) O0, [256+D,256+2D) O1;
// the probabilities P_t (16-bit, two per column) overwrite the first 64 columns
// of S_t and are fed to the second product straight from TMEM.  With D = 64 there
// are 128 columns to spare: P_t then has columns of its own and the next score
// product does not wait for P V (Cfg::kSplitP).  Tensor memory is allocated once per CTA.
//
// Between items nothing is torn down: the tensor pipe goes from the last P V of one item to the
// first Q K^T of the next (its Q and first key tile are already in shared memory), and the first
// P V of the next item only waits until the epilogue warps hold the previous O in registers.
//
// Online softmax in the exp2 domain on raw scores: p = 2^(s*c - m*c) with
// c = scale*log2(e); the running maximum m is only raised when it grows by more
// than 2^8, so O is rarely rescaled.  All statistics and O stay fp32; P is
// rounded to the input dtype exactly once, as upstream rounds its
// probabilities (torch_neuronx/_sdpa_math.py:94).  Rows without a visible key
// give out = 0, lse = -inf (:85-91).  The causal rule is j <= i + shift with
// shift = q_offset - k_offset (0 reproduces the top-left aligned triangle of
// :20-28); kv_lens masks right padding; key tiles that no row of the item can
// see are never loaded.
//
// Every wait is bounded: on expiry the role raises a CTA-wide abort flag, every
// other role drains, the CTA waits for the copies and MMAs it issued, tensor memory is freed and
// the status word reports B200_SDPA_ERR_TIMEOUT.
#include "tc_common.cuh"
#include "debug.cuh"

#include <cstdlib>
#include <type_traits>

namespace b200 {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kBlockM = 128;   // rows per query tile (= TMEM lanes)
constexpr int kBlockN = 128;   // keys per tile
constexpr int kTilesPerCta = 2;
constexpr int kRowsPerCta = kBlockM * kTilesPerCta;
constexpr int kThreads = 512;
constexpr int kEpilogueWarp0 = 8;
constexpr int kProducerWarp = 12;
constexpr int kMmaWarp = 13;
constexpr int kItemSlots = 4;
constexpr int kConsumerThreads = 256 + 128 + 32;   // softmax + epilogue + MMA warp read every item
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;         // in units of log2
// Registers per thread after the set-up: softmax warpgroups, epilogue warpgroup, producer/MMA warpgroup;
// each split adds up to the 64 K registers of the SM (2 x 128 softmax threads + 128 + 128).  The softmax
// loop and the MMA issue loop are the two places where a spilled register costs time on the critical
// path, so they get what they need and the epilogue (which only has to keep up) what is left.  Measured
// on the bench shapes against 192/80/48, 168/104/72, 160/104/88, 152/120/88, 176/40/120, 184/40/104.
// The bias variants keep sixteen more 16-byte bias pieces per softmax thread.
template <bool BIAS> struct Regs {
  static constexpr int kSoftmax = BIAS ? 192 : 176, kEpilogue = BIAS ? 40 : 56, kControl = BIAS ? 88 : 104;
  static_assert(2 * 128 * kSoftmax + 128 * kEpilogue + 128 * kControl <= 65536, "register file");
};

template <int D> struct Cfg {
  static constexpr int kBoxes = D / 64;                      // TMA boxes per tile
  static constexpr int kTileBytes = kBlockN * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 8;         // K/V ring slots
  static constexpr int kSmemTiles = (kTilesPerCta + kStages) * kTileBytes;
  static constexpr int kStatBytes = kTilesPerCta * kBlockM * 2 * 4;   // two output weights for every row of both tiles
  // Kept under 195 KB on purpose: with the 1 KB the system reserves per CTA the request must fit the
  // 196 KB shared-memory configuration of the SM, or the L1 cache (which holds the spilled registers of
  // the softmax loop) shrinks from 60 KB to 28 KB and every spill turns into an L2 round trip.  That is
  // why there is no slack for rounding the tile area up to 1024 bytes: the dynamic shared memory is
  // declared with that alignment and the kernel checks it.
  static constexpr int kSmemBytes = kSmemTiles + kStatBytes + 640 /*barriers, items*/;
  static_assert(kSmemBytes + 1024 <= 196 * 1024, "must fit the 196 KB shared-memory configuration");
  // With D = 64 the two O accumulators leave 128 tensor-memory columns free: P_t gets columns of its
  // own ([384,448) / [448,512)) instead of overwriting S_t, so Q_t K(j+1)^T no longer has to wait for
  // P_t(j) V(j) -- it is issued as soon as the softmax warps have copied S_t(j) into registers.
  static constexpr bool kSplitP = (D == 64);
};

// One work item as the scheduler publishes it in shared memory (decoded once, read by every role).
struct ItemRec {
  int idx;                 // position in the item list, or -1: no more work
  int b, hk;
  int head0, head1;        // query head of each tile
  int row0_0, row0_1;      // first query row of each tile
  int nt0, nt1;            // key tiles of each tile (0: nothing visible, or tile beyond L)
  int lim0, lim1;          // visible-key count of each tile's first row (may be <= 0)
  int in_range;            // bit t: tile t starts inside L
  int kv_limit;
};

struct Sync {
  uint64_t item_full[kItemSlots];   // the scheduler published an item index
  uint64_t item_empty[kItemSlots];  // every consumer thread has read it
  uint64_t q_full[2];      // Q_t of an item has landed
  uint64_t q_free[2];      // the last Q_t K^T of an item has retired: the slot may take the next item's Q
  uint64_t kv_full[8];
  uint64_t kv_empty[8];
  uint64_t s_full[2];
  uint64_t p_ready[2][2];  // [tile][half of P]
  uint64_t s_free[2];      // (D = 64) the softmax warps hold S_t(j) in registers
  uint64_t pv_done[2];     // (D = 64) P_t(j) V(j) has retired
  uint64_t o_done[2];      // the last P_t V of an item has retired
  uint64_t stats_ready[2]; // the softmax warps have left the item's row statistics in shared memory
  uint64_t o_free[2];      // the epilogue warps hold O_t (and the statistics) in registers
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  ItemRec item[kItemSlots];
};

static_assert(sizeof(Sync) <= 640, "barrier block must fit its reserve");

template <int N> __device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

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

// Item order: the (batch, kv head) key/value streams are taken `streams_per_wave` at a time, so that
// what the CTAs in flight read together fits in L2 (all streams at once when they do); inside a wave
// longest (latest) query blocks first, heads of one kv group adjacent.  Two layouts of the two tiles:
//   pair_heads == 0: rows [256 q, +128) and [256 q + 128, +128) of one query head;
//   pair_heads == 1: the same 128 rows of two query heads that share a kv head
//     (even group size) -- both tiles then see exactly the same keys, so under a
//     causal mask neither waits for the other's extra diagonal tile.
__device__ __forceinline__ ItemRec decode_item(const Problem& p, int idx, int n_qblk, int pair_heads, int streams_per_wave) {
  ItemRec it;
  it.idx = idx;
  const int heads_per_cta = pair_heads ? 2 : 1;
  const int ctas_per_stream = p.group / heads_per_cta;            // per query block
  const int n_streams = p.Hkv * p.B;
  const int full_wave = n_qblk * streams_per_wave * ctas_per_stream;
  const int wave = idx / full_wave;
  const int in_wave = idx - wave * full_wave;
  const int first_stream = wave * streams_per_wave;
  const int wave_streams = (n_streams - first_stream) < streams_per_wave ? (n_streams - first_stream) : streams_per_wave;
  const int per_blk = wave_streams * ctas_per_stream;
  const int qblk = n_qblk - 1 - in_wave / per_blk;
  const int rem = in_wave % per_blk;
  const int stream = first_stream + rem / ctas_per_stream;
  it.hk = stream % p.Hkv;
  it.b = stream / p.Hkv;
  const int hq0 = it.hk * p.group + (rem % ctas_per_stream) * heads_per_cta;
  it.head0 = hq0;
  it.head1 = pair_heads ? hq0 + 1 : hq0;
  it.kv_limit = valid_keys(p, it.b);
  const int rows_per_item = pair_heads ? kBlockM : kRowsPerCta;
  const TileGeom g0 = tile_geometry(p, qblk * rows_per_item, it.kv_limit);
  const TileGeom g1 = tile_geometry(p, qblk * rows_per_item + (pair_heads ? 0 : kBlockM), it.kv_limit);
  it.row0_0 = g0.row0;
  it.row0_1 = g1.row0;
  it.nt0 = g0.n_tiles;
  it.nt1 = g1.n_tiles;
  it.lim0 = g0.min_lim;
  it.lim1 = g1.min_lim;
  it.in_range = (g0.in_range ? 1 : 0) | (g1.in_range ? 2 : 0);
  return it;
}

// ACC: the accumulating form (a ring step folded into a running fp32 result).  A template parameter, not a
// run-time branch: the softmax loop has no register to spare for state it does not use.
template <int D, bool BF16, bool BIAS, bool ACC>
__global__ void __launch_bounds__(kThreads, 1)
prefill_persistent_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const Problem p, const int n_qblk, const int pair_heads,
               const int streams_per_wave, const int n_items, unsigned int* __restrict__ next_item,
               const long long wait_limit) {
  using C = Cfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tiles = smem_u32(smem_raw);                     // tile area: 1024-byte aligned (swizzled TMA boxes)
  if ((tiles & 1023u) != 0u) {                                   // uniform over the CTA; nothing has been started
    if (threadIdx.x == 0) report(p.status, 0, -4, static_cast<int>(tiles & 1023u));
    return;
  }
  // [tile][row][weight of the previous accumulator (accumulating form), weight of O]
  float* stats = reinterpret_cast<float*>(smem_raw + C::kSmemTiles);
  Sync* sync = reinterpret_cast<Sync*>(smem_raw + C::kSmemTiles + C::kStatBytes);
  volatile int* abort_flag = &sync->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  const uint32_t q_smem[2] = {tiles, tiles + C::kTileBytes};
  const uint32_t kv_smem = tiles + kTilesPerCta * C::kTileBytes;

  // ---- set-up, once per CTA
  if (warp == kProducerWarp && lane == 0) {
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(smem_u32(&sync->item_full[s]), 1);
      mbar_init(smem_u32(&sync->item_empty[s]), kConsumerThreads);
    }
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sync->kv_full[s]), 1);
      mbar_init(smem_u32(&sync->kv_empty[s]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&sync->q_full[t]), 1);
      mbar_init(smem_u32(&sync->q_free[t]), 1);
      mbar_init(smem_u32(&sync->s_full[t]), 1);
      mbar_init(smem_u32(&sync->p_ready[t][0]), kBlockM);
      mbar_init(smem_u32(&sync->p_ready[t][1]), kBlockM);
      mbar_init(smem_u32(&sync->s_free[t]), kBlockM);
      mbar_init(smem_u32(&sync->pv_done[t]), 1);
      mbar_init(smem_u32(&sync->o_done[t]), 1);
      mbar_init(smem_u32(&sync->stats_ready[t]), kBlockM);
      mbar_init(smem_u32(&sync->o_free[t]), kBlockM);
    }
    mbar_init(smem_u32(&sync->drain), 1);
    sync->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sync->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sync->tmem_base;

  // what the producer lane has in flight (needed again if the CTA has to drain after an abort)
  int ring_pos = 0;              // K/V tiles issued so far, over all items
  int q_loads[2] = {0, 0};       // Q_t copies issued so far

  // every consumer role reads the next item from the scheduler's ring
  auto next_item_rec = [&](int k, bool* ok) -> ItemRec {
    const int slot = k % kItemSlots;
    ItemRec rec;
    rec.idx = -1;
    *ok = wait_clocked(smem_u32(&sync->item_full[slot]), (k / kItemSlots) & 1, abort_flag, wait_limit);
    if (!*ok) return rec;
    rec = sync->item[slot];
    mbar_arrive(smem_u32(&sync->item_empty[slot]));
    return rec;
  };

  if (warp >= kProducerWarp) {
    setmaxnreg_dec<Regs<BIAS>::kControl>();
    if (warp == kProducerWarp) {
      // ------------------------------------------------- scheduler + TMA producer
      if (lane == 0) {
        bool alive = true;
        // An item is drawn only when this CTA is ready to start copying it, i.e. when the copies of the
        // item before it have all been issued (the ring keeps the producer about two key tiles ahead of the
        // tensor cores, which covers the round trip of the atomic).  Drawing earlier would tie the next
        // item to a CTA that may still be busy for a long time while others run dry.
        auto fetch = [&](int k) -> int {
          const unsigned int i = next_item != nullptr ? atomicAdd(next_item, 1u)
                                                      : blockIdx.x + static_cast<unsigned int>(k) * gridDim.x;
          return i < static_cast<unsigned int>(n_items) ? static_cast<int>(i) : -1;
        };
        for (int k = 0; alive; ++k) {
          const int idx = fetch(k);
          const int slot = k % kItemSlots;
          if (k >= kItemSlots) {
            alive = wait_clocked(smem_u32(&sync->item_empty[slot]), (k / kItemSlots - 1) & 1, abort_flag, wait_limit);
            if (!alive) {
              report(p.status, 1, -2, k);
              break;
            }
          }
          ItemRec it;
          it.idx = -1;
          if (idx >= 0) it = decode_item(p, idx, n_qblk, pair_heads, streams_per_wave);
          sync->item[slot] = it;
          mbar_arrive(smem_u32(&sync->item_full[slot]));
          if (idx < 0) break;
          const int n_iter = it.nt0 > it.nt1 ? it.nt0 : it.nt1;
          // Q tiles: a slot is free again once the last Q K^T of the item that used it has retired.  A tile
          // without visible keys never reads its Q.
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if ((t == 0 ? it.nt0 : it.nt1) == 0 || !alive) continue;
            if (q_loads[t] > 0) {
              alive = wait_clocked(smem_u32(&sync->q_free[t]), (q_loads[t] - 1) & 1, abort_flag, wait_limit);
              if (!alive) {
                report(p.status, 1, -1, t);
                break;
              }
            }
            const uint32_t qbar = smem_u32(&sync->q_full[t]);
            mbar_arrive_expect_tx(qbar, C::kTileBytes);
            for (int bx = 0; bx < C::kBoxes; ++bx)
              tma_load_4d(q_smem[t] + bx * kBoxBytes, &tm_q, qbar, bx * 64, t == 0 ? it.row0_0 : it.row0_1,
                          t == 0 ? it.head0 : it.head1, it.b);
            ++q_loads[t];
          }
          for (int item = 0; item < 2 * n_iter && alive; ++item) {
            const int j = item >> 1;
            const int stage = ring_pos % C::kStages;
            const uint32_t round = static_cast<uint32_t>(ring_pos / C::kStages);
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
            for (int bx = 0; bx < C::kBoxes; ++bx)
              tma_load_4d(dst + bx * kBoxBytes, map, bar, bx * 64, j * kBlockN, it.hk, it.b);
            ++ring_pos;
          }
        }
      }
      __syncwarp();
    } else if (warp == kMmaWarp) {
      // -------------------------------------------------------------- MMA issuer
      // The whole warp runs the control flow (waits included) so that addresses and
      // descriptors stay in the uniform datapath; one elected lane issues.  The tile
      // index is a compile-time constant everywhere for the same reason.
      constexpr uint32_t idesc_qk = make_idesc(BF16, false, kBlockM, kBlockN);
      constexpr uint32_t idesc_pv = make_idesc(BF16, true, kBlockM, D);
      // descriptors: fixed fields once, then only the 16-byte-unit start address moves
      const uint64_t q_desc0 = smem_desc_sw128(q_smem[0], 16, 1024), q_desc1 = smem_desc_sw128(q_smem[1], 16, 1024);
      const uint64_t kv_desc_k = smem_desc_sw128(kv_smem, 16, 1024);          // K tile as K-major B operand
      const uint64_t kv_desc_v = smem_desc_sw128(kv_smem, kBoxBytes, 1024);   // V tile as MN-major B operand
      auto issue_qk = [&](auto tile_const, uint32_t stage) {
        constexpr int t = decltype(tile_const)::value;
        const uint64_t qd = t == 0 ? q_desc0 : q_desc1;
        const uint64_t kd = kv_desc_k + static_cast<uint64_t>(stage * (C::kTileBytes >> 4));
        const uint32_t d_addr = tmem_base + static_cast<uint32_t>(t * 128);
        if (elect_one() && dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 1, d_addr, tmem_base, 128, kTmemCols)) {
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
        if (elect_one() && dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 2, d_addr, tmem_base, D, kTmemCols) &&
            dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 3, a_addr, tmem_base, 32, kTmemCols)) {
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
      const std::integral_constant<int, 0> T0{};
      const std::integral_constant<int, 1> T1{};

      bool alive = true;
      int ring_c = 0;                 // K/V tiles consumed so far (position in the ring), over all items
      int n_q[2] = {0, 0};            // items for which Q_t was awaited
      int n_p[2] = {0, 0};            // P tiles consumed per tile
      int n_sfree[2] = {0, 0};        // (D = 64) score tiles released by the softmax warps and consumed here
      int n_o[2] = {0, 0};            // items whose O_t was completed
      auto wait_full = [&](int pos) -> bool {
        const int stage = pos % C::kStages;
        const uint32_t round = static_cast<uint32_t>(pos / C::kStages);
        const bool ok = wait_clocked(smem_u32(&sync->kv_full[stage]), round & 1u, abort_flag, wait_limit);
        if (!ok && lane == 0) report(p.status, 2, pos, stage);
        return ok;
      };
      auto stage_of = [&](int pos) { return static_cast<uint32_t>(pos % C::kStages); };
      auto empty_bar = [&](int pos) { return smem_u32(&sync->kv_empty[pos % C::kStages]); };

      for (int k = 0; alive; ++k) {
        const ItemRec it = next_item_rec(k, &alive);
        if (!alive) {
          if (lane == 0) report(p.status, 2, -3, k);
          break;
        }
        if (it.idx < 0) break;
        const int nt0 = it.nt0, nt1 = it.nt1;
        const int n_iter = nt0 > nt1 ? nt0 : nt1;
        if (n_iter == 0) continue;
        const int base = ring_c;       // ring position of K(0) of this item: K(j) at base + 2 j, V(j) at base + 2 j + 1
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if ((t == 0 ? nt0 : nt1) == 0 || !alive) continue;
          alive = wait_clocked(smem_u32(&sync->q_full[t]), n_q[t] & 1, abort_flag, wait_limit);
          if (!alive && lane == 0) report(p.status, 2, -1, t);
          ++n_q[t];
        }
        if (alive) alive = wait_full(base);
        if (!alive) break;
        tc_fence_after_sync();
        if (nt0 > 0) {
          issue_qk(T0, stage_of(base));
          commit(smem_u32(&sync->s_full[0]));
          if (nt0 == 1) commit(smem_u32(&sync->q_free[0]));
        }
        if (nt1 > 0) {
          issue_qk(T1, stage_of(base));
          commit(smem_u32(&sync->s_full[1]));
          if (nt1 == 1) commit(smem_u32(&sync->q_free[1]));
        }
        commit(empty_bar(base));
        for (int j = 0; j < n_iter && alive; ++j) {
          const int pos_v = base + 2 * j + 1, pos_kn = base + 2 * j + 2;
          const bool has_next = j + 1 < n_iter;
          alive = wait_full(pos_v);
          if (!alive) break;
          // one tile: P_t(j) V(j) in two halves as the halves of P arrive, then Q_t K(j+1)^T
          auto serve = [&](auto tile_const) {
            constexpr int t = decltype(tile_const)::value;
            const int nt = t == 0 ? nt0 : nt1;
            if (C::kSplitP) {
              // next scores first: S_t(j) only has to be out of tensor memory, not consumed
              if (t == 0 && has_next) {
                alive = wait_full(pos_kn);
                if (!alive) return;
              }
              if (j + 1 < nt) {
                alive = wait_clocked(smem_u32(&sync->s_free[t]), n_sfree[t] & 1, abort_flag, wait_limit);
                if (!alive) {
                  if (lane == 0) report(p.status, 9, j, t);
                  return;
                }
                tc_fence_after_sync();
                issue_qk(tile_const, stage_of(pos_kn));
                commit(smem_u32(&sync->s_full[t]));
                if (j + 2 == nt) commit(smem_u32(&sync->q_free[t]));
              }
              if (j < nt) ++n_sfree[t];   // one release per score tile, awaited or not
            }
            if (j < nt) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                alive = wait_clocked(smem_u32(&sync->p_ready[t][half]), n_p[t] & 1, abort_flag, wait_limit);
                if (!alive) {
                  if (lane == 0) report(p.status, 3, j, t);
                  return;
                }
                if (j == 0 && half == 0 && n_o[t] > 0) {
                  // the first product of an item overwrites O_t: the epilogue warps must hold the last item's
                  alive = wait_clocked(smem_u32(&sync->o_free[t]), (n_o[t] - 1) & 1, abort_flag, wait_limit);
                  if (!alive) {
                    if (lane == 0) report(p.status, 11, j, t);
                    return;
                  }
                }
                tc_fence_after_sync();
                issue_pv_half(tile_const, stage_of(pos_v), half, j > 0);
              }
              ++n_p[t];
            }
            if (C::kSplitP) {
              if (j < nt) {
                commit(smem_u32(&sync->pv_done[t]));
                if (j + 1 >= nt) {
                  commit(smem_u32(&sync->o_done[t]));
                  ++n_o[t];
                }
              }
            } else {
              if (t == 0 && has_next) {
                alive = wait_full(pos_kn);
                if (!alive) return;
                tc_fence_after_sync();
              }
              if (j + 1 < nt) {
                issue_qk(tile_const, stage_of(pos_kn));
                commit(smem_u32(&sync->s_full[t]));
                if (j + 2 == nt) commit(smem_u32(&sync->q_free[t]));
              } else if (j < nt) {
                commit(smem_u32(&sync->o_done[t]));
                ++n_o[t];
              }
            }
          };
          serve(T0);
          if (!alive) break;
          serve(T1);
          if (!alive) break;
          commit(empty_bar(pos_v));
          if (has_next) commit(empty_bar(pos_kn));
        }
        ring_c = base + 2 * n_iter;
      }
      __syncwarp();
    }
  } else if (warp >= kEpilogueWarp0) {
    // ------------------------------------------------------------------ epilogue
    // One thread per query row drains O_t of a finished item (32 columns at a time), normalises with the
    // row statistics the softmax thread of that row left in shared memory, and stores the row in 16-byte
    // pieces with the output's own strides; tensor-memory instructions stay outside per-lane conditions.
    setmaxnreg_dec<Regs<BIAS>::kEpilogue>();
    const int quad = warp & 3;
    const int r = tid & 127;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint16_t* out16 = reinterpret_cast<uint16_t*>(p.out);
    bool alive = true;
    int n_e[2] = {0, 0};   // items of tile t with keys, drained so far
    for (int k = 0; alive; ++k) {
      const ItemRec it = next_item_rec(k, &alive);
      if (!alive) {
        if (lane == 0) report(p.status, 6, -3, k);
        break;
      }
      if (it.idx < 0) break;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int nt = t == 0 ? it.nt0 : it.nt1;
        const int head = t == 0 ? it.head0 : it.head1;
        if (((it.in_range >> t) & 1) == 0 || !alive) continue;
        const int row_g = (t == 0 ? it.row0_0 : it.row0_1) + r;
        const bool row_ok = row_g < p.L;
        uint16_t* orow = out16 + it.b * p.os[0] + static_cast<long long>(head) * p.os[1] +
                         static_cast<long long>(row_g) * p.os[2];
        float* arow = p.acc + it.b * p.as[0] + static_cast<long long>(head) * p.as[1] + static_cast<long long>(row_g) * p.as[2];
        if (ACC && nt == 0 && p.acc_mode == 2) continue;      // accumulating form: no visible key here, nothing to fold
        float w_acc = 0.f, inv = 0.f;
        if (nt > 0) {
          bool ok = wait_relaxed(smem_u32(&sync->o_done[t]), n_e[t] & 1, abort_flag, wait_limit);
          ok = ok && wait_relaxed(smem_u32(&sync->stats_ready[t]), n_e[t] & 1, abort_flag, wait_limit);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) report(p.status, 6 + t, k, quad);
            alive = false;
            continue;
          }
          tc_fence_after_sync();
          ++n_e[t];
          w_acc = stats[(t * kBlockM + r) * 2];
          inv = stats[(t * kBlockM + r) * 2 + 1];
        }
        const uint32_t o_addr = tmem_base + lane_off + 256u + static_cast<uint32_t>(t) * D;
        // checked build: the columns drained below, and the row this thread is about to store
        if (!dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 4, o_addr, tmem_base, D, kTmemCols)) *abort_flag = 1;
        const bool store_ok = dbg_bhrc(p.status, DBG_PREFILL_PERSISTENT * 100 + 5, it.b, p.B, head, p.Hq, row_ok ? row_g : 0, p.L, 0, D, p.Dv);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          if (nt > 0) {
            tmem_ld_32x32(o_addr + c * 32, v);
            tmem_ld_wait();
            if (c == D / 32 - 1) {
              // O_t and the weights are in registers: the next item may overwrite both
              tc_fence_before_sync();
              mbar_arrive(smem_u32(&sync->o_free[t]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (ACC && row_ok && store_ok) {
            // running fp32 result: acc = acc * w_acc + O * w_o, four columns at a time
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              float4* dst = reinterpret_cast<float4*>(arow + c * 32 + u * 4);
              float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
              if (p.acc_mode == 2) a = *dst;
              a.x = fmaf(a.x, w_acc, __uint_as_float(v[4 * u]) * inv);
              a.y = fmaf(a.y, w_acc, __uint_as_float(v[4 * u + 1]) * inv);
              a.z = fmaf(a.z, w_acc, __uint_as_float(v[4 * u + 2]) * inv);
              a.w = fmaf(a.w, w_acc, __uint_as_float(v[4 * u + 3]) * inv);
              *dst = a;
            }
          } else if (!ACC && row_ok && store_ok) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              w.x = pack2<BF16>(__uint_as_float(v[8 * u]) * inv, __uint_as_float(v[8 * u + 1]) * inv);
              w.y = pack2<BF16>(__uint_as_float(v[8 * u + 2]) * inv, __uint_as_float(v[8 * u + 3]) * inv);
              w.z = pack2<BF16>(__uint_as_float(v[8 * u + 4]) * inv, __uint_as_float(v[8 * u + 5]) * inv);
              w.w = pack2<BF16>(__uint_as_float(v[8 * u + 6]) * inv, __uint_as_float(v[8 * u + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
            }
          }
        }
        // (rows that saw keys get their lse from the softmax thread that owns the row statistics)
        if (nt == 0 && row_ok && store_ok) {
          if (ACC && p.acc_mode == 1) p.acc_lse[it.b * p.als[0] + head * p.als[1] + row_g * p.als[2]] = -CUDART_INF_F;
          if (!ACC && p.lse != nullptr) p.lse[it.b * p.ls[0] + head * p.ls[1] + row_g * p.ls[2]] = -CUDART_INF_F;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax roles
    setmaxnreg_inc<Regs<BIAS>::kSoftmax>();
    const int t = warp >> 2;                 // which 128-row tile
    const int quad = warp & 3;               // TMEM lane quadrant this warp may touch
    const int r = tid & 127;                 // row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + static_cast<uint32_t>(t) * 128u;
    const uint32_t o_addr = tmem_base + lane_off + 256u + static_cast<uint32_t>(t) * D;
    const uint32_t p_addr = C::kSplitP ? tmem_base + lane_off + 384u + static_cast<uint32_t>(t) * 64u : s_addr;
    // checked build: the three column ranges this thread reads and writes; a violation drains the CTA
    if (!dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 6, s_addr, tmem_base, 128, kTmemCols) ||
        !dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 7, o_addr, tmem_base, D, kTmemCols) ||
        !dbg_tmem(p.status, DBG_PREFILL_PERSISTENT * 100 + 8, p_addr, tmem_base, 64, kTmemCols))
      *abort_flag = 1;
    // With an additive bias the logits s * scale + bias are formed when the scores are read;
    // everything after that then works on them with scale 1 (log2 e in the exponent).
    const float sl2_in = BIAS ? p.scale : p.scale * kLog2e;
    const float sl2 = BIAS ? kLog2e : sl2_in;
    const bool bias_wide = BIAS && bias_rows_32b(p);
    bool alive = true;
    int n_s = 0;        // score tiles of this tile consumed so far, over all items
    int n_done = 0;     // items (with keys) of this tile finished so far

    for (int k = 0; alive; ++k) {
      const ItemRec it = next_item_rec(k, &alive);
      if (!alive) {
        if (lane == 0) report(p.status, 4 + t, -3, k);
        break;
      }
      if (it.idx < 0) break;
      const int n_tiles = t == 0 ? it.nt0 : it.nt1;
      if (n_tiles == 0) continue;
      const int min_lim = t == 0 ? it.lim0 : it.lim1;
      const int head = t == 0 ? it.head0 : it.head1;
      const int b = it.b;
      const int row_g = (t == 0 ? it.row0_0 : it.row0_1) + r;
      int lim = it.kv_limit;                   // keys [0, lim) are visible to this row
      if (p.causal) {
        const long long c = static_cast<long long>(row_g) + p.causal_shift + 1;
        lim = c < lim ? static_cast<int>(c < 0 ? 0 : c) : lim;
      }
      float m_run = -CUDART_INF_F, l_run = 0.f;
      // accumulating form: the row's running lse is fetched now and used after the last key tile
      float* acc_lse_row = nullptr;
      float old_lse = -CUDART_INF_F;
      if constexpr (ACC) {
        if (row_g < p.L) {
          acc_lse_row = p.acc_lse + b * p.als[0] + head * p.als[1] + row_g * p.als[2];
          if (p.acc_mode == 2) old_lse = *acc_lse_row;
        }
      }
      // this row of the bias, 16-bit elements in the query's dtype, unit stride along the keys
      const uint4* bias_row = nullptr;
      if constexpr (BIAS) {
        if (row_g < p.L)
          bias_row = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + b * p.bs[0] +
                                                    static_cast<long long>(head) * p.bs[1] +
                                                    static_cast<long long>(row_g) * p.bs[2]);
      }

      for (int j = 0; j < n_tiles; ++j) {
        uint4 bv[BIAS ? kBlockN / 8 : 1];
        if constexpr (BIAS) {
          // the bias of this key tile travels while the scores are awaited
          load_bias_row(bv, bias_row, j * kBlockN, p.S, bias_wide);
        }
        bool ok = wait_clocked(smem_u32(&sync->s_full[t]), n_s & 1, abort_flag, wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 4 + t, j, quad);
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const int col0 = j * kBlockN;
        const bool need_mask = col0 + kBlockN > min_lim;

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
        if (C::kSplitP && n_s > 0) {
          // here S can be ready before P V of the previous score tile (of this item or of the last one) has
          // retired, and that product still reads the P columns and writes O_t: wait for it before touching either
          bool pv_ok = wait_clocked(smem_u32(&sync->pv_done[t]), (n_s - 1) & 1, abort_flag, wait_limit);
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
        const uint64_t sl2_2 = f2_pack(sl2, sl2), nms_2 = f2_pack(nms, nms);
        uint64_t sum2[2] = {0ull, 0ull};           // two packed accumulators = four chains
#pragma unroll
        for (int c = 0; c < kBlockN / 32; ++c) {
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
        if (j + 1 == n_tiles) {
          // last key tile of the item: leave 1 / (row sum) for the epilogue warps before the product they
          // wait for can be issued, and write the row's lse.  The epilogue must be done with the previous
          // item's figures.
          if (n_done > 0) {
            bool free_ok = wait_clocked(smem_u32(&sync->o_free[t]), (n_done - 1) & 1, abort_flag, wait_limit);
            free_ok = __all_sync(0xffffffffu, free_ok);
            if (!free_ok) {
              if (lane == 0) report(p.status, 12, j, t);
              alive = false;
              break;
            }
          }
          // one rounding at the magnitude of the maximum: m*scale + ln(l)
          const float lse = l_run > 0.f ? fmaf(m_run, BIAS ? 1.f : p.scale, lg2(l_run) * kLn2) : -CUDART_INF_F;
          float w_acc = 0.f, w_o = l_run > 0.f ? 1.f / l_run : 0.f;
          if (ACC && acc_lse_row != nullptr) {
            // accumulating form: fold this block's (result, lse) into the running pair for the row
            float* al = acc_lse_row;
            const float old = old_lse;
            const float hi = fmaxf(old, lse);
            float merged = -CUDART_INF_F;
            if (hi != -CUDART_INF_F) {
              const float e_old = ex2((old - hi) * kLog2e), e_new = ex2((lse - hi) * kLog2e);   // -inf -> 0
              merged = hi + lg2(e_old + e_new) * kLn2;
              w_acc = ex2((old - merged) * kLog2e);
              w_o *= ex2((lse - merged) * kLog2e);
            } else {
              w_o = 0.f;
            }
            *al = merged;
          }
          stats[(t * kBlockM + r) * 2] = w_acc;
          stats[(t * kBlockM + r) * 2 + 1] = w_o;
          mbar_arrive(smem_u32(&sync->stats_ready[t]));
          ++n_done;
          if (!ACC && p.lse != nullptr && row_g < p.L &&
              dbg_bhrc(p.status, DBG_PREFILL_PERSISTENT * 100 + 9, b, p.B, head, p.Hq, row_g, p.L, 0, 0, 1))
            p.lse[b * p.ls[0] + head * p.ls[1] + row_g * p.ls[2]] = lse;
        }
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&sync->p_ready[t][1]));
        ++n_s;
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
      for (int t = 0; t < 2; ++t)
        if (q_loads[t] > 0) wait_drain(smem_u32(&sync->q_full[t]), (q_loads[t] - 1) & 1);
      for (int s = 0; s < C::kStages && s < ring_pos; ++s) {
        const uint32_t last_round = static_cast<uint32_t>((ring_pos - 1 - s) / C::kStages);
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

// CTAs of the persistent grid: one per SM, never more than there are items.  The planner is host-only
// and assumes the 148 SMs of a B200; the launcher asks the device.
constexpr int kAssumedSms = 148;

int sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) {
    cudaGetLastError();
    return kAssumedSms;
  }
  return sms;
}

struct PrefillGeom {
  int pair_heads, rows, n_qblk;
  long long n_items;
};

PrefillGeom prefill_geometry(const Problem& p) {
  PrefillGeom g;
  g.pair_heads = pair_heads_mode(p);
  g.rows = g.pair_heads ? kBlockM : kRowsPerCta;
  g.n_qblk = (p.L + g.rows - 1) / g.rows;
  g.n_items = static_cast<long long>(g.n_qblk) * (p.Hq / (g.pair_heads ? 2 : 1)) * p.B;
  return g;
}

template <int D, bool BF16, bool BIAS, bool ACC>
int launch_variant(const Problem& p, void* workspace, uint64_t workspace_bytes, cudaStream_t stream) {
  using C = Cfg<D>;
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, p.q, BF16, D, p.L, p.Hq, p.B, p.qs) || !make_map(&tk, p.k, BF16, D, p.S, p.Hkv, p.B, p.ks) ||
      !make_map(&tv, p.v, BF16, D, p.S, p.Hkv, p.B, p.vs))
    return B200_SDPA_ERR_CUDA;
  auto kern = prefill_persistent_kernel<D, BF16, BIAS, ACC>;
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute: set on every
  // launch (a cheap host-side call), so a process that drives several GPUs gets it on each of them
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  const PrefillGeom g = prefill_geometry(p);
  if (g.n_items <= 0 || g.n_items > 0x3fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  const int sms = sm_count();
  const int grid = g.n_items < sms ? static_cast<int>(g.n_items) : sms;
  // With scratch for one counter the items are handed out one at a time (longest first, whoever is free
  // takes the next); without it every CTA takes items c, c + grid, c + 2 grid, ... of the same list.
  unsigned int* counter = nullptr;
  if (workspace != nullptr && workspace_bytes >= sizeof(unsigned int) && reinterpret_cast<uintptr_t>(workspace) % 4 == 0) {
    counter = reinterpret_cast<unsigned int*>(workspace);
    if (cudaMemsetAsync(counter, 0, sizeof(unsigned int), stream) != cudaSuccess) {
      cudaGetLastError();
      return B200_SDPA_ERR_CUDA;
    }
  }
  const int per_wave = kv_streams_per_wave(static_cast<long long>(p.S) * 2 * D * 2, static_cast<long long>(p.Hkv) * p.B);
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p, g.n_qblk, g.pair_heads, per_wave,
                                                  static_cast<int>(g.n_items), counter, wait_limit_cycles());
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_PREFILL);
  return B200_SDPA_OK;
}

}  // namespace

// How the two prefill kernels share the work.  What the persistent kernel saves is the cost of going from
// one work item to the next (no CTA launch, set-up or tear-down; the next item's Q and first key tile
// already in flight; the epilogue on its own warps); what it pays is a heavier steady state (sixteen warps
// share the register file, and under a power cap it clocks a little lower).  Measured on one B200: with up
// to 32 key tiles per item it is 3-5 % faster in bursts (8-14 % with a bias) and about 2 % slower when the
// GPU sits at its power cap for seconds; with 256 key tiles per item (32768 keys, and the blocks of a ring
// over 131072) the per-CTA kernel is 5 % faster either way.  So: head dimension 128, at least three items
// per SM, and at most 64 key tiles per item.  B200_SDPA_PREFILL = "persistent" or "per_cta" overrides the
// choice where both kernels can serve the request (for tests and measurements).
// (acc, acc_lse) of the accumulating form: fp32 rows read and written as 16-byte pieces
bool prefill_accumulate_eligible(const Problem& p) {
  if (p.E != 128 || p.Dv != 128 || p.acc == nullptr || p.acc_lse == nullptr || p.bias != nullptr) return false;
  if (reinterpret_cast<uintptr_t>(p.acc) % 16 != 0) return false;
  const int n[3] = {p.B, p.Hq, p.L};
  for (int i = 0; i < 3; ++i)
    if (n[i] > 1 && (p.as[i] <= 0 || p.as[i] % 4 != 0 || p.als[i] <= 0)) return false;
  return true;
}

bool prefill_persistent_wanted(const Problem& p) {
  if (p.E != 128 || p.Dv != 128) return false;
  const char* e = getenv("B200_SDPA_PREFILL");
  if (e != nullptr && e[0] == 'p' && e[1] == 'e' && e[2] == 'r' && e[3] == 's') return true;    // "persistent"
  if (e != nullptr && e[0] == 'p' && e[1] == 'e' && e[2] == 'r' && e[3] == '_') return false;   // "per_cta"
  // The accumulating form (ring steps) runs for seconds with the GPU at its power cap, where the kernel with
  // one item per CTA was the faster one at every block size measured (eight ranks' blocks: 272.7 ms against
  // 291.5 ms for this kernel).
  if (p.acc_mode != 0) return false;
  return prefill_geometry(p).n_items >= 3LL * kAssumedSms && (p.S + kBlockN - 1) / kBlockN <= 64;
}

void plan_prefill_persistent(const Problem& p, B200SdpaPlan* plan) {
  const PrefillGeom g = prefill_geometry(p);
  plan->path = B200_SDPA_PATH_PREFILL;
  plan->block_m = g.rows;
  plan->block_n = kBlockN;
  plan->grid_x = static_cast<int32_t>(g.n_items < kAssumedSms ? g.n_items : kAssumedSms);
  plan->grid_y = plan->grid_z = 1;
  plan->threads = kThreads;
  plan->smem_bytes = Cfg<128>::kSmemBytes;
  plan->kv_splits = 1;
  plan->launches = 1;
  // optional: with 16 bytes of scratch the CTAs draw their work items from a shared counter
  plan->workspace_bytes = 16;
}

// The caller has checked prefill_eligible() and prefill_persistent_wanted().
int launch_prefill_persistent(const Problem& p, int dtype, void* workspace, uint64_t workspace_bytes,
                              cudaStream_t stream) {
  const bool bf16 = dtype == B200_SDPA_BF16;
  if (p.acc_mode != 0) {
    if (p.bias != nullptr) return B200_SDPA_ERR_UNSUPPORTED;
    return bf16 ? launch_variant<128, true, false, true>(p, workspace, workspace_bytes, stream)
                : launch_variant<128, false, false, true>(p, workspace, workspace_bytes, stream);
  }
  if (p.bias != nullptr)
    return bf16 ? launch_variant<128, true, true, false>(p, workspace, workspace_bytes, stream)
                : launch_variant<128, false, true, false>(p, workspace, workspace_bytes, stream);
  return bf16 ? launch_variant<128, true, false, false>(p, workspace, workspace_bytes, stream)
              : launch_variant<128, false, false, false>(p, workspace, workspace_bytes, stream);
}

}  // namespace b200
