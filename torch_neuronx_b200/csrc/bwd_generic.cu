// Generic flash-attention backward on CUDA cores (fp32 arithmetic throughout).
//
// Two kernels, neither of which ever holds an [L,S] matrix in global memory:
//   * bwd_dq_kernel : one CTA per (batch, query head, block of query rows); walks the
//     key blocks and accumulates dQ in registers (optionally writes the gradient of
//     the logits for an additive bias);
//   * bwd_dkv_kernel: one CTA per (batch, kv head, block of keys); walks the query
//     heads of the group and their row blocks and accumulates dK and dV in registers,
//     so grouped-query gradients are summed without atomics and in a fixed order.
// Arithmetic follows torch_neuronx/_sdpa_math.py:133-176: probabilities are rebuilt
// from the forward's log-sum-exp (rows with lse = -inf give zeros), dV = P^T dO,
// dP = dO V^T, dS = P * (dP - delta) * scale, dQ = dS K, dK = dS^T Q.  The row term
// `delta` is sum_d dO_d * out_d, which is what upstream's two-part `sum_reduction`
// (:161-163) adds up to; each CTA recomputes it for the rows it holds, so no scratch
// is needed.
#include "common.cuh"
#include "debug.cuh"

namespace b200 {

namespace {

constexpr int kThreads = 256;

// Everything a CTA needs about one block of query rows: Q and dO tiles in shared
// memory plus lse and delta per row.
template <typename T, int TILE>
__device__ __forceinline__ void load_query_block(const BwdProblem& bp, int b, int h, int row0, int ldq, int ldv,
                                                 float* Qs, float* dOs, float* row_lse, float* row_delta) {
  const Problem& p = bp.f;
  constexpr int TPR = kThreads / TILE;
  const int tid = threadIdx.x;
  const T* __restrict__ q = reinterpret_cast<const T*>(p.q);
  const T* __restrict__ go = reinterpret_cast<const T*>(bp.dout);
  const T* __restrict__ o = reinterpret_cast<const T*>(p.out);
  const int64_t q_base = b * p.qs[0] + h * p.qs[1];
  const int64_t g_base = b * bp.dos[0] + h * bp.dos[1];
  const int64_t o_base = b * p.os[0] + h * p.os[1];
  for (int idx = tid; idx < TILE * p.E; idx += kThreads) {
    const int r = idx / p.E, e = idx - r * p.E;
    const int gi = row0 + r;
    Qs[r * ldq + e] = gi < p.L ? to_f32<T>(q[q_base + gi * p.qs[2] + e * p.qs[3]]) : 0.f;
  }
  for (int idx = tid; idx < TILE * ldv; idx += kThreads) {
    const int r = idx / ldv, e = idx - r * ldv;
    const int gi = row0 + r;
    dOs[idx] = (gi < p.L && e < p.Dv) ? to_f32<T>(go[g_base + gi * bp.dos[2] + e * bp.dos[3]]) : 0.f;
  }
  __syncthreads();
  {
    const int r = tid / TPR, sub = tid % TPR;
    const int gi = row0 + r;
    float d = 0.f;
    if (gi < p.L) {
      for (int e = sub; e < p.Dv; e += TPR) d = fmaf(dOs[r * ldv + e], to_f32<T>(o[o_base + gi * p.os[2] + e * p.os[3]]), d);
    }
#pragma unroll
    for (int off = TPR / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
    if (sub == 0) {
      row_delta[r] = d;
      row_lse[r] = gi < p.L ? p.lse[b * p.ls[0] + h * p.ls[1] + gi * p.ls[2]] : -CUDART_INF_F;
    }
  }
  __syncthreads();
}

template <typename T, int TILE>
__device__ __forceinline__ void load_key_block(const Problem& p, int b, int hk, int64_t j0, int64_t j_end, int ldq,
                                               int ldv, float* Ks, float* Vs) {
  const int tid = threadIdx.x;
  const T* __restrict__ k = reinterpret_cast<const T*>(p.k);
  const T* __restrict__ v = reinterpret_cast<const T*>(p.v);
  const int64_t k_base = b * p.ks[0] + hk * p.ks[1];
  const int64_t v_base = b * p.vs[0] + hk * p.vs[1];
  for (int idx = tid; idx < TILE * p.E; idx += kThreads) {
    const int r = idx / p.E, e = idx - r * p.E;
    const int64_t gj = j0 + r;
    Ks[r * ldq + e] = gj < j_end ? to_f32<T>(k[k_base + gj * p.ks[2] + e * p.ks[3]]) : 0.f;
  }
  for (int idx = tid; idx < TILE * ldv; idx += kThreads) {
    const int r = idx / ldv, e = idx - r * ldv;
    const int64_t gj = j0 + r;
    Vs[idx] = (gj < j_end && e < p.Dv) ? to_f32<T>(v[v_base + gj * p.vs[2] + e * p.vs[3]]) : 0.f;
  }
}

// Thread (ty, tx) rebuilds the probabilities of its R x R patch (rows ty*R+i, key
// columns tx+16j) and turns them into dS (before the scale).  `pr` and `ds` come back
// in registers.
template <int TILE>
__device__ __forceinline__ void score_patch(const BwdProblem& bp, int b, int h, int row0, int64_t j0, int n_keys,
                                            int ldq, int ldv, const float* Qs, const float* dOs, const float* Ks,
                                            const float* Vs, const float* row_lse, const float* row_delta,
                                            float (&pr)[TILE / 16][TILE / 16], float (&ds)[TILE / 16][TILE / 16]) {
  constexpr int R = TILE / 16;
  const Problem& p = bp.f;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float s[R][R], dp[R][R];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int j = 0; j < R; ++j) s[i][j] = dp[i][j] = 0.f;
#pragma unroll 4
  for (int e = 0; e < p.E; ++e) {
    float qv[R], kv[R];
#pragma unroll
    for (int i = 0; i < R; ++i) qv[i] = Qs[(ty * R + i) * ldq + e];
#pragma unroll
    for (int j = 0; j < R; ++j) kv[j] = Ks[(tx + 16 * j) * ldq + e];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < R; ++j) s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
  }
#pragma unroll 4
  for (int e = 0; e < p.Dv; ++e) {
    float gv[R], vv[R];
#pragma unroll
    for (int i = 0; i < R; ++i) gv[i] = dOs[(ty * R + i) * ldv + e];
#pragma unroll
    for (int j = 0; j < R; ++j) vv[j] = Vs[(tx + 16 * j) * ldv + e];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < R; ++j) dp[i][j] = fmaf(gv[i], vv[j], dp[i][j]);
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = ty * R + i;
    const int gi = row0 + r;
    const float lse = row_lse[r];
    const float delta = row_delta[r];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int64_t gj = j0 + tx + 16 * j;
      float val = s[i][j] * p.scale;
      const bool visible =
          gi < p.L && gj < n_keys && lse != -CUDART_INF_F && (!p.causal || gj <= gi + p.causal_shift);
      if (visible && p.bias != nullptr) {
        val += load_as_f32(p.bias, b * p.bs[0] + h * p.bs[1] + gi * p.bs[2] + gj * p.bs[3], p.bias_dtype);
      }
      const float prob = visible ? expf(val - lse) : 0.f;
      pr[i][j] = prob;
      ds[i][j] = prob * (dp[i][j] - delta);
    }
  }
}

template <typename T, int TILE, int NC>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(const BwdProblem bp, const int ldq, const int ldv) {
  constexpr int R = TILE / 16;
  constexpr int LDS = TILE + 1;
  const Problem& p = bp.f;
  extern __shared__ float smem[];
  float* Qs = smem;
  float* Ks = Qs + TILE * ldq;
  float* dOs = Ks + TILE * ldq;
  float* Vs = dOs + TILE * ldv;
  float* Ds = Vs + TILE * ldv;
  float* row_lse = Ds + TILE * LDS;
  float* row_delta = row_lse + TILE;

  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  const int n_mblk = (p.L + TILE - 1) / TILE;
  int64_t bid = blockIdx.x;
  const int mblk = static_cast<int>(bid % n_mblk);
  bid /= n_mblk;
  const int h = static_cast<int>(bid % p.Hq);
  const int b = static_cast<int>(bid / p.Hq);
  const int hk = h / p.group;
  const int row0 = mblk * TILE;
  const int last_row = (row0 + TILE < p.L ? row0 + TILE : p.L) - 1;

  const int n_keys = valid_keys(p, b);
  int64_t k_end = n_keys;
  if (p.causal) {
    const int64_t lim = static_cast<int64_t>(last_row) + p.causal_shift + 1;
    k_end = lim < k_end ? lim : k_end;
  }
  if (k_end < 0) k_end = 0;
  // The logit gradient must be written for every key, visible or not.
  const int64_t k_walk = bp.dbias != nullptr ? p.S : k_end;

  load_query_block<T, TILE>(bp, b, h, row0, ldq, ldv, Qs, dOs, row_lse, row_delta);

  float acc[R][NC];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;

  T* __restrict__ gb = reinterpret_cast<T*>(bp.dbias);
  for (int64_t j0 = 0; j0 < k_walk; j0 += TILE) {
    load_key_block<T, TILE>(p, b, hk, j0, p.S, ldq, ldv, Ks, Vs);
    __syncthreads();
    float pr[R][R], ds[R][R];
    score_patch<TILE>(bp, b, h, row0, j0, n_keys, ldq, ldv, Qs, dOs, Ks, Vs, row_lse, row_delta, pr, ds);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = ty * R + i;
      const int gi = row0 + r;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int c = tx + 16 * j;
        Ds[r * LDS + c] = ds[i][j];
        if (gb != nullptr && gi < p.L && j0 + c < p.S &&
            dbg_bhrc(p.status, DBG_GENERIC_BWD * 100 + 1, b, p.B, h, p.Hq, gi, p.L, j0 + c, 1, p.S)) {
          gb[b * bp.dbs[0] + h * bp.dbs[1] + gi * bp.dbs[2] + (j0 + c) * bp.dbs[3]] = from_f32<T>(ds[i][j]);
        }
      }
    }
    __syncthreads();
#pragma unroll 2
    for (int kk = 0; kk < TILE; ++kk) {
      float dv_[R];
#pragma unroll
      for (int i = 0; i < R; ++i) dv_[i] = Ds[(ty * R + i) * LDS + kk];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int col = tx + 16 * c;
        const float kv = col < p.E ? Ks[kk * ldq + col] : 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) acc[i][c] = fmaf(dv_[i], kv, acc[i][c]);
      }
    }
    __syncthreads();
  }

  T* __restrict__ gq = reinterpret_cast<T*>(bp.dq);
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int gi = row0 + ty * R + i;
    if (gi >= p.L) continue;
    const int64_t base = b * bp.dqs[0] + h * bp.dqs[1] + gi * bp.dqs[2];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int col = tx + 16 * c;
      if (col < p.E && dbg_bhrc(p.status, DBG_GENERIC_BWD * 100 + 2, b, p.B, h, p.Hq, gi, p.L, col, 1, p.E))
        gq[base + col * bp.dqs[3]] = from_f32<T>(acc[i][c] * p.scale);
    }
  }
}

template <typename T, int TILE, int NC>
__global__ void __launch_bounds__(kThreads) bwd_dkv_kernel(const BwdProblem bp, const int ldq, const int ldv) {
  constexpr int R = TILE / 16;
  constexpr int LDS = TILE + 1;
  const Problem& p = bp.f;
  extern __shared__ float smem[];
  float* Qs = smem;
  float* Ks = Qs + TILE * ldq;
  float* dOs = Ks + TILE * ldq;
  float* Vs = dOs + TILE * ldv;
  float* Ds = Vs + TILE * ldv;
  float* Ps = Ds + TILE * LDS;
  float* row_lse = Ps + TILE * LDS;
  float* row_delta = row_lse + TILE;

  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  const int n_nblk = (p.S + TILE - 1) / TILE;
  int64_t bid = blockIdx.x;
  const int nblk = static_cast<int>(bid % n_nblk);
  bid /= n_nblk;
  const int hk = static_cast<int>(bid % p.Hkv);
  const int b = static_cast<int>(bid / p.Hkv);
  const int64_t j0 = static_cast<int64_t>(nblk) * TILE;
  const int n_keys = valid_keys(p, b);

  load_key_block<T, TILE>(p, b, hk, j0, p.S, ldq, ldv, Ks, Vs);

  float acc_k[R][NC], acc_v[R][NC];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc_k[i][c] = acc_v[i][c] = 0.f;

  // First query row that can see any key of this block.
  int row_start = 0;
  if (p.causal) {
    const int64_t first = j0 - p.causal_shift;
    row_start = first > 0 ? static_cast<int>((first < p.L ? first : p.L) / TILE) * TILE : 0;
  }
  const bool any_key = j0 < n_keys;

  for (int g = 0; g < p.group && any_key; ++g) {
    const int h = hk * p.group + g;
    for (int row0 = row_start; row0 < p.L; row0 += TILE) {
      __syncthreads();  // previous tile's readers of Qs/dOs/Ps/Ds are done
      load_query_block<T, TILE>(bp, b, h, row0, ldq, ldv, Qs, dOs, row_lse, row_delta);
      float pr[R][R], ds[R][R];
      score_patch<TILE>(bp, b, h, row0, j0, n_keys, ldq, ldv, Qs, dOs, Ks, Vs, row_lse, row_delta, pr, ds);
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) {
          Ps[(ty * R + i) * LDS + tx + 16 * j] = pr[i][j];
          Ds[(ty * R + i) * LDS + tx + 16 * j] = ds[i][j];
        }
      __syncthreads();
      // This thread now owns keys ty*R+i and feature columns tx+16c.
#pragma unroll 2
      for (int ii = 0; ii < TILE; ++ii) {
        float pv[R], dv_[R];
#pragma unroll
        for (int i = 0; i < R; ++i) {
          pv[i] = Ps[ii * LDS + ty * R + i];
          dv_[i] = Ds[ii * LDS + ty * R + i];
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int col = tx + 16 * c;
          const float gv = dOs[ii * ldv + col];  // zero beyond Dv
          const float qv = col < p.E ? Qs[ii * ldq + col] : 0.f;
#pragma unroll
          for (int i = 0; i < R; ++i) {
            acc_v[i][c] = fmaf(pv[i], gv, acc_v[i][c]);
            acc_k[i][c] = fmaf(dv_[i], qv, acc_k[i][c]);
          }
        }
      }
    }
  }

  T* __restrict__ gk = reinterpret_cast<T*>(bp.dk);
  T* __restrict__ gv = reinterpret_cast<T*>(bp.dv);
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int64_t gj = j0 + ty * R + i;
    if (gj >= p.S) continue;
    const int64_t kb = b * bp.dks[0] + hk * bp.dks[1] + gj * bp.dks[2];
    const int64_t vb = b * bp.dvs[0] + hk * bp.dvs[1] + gj * bp.dvs[2];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int col = tx + 16 * c;
      if (col < p.E && dbg_bhrc(p.status, DBG_GENERIC_BWD * 100 + 3, b, p.B, hk, p.Hkv, gj, p.S, col, 1, p.E))
        gk[kb + col * bp.dks[3]] = from_f32<T>(acc_k[i][c] * p.scale);
      if (col < p.Dv && dbg_bhrc(p.status, DBG_GENERIC_BWD * 100 + 4, b, p.B, hk, p.Hkv, gj, p.S, col, 1, p.Dv))
        gv[vb + col * bp.dvs[3]] = from_f32<T>(acc_v[i][c]);
    }
  }
}

struct BwdConfig {
  int tile, nc, ldq, ldv, smem_dq, smem_dkv;
};

bool pick_bwd_config(const Problem& p, BwdConfig* cfg) {
  const int dmax = p.E > p.Dv ? p.E : p.Dv;
  if (dmax > 256) return false;
  int nc = (dmax + 15) / 16;
  nc = nc <= 4 ? 4 : nc <= 8 ? 8 : 16;
  const int tile = nc <= 8 ? 64 : 32;
  cfg->tile = tile;
  cfg->nc = nc;
  cfg->ldq = p.E | 1;
  cfg->ldv = 16 * nc + 1;  // odd: rows are read both along and across the feature axis
  const int common = 2 * tile * cfg->ldq + 2 * tile * cfg->ldv + 2 * tile;
  cfg->smem_dq = static_cast<int>(sizeof(float)) * (common + tile * (tile + 1));
  cfg->smem_dkv = static_cast<int>(sizeof(float)) * (common + 2 * tile * (tile + 1));
  return cfg->smem_dkv <= 227 * 1024;
}

template <typename T, int TILE, int NC>
int launch_pair(const BwdProblem& bp, const BwdConfig& cfg, cudaStream_t stream) {
  const Problem& p = bp.f;
  const int64_t grid_q = static_cast<int64_t>((p.L + TILE - 1) / TILE) * p.Hq * p.B;
  const int64_t grid_kv = static_cast<int64_t>((p.S + TILE - 1) / TILE) * p.Hkv * p.B;
  if (grid_q > 0x7fffffffLL || grid_kv > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  auto kq = bwd_dq_kernel<T, TILE, NC>;
  auto kkv = bwd_dkv_kernel<T, TILE, NC>;
  if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_dq) != cudaSuccess ||
      cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_dkv) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  kq<<<static_cast<unsigned>(grid_q), kThreads, cfg.smem_dq, stream>>>(bp, cfg.ldq, cfg.ldv);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_BWD_DQ);
  if (grid_kv > 0) {
    kkv<<<static_cast<unsigned>(grid_kv), kThreads, cfg.smem_dkv, stream>>>(bp, cfg.ldq, cfg.ldv);
    if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
    count_launch(KID_BWD_DKV);
  }
  return B200_SDPA_OK;
}

template <typename T>
int launch_bwd_typed(const BwdProblem& bp, const BwdConfig& cfg, cudaStream_t stream) {
  if (cfg.nc == 4) return launch_pair<T, 64, 4>(bp, cfg, stream);
  if (cfg.nc == 8) return launch_pair<T, 64, 8>(bp, cfg, stream);
  return launch_pair<T, 32, 16>(bp, cfg, stream);
}

}  // namespace

int plan_bwd_generic(const BwdProblem& bp, int dtype, B200SdpaPlan* plan) {
  (void)dtype;
  BwdConfig cfg;
  if (!pick_bwd_config(bp.f, &cfg)) return B200_SDPA_ERR_UNSUPPORTED;
  const Problem& p = bp.f;
  const int64_t grid_q = static_cast<int64_t>((p.L + cfg.tile - 1) / cfg.tile) * p.Hq * p.B;
  const int64_t grid_kv = static_cast<int64_t>((p.S + cfg.tile - 1) / cfg.tile) * p.Hkv * p.B;
  if (grid_q > 0x7fffffffLL || grid_kv > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  plan->path = B200_SDPA_PATH_GENERIC;
  plan->block_m = plan->block_n = cfg.tile;
  plan->grid_x = static_cast<int32_t>(grid_q);
  plan->grid_y = static_cast<int32_t>(grid_kv);
  plan->grid_z = 1;
  plan->threads = kThreads;
  plan->smem_bytes = cfg.smem_dkv;
  plan->kv_splits = 1;
  plan->launches = grid_kv > 0 ? 2 : 1;
  plan->workspace_bytes = 0;
  return B200_SDPA_OK;
}

int launch_bwd_generic(const BwdProblem& bp, int dtype, cudaStream_t stream) {
  BwdConfig cfg;
  if (!pick_bwd_config(bp.f, &cfg)) return B200_SDPA_ERR_UNSUPPORTED;
  switch (dtype) {
    case B200_SDPA_F32: return launch_bwd_typed<float>(bp, cfg, stream);
    case B200_SDPA_F16: return launch_bwd_typed<__half>(bp, cfg, stream);
    case B200_SDPA_BF16: return launch_bwd_typed<__nv_bfloat16>(bp, cfg, stream);
    default: return B200_SDPA_ERR_DTYPE;
  }
}

}  // namespace b200
