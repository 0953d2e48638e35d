// Generic flash-attention forward on CUDA cores (fp32 arithmetic throughout).
//
// Serves every request the specialised kernels do not take: fp32 inputs (the
// <=1e-5 parity case), additive bias, arbitrary strides, head dims up to 512,
// negative scale.  Online softmax over TILE x TILE score blocks; scores never
// leave shared memory.  Arithmetic follows torch_neuronx/_sdpa_math.py:79-95:
// scale, causal mask, bias, row max with the dead-row guard, exp, sum,
// lse = max + log(sum); the only difference is that probabilities stay fp32 for
// the second product (upstream rounds them to the input dtype first).
#include "common.cuh"
#include "debug.cuh"

namespace b200 {

namespace {

constexpr int kThreads = 256;

template <typename T, int TILE, int NC>
__global__ void __launch_bounds__(kThreads) generic_fwd_kernel(const Problem p, const int ldq, const int ldv) {
  constexpr int R = TILE / 16;          // rows (and score columns) per thread
  constexpr int LDS = TILE + 1;
  constexpr int TPR = kThreads / TILE;  // threads cooperating on one softmax row
  extern __shared__ float smem[];
  float* Qs = smem;
  float* Ks = Qs + TILE * ldq;
  float* Vs = Ks + TILE * ldq;
  float* Ss = Vs + TILE * ldv;
  float* row_m = Ss + TILE * LDS;
  float* row_l = row_m + TILE;
  float* row_a = row_l + TILE;

  const T* __restrict__ q = reinterpret_cast<const T*>(p.q);
  const T* __restrict__ k = reinterpret_cast<const T*>(p.k);
  const T* __restrict__ v = reinterpret_cast<const T*>(p.v);
  T* __restrict__ out = reinterpret_cast<T*>(p.out);

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

  const int64_t q_base = b * p.qs[0] + h * p.qs[1];
  const int64_t k_base = b * p.ks[0] + hk * p.ks[1];
  const int64_t v_base = b * p.vs[0] + hk * p.vs[1];

  for (int idx = tid; idx < TILE * p.E; idx += kThreads) {
    const int r = idx / p.E, e = idx - r * p.E;
    const int gi = row0 + r;
    Qs[r * ldq + e] = gi < p.L ? to_f32<T>(q[q_base + gi * p.qs[2] + e * p.qs[3]]) : 0.f;
  }
  if (tid < TILE) {
    row_m[tid] = -CUDART_INF_F;
    row_l[tid] = 0.f;
    row_a[tid] = 0.f;
  }
  float acc[R][NC];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
  __syncthreads();

  for (int64_t j0 = 0; j0 < k_end; j0 += TILE) {
    for (int idx = tid; idx < TILE * p.E; idx += kThreads) {
      const int r = idx / p.E, e = idx - r * p.E;
      const int64_t gj = j0 + r;
      Ks[r * ldq + e] = gj < k_end ? to_f32<T>(k[k_base + gj * p.ks[2] + e * p.ks[3]]) : 0.f;
    }
    for (int idx = tid; idx < TILE * ldv; idx += kThreads) {
      const int r = idx / ldv, e = idx - r * ldv;
      const int64_t gj = j0 + r;
      Vs[idx] = (gj < k_end && e < p.Dv) ? to_f32<T>(v[v_base + gj * p.vs[2] + e * p.vs[3]]) : 0.f;
    }
    __syncthreads();

    float s[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < R; ++j) s[i][j] = 0.f;
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
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = ty * R + i;
      const int gi = row0 + r;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int c = tx + 16 * j;
        const int64_t gj = j0 + c;
        float val = s[i][j] * p.scale;
        bool visible = gi < p.L && gj < n_keys && (!p.causal || gj <= gi + p.causal_shift);
        if (visible && p.bias != nullptr) {
          val += load_as_f32(p.bias, b * p.bs[0] + h * p.bs[1] + gi * p.bs[2] + gj * p.bs[3], p.bias_dtype);
        }
        Ss[r * LDS + c] = visible ? val : -CUDART_INF_F;
      }
    }
    __syncthreads();

    {
      const int r = tid / TPR, sub = tid % TPR;
      const float m_old = row_m[r];
      float mx = -CUDART_INF_F;
      for (int c = sub; c < TILE; c += TPR) mx = fmaxf(mx, Ss[r * LDS + c]);
#pragma unroll
      for (int off = TPR / 2; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_old, mx);
      const float m_safe = (m_new == -CUDART_INF_F) ? 0.f : m_new;
      const float alpha = (m_old == -CUDART_INF_F) ? 0.f : expf(m_old - m_safe);
      float sum = 0.f;
      for (int c = sub; c < TILE; c += TPR) {
        const float pr = expf(Ss[r * LDS + c] - m_safe);
        Ss[r * LDS + c] = pr;
        sum += pr;
      }
#pragma unroll
      for (int off = TPR / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (sub == 0) {
        row_l[r] = row_l[r] * alpha + sum;
        row_m[r] = m_new;
        row_a[r] = alpha;
      }
    }
    __syncthreads();

#pragma unroll
    for (int i = 0; i < R; ++i) {
      const float a = row_a[ty * R + i];
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[i][c] *= a;
    }
#pragma unroll 2
    for (int kk = 0; kk < TILE; ++kk) {
      float pv[R];
#pragma unroll
      for (int i = 0; i < R; ++i) pv[i] = Ss[(ty * R + i) * LDS + kk];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const float vv = Vs[kk * ldv + tx + 16 * c];
#pragma unroll
        for (int i = 0; i < R; ++i) acc[i][c] = fmaf(pv[i], vv, acc[i][c]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = ty * R + i;
    const int gi = row0 + r;
    if (gi >= p.L) continue;
    const float l = row_l[r];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int64_t o_base = b * p.os[0] + h * p.os[1] + gi * p.os[2];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int col = tx + 16 * c;
      if (col < p.Dv && dbg_bhrc(p.status, DBG_GENERIC_FWD * 100 + 1, b, p.B, h, p.Hq, gi, p.L, col, 1, p.Dv))
        out[o_base + col * p.os[3]] = from_f32<T>(acc[i][c] * inv);
    }
    if (p.lse != nullptr && tx == 0 && dbg_bhrc(p.status, DBG_GENERIC_FWD * 100 + 2, b, p.B, h, p.Hq, gi, p.L, 0, 0, 1)) {
      const float m = row_m[r];
      p.lse[b * p.ls[0] + h * p.ls[1] + gi * p.ls[2]] = (m == -CUDART_INF_F) ? -CUDART_INF_F : m + logf(l);
    }
  }
}

struct GenericConfig {
  int tile, nc, ldq, ldv, smem;
};

bool pick_config(const Problem& p, GenericConfig* cfg) {
  if (p.E > 512 || p.Dv > 512) return false;
  int nc = (p.Dv + 15) / 16;
  nc = nc <= 4 ? 4 : nc <= 8 ? 8 : nc <= 16 ? 16 : 32;
  const int tile = (p.E <= 256 && nc <= 16) ? 64 : 32;
  cfg->tile = tile;
  cfg->nc = nc;
  cfg->ldq = p.E | 1;
  cfg->ldv = 16 * nc;
  cfg->smem = static_cast<int>(sizeof(float)) * (2 * tile * cfg->ldq + tile * cfg->ldv + tile * (tile + 1) + 3 * tile);
  return cfg->smem <= 227 * 1024;
}

template <typename T, int TILE, int NC>
int launch_one(const Problem& p, const GenericConfig& cfg, int64_t grid, cudaStream_t stream) {
  auto kern = generic_fwd_kernel<T, TILE, NC>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem) != cudaSuccess) {
    cudaGetLastError();
    return B200_SDPA_ERR_CUDA;
  }
  kern<<<static_cast<unsigned>(grid), kThreads, cfg.smem, stream>>>(p, cfg.ldq, cfg.ldv);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_GENERIC);
  return B200_SDPA_OK;
}

template <typename T>
int launch_typed(const Problem& p, const GenericConfig& cfg, int64_t grid, cudaStream_t stream) {
  if (cfg.tile == 64) {
    if (cfg.nc == 4) return launch_one<T, 64, 4>(p, cfg, grid, stream);
    if (cfg.nc == 8) return launch_one<T, 64, 8>(p, cfg, grid, stream);
    return launch_one<T, 64, 16>(p, cfg, grid, stream);
  }
  if (cfg.nc == 4) return launch_one<T, 32, 4>(p, cfg, grid, stream);
  if (cfg.nc == 8) return launch_one<T, 32, 8>(p, cfg, grid, stream);
  if (cfg.nc == 16) return launch_one<T, 32, 16>(p, cfg, grid, stream);
  return launch_one<T, 32, 32>(p, cfg, grid, stream);
}

}  // namespace

int plan_generic(const Problem& p, int dtype, B200SdpaPlan* plan) {
  (void)dtype;
  GenericConfig cfg;
  if (!pick_config(p, &cfg)) return B200_SDPA_ERR_UNSUPPORTED;
  const int64_t grid = static_cast<int64_t>((p.L + cfg.tile - 1) / cfg.tile) * p.Hq * p.B;
  if (grid > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  plan->path = B200_SDPA_PATH_GENERIC;
  plan->block_m = cfg.tile;
  plan->block_n = cfg.tile;
  plan->grid_x = static_cast<int32_t>(grid);
  plan->grid_y = plan->grid_z = 1;
  plan->threads = kThreads;
  plan->smem_bytes = cfg.smem;
  plan->kv_splits = 1;
  plan->launches = 1;
  plan->workspace_bytes = 0;
  return B200_SDPA_OK;
}

int launch_generic(const Problem& p, int dtype, cudaStream_t stream) {
  GenericConfig cfg;
  if (!pick_config(p, &cfg)) return B200_SDPA_ERR_UNSUPPORTED;
  const int64_t grid = static_cast<int64_t>((p.L + cfg.tile - 1) / cfg.tile) * p.Hq * p.B;
  if (grid > 0x7fffffffLL) return B200_SDPA_ERR_UNSUPPORTED;
  switch (dtype) {
    case B200_SDPA_F32: return launch_typed<float>(p, cfg, grid, stream);
    case B200_SDPA_F16: return launch_typed<__half>(p, cfg, grid, stream);
    case B200_SDPA_BF16: return launch_typed<__nv_bfloat16>(p, cfg, grid, stream);
    default: return B200_SDPA_ERR_DTYPE;
  }
}

}  // namespace b200
