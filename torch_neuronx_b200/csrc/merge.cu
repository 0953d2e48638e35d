// Merge of two partial attention results over disjoint key sets (one ring
// step), fp32 running accumulator.  Pure streaming work: one thread per four
// output elements, one log-sum-exp update per row.
#include "common.cuh"

namespace b200 {

namespace {

template <typename T>
__global__ void __launch_bounds__(256) merge_kernel(const B200SdpaMergeParams m, const int64_t rows) {
  const int vec_per_row = (m.Dv + 3) / 4;
  const int64_t total = rows * vec_per_row;
  const T* __restrict__ part = reinterpret_cast<const T*>(m.part);
  T* __restrict__ fin = reinterpret_cast<T*>(m.final_out);
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = idx / vec_per_row;
    const int c0 = static_cast<int>(idx - row * vec_per_row) * 4;
    const int i = static_cast<int>(row % m.L);
    const int h = static_cast<int>((row / m.L) % m.Hq);
    const int b = static_cast<int>(row / (static_cast<int64_t>(m.L) * m.Hq));
    const float lb = m.part_lse[b * m.part_lse_stride[0] + h * m.part_lse_stride[1] + i * m.part_lse_stride[2]];
    const int64_t abase = b * m.acc_stride[0] + h * m.acc_stride[1] + i * m.acc_stride[2];
    float wa, wb, lnew;
    if (m.first) {
      wa = 0.f;
      wb = 1.f;
      lnew = lb;
    } else {
      const float la = m.acc_lse[b * m.acc_lse_stride[0] + h * m.acc_lse_stride[1] + i * m.acc_lse_stride[2]];
      const float mx = fmaxf(la, lb);
      if (mx == -CUDART_INF_F) {
        wa = wb = 0.f;
        lnew = -CUDART_INF_F;
      } else {
        const float ea = expf(la - mx), eb = expf(lb - mx);
        lnew = mx + logf(ea + eb);
        wa = expf(la - lnew);
        wb = expf(lb - lnew);
      }
    }
    const int64_t pbase = b * m.part_stride[0] + h * m.part_stride[1] + i * m.part_stride[2];
    const int64_t fbase = b * m.final_stride[0] + h * m.final_stride[1] + i * m.final_stride[2];
#pragma unroll
    for (int c = c0; c < c0 + 4; ++c) {
      if (c >= m.Dv) break;
      const float pv = to_f32<T>(part[pbase + c * m.part_stride[3]]);
      const float av = m.first ? 0.f : m.acc[abase + c];
      const float r = av * wa + pv * wb;
      m.acc[abase + c] = r;
      if (fin != nullptr) fin[fbase + c * m.final_stride[3]] = from_f32<T>(r);
    }
    // acc_lse is only read here: several threads share a row, so the new
    // value is written by a second kernel once every reader is done.
  }
}

// Second pass: update acc_lse (stream order guarantees the first pass is done).
__global__ void __launch_bounds__(256) merge_lse_kernel(const B200SdpaMergeParams m, const int64_t rows) {
  for (int64_t row = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; row < rows;
       row += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(row % m.L);
    const int h = static_cast<int>((row / m.L) % m.Hq);
    const int b = static_cast<int>(row / (static_cast<int64_t>(m.L) * m.Hq));
    const float lb = m.part_lse[b * m.part_lse_stride[0] + h * m.part_lse_stride[1] + i * m.part_lse_stride[2]];
    float* al = m.acc_lse + b * m.acc_lse_stride[0] + h * m.acc_lse_stride[1] + i * m.acc_lse_stride[2];
    if (m.first) {
      *al = lb;
    } else {
      const float la = *al;
      const float mx = fmaxf(la, lb);
      *al = (mx == -CUDART_INF_F) ? -CUDART_INF_F : mx + logf(expf(la - mx) + expf(lb - mx));
    }
  }
}

template <typename T>
int launch_t(const B200SdpaMergeParams& m, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(m.B) * m.Hq * m.L;
  if (rows == 0 || m.Dv == 0) return B200_SDPA_OK;
  const int64_t total = rows * ((m.Dv + 3) / 4);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  merge_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(m, rows);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  int64_t lblocks = (rows + 255) / 256;
  if (lblocks > 148 * 16) lblocks = 148 * 16;
  merge_lse_kernel<<<static_cast<unsigned>(lblocks), 256, 0, stream>>>(m, rows);
  if (cudaGetLastError() != cudaSuccess) return B200_SDPA_ERR_CUDA;
  count_launch(KID_MERGE);
  return B200_SDPA_OK;
}

}  // namespace

int launch_merge(const B200SdpaMergeParams& m, cudaStream_t stream) {
  switch (m.dtype) {
    case B200_SDPA_F32: return launch_t<float>(m, stream);
    case B200_SDPA_F16: return launch_t<__half>(m, stream);
    case B200_SDPA_BF16: return launch_t<__nv_bfloat16>(m, stream);
    default: return B200_SDPA_ERR_DTYPE;
  }
}

}  // namespace b200
