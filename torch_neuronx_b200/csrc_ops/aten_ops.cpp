// C++ operator layer: the CUDA kernels of
//   aten::_scaled_dot_product_fused_attention_overrideable
//   aten::_scaled_dot_product_fused_attention_overrideable_backward
// registered with the dispatcher, so that a call from Python crosses into native code once and runs
// without the interpreter lock -- what upstream's native dispatcher does for this op
// (torch_neuronx/csrc/core/dispatch/NeuronDispatcher.cpp:2260-2364 DispatchSdpaCore, :2370-2517
// DispatchSdpaFwdImpl, :2523-2582 DispatchSdpaBwdImpl; the cache-hit path without the GIL :2897-2904).
// The layer validates (same rules and messages as :2380-2458 and python_ops/base.py:1036-1111), computes
// float64 inputs in float32 and casts back (:2418-2434, :2498-2501), allocates the outputs with the
// query's layout through the caching allocator (:2352, python_ops/scaled_dot_product_fused_attention.py:
// 357-358), fills the C-ABI parameter block and launches on the current stream.  There is no fallback:
// non-CUDA tensors are rejected and every launch goes through libb200_sdpa.so.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <algorithm>
#include <array>
#include <cmath>
#include <limits>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/b200_sdpa.h"

namespace {

constexpr int kMaxDevices = 64;

struct PerDevice {
  at::Tensor status;        // int32[4]: first device-side error seen by a kernel
  at::Tensor philox_seed;   // int32 scalar zeros (dropout is off)
  at::Tensor philox_offset;
};

std::once_flag g_once[kMaxDevices];
PerDevice g_dev[kMaxDevices];

// Created once per device, by whichever thread gets there first (calls arrive without the interpreter
// lock, so several threads may race here).
PerDevice& device_state(int dev) {
  TORCH_CHECK(dev >= 0 && dev < kMaxDevices, "b200_sdpa: device index out of range");
  PerDevice& d = g_dev[dev];
  std::call_once(g_once[dev], [&] {
    const auto opts = at::TensorOptions().device(at::kCUDA, dev).dtype(at::kInt);
    d.philox_seed = at::zeros({}, opts);
    d.philox_offset = at::zeros({}, opts);
    d.status = at::zeros({4}, opts);
  });
  return d;
}

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200_SDPA_F32;
    case at::kHalf: return B200_SDPA_F16;
    case at::kBFloat16: return B200_SDPA_BF16;
    default: return -1;
  }
}

// Scratch for one call: a fresh block from the caching allocator (stream-ordered, so the block can be
// reused by the next call on the same stream as soon as this one has been queued).
at::Tensor scratch(int dev, uint64_t bytes) {
  return at::empty({static_cast<int64_t>(bytes < 16 ? 16 : bytes)},
                   at::TensorOptions().device(at::kCUDA, dev).dtype(at::kByte));
}

void validate(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
              const c10::optional<at::Tensor>& attn_bias, double dropout_p, bool is_causal, bool return_debug_mask) {
  if (return_debug_mask)
    C10_THROW_ERROR(NotImplementedError,
                    "return_debug_mask=True is not supported: the fused kernel keeps no attention matrix");
  TORCH_CHECK(!(attn_bias.has_value() && attn_bias->defined() && is_causal),
              "_scaled_dot_product_fused_attention_overrideable: Explicit attn_mask should not be set when "
              "is_causal=True");
  TORCH_CHECK(query.device().type() == key.device().type() && key.device().type() == value.device().type(),
              "Expected query, key, and value to have the same device type");
  const auto dt = query.scalar_type();
  TORCH_CHECK(dt == at::kFloat || dt == at::kHalf || dt == at::kBFloat16 || dt == at::kDouble,
              "SDPA: query dtype must be float32, float16, or bfloat16, got ", dt);
  TORCH_CHECK(dt == key.scalar_type() && dt == value.scalar_type(),
              "Expected query, key, and value to have the same dtype");
  TORCH_CHECK(query.dim() == 4 && key.dim() == 4 && value.dim() == 4,
              "SDPA: query, key and value must be 4D tensors (B, H, S, D)");
  TORCH_CHECK(query.size(0) == key.size(0) && key.size(0) == value.size(0), "SDPA: batch sizes must match");
  TORCH_CHECK(key.size(1) == value.size(1), "SDPA: key and value must have the same number of heads");
  TORCH_CHECK(key.size(2) == value.size(2), "SDPA: key and value must have the same sequence length");
  TORCH_CHECK(query.size(3) == key.size(3), "SDPA: query and key must have the same embedding dimension");
  TORCH_CHECK(key.size(1) != 0 && query.size(1) % key.size(1) == 0,
              "SDPA: Number of heads in key and value must divide the number of heads in query");
  if (dropout_p < 0.0 || dropout_p > 1.0)
    C10_THROW_ERROR(ValueError, "dropout_p=" + std::to_string(dropout_p) + " is outside [0, 1]. Pass a value in [0, 1].");
  if (dropout_p != 0.0)
    C10_THROW_ERROR(NotImplementedError, "dropout_p != 0 is not supported by the B200 fused attention path");
  if (!query.is_cuda()) C10_THROW_ERROR(ValueError, "Expected CUDA device, got " + query.device().str());
  TORCH_CHECK(query.device() == key.device() && key.device() == value.device(),
              "Expected query, key, and value to be on the same device");
}

// Output buffer laid out like the query: identical strides when the shapes agree, otherwise dense strides
// in the query's dimension order (the rule of torch's own meta kernel for this op).
at::Tensor alloc_like_query(const at::Tensor& query, std::array<int64_t, 4> shape) {
  if (query.sizes() == at::IntArrayRef(shape.data(), 4)) return at::empty_like(query);
  std::array<int, 4> order = {0, 1, 2, 3};
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return query.stride(a) > query.stride(b); });
  std::array<int64_t, 4> permuted, back;
  for (int i = 0; i < 4; ++i) permuted[i] = shape[order[i]];
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j)
      if (order[j] == i) back[i] = j;
  return at::empty(at::IntArrayRef(permuted.data(), 4), query.options()).permute(at::IntArrayRef(back.data(), 4));
}

// Strides of `bias` viewed as broadcast to (B, Hq, L, S): 0 where broadcast.
void bias_strides(const at::Tensor& bias, const std::array<int64_t, 4>& target, int64_t* out) {
  TORCH_CHECK(bias.dim() <= 4, "attn_mask must have at most 4 dimensions");
  const int pad = 4 - static_cast<int>(bias.dim());
  for (int i = 0; i < 4; ++i) {
    const int64_t s = i < pad ? 1 : bias.size(i - pad);
    const int64_t st = i < pad ? 0 : bias.stride(i - pad);
    if (s == target[i]) {
      out[i] = s != 1 ? st : 0;
    } else {
      TORCH_CHECK(s == 1, "attn_mask of shape ", bias.sizes(), " is not broadcastable to (", target[0], ", ", target[1],
                  ", ", target[2], ", ", target[3], ")");
      out[i] = 0;
    }
  }
}

template <size_t N> void copy_strides(const at::Tensor& t, int64_t (&dst)[N]) {
  for (size_t i = 0; i < N; ++i) dst[i] = t.stride(static_cast<int64_t>(i));
}

// bool mask (true = keep) -> 0 / -inf in the query dtype; float masks as they are; other float widths -> fp32
at::Tensor additive_bias(const at::Tensor& mask, const at::Tensor& query) {
  if (mask.scalar_type() == at::kBool) {
    return at::where(mask, at::zeros({}, query.options().dtype(at::kFloat)),
                     at::full({}, -std::numeric_limits<float>::infinity(), query.options().dtype(at::kFloat)))
        .to(query.scalar_type());
  }
  if (dtype_code(mask.scalar_type()) < 0) return mask.to(at::kFloat);
  return mask;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor, at::Tensor, at::Tensor>
fused_attention_overrideable(const at::Tensor& query_in, const at::Tensor& key_in, const at::Tensor& value_in,
                             const c10::optional<at::Tensor>& attn_bias, double dropout_p, bool is_causal,
                             bool return_debug_mask, c10::optional<double> scale) {
  validate(query_in, key_in, value_in, attn_bias, dropout_p, is_causal, return_debug_mask);
  TORCH_CHECK(query_in.numel() != 0 && key_in.size(3) != 0 && value_in.size(3) != 0,
              "SDPA: zero-size inputs are not routed to the fused kernel");
  const bool f64 = query_in.scalar_type() == at::kDouble;
  const at::Tensor query = f64 ? query_in.to(at::kFloat) : query_in;
  const at::Tensor key = f64 ? key_in.to(at::kFloat) : key_in;
  const at::Tensor value = f64 ? value_in.to(at::kFloat) : value_in;
  const c10::cuda::CUDAGuard guard(query.device());
  const int dev = query.device().index();
  PerDevice& st = device_state(dev);

  const int64_t B = query.size(0), Hq = query.size(1), L = query.size(2), E = query.size(3);
  const int64_t Hkv = key.size(1), S = key.size(2), Dv = value.size(3);
  at::Tensor out = alloc_like_query(query, {B, Hq, L, Dv});
  at::Tensor lse = at::empty({B, Hq, L}, query.options().dtype(at::kFloat));

  B200SdpaParams p{};
  p.struct_size = sizeof(B200SdpaParams);
  p.dtype = dtype_code(query.scalar_type());
  p.device = dev;
  p.force_path = B200_SDPA_PATH_AUTO;
  p.q = query.data_ptr();
  p.k = key.data_ptr();
  p.v = value.data_ptr();
  p.out = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  copy_strides(query, p.q_stride);
  copy_strides(key, p.k_stride);
  copy_strides(value, p.v_stride);
  copy_strides(out, p.out_stride);
  copy_strides(lse, p.lse_stride);
  p.B = static_cast<int32_t>(B);
  p.Hq = static_cast<int32_t>(Hq);
  p.Hkv = static_cast<int32_t>(Hkv);
  p.L = static_cast<int32_t>(L);
  p.S = static_cast<int32_t>(S);
  p.E = static_cast<int32_t>(E);
  p.Dv = static_cast<int32_t>(Dv);
  p.scale = static_cast<float>(scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(E)));
  p.is_causal = is_causal ? 1 : 0;
  at::Tensor bias;   // keeps a converted mask alive until the launch is queued
  if (attn_bias.has_value() && attn_bias->defined()) {
    bias = additive_bias(f64 && attn_bias->scalar_type() == at::kDouble ? attn_bias->to(at::kFloat) : *attn_bias, query);
    p.bias = bias.data_ptr();
    p.bias_dtype = dtype_code(bias.scalar_type());
    bias_strides(bias, {B, Hq, L, S}, p.bias_stride);
  }
  p.status = st.status.data_ptr<int32_t>();

  B200SdpaPlan plan{};
  plan.struct_size = sizeof(B200SdpaPlan);
  int rc = b200_sdpa_query_plan(&p, &plan);
  TORCH_CHECK(rc == B200_SDPA_OK, "b200_sdpa_query_plan: ", b200_sdpa_strerror(rc));
  at::Tensor ws;
  if (plan.workspace_bytes != 0) {
    ws = scratch(dev, plan.workspace_bytes);
    p.workspace = ws.data_ptr();
    p.workspace_bytes = static_cast<uint64_t>(ws.numel());
  }
  rc = b200_sdpa_fwd(&p, c10::cuda::getCurrentCUDAStream(dev).stream());
  TORCH_CHECK(rc == B200_SDPA_OK, "b200_sdpa_fwd: ", b200_sdpa_strerror(rc));
  if (f64) out = out.to(at::kDouble);
  return std::make_tuple(out, lse, at::Tensor(), at::Tensor(), c10::SymInt(L), c10::SymInt(S), st.philox_seed,
                         st.philox_offset, at::Tensor());
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> fused_attention_overrideable_backward(
    const at::Tensor& grad_out_in, const at::Tensor& query_in, const at::Tensor& key_in, const at::Tensor& value_in,
    const at::Tensor& attn_bias, std::array<bool, 4> grad_input_mask, const at::Tensor& out_in,
    const at::Tensor& logsumexp, const at::Tensor& /*cum_seq_q*/, const at::Tensor& /*cum_seq_k*/,
    c10::SymInt /*max_q*/, c10::SymInt /*max_k*/, double dropout_p, bool is_causal, const at::Tensor& /*philox_seed*/,
    const at::Tensor& /*philox_offset*/, c10::optional<double> scale) {
  if (!query_in.is_cuda()) C10_THROW_ERROR(ValueError, "Expected CUDA device, got " + query_in.device().str());
  TORCH_CHECK(key_in.size(1) != 0 && query_in.size(1) % key_in.size(1) == 0,
              "SDPA: Number of heads in key and value must divide the number of heads in query");
  if (dropout_p != 0.0)
    C10_THROW_ERROR(NotImplementedError, "dropout_p != 0 is not supported by the B200 fused attention path");
  const bool f64 = query_in.scalar_type() == at::kDouble;
  auto f32 = [&](const at::Tensor& t) { return f64 ? t.to(at::kFloat) : t; };
  at::Tensor grad_out = f32(grad_out_in);
  const at::Tensor query = f32(query_in), key = f32(key_in), value = f32(value_in), out = f32(out_in);
  const c10::cuda::CUDAGuard guard(query.device());
  const int dev = query.device().index();
  PerDevice& st = device_state(dev);

  const int64_t B = query.size(0), Hq = query.size(1), L = query.size(2), E = query.size(3);
  const int64_t Hkv = key.size(1), S = key.size(2), Dv = value.size(3);
  TORCH_CHECK(grad_out.sizes() == at::IntArrayRef({B, Hq, L, Dv}) && out.sizes() == at::IntArrayRef({B, Hq, L, Dv}),
              "SDPA backward: grad_out and out must have shape (B, Hq, L, Dv)");
  TORCH_CHECK(grad_out.scalar_type() == query.scalar_type() && out.scalar_type() == query.scalar_type(),
              "SDPA backward: grad_out and out must have the dtype of query");
  TORCH_CHECK(logsumexp.scalar_type() == at::kFloat && logsumexp.sizes() == at::IntArrayRef({B, Hq, L}),
              "SDPA backward: logsumexp must be a float32 tensor of shape (B, Hq, L)");
  // only an undefined or empty tensor means "no bias" (python_ops/scaled_dot_product_fused_attention.py:178)
  const bool has_bias = attn_bias.defined() && attn_bias.numel() != 0;
  const bool want_bias_grad = has_bias && grad_input_mask[3];
  // e.g. the expanded gradient of a reduction: stride 0 everywhere
  const int64_t es = grad_out.element_size();
  if (grad_out.stride(3) != 1 || (grad_out.stride(0) * es) % 16 != 0 || (grad_out.stride(1) * es) % 16 != 0 ||
      (grad_out.stride(2) * es) % 16 != 0)
    grad_out = grad_out.contiguous();
  at::Tensor gq = at::empty_like(query), gk = at::empty_like(key), gv = at::empty_like(value), gb;
  if (want_bias_grad) gb = at::empty({B, Hq, L, S}, query.options());

  B200SdpaBwdParams p{};
  p.struct_size = sizeof(B200SdpaBwdParams);
  p.dtype = dtype_code(query.scalar_type());
  p.device = dev;
  p.force_path = B200_SDPA_PATH_AUTO;
  p.grad_out = grad_out.data_ptr();
  p.q = query.data_ptr();
  p.k = key.data_ptr();
  p.v = value.data_ptr();
  p.out = out.data_ptr();
  p.lse = logsumexp.data_ptr<float>();
  p.grad_q = gq.data_ptr();
  p.grad_k = gk.data_ptr();
  p.grad_v = gv.data_ptr();
  copy_strides(grad_out, p.grad_out_stride);
  copy_strides(query, p.q_stride);
  copy_strides(key, p.k_stride);
  copy_strides(value, p.v_stride);
  copy_strides(out, p.out_stride);
  copy_strides(logsumexp, p.lse_stride);
  copy_strides(gq, p.grad_q_stride);
  copy_strides(gk, p.grad_k_stride);
  copy_strides(gv, p.grad_v_stride);
  if (gb.defined()) {
    p.grad_bias = gb.data_ptr();
    copy_strides(gb, p.grad_bias_stride);
  }
  p.B = static_cast<int32_t>(B);
  p.Hq = static_cast<int32_t>(Hq);
  p.Hkv = static_cast<int32_t>(Hkv);
  p.L = static_cast<int32_t>(L);
  p.S = static_cast<int32_t>(S);
  p.E = static_cast<int32_t>(E);
  p.Dv = static_cast<int32_t>(Dv);
  p.scale = static_cast<float>(scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(E)));
  p.is_causal = is_causal ? 1 : 0;
  at::Tensor bias;
  if (has_bias) {
    bias = dtype_code(attn_bias.scalar_type()) < 0 ? attn_bias.to(at::kFloat) : attn_bias;
    p.bias = bias.data_ptr();
    p.bias_dtype = dtype_code(bias.scalar_type());
    bias_strides(bias, {B, Hq, L, S}, p.bias_stride);
  }
  p.status = st.status.data_ptr<int32_t>();

  B200SdpaPlan plan{};
  plan.struct_size = sizeof(B200SdpaPlan);
  int rc = b200_sdpa_bwd_query_plan(&p, &plan);
  TORCH_CHECK(rc == B200_SDPA_OK, "b200_sdpa_bwd_query_plan: ", b200_sdpa_strerror(rc));
  at::Tensor ws;
  if (plan.workspace_bytes != 0) {
    ws = scratch(dev, plan.workspace_bytes);
    p.workspace = ws.data_ptr();
    p.workspace_bytes = static_cast<uint64_t>(ws.numel());
  }
  rc = b200_sdpa_bwd(&p, c10::cuda::getCurrentCUDAStream(dev).stream());
  TORCH_CHECK(rc == B200_SDPA_OK, "b200_sdpa_bwd: ", b200_sdpa_strerror(rc));
  if (f64) {
    gq = gq.to(at::kDouble);
    gk = gk.to(at::kDouble);
    gv = gv.to(at::kDouble);
    if (gb.defined()) gb = gb.to(at::kDouble);
  }
  return std::make_tuple(gq, gk, gv, gb);
}

// The status word of a device (int32[4] on that device), shared with the Python layer so that both
// report device-side errors through the same place.
at::Tensor status_word(int64_t device) { return device_state(static_cast<int>(device)).status; }

}  // namespace

TORCH_LIBRARY_IMPL(aten, CUDA, m) {
  m.impl("_scaled_dot_product_fused_attention_overrideable", &fused_attention_overrideable);
  m.impl("_scaled_dot_product_fused_attention_overrideable_backward", &fused_attention_overrideable_backward);
}

TORCH_LIBRARY(b200_sdpa_native, m) {
  m.def("status_word(int device) -> Tensor", &status_word);
}
