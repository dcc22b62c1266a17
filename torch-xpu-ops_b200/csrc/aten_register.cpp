// ATen dispatcher registration: the CUDA-key kernels of the row-wise normalization / softmax
// operator family, re-implemented on top of the b200norm C ABI.  This file plays the role of
// intel/torch-xpu-ops' host wrappers (src/ATen/native/xpu/LayerNorm.cpp, SoftMax.cpp, LossNLL.cpp):
// argument checks, contiguity, output allocation, stat reshaping — no device code.  Loading the
// shared object replaces PyTorch's own CUDA kernels for exactly these operators; the ATen schemas
// are untouched, so autograd formulas and every caller keep working.
//
// There is no fallback: a non-zero status from the C ABI becomes a c10::Error.
#include <limits>
#include <ATen/ATen.h>
#include <ATen/AccumulateType.h>
#include <ATen/ExpandUtils.h>
#include <ATen/WrapDimUtils.h>
#include <ATen/native/Resize.h>
#include <ATen/native/layer_norm.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/autograd.h>
#include <torch/library.h>
#include <ATen/ops/cross_entropy_loss_native.h>

#include <array>
#include <tuple>
#include <vector>

#include "b200norm.h"

namespace b200norm {

using at::Tensor;

static int to_b2n_dtype(at::ScalarType t, const char* what) {
  switch (t) {
    case at::kFloat: return B2N_F32;
    case at::kHalf: return B2N_F16;
    case at::kBFloat16: return B2N_BF16;
    case at::kDouble: return B2N_F64;
    default: TORCH_CHECK(false, "b200norm: ", what, ": unsupported dtype ", t);
  }
}

// What a kernel could not report by trapping — an nll_loss target outside [0, C), a bounded wait that
// gave up — sits in the library's device status word.  The operators that can set it enqueue a
// non-blocking copy of the word behind their kernels (note_possible_device_failure); every later
// operator call on that device looks at the copy once it has arrived and raises.  So the error
// reaches the caller without any synchronisation on the hot path, one call late — the same way a
// CUDA launch failure does.  The reference fails in the kernel instead (SYCL_KERNEL_ASSERT,
// src/ATen/native/xpu/sycl/LossNLLKernel.cpp:30-35).
static void raise_if_earlier_kernel_failed() {
  const int st = b2n_status_poll();
  TORCH_CHECK(st == B2N_OK, "b200norm: an earlier kernel on this device reported: ", b2n_strerror(st),
              st == B2N_ERR_TARGET_RANGE ? " (nll_loss / cross_entropy: a target is outside [0, n_classes) and is not ignore_index; that row contributed nothing)" : "",
              st == B2N_ERR_TIMEOUT ? " (the kernel left early: its output is incomplete)" : "");
}

static void check_status(int st, const char* op) {
  TORCH_CHECK(st == B2N_OK, "b200norm::", op, " failed: ", b2n_strerror(st),
              st == B2N_ERR_CUDA ? " (cudaError " : "", st == B2N_ERR_CUDA ? std::to_string(b2n_last_cuda_error()) : "",
              st == B2N_ERR_CUDA ? ")" : "");
  raise_if_earlier_kernel_failed();
}

static void* cur_stream() { return static_cast<void*>(c10::cuda::getCurrentCUDAStream().stream()); }

static void note_possible_device_failure() { b2n_status_post(cur_stream()); }

static at::ScalarType acc_type_of(at::ScalarType t) { return t == at::kDouble ? at::kDouble : at::kFloat; }

static std::vector<int64_t> stat_shape_of(const Tensor& input, size_t normalized_ndim) {
  // input.shape[:axis] + [1] * normalized_ndim  (LayerNorm.cpp:82-94 of the reference)
  const size_t axis = input.dim() - normalized_ndim;
  std::vector<int64_t> shape;
  for (size_t i = 0; i < axis; ++i) shape.push_back(input.size(i));
  for (size_t i = axis; i < static_cast<size_t>(input.dim()); ++i) shape.push_back(1);
  return shape;
}

static int weight_dtype(const Tensor& input, const Tensor& weight, const Tensor& bias, const char* op) {
  if (weight.defined() && bias.defined()) {
    TORCH_CHECK(weight.scalar_type() == bias.scalar_type(), op, ": weight and bias must have the same dtype");
  }
  const Tensor& w = weight.defined() ? weight : bias;
  if (!w.defined()) return to_b2n_dtype(input.scalar_type(), op);
  TORCH_CHECK(w.scalar_type() == input.scalar_type() || w.scalar_type() == at::kFloat, op,
              ": weight dtype must equal the input dtype or be float32, got ", w.scalar_type(), " for input ",
              input.scalar_type());
  return to_b2n_dtype(w.scalar_type(), op);
}

// ---- native_layer_norm ---------------------------------------------------------------------------
std::tuple<Tensor, Tensor, Tensor> native_layer_norm(const Tensor& input, at::IntArrayRef normalized_shape,
                                                     const std::optional<Tensor>& weight_opt,
                                                     const std::optional<Tensor>& bias_opt, double eps) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  c10::MaybeOwned<Tensor> bias_mo = at::borrow_from_optional_tensor(bias_opt);
  const Tensor& weight = *weight_mo;
  const Tensor& bias = *bias_mo;
  TORCH_CHECK(input.is_cuda(), "native_layer_norm: expected a CUDA tensor");
  TORCH_CHECK(!weight.defined() || weight.device() == input.device(), "native_layer_norm: weight on another device");
  TORCH_CHECK(!bias.defined() || bias.device() == input.device(), "native_layer_norm: bias on another device");
  const c10::cuda::CUDAGuard guard(input.device());

  auto M_N = at::native::_check_layer_norm_inputs(input, normalized_shape, weight, bias);
  const int64_t M = M_N.first, N = M_N.second;
  auto X = input.expect_contiguous();
  auto gamma = weight.expect_contiguous();
  auto beta = bias.expect_contiguous();

  Tensor Y = at::empty_like(*X, at::MemoryFormat::Contiguous);
  const auto acc = acc_type_of(input.scalar_type());
  Tensor mean = at::empty({M}, X->options().dtype(acc));
  Tensor rstd = at::empty({M}, X->options().dtype(acc));
  if (M > 0) {
    const int xdt = to_b2n_dtype(input.scalar_type(), "native_layer_norm");
    const int wdt = weight_dtype(input, weight, bias, "native_layer_norm");
    check_status(b2n_layer_norm_fwd(X->const_data_ptr(), gamma->defined() ? gamma->const_data_ptr() : nullptr,
                                    beta->defined() ? beta->const_data_ptr() : nullptr, Y.mutable_data_ptr(),
                                    mean.mutable_data_ptr(), rstd.mutable_data_ptr(), M, N, eps, xdt, wdt,
                                    cur_stream()),
                 "layer_norm_fwd");
  }
  const auto stat_shape = stat_shape_of(input, normalized_shape.size());
  return std::make_tuple(std::move(Y), mean.view(stat_shape), rstd.view(stat_shape));
}

std::tuple<Tensor, Tensor, Tensor> native_layer_norm_backward(
    const Tensor& grad_out, const Tensor& input, at::IntArrayRef normalized_shape, const Tensor& mean,
    const Tensor& rstd, const std::optional<Tensor>& weight_opt, const std::optional<Tensor>& bias_opt,
    std::array<bool, 3> mask) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  c10::MaybeOwned<Tensor> bias_mo = at::borrow_from_optional_tensor(bias_opt);
  const Tensor& weight = *weight_mo;
  const Tensor& bias = *bias_mo;
  TORCH_CHECK(input.is_cuda() && grad_out.is_cuda(), "native_layer_norm_backward: expected CUDA tensors");
  const c10::cuda::CUDAGuard guard(input.device());

  auto M_N = at::native::_check_layer_norm_inputs(input, normalized_shape, weight, bias);
  const int64_t M = M_N.first, N = M_N.second;
  auto X = input.expect_contiguous();
  auto gamma = weight.expect_contiguous();
  auto beta = bias.expect_contiguous();
  Tensor dY = grad_out.contiguous();
  TORCH_CHECK(dY.scalar_type() == X->scalar_type(), "native_layer_norm_backward: grad_out dtype ", dY.scalar_type(),
              " does not match input dtype ", X->scalar_type());
  const auto acc = acc_type_of(input.scalar_type());
  Tensor mean_c = mean.to(acc).contiguous();
  Tensor rstd_c = rstd.to(acc).contiguous();

  Tensor dX, dgamma, dbeta;
  if (mask[0]) dX = at::empty_like(*X, at::MemoryFormat::Contiguous);
  // a gradient for an absent weight/bias is returned as an undefined tensor when it is not asked
  // for, and with the weight's shape (zeros when M == 0) when it is — LayerNorm.cpp:150-181
  if (mask[1] && gamma->defined()) dgamma = M > 0 ? at::empty_like(*gamma, at::MemoryFormat::Contiguous)
                              : at::zeros_like(*gamma, at::MemoryFormat::Contiguous);
  if (mask[2] && beta->defined()) dbeta = M > 0 ? at::empty_like(*beta, at::MemoryFormat::Contiguous)
                             : at::zeros_like(*beta, at::MemoryFormat::Contiguous);
  if (M > 0 && N > 0) {
    const int xdt = to_b2n_dtype(input.scalar_type(), "native_layer_norm_backward");
    const int wdt = weight_dtype(input, weight, bias, "native_layer_norm_backward");
    const bool want_w = dgamma.defined() || dbeta.defined();
    const size_t ws_bytes = b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, want_w);
    Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, X->options().dtype(at::kByte));
    check_status(b2n_layer_norm_bwd(dY.const_data_ptr(), X->const_data_ptr(), mean_c.const_data_ptr(),
                                    rstd_c.const_data_ptr(), gamma->defined() ? gamma->const_data_ptr() : nullptr,
                                    dX.defined() ? dX.mutable_data_ptr() : nullptr,
                                    dgamma.defined() ? dgamma.mutable_data_ptr() : nullptr,
                                    dbeta.defined() ? dbeta.mutable_data_ptr() : nullptr,
                                    ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, M, N, xdt, wdt, cur_stream()),
                 "layer_norm_bwd");
  }
  return std::make_tuple(std::move(dX), std::move(dgamma), std::move(dbeta));
}

// ---- _fused_rms_norm -----------------------------------------------------------------------------
std::tuple<Tensor, Tensor> fused_rms_norm(const Tensor& input, at::IntArrayRef normalized_shape,
                                          const std::optional<Tensor>& weight_opt, std::optional<double> eps_opt) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  TORCH_CHECK(input.is_cuda(), "_fused_rms_norm: expected a CUDA tensor");
  const c10::cuda::CUDAGuard guard(input.device());
  auto M_N = at::native::_check_layer_norm_inputs(input, normalized_shape, weight, weight);
  const int64_t M = M_N.first, N = M_N.second;
  auto X = input.expect_contiguous();
  auto gamma = weight.expect_contiguous();
  const auto acc = acc_type_of(input.scalar_type());
  // default eps = machine epsilon of the accumulate type (LayerNorm.cpp:218-224)
  const double eps = eps_opt.value_or(acc == at::kFloat ? static_cast<double>(std::numeric_limits<float>::epsilon())
                                                        : std::numeric_limits<double>::epsilon());
  Tensor Y = at::empty_like(*X, at::MemoryFormat::Contiguous);
  Tensor rstd = at::empty({M}, X->options().dtype(acc));
  if (M > 0) {
    const int xdt = to_b2n_dtype(input.scalar_type(), "_fused_rms_norm");
    const int wdt = weight_dtype(input, weight, Tensor(), "_fused_rms_norm");
    check_status(b2n_rms_norm_fwd(X->const_data_ptr(), gamma->defined() ? gamma->const_data_ptr() : nullptr,
                                  Y.mutable_data_ptr(), rstd.mutable_data_ptr(), M, N, eps, xdt, wdt, cur_stream()),
                 "rms_norm_fwd");
  }
  return std::make_tuple(std::move(Y), rstd.view(stat_shape_of(input, normalized_shape.size())));
}

std::tuple<Tensor, Tensor> fused_rms_norm_backward(const Tensor& grad_out, const Tensor& input,
                                                   at::IntArrayRef normalized_shape, const Tensor& rstd,
                                                   const std::optional<Tensor>& weight_opt, std::array<bool, 2> mask) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  TORCH_CHECK(input.is_cuda() && grad_out.is_cuda(), "_fused_rms_norm_backward: expected CUDA tensors");
  const c10::cuda::CUDAGuard guard(input.device());
  auto M_N = at::native::_check_layer_norm_inputs(input, normalized_shape, weight, weight);
  const int64_t M = M_N.first, N = M_N.second;
  auto X = input.expect_contiguous();
  auto gamma = weight.expect_contiguous();
  Tensor dY = grad_out.contiguous();
  TORCH_CHECK(dY.scalar_type() == X->scalar_type(), "_fused_rms_norm_backward: grad_out dtype ", dY.scalar_type(),
              " does not match input dtype ", X->scalar_type());
  Tensor rstd_c = rstd.to(acc_type_of(input.scalar_type())).contiguous();
  Tensor dX, dgamma;
  if (mask[0]) dX = at::empty_like(*X, at::MemoryFormat::Contiguous);
  if (mask[1] && gamma->defined()) dgamma = M > 0 ? at::empty_like(*gamma, at::MemoryFormat::Contiguous)
                              : at::zeros_like(*gamma, at::MemoryFormat::Contiguous);
  if (M > 0 && N > 0) {
    const int xdt = to_b2n_dtype(input.scalar_type(), "_fused_rms_norm_backward");
    const int wdt = weight_dtype(input, weight, Tensor(), "_fused_rms_norm_backward");
    const size_t ws_bytes = b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, dgamma.defined());
    Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, X->options().dtype(at::kByte));
    check_status(b2n_rms_norm_bwd(dY.const_data_ptr(), X->const_data_ptr(), rstd_c.const_data_ptr(),
                                  gamma->defined() ? gamma->const_data_ptr() : nullptr,
                                  dX.defined() ? dX.mutable_data_ptr() : nullptr,
                                  dgamma.defined() ? dgamma.mutable_data_ptr() : nullptr,
                                  ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, M, N, xdt, wdt, cur_stream()),
                 "rms_norm_bwd");
  }
  return std::make_tuple(std::move(dX), std::move(dgamma));
}

// ---- native_group_norm, batch_norm_stats, batch_norm_update_stats ----------------------------------
// Host wrapper of upstream's native_group_norm (aten/src/ATen/native/group_norm.cpp) around the kernel the
// reference registers for its GroupNormKernel stub (src/ATen/native/xpu/GroupNorm.cpp:20): same checks, the
// statistics in the weights' dtype when the input is 16-bit and the weights are float (mixed type), else the input's.
std::tuple<Tensor, Tensor, Tensor> native_group_norm(const Tensor& input, const std::optional<Tensor>& weight_opt,
                                                     const std::optional<Tensor>& bias_opt, int64_t N, int64_t C,
                                                     int64_t HxW, int64_t group, double eps) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  c10::MaybeOwned<Tensor> bias_mo = at::borrow_from_optional_tensor(bias_opt);
  const Tensor& weight = *weight_mo;
  const Tensor& bias = *bias_mo;
  const char* op = "native_group_norm";
  TORCH_CHECK(input.is_cuda(), op, ": expected a CUDA tensor");
  TORCH_CHECK(group > 0, "Expected num groups to be greater than 0, got ", group);
  TORCH_CHECK(C % group == 0, "Expected number of channels in input to be divisible by num_groups, but got input of shape ",
              input.sizes(), " and num_groups=", group);
  TORCH_CHECK(!weight.defined() || (weight.dim() == 1 && weight.numel() == C),
              "Expected weight to be a vector of size equal to the number of channels in input, but got weight of shape ",
              weight.sizes(), " and input of shape ", input.sizes());
  TORCH_CHECK(!bias.defined() || (bias.dim() == 1 && bias.numel() == C),
              "Expected bias to be a vector of size equal to the number of channels in input, but got bias of shape ",
              bias.sizes(), " and input of shape ", input.sizes());
  TORCH_CHECK(input.numel() == N * C * HxW, op, ": input has ", input.numel(), " elements, expected N*C*HxW = ", N * C * HxW);
  const c10::cuda::CUDAGuard guard(input.device());
  Tensor X = input.contiguous();
  auto gamma = weight.expect_contiguous();
  auto beta = bias.expect_contiguous();
  const int xdt = to_b2n_dtype(X.scalar_type(), op);
  const int wdt = weight_dtype(X, weight, bias, op);
  const bool mixed = wdt == B2N_F32 && xdt != B2N_F32 && (weight.defined() || bias.defined());
  const auto stat_type = mixed ? at::kFloat : X.scalar_type();
  Tensor Y = at::empty_like(X, at::MemoryFormat::Contiguous);
  Tensor mean = at::empty({N, group}, X.options().dtype(stat_type));
  Tensor rstd = at::empty({N, group}, X.options().dtype(stat_type));
  if (X.numel() > 0) {
    check_status(b2n_group_norm_fwd(X.const_data_ptr(), gamma->defined() ? gamma->const_data_ptr() : nullptr,
                                    beta->defined() ? beta->const_data_ptr() : nullptr, Y.mutable_data_ptr(),
                                    mean.mutable_data_ptr(), rstd.mutable_data_ptr(), N, C, HxW, group, eps, xdt, wdt,
                                    to_b2n_dtype(stat_type, op), cur_stream()),
                 "group_norm_fwd");
  }
  return std::make_tuple(std::move(Y), std::move(mean), std::move(rstd));
}

// Host wrapper of upstream's native_group_norm_backward (aten/src/ATen/native/group_norm.cpp) around the kernel the
// reference registers for its GroupNormBackwardKernel stub (src/ATen/native/xpu/GroupNorm.cpp:23): dX like X, dgamma /
// dbeta like the weight (undefined without one, or when masked off).
std::tuple<Tensor, Tensor, Tensor> native_group_norm_backward(const Tensor& grad_out, const Tensor& input, const Tensor& mean,
                                                              const Tensor& rstd, const std::optional<Tensor>& weight_opt,
                                                              int64_t N, int64_t C, int64_t HxW, int64_t group,
                                                              std::array<bool, 3> mask) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  const char* op = "native_group_norm_backward";
  TORCH_CHECK(input.is_cuda() && grad_out.is_cuda(), op, ": expected CUDA tensors");
  TORCH_CHECK(group > 0 && C % group == 0, "Expected number of channels in input to be divisible by num_groups, but got input of shape ",
              input.sizes(), " and num_groups=", group);
  TORCH_CHECK(input.numel() == N * C * HxW && grad_out.numel() == input.numel(), op, ": input and grad_out must have N*C*HxW = ",
              N * C * HxW, " elements");
  TORCH_CHECK(mean.numel() == N * group && rstd.numel() == N * group && mean.scalar_type() == rstd.scalar_type(), op,
              ": mean and rstd must be [N, group] tensors of one dtype");
  TORCH_CHECK(!weight.defined() || (weight.dim() == 1 && weight.numel() == C),
              "Expected weight to be a vector of size equal to the number of channels in input, but got weight of shape ",
              weight.sizes(), " and input of shape ", input.sizes());
  const c10::cuda::CUDAGuard guard(input.device());
  Tensor X = input.contiguous();
  Tensor dY = grad_out.to(X.scalar_type()).contiguous();
  Tensor M = mean.contiguous(), R = rstd.contiguous();
  auto gamma = weight.expect_contiguous();
  const int xdt = to_b2n_dtype(X.scalar_type(), op);
  const int wdt = weight_dtype(X, weight, Tensor(), op);
  Tensor dX, dgamma, dbeta;
  if (mask[0]) dX = at::empty_like(X, at::MemoryFormat::Contiguous);
  if (mask[1] && weight.defined()) dgamma = at::empty_like(*gamma, at::MemoryFormat::Contiguous);
  if (mask[2] && weight.defined()) dbeta = at::empty_like(*gamma, at::MemoryFormat::Contiguous);
  if (X.numel() == 0) {
    if (dgamma.defined()) dgamma.zero_();
    if (dbeta.defined()) dbeta.zero_();
  } else if (dX.defined() || dgamma.defined() || dbeta.defined()) {
    const size_t ws_bytes = (dgamma.defined() || dbeta.defined()) ? b2n_group_norm_bwd_workspace_bytes(N, C, HxW, xdt) : 0;
    Tensor ws = ws_bytes ? at::empty({static_cast<int64_t>(ws_bytes)}, X.options().dtype(at::kByte)) : Tensor();
    check_status(b2n_group_norm_bwd_ws(dY.const_data_ptr(), X.const_data_ptr(), M.const_data_ptr(), R.const_data_ptr(),
                                       gamma->defined() ? gamma->const_data_ptr() : nullptr,
                                       dX.defined() ? dX.mutable_data_ptr() : nullptr,
                                       dgamma.defined() ? dgamma.mutable_data_ptr() : nullptr,
                                       dbeta.defined() ? dbeta.mutable_data_ptr() : nullptr, N, C, HxW, group, xdt, wdt,
                                       to_b2n_dtype(M.scalar_type(), op), ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes,
                                       cur_stream()),
                 "group_norm_bwd");
  }
  return std::make_tuple(std::move(dX), std::move(dgamma), std::move(dbeta));
}

static void bn_dims(const Tensor& input, const char* op, int64_t& N, int64_t& C, int64_t& HxW) {
  TORCH_CHECK(input.dim() >= 2, op, ": expected an input with at least two dimensions [N, C, ...]");
  N = input.size(0);
  C = input.size(1);
  HxW = 1;
  for (int64_t i = 2; i < input.dim(); ++i) HxW *= input.size(i);
  TORCH_CHECK(C == 0 || (N > 0 && HxW > 0), op, ": expected a non-empty input, got ", input.sizes());
}

// batch_norm_stats_xpu (src/ATen/native/xpu/BatchNorm.cpp:20): per-channel mean and 1/sqrt(var + eps), float.
std::tuple<Tensor, Tensor> batch_norm_stats(const Tensor& input, double eps) {
  const char* op = "batch_norm_stats";
  TORCH_CHECK(input.is_cuda(), op, ": expected a CUDA tensor");
  const c10::cuda::CUDAGuard guard(input.device());
  int64_t N, C, HxW;
  bn_dims(input, op, N, C, HxW);
  Tensor X = input.contiguous();
  Tensor mean = at::empty({C}, X.options().dtype(at::kFloat));
  Tensor invstd = at::empty({C}, X.options().dtype(at::kFloat));
  if (C > 0) {
    const int xdt = to_b2n_dtype(X.scalar_type(), op);
    const size_t ws_bytes = b2n_batch_norm_stats_workspace_bytes(N, C, HxW, xdt);  // several CTAs per channel need scratch
    Tensor ws = ws_bytes ? at::empty({static_cast<int64_t>(ws_bytes)}, X.options().dtype(at::kByte)) : Tensor();
    check_status(b2n_batch_norm_stats_ws(X.const_data_ptr(), mean.mutable_data_ptr<float>(), invstd.mutable_data_ptr<float>(),
                                         nullptr, nullptr, N, C, HxW, eps, 0.0, 0, xdt, B2N_F32,
                                         ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, cur_stream()),
                 op);
  }
  return std::make_tuple(std::move(mean), std::move(invstd));
}

// batch_norm_update_stats_xpu (BatchNorm.cpp:76): per-channel mean and biased variance, float; the running
// statistics blended in place with `momentum`.
std::tuple<Tensor, Tensor> batch_norm_update_stats(const Tensor& input, const std::optional<Tensor>& running_mean_opt,
                                                   const std::optional<Tensor>& running_var_opt, double momentum) {
  const char* op = "batch_norm_update_stats";
  c10::MaybeOwned<Tensor> rm_mo = at::borrow_from_optional_tensor(running_mean_opt);
  c10::MaybeOwned<Tensor> rv_mo = at::borrow_from_optional_tensor(running_var_opt);
  const Tensor& rm = *rm_mo;
  const Tensor& rv = *rv_mo;
  TORCH_CHECK(input.is_cuda(), op, ": expected a CUDA tensor");
  const c10::cuda::CUDAGuard guard(input.device());
  int64_t N, C, HxW;
  bn_dims(input, op, N, C, HxW);
  Tensor X = input.contiguous();
  TORCH_CHECK(!rm.defined() || (rm.is_contiguous() && rm.numel() == C), op, ": running_mean must be a contiguous [C] tensor");
  TORCH_CHECK(!rv.defined() || (rv.is_contiguous() && rv.numel() == C), op, ": running_var must be a contiguous [C] tensor");
  TORCH_CHECK(!rm.defined() || !rv.defined() || rm.scalar_type() == rv.scalar_type(), op,
              ": running_mean and running_var must have the same dtype");
  const Tensor& r = rm.defined() ? rm : rv;
  Tensor mean = at::empty({C}, X.options().dtype(at::kFloat));
  Tensor var = at::empty({C}, X.options().dtype(at::kFloat));
  if (C > 0) {
    const int xdt = to_b2n_dtype(X.scalar_type(), op);
    const size_t ws_bytes = b2n_batch_norm_stats_workspace_bytes(N, C, HxW, xdt);
    Tensor ws = ws_bytes ? at::empty({static_cast<int64_t>(ws_bytes)}, X.options().dtype(at::kByte)) : Tensor();
    check_status(b2n_batch_norm_stats_ws(X.const_data_ptr(), mean.mutable_data_ptr<float>(), var.mutable_data_ptr<float>(),
                                         rm.defined() ? rm.mutable_data_ptr() : nullptr,
                                         rv.defined() ? rv.mutable_data_ptr() : nullptr, N, C, HxW, 0.0, momentum, 1, xdt,
                                         r.defined() ? to_b2n_dtype(r.scalar_type(), op) : B2N_F32,
                                         ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, cur_stream()),
                 op);
  }
  return std::make_tuple(std::move(mean), std::move(var));
}

// ---- softmax family ------------------------------------------------------------------------------
struct SoftmaxDims { int64_t outer, n, inner; };
static SoftmaxDims softmax_dims(const Tensor& t, int64_t dim) {
  // a 0-dim tensor is treated as one element (SoftMaxKernels.cpp:2143-2148 of the reference)
  if (t.dim() == 0) return {1, 1, 1};
  SoftmaxDims d{1, t.size(dim), 1};
  for (int64_t i = 0; i < dim; ++i) d.outer *= t.size(i);
  for (int64_t i = dim + 1; i < t.dim(); ++i) d.inner *= t.size(i);
  return d;
}

static void softmax_forward_into(const Tensor& input, int64_t dim_, bool half_to_float, int mode, const Tensor& out,
                                 const char* op) {
  const c10::cuda::CUDAGuard guard(input.device());
  if (half_to_float) {
    TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16, op,
                ": conversion is supported for Half and BFloat16 type only");
  }
  const int64_t dim = at::maybe_wrap_dim(dim_, input.dim());
  TORCH_CHECK(dim >= 0 && dim < std::max<int64_t>(input.dim(), 1), op, ": dim must be non-negative and less than input dimensions");
  TORCH_CHECK(out.is_contiguous(), op, ": output must be contiguous");
  if (input.numel() == 0) return;
  Tensor x = input.contiguous();
  const SoftmaxDims d = softmax_dims(x, dim);
  check_status(b2n_softmax_fwd(x.const_data_ptr(), out.mutable_data_ptr(), d.outer, d.n, d.inner,
                               to_b2n_dtype(x.scalar_type(), op), to_b2n_dtype(out.scalar_type(), op), mode,
                               cur_stream()),
               op);
}

static Tensor softmax_forward(const Tensor& input, int64_t dim, bool half_to_float, int mode, const char* op) {
  TORCH_CHECK(input.is_cuda(), op, ": expected a CUDA tensor");
  const c10::cuda::CUDAGuard guard(input.device());
  Tensor out = at::empty_like(input, input.options().dtype(half_to_float ? at::kFloat : input.scalar_type()),
                              at::MemoryFormat::Contiguous);
  softmax_forward_into(input, dim, half_to_float, mode, out, op);
  return out;
}

static Tensor& softmax_forward_out(const Tensor& input, int64_t dim, bool half_to_float, int mode, Tensor& out,
                                   const char* op) {
  TORCH_CHECK(input.is_cuda() && out.is_cuda(), op, ": expected CUDA tensors");
  const auto want = half_to_float ? at::kFloat : input.scalar_type();
  TORCH_CHECK(out.scalar_type() == want, op, ": expected out dtype ", want, " but got ", out.scalar_type());
  at::native::resize_output(out, input.sizes());
  if (out.is_contiguous()) {
    softmax_forward_into(input, dim, half_to_float, mode, out, op);
  } else {
    Tensor tmp = at::empty_like(input, input.options().dtype(want), at::MemoryFormat::Contiguous);
    softmax_forward_into(input, dim, half_to_float, mode, tmp, op);
    out.copy_(tmp);
  }
  return out;
}

static void softmax_backward_into(const Tensor& grad, const Tensor& output, int64_t dim_, at::ScalarType input_dtype,
                                  bool is_log, const Tensor& grad_input, const char* op) {
  const c10::cuda::CUDAGuard guard(grad.device());
  const bool half_to_float = grad.scalar_type() != input_dtype;
  if (half_to_float) {
    TORCH_CHECK(grad.scalar_type() == at::kFloat && (input_dtype == at::kHalf || input_dtype == at::kBFloat16), op,
                ": expected input and grad types to match, or input to be at::Half/BFloat16 and grad to be at::Float");
  }
  TORCH_CHECK(grad.sizes() == output.sizes(), op, ": grad and output sizes differ");
  const int64_t dim = at::maybe_wrap_dim(dim_, grad.dim());
  TORCH_CHECK(dim >= 0 && dim < std::max<int64_t>(grad.dim(), 1), op, ": dim must be non-negative and less than input dimensions");
  if (grad.numel() == 0) return;
  Tensor g = grad.contiguous();
  Tensor y = output.to(g.scalar_type()).contiguous();
  const SoftmaxDims d = softmax_dims(g, dim);
  check_status(b2n_softmax_bwd(g.const_data_ptr(), y.const_data_ptr(), grad_input.mutable_data_ptr(), d.outer, d.n,
                               d.inner, to_b2n_dtype(g.scalar_type(), op), to_b2n_dtype(grad_input.scalar_type(), op),
                               is_log ? 1 : 0, cur_stream()),
               op);
}

static Tensor softmax_backward(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType input_dtype,
                               bool is_log, const char* op) {
  TORCH_CHECK(grad.is_cuda() && output.is_cuda(), op, ": expected CUDA tensors");
  const c10::cuda::CUDAGuard guard(grad.device());
  Tensor gi = at::empty_like(grad, grad.options().dtype(input_dtype), at::MemoryFormat::Contiguous);
  softmax_backward_into(grad, output, dim, input_dtype, is_log, gi, op);
  return gi;
}

static Tensor& softmax_backward_out(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType input_dtype,
                                    bool is_log, Tensor& grad_input, const char* op) {
  TORCH_CHECK(grad.is_cuda() && output.is_cuda() && grad_input.is_cuda(), op, ": expected CUDA tensors");
  TORCH_CHECK(grad_input.scalar_type() == input_dtype, op, ": expected grad_input dtype ", input_dtype, " but got ",
              grad_input.scalar_type());
  at::native::resize_output(grad_input, grad.sizes());
  if (grad_input.is_contiguous()) {
    softmax_backward_into(grad, output, dim, input_dtype, is_log, grad_input, op);
  } else {
    Tensor tmp = at::empty_like(grad, grad.options().dtype(input_dtype), at::MemoryFormat::Contiguous);
    softmax_backward_into(grad, output, dim, input_dtype, is_log, tmp, op);
    grad_input.copy_(tmp);
  }
  return grad_input;
}

Tensor softmax(const Tensor& self, int64_t dim, bool h2f) { return softmax_forward(self, dim, h2f, 0, "_softmax"); }
Tensor& softmax_out(const Tensor& self, int64_t dim, bool h2f, Tensor& out) {
  return softmax_forward_out(self, dim, h2f, 0, out, "_softmax.out");
}
Tensor log_softmax(const Tensor& self, int64_t dim, bool h2f) { return softmax_forward(self, dim, h2f, 1, "_log_softmax"); }
Tensor& log_softmax_out(const Tensor& self, int64_t dim, bool h2f, Tensor& out) {
  return softmax_forward_out(self, dim, h2f, 1, out, "_log_softmax.out");
}
// aten::_safe_softmax: softmax whose fully masked (all -inf) rows come out as zeros.  Mirrors
// _safe_softmax_xpu (src/ATen/native/xpu/SoftMax.cpp:102-110): Half input with dtype Float takes the
// half_to_float kernel, any other dtype is a conversion first.
Tensor safe_softmax(const Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype) {
  if ((self.scalar_type() == at::kHalf || self.scalar_type() == at::kBFloat16) && dtype == at::kFloat)
    return softmax_forward(self, dim, true, 2, "_safe_softmax");
  Tensor converted = dtype.has_value() ? self.toType(dtype.value()) : self;
  return softmax_forward(converted, dim, false, 2, "_safe_softmax");
}
Tensor softmax_backward_data(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType input_dtype) {
  return softmax_backward(grad, output, dim, input_dtype, false, "_softmax_backward_data");
}
Tensor& softmax_backward_data_out(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType input_dtype,
                                  Tensor& grad_input) {
  return softmax_backward_out(grad, output, dim, input_dtype, false, grad_input, "_softmax_backward_data.out");
}
Tensor log_softmax_backward_data(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType input_dtype) {
  return softmax_backward(grad, output, dim, input_dtype, true, "_log_softmax_backward_data");
}
Tensor& log_softmax_backward_data_out(const Tensor& grad, const Tensor& output, int64_t dim,
                                      at::ScalarType input_dtype, Tensor& grad_input) {
  return softmax_backward_out(grad, output, dim, input_dtype, true, grad_input, "_log_softmax_backward_data.out");
}

// ---- masked softmax ------------------------------------------------------------------------------
// Same checks and mask layouts as masked_softmax_kernel / masked_softmax_backward_kernel
// (src/ATen/native/xpu/sycl/SoftMaxKernels.cpp:2301-2407).
Tensor masked_softmax(const Tensor& input_, const Tensor& mask_, std::optional<int64_t> dim_,
                      std::optional<int64_t> mask_type_) {
  const char* op = "_masked_softmax";
  TORCH_CHECK(input_.is_cuda() && mask_.is_cuda(), op, ": expected CUDA tensors");
  TORCH_CHECK(mask_.scalar_type() == at::kBool, "Mask should be a boolean tensor");
  TORCH_CHECK(mask_type_.has_value(), "Mask Type should be defined");
  const int64_t mask_type = mask_type_.value();
  TORCH_CHECK(mask_type == 0 || mask_type == 1 || mask_type == 2,
              "Mask Type should be 0 (src_mask), 1 (src_key_padding_mask), or 2 (default_mask)");
  const bool is_BxT = mask_type == 1 && input_.dim() == 4 && mask_.dim() == 2 && input_.size(0) == mask_.size(0) &&
                      input_.size(2) == mask_.size(1) && input_.size(3) == mask_.size(1);
  const bool is_TxT = mask_type == 0 && input_.dim() == 4 && mask_.dim() == 2 && input_.size(3) == mask_.size(1) &&
                      input_.size(2) == mask_.size(0) && mask_.size(0) == mask_.size(1);
  const bool same = mask_.sizes() == input_.sizes();
  TORCH_CHECK(same || is_BxT || is_TxT, "Mask shape should match input. mask: ", mask_.sizes(),
              " input: ", input_.sizes());
  const c10::cuda::CUDAGuard guard(input_.device());
  Tensor input = input_.dim() == 0 ? input_.view(1) : input_;
  const int64_t dim = dim_.has_value() ? at::maybe_wrap_dim(dim_.value(), input.dim()) : input.dim() - 1;
  if (dim != input.dim() - 1) {
    // other dims: the mask applied up front, then the plain kernels (masked elements come out as exp(-inf) = 0)
    Tensor full = same ? (mask_.dim() == 0 ? mask_.view(1) : mask_)
                       : (is_BxT ? mask_.view({mask_.size(0), 1, 1, mask_.size(1)}) : mask_).expand_as(input);
    return softmax_forward(input.masked_fill(full, -std::numeric_limits<double>::infinity()), dim, false, 0, op)
        .view(input_.sizes());
  }
  Tensor x = input.contiguous();
  Tensor mask = mask_.contiguous();
  Tensor out = at::empty_like(x, x.options(), at::MemoryFormat::Contiguous);
  if (x.numel() == 0) return out.view(input_.sizes());
  const int64_t n = x.size(-1), rows = x.numel() / n;
  int64_t row_div = 1, row_mod = rows;
  if (!same && is_BxT) { row_div = x.size(1) * x.size(2); row_mod = x.size(0); }
  if (!same && is_TxT) { row_div = 1; row_mod = mask.size(0); }
  check_status(b2n_masked_softmax_fwd(x.const_data_ptr(), mask.const_data_ptr(), out.mutable_data_ptr(), rows, n,
                                      row_div, row_mod, to_b2n_dtype(x.scalar_type(), op), cur_stream()),
               op);
  return out.view(input_.sizes());
}

Tensor masked_softmax_backward(const Tensor& grad_, const Tensor& output_, const Tensor& mask_,
                               std::optional<int64_t> dim_) {
  const char* op = "_masked_softmax_backward";
  TORCH_CHECK(grad_.is_cuda() && output_.is_cuda() && mask_.is_cuda(), op, ": expected CUDA tensors");
  const c10::cuda::CUDAGuard guard(grad_.device());
  if (grad_.numel() == 0) return at::empty_like(grad_, grad_.options());
  Tensor grad = grad_.contiguous(), output = output_.contiguous(), mask = mask_.contiguous();
  const int64_t dim = dim_.has_value() ? at::maybe_wrap_dim(dim_.value(), output.dim()) : output.dim() - 1;
  if (grad.dim() == 0) { grad = grad.view(1); mask = mask.view(1); output = output.view(1); }
  TORCH_CHECK(dim >= 0 && dim < grad.dim(), "dim must be non-negative and less than input dimensions");
  TORCH_CHECK(grad.sizes() == mask.sizes(), "Mask shape should match grad shape");
  TORCH_CHECK(mask.scalar_type() == at::kBool, "Mask should be a boolean tensor");
  TORCH_CHECK(output.scalar_type() == grad.scalar_type() && output.sizes() == grad.sizes(), op,
              ": grad_output and output must agree in dtype and shape");
  if (dim != grad.dim() - 1) {
    Tensor gi = softmax_backward(grad.masked_fill(mask, 0), output.masked_fill(mask, 0), dim, grad.scalar_type(),
                                 false, op);
    return gi.masked_fill(mask, 0).view(grad_.sizes());
  }
  Tensor gi = at::empty_like(grad, grad.options(), at::MemoryFormat::Contiguous);
  const int64_t n = grad.size(-1), rows = grad.numel() / n;
  check_status(b2n_masked_softmax_bwd(grad.const_data_ptr(), output.const_data_ptr(), mask.const_data_ptr(),
                                      gi.mutable_data_ptr(), rows, n, to_b2n_dtype(grad.scalar_type(), op),
                                      cur_stream()),
               op);
  return gi.view(grad_.sizes());
}

// ---- nll_loss ------------------------------------------------------------------------------------
// Shape rules of the upstream meta function for nll_loss_forward.
static void nll_check(const Tensor& self, const Tensor& target, const Tensor& weight) {
  TORCH_CHECK(self.dim() > 0 && self.dim() <= 2, "input tensor should be 1D or 2D");
  TORCH_CHECK(target.dim() <= 1, "0D or 1D target tensor expected, multi-target not supported");
  const bool no_batch = self.dim() == 1 && target.dim() == 0;
  TORCH_CHECK(no_batch || (self.size(0) == target.size(0)), "size mismatch (got input: ", self.sizes(),
              ", target: ", target.sizes(), ")");
  const int64_t C = self.size(-1);
  TORCH_CHECK(!weight.defined() || (weight.dim() == 1 && weight.numel() == C),
              "weight tensor should be defined either for all ", C, " classes or no classes but got weight tensor of shape: ",
              weight.sizes());
  TORCH_CHECK(target.scalar_type() == at::kLong || target.scalar_type() == at::kByte,
              "expected target dtype Long or Byte but got ", target.scalar_type());
}

static void nll_forward_into(const Tensor& self, const Tensor& target, const Tensor& weight, int64_t reduction,
                             int64_t ignore_index, const Tensor& output, const Tensor& total_weight) {
  const c10::cuda::CUDAGuard guard(self.device());
  const int64_t C = self.size(-1);
  const int64_t M = self.dim() == 1 ? 1 : self.size(0);
  Tensor x = self.contiguous();
  Tensor t = target.contiguous();
  Tensor w = weight.defined() ? weight.to(self.scalar_type()).contiguous() : Tensor();
  const size_t ws_bytes = b2n_nll_loss_workspace_bytes(M);
  Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, self.options().dtype(at::kByte));
  if (reduction == at::Reduction::None) total_weight.zero_();
  check_status(b2n_nll_loss_fwd(x.const_data_ptr(), t.const_data_ptr(), w.defined() ? w.const_data_ptr() : nullptr,
                                output.mutable_data_ptr(), total_weight.mutable_data_ptr(), nullptr,
                                ws.mutable_data_ptr(), ws_bytes, M, C, static_cast<int>(reduction), ignore_index,
                                to_b2n_dtype(self.scalar_type(), "nll_loss_forward"),
                                t.scalar_type() == at::kByte ? 1 : 0, cur_stream()),
               "nll_loss_fwd");
  note_possible_device_failure();
}

std::tuple<Tensor, Tensor> nll_loss_forward(const Tensor& self, const Tensor& target,
                                            const std::optional<Tensor>& weight_opt, int64_t reduction,
                                            int64_t ignore_index) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  TORCH_CHECK(self.is_cuda() && target.is_cuda(), "nll_loss_forward: expected CUDA tensors");
  nll_check(self, target, weight);
  const c10::cuda::CUDAGuard guard(self.device());
  const bool batched_none = reduction == at::Reduction::None && self.dim() == 2;
  Tensor output = batched_none ? at::empty({self.size(0)}, self.options()) : at::empty({}, self.options());
  Tensor total_weight = at::empty({}, self.options());
  nll_forward_into(self, target, weight, reduction, ignore_index, output, total_weight);
  return std::make_tuple(std::move(output), std::move(total_weight));
}

std::tuple<Tensor&, Tensor&> nll_loss_forward_out(const Tensor& self, const Tensor& target,
                                                  const std::optional<Tensor>& weight_opt, int64_t reduction,
                                                  int64_t ignore_index, Tensor& output, Tensor& total_weight) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  TORCH_CHECK(self.is_cuda() && target.is_cuda(), "nll_loss_forward: expected CUDA tensors");
  nll_check(self, target, weight);
  const bool batched_none = reduction == at::Reduction::None && self.dim() == 2;
  at::native::resize_output(output, batched_none ? at::IntArrayRef({self.size(0)}) : at::IntArrayRef({}));
  at::native::resize_output(total_weight, {});
  TORCH_CHECK(output.scalar_type() == self.scalar_type() && total_weight.scalar_type() == self.scalar_type(),
              "nll_loss_forward.output: out tensors must have the input dtype");
  TORCH_CHECK(output.is_contiguous(), "nll_loss_forward.output: output must be contiguous");
  nll_forward_into(self, target, weight, reduction, ignore_index, output, total_weight);
  return std::forward_as_tuple(output, total_weight);
}

static void nll_backward_into(const Tensor& grad_output, const Tensor& self, const Tensor& target,
                              const Tensor& weight, int64_t reduction, int64_t ignore_index,
                              const Tensor& total_weight, const Tensor& grad_input) {
  const c10::cuda::CUDAGuard guard(self.device());
  const int64_t C = self.size(-1);
  const int64_t M = self.dim() == 1 ? 1 : self.size(0);
  Tensor g = grad_output.to(self.scalar_type()).contiguous();
  Tensor t = target.contiguous();
  Tensor w = weight.defined() ? weight.to(self.scalar_type()).contiguous() : Tensor();
  Tensor tw = total_weight.to(self.scalar_type()).contiguous();
  if (reduction == at::Reduction::None && self.dim() == 2) {
    TORCH_CHECK(g.dim() == 1 && g.size(0) == M, "Expected a tensor of dimension 1 and tensor.size[0] == ", M,
                " but got: dimension ", g.dim(), " and tensor.size[0] == ", g.dim() ? g.size(0) : 0);
  } else {
    TORCH_CHECK(g.numel() == 1, "Expected a single element grad_output tensor, but got: ", g.sizes());
  }
  check_status(b2n_nll_loss_bwd(g.const_data_ptr(), t.const_data_ptr(), w.defined() ? w.const_data_ptr() : nullptr,
                                tw.const_data_ptr(), grad_input.mutable_data_ptr(), M, C,
                                static_cast<int>(self.dim() == 1 && reduction == at::Reduction::None ? at::Reduction::Sum
                                                                                                    : reduction),
                                ignore_index, to_b2n_dtype(self.scalar_type(), "nll_loss_backward"),
                                t.scalar_type() == at::kByte ? 1 : 0, cur_stream()),
               "nll_loss_bwd");
  note_possible_device_failure();
}

Tensor nll_loss_backward(const Tensor& grad_output, const Tensor& self, const Tensor& target,
                         const std::optional<Tensor>& weight_opt, int64_t reduction, int64_t ignore_index,
                         const Tensor& total_weight) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  TORCH_CHECK(self.is_cuda() && target.is_cuda() && grad_output.is_cuda(), "nll_loss_backward: expected CUDA tensors");
  nll_check(self, target, weight);
  const c10::cuda::CUDAGuard guard(self.device());
  Tensor grad_input = at::empty_like(self, at::MemoryFormat::Contiguous);
  nll_backward_into(grad_output, self, target, weight, reduction, ignore_index, total_weight, grad_input);
  return grad_input;
}

Tensor& nll_loss_backward_out(const Tensor& grad_output, const Tensor& self, const Tensor& target,
                              const std::optional<Tensor>& weight_opt, int64_t reduction, int64_t ignore_index,
                              const Tensor& total_weight, Tensor& grad_input) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  TORCH_CHECK(self.is_cuda() && target.is_cuda() && grad_output.is_cuda(), "nll_loss_backward: expected CUDA tensors");
  nll_check(self, target, weight);
  at::native::resize_output(grad_input, self.sizes());
  TORCH_CHECK(grad_input.scalar_type() == self.scalar_type() && grad_input.is_contiguous(),
              "nll_loss_backward.grad_input: grad_input must be contiguous and have the input dtype");
  nll_backward_into(grad_output, self, target, weight, reduction, ignore_index, total_weight, grad_input);
  return grad_input;
}

// ---- cross_entropy_loss: the fused backward for autograd users ---------------------------------------
// aten::cross_entropy_loss is a composite: log_softmax, then nll_loss, whose derivative formulas call
// nll_loss_backward (a dense, almost all-zero gradient of the log-probabilities: 3.9 GiB written and read back
// for 16384 x 128256 bf16) and then _log_softmax_backward_data.  For class-index targets without label smoothing
// this autograd kernel keeps the same forward operators and replaces the two backward steps by
// b2n_cross_entropy_bwd, which never materialises that gradient.  Everything else (probability targets, label
// smoothing, class dimension not last) goes to the composite unchanged.
class FusedCrossEntropy : public torch::autograd::Function<FusedCrossEntropy> {
 public:
  static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& self, const Tensor& target,
                        const std::optional<Tensor>& weight, int64_t reduction, int64_t ignore_index) {
    at::AutoDispatchBelowADInplaceOrView below_autograd;
    Tensor logp = at::_log_softmax(self, -1, false);
    auto [loss, total_weight] = at::nll_loss_forward(logp, target, weight, reduction, ignore_index);
    // (an absent weight is saved as an empty tensor: the saved list holds defined tensors only)
    ctx->save_for_backward({logp, target, weight.has_value() && weight->defined() ? *weight : at::empty({0}, logp.options()),
                            total_weight});
    ctx->saved_data["has_weight"] = weight.has_value() && weight->defined();
    ctx->saved_data["reduction"] = reduction;
    ctx->saved_data["ignore_index"] = ignore_index;
    return loss;
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list grads) {
    const auto saved = ctx->get_saved_variables();
    const Tensor& logp = saved[0];
    const Tensor& target = saved[1];
    const Tensor& weight = saved[2];
    const Tensor& total_weight = saved[3];
    int64_t reduction = ctx->saved_data["reduction"].toInt();
    const int64_t ignore_index = ctx->saved_data["ignore_index"].toInt();
    const c10::cuda::CUDAGuard guard(logp.device());
    const int64_t C = logp.size(-1), M = logp.dim() == 1 ? 1 : logp.size(0);
    if (logp.dim() == 1 && reduction == at::Reduction::None) reduction = at::Reduction::Sum;  // one row: the scalar applies as is
    Tensor y = logp.contiguous();
    Tensor g = grads[0].to(y.scalar_type()).contiguous();
    Tensor t = target.contiguous();
    Tensor w = ctx->saved_data["has_weight"].toBool() ? weight.to(y.scalar_type()).contiguous() : Tensor();
    Tensor tw = total_weight.to(y.scalar_type()).contiguous();
    Tensor dx = at::empty_like(y);
    if (y.numel() > 0) {
      check_status(b2n_cross_entropy_bwd(y.const_data_ptr(), t.const_data_ptr(), w.defined() ? w.const_data_ptr() : nullptr,
                                         g.const_data_ptr(), tw.const_data_ptr(), dx.mutable_data_ptr(), M, C,
                                         static_cast<int>(reduction), ignore_index,
                                         to_b2n_dtype(y.scalar_type(), "cross_entropy_loss backward"),
                                         t.scalar_type() == at::kByte ? 1 : 0, cur_stream()),
                   "cross_entropy_bwd");
      note_possible_device_failure();
    }
    return {dx, Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

Tensor cross_entropy_loss_autograd(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight_opt,
                                   int64_t reduction, c10::SymInt ignore_index, double label_smoothing) {
  c10::MaybeOwned<Tensor> weight_mo = at::borrow_from_optional_tensor(weight_opt);
  const Tensor& weight = *weight_mo;
  const auto dt = self.scalar_type();
  const bool class_indices = (target.scalar_type() == at::kLong || target.scalar_type() == at::kByte) &&
                             target.dim() == self.dim() - 1 && (self.dim() == 1 || self.size(0) == target.size(0));
  const bool fused = self.is_cuda() && target.is_cuda() && (self.dim() == 1 || self.dim() == 2) && class_indices &&
                     label_smoothing == 0.0 && self.numel() > 0 &&
                     (dt == at::kFloat || dt == at::kHalf || dt == at::kBFloat16 || dt == at::kDouble) &&
                     (!weight.defined() || (weight.is_cuda() && weight.dim() == 1 && weight.numel() == self.size(-1)));
  if (!fused) return at::native::cross_entropy_loss_symint(self, target, weight_opt, reduction, std::move(ignore_index), label_smoothing);
  return FusedCrossEntropy::apply(self, target, weight.defined() ? std::optional<Tensor>(weight) : std::nullopt, reduction,
                                  ignore_index.expect_int());
}

}  // namespace b200norm

TORCH_LIBRARY_IMPL(aten, AutogradCUDA, m) {
  m.impl("cross_entropy_loss", TORCH_FN(b200norm::cross_entropy_loss_autograd));
}

TORCH_LIBRARY_IMPL(aten, CUDA, m) {
  using namespace b200norm;
  m.impl("native_layer_norm", TORCH_FN(native_layer_norm));
  m.impl("native_layer_norm_backward", TORCH_FN(native_layer_norm_backward));
  m.impl("_fused_rms_norm", TORCH_FN(fused_rms_norm));
  m.impl("_fused_rms_norm_backward", TORCH_FN(fused_rms_norm_backward));
  m.impl("native_group_norm", TORCH_FN(native_group_norm));
  m.impl("native_group_norm_backward", TORCH_FN(native_group_norm_backward));
  m.impl("batch_norm_stats", TORCH_FN(batch_norm_stats));
  m.impl("batch_norm_update_stats", TORCH_FN(batch_norm_update_stats));
  m.impl("_softmax", TORCH_FN(softmax));
  m.impl("_safe_softmax", TORCH_FN(safe_softmax));
  m.impl("_masked_softmax", TORCH_FN(masked_softmax));
  m.impl("_masked_softmax_backward", TORCH_FN(masked_softmax_backward));
  m.impl("_softmax.out", TORCH_FN(softmax_out));
  m.impl("_log_softmax", TORCH_FN(log_softmax));
  m.impl("_log_softmax.out", TORCH_FN(log_softmax_out));
  m.impl("_softmax_backward_data", TORCH_FN(softmax_backward_data));
  m.impl("_softmax_backward_data.out", TORCH_FN(softmax_backward_data_out));
  m.impl("_log_softmax_backward_data", TORCH_FN(log_softmax_backward_data));
  m.impl("_log_softmax_backward_data.out", TORCH_FN(log_softmax_backward_data_out));
  m.impl("nll_loss_forward", TORCH_FN(nll_loss_forward));
  m.impl("nll_loss_forward.output", TORCH_FN(nll_loss_forward_out));
  m.impl("nll_loss_backward", TORCH_FN(nll_loss_backward));
  m.impl("nll_loss_backward.grad_input", TORCH_FN(nll_loss_backward_out));
}
