// nll_loss forward / backward.
//
// Forward follows at::native::xpu::nll_loss_forward_kernel
// (src/ATen/native/xpu/sycl/LossNLLKernel.cpp:391-535): out = sum_i -w[t_i] * x[i, t_i] (divided by
// sum_i w[t_i] for mean), rows whose target equals ignore_index are skipped, an empty batch gives
// NaN (mean) or 0 (sum).  The reference reduces in ONE work-group (:496-533); here many CTAs write
// per-CTA partial sums and a second one-CTA kernel folds them in index order, so the result is
// deterministic and the gather is spread over the machine.
#include "common.cuh"
#include "launchers.h"

namespace b2n {

namespace {

constexpr int kNllThreads = 256;
constexpr int kNllMaxBlocks = 1024;

template <typename A> __device__ __forceinline__ A quiet_nan();
template <> __device__ __forceinline__ float quiet_nan<float>() { return __int_as_float(0x7fc00000); }
template <> __device__ __forceinline__ double quiet_nan<double>() { return __longlong_as_double(0x7ff8000000000000LL); }

template <typename IdxT> __device__ __forceinline__ int64_t load_target(const void* target, int64_t i) {
  return static_cast<int64_t>(static_cast<const IdxT*>(target)[i]);
}

template <typename T, typename IdxT>
__global__ void nll_fwd_none_kernel(const T* __restrict__ logp, const void* __restrict__ target,
                                    const T* __restrict__ weight, T* __restrict__ out, int64_t M, int64_t C,
                                    int64_t ignore_index, int* status) {
  using A = acc_t<T>;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < M;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = load_target<IdxT>(target, i);
    A v = 0;
    if (t != ignore_index) {
      if (t >= 0 && t < C) {
        const A w = weight ? to_acc<A>(weight[t]) : A(1);
        v = -w * to_acc<A>(logp[i * C + t]);
      } else {
        record_status(status, B2N_ERR_TARGET_RANGE);
      }
    }
    out[i] = from_acc<T>(v);
  }
}

// partial[2*b] = sum over CTA b's rows of -w*x ; partial[2*b+1] = sum of w
template <typename T, typename IdxT>
__global__ void nll_fwd_partial_kernel(const T* __restrict__ logp, const void* __restrict__ target,
                                       const T* __restrict__ weight, acc_t<T>* __restrict__ partial,
                                       int64_t M, int64_t C, int64_t ignore_index, int* status) {
  using A = acc_t<T>;
  __shared__ A scratch[32];
  A s = 0, ws = 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < M;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = load_target<IdxT>(target, i);
    if (t == ignore_index) continue;
    if (t >= 0 && t < C) {
      const A w = weight ? to_acc<A>(weight[t]) : A(1);
      s -= w * to_acc<A>(logp[i * C + t]);
      ws += w;
    } else {
      record_status(status, B2N_ERR_TARGET_RANGE);
    }
  }
  s = block_reduce(s, scratch, SumOp());
  ws = block_reduce(ws, scratch, SumOp());
  if (threadIdx.x == 0) {
    partial[2 * blockIdx.x] = s;
    partial[2 * blockIdx.x + 1] = ws;
  }
}

template <typename T>
__global__ void nll_fwd_fold_kernel(const acc_t<T>* __restrict__ partial, int nblocks, T* __restrict__ out,
                                    T* __restrict__ total_weight, float* __restrict__ sums_f32, int reduction,
                                    int64_t M) {
  using A = acc_t<T>;
  __shared__ A scratch[32];
  A s = 0, ws = 0;
  // fixed assignment of partials to threads and fixed combine order: deterministic
  for (int b = threadIdx.x; b < nblocks; b += blockDim.x) {
    s += partial[2 * b];
    ws += partial[2 * b + 1];
  }
  s = block_reduce(s, scratch, SumOp());
  ws = block_reduce(ws, scratch, SumOp());
  if (threadIdx.x == 0) {
    if (sums_f32) {
      sums_f32[0] = static_cast<float>(s);
      sums_f32[1] = static_cast<float>(ws);
    }
    if (total_weight) *total_weight = from_acc<T>(ws);
    A r = s;
    if (reduction == B2N_REDUCE_MEAN) r = (M == 0) ? quiet_nan<A>() : s / ws;
    if (out) *out = from_acc<T>(r);
  }
}

// grad_input was zero-filled; scatter one value per row.
template <typename T, typename IdxT>
__global__ void nll_bwd_kernel(const T* __restrict__ grad_out, const void* __restrict__ target,
                               const T* __restrict__ weight, const T* __restrict__ total_weight,
                               T* __restrict__ grad_input, int64_t M, int64_t C, int reduction,
                               int64_t ignore_index, int* status) {
  using A = acc_t<T>;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < M;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = load_target<IdxT>(target, i);
    if (t == ignore_index) continue;
    if (t < 0 || t >= C) {
      record_status(status, B2N_ERR_TARGET_RANGE);
      continue;
    }
    const A w = weight ? to_acc<A>(weight[t]) : A(1);
    A g = to_acc<A>(reduction == B2N_REDUCE_NONE ? grad_out[i] : grad_out[0]);
    if (reduction == B2N_REDUCE_MEAN) g = g / to_acc<A>(*total_weight);
    grad_input[i * C + t] = from_acc<T>(-w * g);
  }
}

template <typename T, typename IdxT>
int nll_fwd_typed(const void* logp, const void* target, const void* weight, void* out, void* total_weight,
                  float* sums_f32, void* workspace, int64_t M, int64_t C, int reduction, int64_t ignore_index,
                  cudaStream_t st) {
  using A = acc_t<T>;
  int* status = device_status_ptr();
  if (reduction == B2N_REDUCE_NONE) {
    if (M == 0) return B2N_OK;
    const int64_t blocks = (M + kNllThreads - 1) / kNllThreads;
    const int grid = static_cast<int>(blocks < kNllMaxBlocks ? blocks : kNllMaxBlocks);
    nll_fwd_none_kernel<T, IdxT><<<grid, kNllThreads, 0, st>>>(static_cast<const T*>(logp), target,
                                                               static_cast<const T*>(weight),
                                                               static_cast<T*>(out), M, C, ignore_index, status);
    return launched();
  }
  int64_t blocks = (M + kNllThreads - 1) / kNllThreads;
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks < kNllMaxBlocks ? blocks : kNllMaxBlocks);
  nll_fwd_partial_kernel<T, IdxT><<<grid, kNllThreads, 0, st>>>(static_cast<const T*>(logp), target,
                                                                static_cast<const T*>(weight),
                                                                static_cast<A*>(workspace), M, C, ignore_index,
                                                                status);
  if (int e = launched()) return e;
  nll_fwd_fold_kernel<T><<<1, kNllThreads, 0, st>>>(static_cast<const A*>(workspace), grid, static_cast<T*>(out),
                                                    static_cast<T*>(total_weight), sums_f32, reduction, M);
  return launched();
}

template <typename T, typename IdxT>
int nll_bwd_typed(const void* grad_out, const void* target, const void* weight, const void* total_weight,
                  void* grad_input, int64_t M, int64_t C, int reduction, int64_t ignore_index, cudaStream_t st) {
  if (int e = check_cuda(cudaMemsetAsync(grad_input, 0, static_cast<size_t>(M) * C * sizeof(T), st))) return e;
  if (M == 0) return B2N_OK;
  const int64_t blocks = (M + kNllThreads - 1) / kNllThreads;
  const int grid = static_cast<int>(blocks < kNllMaxBlocks ? blocks : kNllMaxBlocks);
  nll_bwd_kernel<T, IdxT><<<grid, kNllThreads, 0, st>>>(
      static_cast<const T*>(grad_out), target, static_cast<const T*>(weight), static_cast<const T*>(total_weight),
      static_cast<T*>(grad_input), M, C, reduction, ignore_index, device_status_ptr());
  return launched();
}

}  // namespace

size_t nll_loss_workspace_bytes(int64_t M) {
  (void)M;
  return static_cast<size_t>(kNllMaxBlocks) * 2 * sizeof(double);
}

#define B2N_NLL_DISPATCH(FN, ...)                                                  \
  switch (dtype) {                                                                 \
    case B2N_F32: return u8 ? FN<float, uint8_t>(__VA_ARGS__) : FN<float, int64_t>(__VA_ARGS__);   \
    case B2N_F16: return u8 ? FN<f16, uint8_t>(__VA_ARGS__) : FN<f16, int64_t>(__VA_ARGS__);       \
    case B2N_BF16: return u8 ? FN<bf16, uint8_t>(__VA_ARGS__) : FN<bf16, int64_t>(__VA_ARGS__);    \
    case B2N_F64: return u8 ? FN<double, uint8_t>(__VA_ARGS__) : FN<double, int64_t>(__VA_ARGS__); \
    default: return B2N_ERR_UNSUPPORTED_DTYPE;                                     \
  }

int launch_nll_loss_fwd(const void* logp, const void* target, const void* weight, void* out, void* total_weight,
                        float* sums_f32, void* workspace, size_t workspace_bytes, int64_t M, int64_t C,
                        int reduction, int64_t ignore_index, int dtype, bool u8, cudaStream_t st) {
  if (reduction != B2N_REDUCE_NONE && (workspace == nullptr || workspace_bytes < nll_loss_workspace_bytes(M)))
    return B2N_ERR_WORKSPACE;
  B2N_NLL_DISPATCH(nll_fwd_typed, logp, target, weight, out, total_weight, sums_f32, workspace, M, C, reduction,
                   ignore_index, st)
}

int launch_nll_loss_bwd(const void* grad_out, const void* target, const void* weight, const void* total_weight,
                        void* grad_input, int64_t M, int64_t C, int reduction, int64_t ignore_index, int dtype,
                        bool u8, cudaStream_t st) {
  B2N_NLL_DISPATCH(nll_bwd_typed, grad_out, target, weight, total_weight, grad_input, M, C, reduction,
                   ignore_index, st)
}

}  // namespace b2n
