// dtype dispatch for softmax / log-softmax.
#include "softmax_launch.cuh"

namespace b2n {

int launch_softmax_fwd(const void* x, void* y, int64_t outer, int64_t N, int64_t inner, int in_dtype,
                       int out_dtype, bool is_log, cudaStream_t st) {
  if (in_dtype == out_dtype) {
    switch (in_dtype) {
      case B2N_F32: return softmax_fwd_f32(is_log, x, y, outer, N, inner, st);
      case B2N_F16: return softmax_fwd_f16(is_log, x, y, outer, N, inner, st);
      case B2N_BF16: return softmax_fwd_bf16(is_log, x, y, outer, N, inner, st);
      case B2N_F64: return softmax_fwd_f64(is_log, x, y, outer, N, inner, st);
      default: return B2N_ERR_UNSUPPORTED_DTYPE;
    }
  }
  if (out_dtype == B2N_F32 && in_dtype == B2N_F16) return softmax_fwd_f16_f32(is_log, x, y, outer, N, inner, st);
  if (out_dtype == B2N_F32 && in_dtype == B2N_BF16) return softmax_fwd_bf16_f32(is_log, x, y, outer, N, inner, st);
  return B2N_ERR_UNSUPPORTED_DTYPE;
}

int launch_softmax_bwd(const void* dy, const void* y, void* dx, int64_t outer, int64_t N, int64_t inner,
                       int grad_dtype, int dx_dtype, bool is_log, cudaStream_t st) {
  if (grad_dtype == dx_dtype) {
    switch (grad_dtype) {
      case B2N_F32: return softmax_bwd_f32(is_log, dy, y, dx, outer, N, inner, st);
      case B2N_F16: return softmax_bwd_f16(is_log, dy, y, dx, outer, N, inner, st);
      case B2N_BF16: return softmax_bwd_bf16(is_log, dy, y, dx, outer, N, inner, st);
      case B2N_F64: return softmax_bwd_f64(is_log, dy, y, dx, outer, N, inner, st);
      default: return B2N_ERR_UNSUPPORTED_DTYPE;
    }
  }
  if (grad_dtype == B2N_F32 && dx_dtype == B2N_F16) return softmax_bwd_f16_f32(is_log, dy, y, dx, outer, N, inner, st);
  if (grad_dtype == B2N_F32 && dx_dtype == B2N_BF16) return softmax_bwd_bf16_f32(is_log, dy, y, dx, outer, N, inner, st);
  return B2N_ERR_UNSUPPORTED_DTYPE;
}

}  // namespace b2n
