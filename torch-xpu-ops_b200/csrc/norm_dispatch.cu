// dtype dispatch for layer norm / RMS norm: picks the (x type, weight type) instantiation.
#include "norm_launch.cuh"

namespace b2n {

namespace {
enum Combo { C_F32, C_F16, C_F16_W32, C_BF16, C_BF16_W32, C_F64, C_NONE };
Combo combo_of(int x_dtype, int w_dtype) {
  if (x_dtype == B2N_F32 && w_dtype == B2N_F32) return C_F32;
  if (x_dtype == B2N_F16 && w_dtype == B2N_F16) return C_F16;
  if (x_dtype == B2N_F16 && w_dtype == B2N_F32) return C_F16_W32;
  if (x_dtype == B2N_BF16 && w_dtype == B2N_BF16) return C_BF16;
  if (x_dtype == B2N_BF16 && w_dtype == B2N_F32) return C_BF16_W32;
  if (x_dtype == B2N_F64 && w_dtype == B2N_F64) return C_F64;
  return C_NONE;
}
}  // namespace

int launch_norm_fwd(bool rms, const void* x, const void* gamma, const void* beta, void* y, void* mean,
                    void* rstd, int64_t M, int64_t N, double eps, int x_dtype, int w_dtype, cudaStream_t st) {
  switch (combo_of(x_dtype, w_dtype)) {
    case C_F32: return norm_fwd_f32(rms, x, gamma, beta, y, mean, rstd, M, N, eps, st);
    case C_F16: return norm_fwd_f16(rms, x, gamma, beta, y, mean, rstd, M, N, eps, st);
    case C_F16_W32: return norm_fwd_f16_w32(rms, x, gamma, beta, y, mean, rstd, M, N, eps, st);
    case C_BF16: return norm_fwd_bf16(rms, x, gamma, beta, y, mean, rstd, M, N, eps, st);
    case C_BF16_W32: return norm_fwd_bf16_w32(rms, x, gamma, beta, y, mean, rstd, M, N, eps, st);
    case C_F64: return norm_fwd_f64(rms, x, gamma, beta, y, mean, rstd, M, N, eps, st);
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

size_t norm_bwd_workspace_bytes(int64_t M, int64_t N, int x_dtype, int w_dtype, int want_wgrad) {
  (void)w_dtype;
  if (!want_wgrad || M <= 0 || N <= 0) return 0;
  switch (x_dtype) {
    case B2N_F32: return norm_bwd_ws_f32(M, N);
    case B2N_F16: return norm_bwd_ws_f16(M, N);
    case B2N_BF16: return norm_bwd_ws_bf16(M, N);
    case B2N_F64: return norm_bwd_ws_f64(M, N);
    default: return 0;
  }
}

int launch_norm_bwd(bool rms, const void* dy, const void* x, const void* mean, const void* rstd,
                    const void* gamma, void* dx, void* dgamma, void* dbeta, void* ws, size_t ws_bytes,
                    int64_t M, int64_t N, int x_dtype, int w_dtype, cudaStream_t st, int64_t* partials_out) {
  switch (combo_of(x_dtype, w_dtype)) {
    case C_F32: return norm_bwd_f32(rms, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out);
    case C_F16: return norm_bwd_f16(rms, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out);
    case C_F16_W32: return norm_bwd_f16_w32(rms, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out);
    case C_BF16: return norm_bwd_bf16(rms, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out);
    case C_BF16_W32: return norm_bwd_bf16_w32(rms, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out);
    case C_F64: return norm_bwd_f64(rms, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out);
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

int launch_norm_wgrad_fold(const void* ws, int64_t P, int64_t N, void* dgamma, void* dbeta, int x_dtype, int w_dtype,
                           cudaStream_t st) {
  switch (combo_of(x_dtype, w_dtype)) {
    case C_F32: return norm_fold_f32(ws, P, N, dgamma, dbeta, st);
    case C_F16: return norm_fold_f16(ws, P, N, dgamma, dbeta, st);
    case C_F16_W32: return norm_fold_f16_w32(ws, P, N, dgamma, dbeta, st);
    case C_BF16: return norm_fold_bf16(ws, P, N, dgamma, dbeta, st);
    case C_BF16_W32: return norm_fold_bf16_w32(ws, P, N, dgamma, dbeta, st);
    case C_F64: return norm_fold_f64(ws, P, N, dgamma, dbeta, st);
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

}  // namespace b2n
