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

// Host-only: the tile geometry softmax_spatial_tma_launch would use (see the header for the fields).
extern "C" int b2n_softmax_tile_plan(int64_t outer, int64_t N, int64_t inner, int elem_size, int backward, int sm_count,
                                     int64_t max_smem_bytes, int* out) {
  if (out == nullptr || outer < 1 || N < 1 || inner < 1 || (elem_size != 2 && elem_size != 4) || sm_count < 1 ||
      max_smem_bytes <= b2n::kTmaHeaderBytes)
    return B2N_ERR_BAD_ARG;
  const int nin = backward ? 2 : 1;
  b2n::TmaTilePlan p;
  if (N >= 2 && N <= 65536 && outer <= 0x7fffffffLL && inner <= 0x7fffffffLL && (inner * elem_size) % 16 == 0 &&
      N * inner * elem_size < (1ll << 40))
    p = b2n::plan_tma_tile(outer, N, inner, elem_size, nin, backward != 0, max_smem_bytes - b2n::kTmaHeaderBytes, sm_count);
  const int64_t npad = p.ok ? (N + p.NB - 1) / p.NB * p.NB : 0;
  out[0] = p.ok ? 1 : 0;
  out[1] = p.W;
  out[2] = p.NX;
  out[3] = p.NB;
  out[4] = p.S;
  out[5] = p.segs;
  out[6] = p.reg ? 1 : 0;
  out[7] = p.ok ? static_cast<int>(b2n::kTmaHeaderBytes + static_cast<int64_t>(p.S) * npad * p.W * p.NX * elem_size * nin) : 0;
  return B2N_OK;
}
