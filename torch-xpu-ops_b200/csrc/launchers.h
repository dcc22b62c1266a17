// Internal C++ launchers behind the C ABI (one per operator and direction).  Each returns a
// b2n_status and enqueues on `st` without synchronising.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b2n {

int launch_norm_fwd(bool rms, const void* x, const void* gamma, const void* beta, void* y, void* mean,
                    void* rstd, int64_t M, int64_t N, double eps, int x_dtype, int w_dtype,
                    cudaStream_t st);

size_t norm_bwd_workspace_bytes(int64_t M, int64_t N, int x_dtype, int w_dtype, int want_wgrad);

// `workspace` may be any device memory of the required size; the no-allocation entry point passes
// a file-scope device array here.
int launch_norm_bwd(bool rms, const void* dy, const void* x, const void* mean, const void* rstd,
                    const void* gamma, void* dx, void* dgamma, void* dbeta, void* workspace,
                    size_t workspace_bytes, int64_t M, int64_t N, int x_dtype, int w_dtype,
                    cudaStream_t st, int64_t* partials_out = nullptr);
// partials_out != nullptr: the row kernels leave the weight-gradient partial sums workspace[*partials_out][2][N]
// unfolded (dgamma / dbeta are not touched); launch_norm_wgrad_fold turns them into dgamma / dbeta.
int launch_norm_wgrad_fold(const void* workspace, int64_t partial_rows, int64_t N, void* dgamma, void* dbeta,
                           int x_dtype, int w_dtype, cudaStream_t st);

int launch_softmax_fwd(const void* x, void* y, int64_t outer, int64_t N, int64_t inner, int in_dtype,
                       int out_dtype, bool is_log, cudaStream_t st);
int launch_softmax_bwd(const void* dy, const void* y, void* dx, int64_t outer, int64_t N, int64_t inner,
                       int grad_dtype, int dx_dtype, bool is_log, cudaStream_t st);

size_t nll_loss_workspace_bytes(int64_t M);
int launch_nll_loss_fwd(const void* logp, const void* target, const void* weight, void* out,
                        void* total_weight, float* sums_f32, void* workspace, size_t workspace_bytes,
                        int64_t M, int64_t C, int reduction, int64_t ignore_index, int dtype,
                        bool target_is_u8, cudaStream_t st);
int launch_nll_loss_bwd(const void* grad_out, const void* target, const void* weight,
                        const void* total_weight, void* grad_input, int64_t M, int64_t C, int reduction,
                        int64_t ignore_index, int dtype, bool target_is_u8, cudaStream_t st);
int launch_masked_softmax_fwd(const void* x, const void* mask, void* y, int64_t M, int64_t N, int64_t row_div,
                              int64_t row_mod, int dtype, cudaStream_t st);
int launch_masked_softmax_bwd(const void* dy, const void* y, const void* mask, void* dx, int64_t M, int64_t N,
                              int dtype, cudaStream_t st);
int launch_cross_entropy_bwd(const void* logp, const void* target, const void* weight, const void* grad_out,
                             const void* total_weight, void* dx, int64_t M, int64_t C, int reduction,
                             int64_t ignore_index, int dtype, bool target_is_u8, cudaStream_t st);

}  // namespace b2n
