/*
 * b200norm — C ABI of the sm_100a row-wise normalization / softmax kernels.
 *
 * Every entry point enqueues work on the CUDA stream the caller passes (a cudaStream_t cast to
 * void*; NULL = the legacy default stream) and returns without synchronising the host.  The
 * library allocates nothing unless an entry point's comment says otherwise: every input, output
 * and workspace is a device pointer owned by the caller and borrowed only for the duration of the
 * enqueued work.  All tensors are row-major contiguous.  Return value: B2N_OK (0) or a negative
 * b2n_status.  Nothing here throws, aborts or traps.
 *
 * Each entry point replaces one launcher of intel/torch-xpu-ops; the citation next to it gives the
 * reference declaration (path within that project) whose role it takes.
 */
#ifndef B200NORM_H_
#define B200NORM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2N_ABI_VERSION 1

/* element types; values are part of the ABI */
typedef enum b2n_dtype {
  B2N_F32 = 0,
  B2N_F16 = 1,
  B2N_BF16 = 2,
  B2N_F64 = 3
} b2n_dtype;

typedef enum b2n_status {
  B2N_OK = 0,
  B2N_ERR_BAD_ARG = -1,           /* null pointer, negative size, bad enum */
  B2N_ERR_UNSUPPORTED_DTYPE = -2, /* dtype combination has no kernel */
  B2N_ERR_WORKSPACE = -3,         /* workspace missing or too small */
  B2N_ERR_CUDA = -4,              /* a CUDA runtime call failed; see b2n_last_cuda_error */
  B2N_ERR_TIMEOUT = -5,           /* a bounded device-side wait gave up (read via b2n_device_status) */
  B2N_ERR_TARGET_RANGE = -6,      /* nll_loss: a target outside [0, C) that is not ignore_index */
  B2N_ERR_TOO_LARGE = -7          /* size beyond what the entry point accepts */
} b2n_status;

/* reduction modes of nll_loss; same numbering as at::Reduction */
typedef enum b2n_reduction { B2N_REDUCE_NONE = 0, B2N_REDUCE_MEAN = 1, B2N_REDUCE_SUM = 2 } b2n_reduction;

/* kernel family selection, for tests and profiling; B2N_PATH_AUTO is what production uses */
typedef enum b2n_path {
  B2N_PATH_AUTO = 0,
  B2N_PATH_GENERIC = 1, /* global-memory multi-pass kernels: any alignment, any N */
  B2N_PATH_RING = 2,    /* persistent CTAs, bulk-async (TMA) shared-memory ring, register-resident rows */
  B2N_PATH_CLUSTER = 3, /* long rows split over a thread-block cluster, slices resident in shared memory */
  B2N_PATH_TWOPASS = 4  /* long rows streamed through the ring twice, second pass served from L2 */
} b2n_path;

int b2n_abi_version(void);
const char* b2n_strerror(int status);
/* cudaError_t of the most recent failing CUDA call made by this thread inside the library */
int b2n_last_cuda_error(void);
/* Force a kernel family for subsequent calls from this thread (b2n_path); returns the previous
 * value.  A forced family that cannot take a given shape makes the call return
 * B2N_ERR_BAD_ARG instead of silently using another one. */
int b2n_set_path(int path);
/* Launch parameters of the ring kernels, per calling thread (0 restores the automatic choice).
 * Values that do not fit a shape are clamped.  Knobs 0-3 are tuning aids for sweeps; the SM margin
 * is for production use. */
typedef enum b2n_tuning_knob {
  B2N_TUNE_ROWS_PER_GROUP = 0, /* rows of a tile each row group works through (1..4) */
  B2N_TUNE_STAGES = 1,         /* upper bound on the ring depth */
  B2N_TUNE_STORE_LAG = 2,      /* bulk stores left in flight before a stage is refilled (1..3) */
  B2N_TUNE_CLUSTER_SIZE = 3,   /* CTAs per row in the cluster kernels (2, 4 or 8) */
  B2N_TUNE_SM_MARGIN = 4,      /* SMs the persistent kernels leave free, e.g. for the kernel of a collective that
                                  runs beside them on another stream (it cannot share an SM with a ring CTA) */
  B2N_TUNE_TILE_KB = 5         /* non-last-dim softmax: shared memory (KB) one staged tile may take (0: automatic) */
} b2n_tuning_knob;
int b2n_set_tuning(int knob, int value);
/* Diagnostic: while a buffer is set (this thread), one consumer thread of CTA 0 of the layer-norm /
 * RMS-norm forward ring kernel appends event records to it.  Layout (64-bit words, zero the buffer
 * first): word 0 = record count (word 1 belongs to a second writer slot that is unused); then the
 * records, at most cap = (bytes - 16) / 32 of them, each {event << 48 | tile index, %globaltimer
 * ns}.  Events: 1/2 consumer wait begin/end, 3 consumer released the tile, 8+k points inside the
 * consumer's arithmetic (16: kernel entry).  NULL switches it off. */
int b2n_set_trace_buffer(void* device_buffer, size_t bytes);
/* Name of the kernel family the most recent launch from this thread used ("generic", "ring", ...). */
const char* b2n_last_path(void);
/* Reads and clears the device-side status word of the current device (synchronises `stream`).
 * 0, or the b2n_status recorded by a kernel (B2N_ERR_TIMEOUT, B2N_ERR_TARGET_RANGE). */
int b2n_device_status(void* stream);
/* The same word for callers that must not block (a dispatcher binding): b2n_status_post enqueues a
 * copy of the word to a pinned host word behind the work already on `stream`; b2n_status_poll
 * returns 0 while that copy is still to run, else the value it carried (and, when non-zero, clears
 * the device word).  Neither synchronises.  The first b2n_status_post on a device allocates the
 * pinned word and one event (cudaHostAlloc / cudaEventCreate) — the one allocation outside the
 * caller's hands, made off the kernels' path; call it once before a stream capture begins if
 * captures are used.  The reference traps on the device instead (SYCL_KERNEL_ASSERT in
 * src/ATen/native/xpu/sycl/LossNLLKernel.cpp:30-35); a trap is not acceptable on a shared GPU, so
 * the failure surfaces on the host, one call late. */
int b2n_status_post(void* stream);
int b2n_status_poll(void);

/* Number of kernels this thread has launched through the library since it was loaded. */
unsigned long long b2n_launch_count(void);
/* Measurement aid.  Between b2n_profile_begin() and b2n_profile_end() every main kernel launched
 * from this thread (not the small fold / scatter kernels) is bracketed by a pair of CUDA events on
 * its stream.  b2n_profile_end synchronises on them and writes one line per kernel name,
 * "name launches total_milliseconds\n", into report (NUL-terminated, truncated to cap). */
int b2n_profile_begin(void);
int b2n_profile_end(char* report, size_t cap);

/* ---- layer norm / RMS norm ------------------------------------------------------------------
 * x, y: [M, N] of x_dtype.  gamma, beta: [N] of w_dtype or NULL (w_dtype == x_dtype or B2N_F32).
 * mean, rstd: [M] of the accumulate type (float; double when x_dtype == B2N_F64).
 *
 * Replaces at::native::xpu::layer_norm_kernel (src/ATen/native/xpu/sycl/LayerNormKernels.h:19-28)
 * behind layer_norm_xpu (src/ATen/native/xpu/LayerNorm.cpp:35). */
int b2n_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, void* mean,
                       void* rstd, int64_t M, int64_t N, double eps, int x_dtype, int w_dtype,
                       void* stream);

/* Replaces at::native::xpu::rms_norm_kernel (sycl/LayerNormKernels.h:42-49) behind
 * _fused_rms_norm_xpu (LayerNorm.cpp:203).  y = gamma * (x * rstd), rstd = 1/sqrt(mean(x^2)+eps). */
int b2n_rms_norm_fwd(const void* x, const void* gamma, void* y, void* rstd, int64_t M, int64_t N,
                     double eps, int x_dtype, int w_dtype, void* stream);

/* Bytes of scratch the two backward entry points need for the weight-gradient partial sums
 * (0 when neither dgamma nor dbeta is requested). */
size_t b2n_norm_bwd_workspace_bytes(int64_t M, int64_t N, int x_dtype, int w_dtype, int want_wgrad);

/* dx (x_dtype, [M,N]), dgamma / dbeta (w_dtype, [N]); any of the three may be NULL (masked off).
 * workspace: >= b2n_norm_bwd_workspace_bytes(...) bytes, 256-byte aligned, contents ignored.
 * The weight gradients are summed in a fixed order: bit-reproducible from run to run.
 *
 * Replaces at::native::xpu::layer_norm_backward_kernel (sycl/LayerNormKernels.h:30-40) behind
 * layer_norm_backward_xpu (LayerNorm.cpp:99). */
int b2n_layer_norm_bwd(const void* dy, const void* x, const void* mean, const void* rstd,
                       const void* gamma, void* dx, void* dgamma, void* dbeta, void* workspace,
                       size_t workspace_bytes, int64_t M, int64_t N, int x_dtype, int w_dtype,
                       void* stream);

/* No counterpart in the reference: the same backward for callers that cannot allocate — an
 * inference engine's plug-in enqueue callback, a serving loop with a frozen memory pool, a
 * process whose device memory already belongs to another allocator — and so have no workspace
 * to pass.  The weight-gradient partial sums live in a fixed device array inside the library
 * (b2n_noalloc_scratch_bytes() = 16 MiB, held by every GPU that loads the library until the
 * process exits); nothing is allocated on the call path.  Problems that need more scratch than
 * that (b2n_norm_bwd_workspace_bytes(...) > 16 MiB) return B2N_ERR_TOO_LARGE.  All calls on a
 * device share the array, so calls that overlap on the GPU race: serialise them.  The first call
 * on a device looks up the array's address; make it before any stream capture begins.  Results
 * equal b2n_layer_norm_bwd's. */
size_t b2n_noalloc_scratch_bytes(void);
int b2n_layer_norm_bwd_noalloc(const void* dy, const void* x, const void* mean, const void* rstd,
                               const void* gamma, void* dx, void* dgamma, void* dbeta, int64_t M,
                               int64_t N, int x_dtype, int w_dtype, void* stream);

/* Replaces at::native::xpu::rms_norm_backward_kernel (sycl/LayerNormKernels.h:51-58) behind
 * _fused_rms_norm_backward_xpu (LayerNorm.cpp:255). */
int b2n_rms_norm_bwd(const void* dy, const void* x, const void* rstd, const void* gamma, void* dx,
                     void* dgamma, void* workspace, size_t workspace_bytes, int64_t M, int64_t N,
                     int x_dtype, int w_dtype, void* stream);

/* The backward in two steps, for a row-sharded caller: the row kernels write dx and leave the
 * weight-gradient partial sums workspace[*partial_rows][2][N] (accumulate type) unfolded;
 * b2n_norm_wgrad_fold adds the partial rows in index order into dgamma / dbeta (either may be NULL;
 * RMS norm has no dbeta).  Together they produce exactly what b2n_layer_norm_bwd / b2n_rms_norm_bwd
 * produce — the one-call entry points run the same two kernels back to back.  Split, the fold (and
 * the all-reduce of its [dgamma | dbeta] output that follows it on every rank) can be enqueued on a
 * second stream behind an event, so the next operator's row kernel starts right behind this one's
 * instead of behind the fold.  rms != 0: RMS norm (mean is ignored).  The workspace must stay
 * untouched until the fold has run.
 *
 * The reference reduces the same way in two stages on one queue: GammaBetaReduceFunctor writes
 * [num_tile_m, N] partial tiles which `blocks.sum(0)` then adds
 * (src/ATen/native/xpu/sycl/LayerNormKernels.cpp:701-874, :1196-1407). */
int b2n_norm_bwd_partials(int rms, const void* dy, const void* x, const void* mean, const void* rstd,
                          const void* gamma, void* dx, void* workspace, size_t workspace_bytes,
                          int64_t M, int64_t N, int x_dtype, int w_dtype, int64_t* partial_rows,
                          void* stream);
int b2n_norm_wgrad_fold(const void* workspace, int64_t partial_rows, int64_t N, void* dgamma,
                        void* dbeta, int x_dtype, int w_dtype, void* stream);

/* No counterpart in the reference (it leaves the gradient exchange to c10d's all-reduce,
 * src/xccl/ProcessGroupXCCL.cpp:1327-1344): b2n_norm_wgrad_fold and the all-reduce(SUM) of its
 * [dgamma | dbeta] result over the ranks of one node as ONE kernel over peer memory.  Every CTA folds
 * its slice of the local partial sums into this rank's exchange buffer, raises a flag in every peer's
 * buffer, waits (bounded: B2N_ERR_TIMEOUT in the device status word) for the peers' flags, reads the
 * peers' slices with plain peer loads and adds all ranks' slices in rank order — every rank ends
 * with the same bits.  No multicast, no library collective.
 *
 * peer_buffers: host array of `world` device pointers, entry r = rank r's exchange buffer as mapped
 * into THIS process (entry `rank` = the local one); each buffer has b2n_wgrad_exchange_bytes(n_max)
 * bytes, zeroed once before first use, 16-byte aligned, mapped so that peer loads and stores from this
 * device are legal (b2n_wgrad_exchange_alloc / _open below do all of that).  world <= 8, N % 4 == 0, N <= n_max.
 * ctas: CTAs to use (1..256): ~128 when the kernel has the GPU to itself, as few as the SMs left
 * free when it runs on a second stream beside persistent kernels.  All ranks must make the same
 * sequence of calls on a buffer, and one buffer serves one (N, ctas) configuration.  dgamma / dbeta
 * of w_dtype (dbeta NULL for RMS norm).  The kernel advances its generation counters itself, so a
 * captured launch can be replayed from a CUDA graph unchanged. */
size_t b2n_wgrad_exchange_bytes(int64_t n_max);
/* The exchange buffers.  These four calls DO allocate / map device memory, once, at set-up:
 * _alloc: cudaMalloc of b2n_wgrad_exchange_bytes(n_max) zeroed bytes on the current device, and its
 *   64-byte CUDA IPC handle for the other ranks (processes) of the node;
 * _open: maps a peer's handle into this process — call it with THIS rank's device current: the
 *   mapping must belong to the context whose kernels use it, and cudaIpcMemLazyEnablePeerAccess then
 *   switches peer access on for that pair (a handle cannot be opened by the process that exported it);
 * _close / _free: undo them, after the last kernel that uses the buffers has finished. */
int b2n_wgrad_exchange_alloc(int64_t n_max, void** local, unsigned char* handle64);
int b2n_wgrad_exchange_open(const unsigned char* handle64, void** mapped);
int b2n_wgrad_exchange_close(void* mapped);
int b2n_wgrad_exchange_free(void* local);
int b2n_norm_wgrad_fold_allreduce(const void* workspace, int64_t partial_rows, int64_t N,
                                  void* const* peer_buffers, int64_t n_max, int rank, int world,
                                  void* dgamma, void* dbeta, int w_dtype, int ctas, void* stream);

/* ---- sibling norms -------------------------------------------------------------------------------
 * GroupNorm forward over a contiguous [N, C, HxW] tensor with G groups (C % G == 0): per (n, g) the
 * mean and 1/sqrt(var + eps) of the D * HxW elements of the group (D = C / G), then
 * y = (x - mean) * rstd * gamma[c] + beta[c] per channel c.  gamma, beta: [C] of w_dtype or NULL
 * (w_dtype == x_dtype, or B2N_F32 with 16-bit x); mean, rstd: [N * G] of stat_dtype (x_dtype, or
 * B2N_F32 when the weights are fp32).  A group may hold at most 2^31 - 1 elements.
 *
 * Replaces at::native::xpu::group_norm_kernel (src/ATen/native/xpu/sycl/GroupNormKernels.h:17-28;
 * moments GroupNormKernels.cpp:73-136, driver :365-499) behind the GroupNormKernel dispatch stub
 * (src/ATen/native/xpu/GroupNorm.cpp:20). */
int b2n_group_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, void* mean,
                       void* rstd, int64_t N, int64_t C, int64_t HxW, int64_t G, double eps,
                       int x_dtype, int w_dtype, int stat_dtype, void* stream);

/* GroupNorm backward from the forward's saved statistics (mean, rstd: [N * G] of stat_dtype):
 * dx [N, C, HxW] of x_dtype, dgamma / dbeta [C] of w_dtype; any of the three may be NULL (not wanted).  gamma may be
 * NULL (ones).  With xhat = (x - mean) * rstd and g = dy * gamma[c]:
 * dx = rstd * (g - (xhat * sum(g * xhat) + sum(g)) / (D * HxW)) per (n, group) row;
 * dgamma[c] = sum over n, HxW of dy * xhat; dbeta[c] = sum dy.  An element of the N = 0 / HxW = 0 corner writes nothing.
 *
 * Replaces at::native::xpu::group_norm_backward_kernel (src/ATen/native/xpu/sycl/GroupNormKernels.h:30-42) behind the
 * GroupNormBackwardKernel dispatch stub (src/ATen/native/xpu/GroupNorm.cpp:23). */
int b2n_group_norm_bwd(const void* dy, const void* x, const void* mean, const void* rstd,
                       const void* gamma, void* dx, void* dgamma, void* dbeta, int64_t N, int64_t C,
                       int64_t HxW, int64_t G, int x_dtype, int w_dtype, int stat_dtype, void* stream);
/* The same with a caller-allocated scratch area (size from b2n_group_norm_bwd_workspace_bytes, 0: none is useful;
 * contents ignored on entry; 16-byte aligned): the weight gradients are then summed by every SM whatever C is, parts
 * added in a fixed order, instead of by one CTA per channel. */
size_t b2n_group_norm_bwd_workspace_bytes(int64_t N, int64_t C, int64_t HxW, int x_dtype);
int b2n_group_norm_bwd_ws(const void* dy, const void* x, const void* mean, const void* rstd,
                          const void* gamma, void* dx, void* dgamma, void* dbeta, int64_t N, int64_t C,
                          int64_t HxW, int64_t G, int x_dtype, int w_dtype, int stat_dtype, void* workspace,
                          size_t workspace_bytes, void* stream);

/* BatchNorm statistics of a contiguous [N, C, HxW] tensor, per channel over N and HxW, in fp32:
 * mean[C] and, mode 0, second[C] = 1 / sqrt(biased var + eps) (batch_norm_stats); mode 1,
 * second[C] = biased var, and running_mean / running_var ([C] of running_dtype = x_dtype or
 * B2N_F32; either may be NULL) are blended in place with `momentum`, the variance unbiased by
 * n / (n - 1) (batch_norm_update_stats).
 *
 * Replaces batch_norm_stats_kernel and batch_norm_update_stats_kernel
 * (src/ATen/native/xpu/sycl/BatchNormKernels.h:19, :52; BatchNormKernels.cpp:992, :3864) behind
 * batch_norm_stats_xpu / batch_norm_update_stats_xpu (src/ATen/native/xpu/BatchNorm.cpp:20, :76). */
int b2n_batch_norm_stats(const void* x, float* mean, float* second, void* running_mean,
                         void* running_var, int64_t N, int64_t C, int64_t HxW, double eps,
                         double momentum, int mode, int x_dtype, int running_dtype, void* stream);

/* The same with a caller-allocated scratch area, which lets several CTAs share a channel (few channels, or
 * channels with much data, would otherwise leave most of the GPU idle: one CTA per channel).  The size comes
 * from b2n_batch_norm_stats_workspace_bytes (0: no scratch is useful for the shape); contents are ignored on
 * entry; `workspace` 16-byte aligned.  With workspace == NULL, or too small, this is b2n_batch_norm_stats.
 * Results do not depend on the order in which the CTAs finish (partial sums are added in a fixed order).
 * The reference reduces a channel inside one work-group or with its own two-stage scheme
 * (sycl/BatchNormKernels.cpp:992 ff.); the scratch is this build's equivalent of its staging buffers. */
size_t b2n_batch_norm_stats_workspace_bytes(int64_t N, int64_t C, int64_t HxW, int x_dtype);
int b2n_batch_norm_stats_ws(const void* x, float* mean, float* second, void* running_mean,
                            void* running_var, int64_t N, int64_t C, int64_t HxW, double eps,
                            double momentum, int mode, int x_dtype, int running_dtype, void* workspace,
                            size_t workspace_bytes, void* stream);

/* ---- softmax / log-softmax --------------------------------------------------------------------
 * The tensor is viewed as [outer, N, inner]; the reduction runs over N (inner == 1 for the last
 * dim).  out_dtype == in_dtype, or B2N_F32 with a 16-bit input ("half_to_float").
 * is_log: 0 softmax, 1 log-softmax, 2 "safe" softmax — a row whose every element is -inf gives
 * zeros instead of NaN (a row that also holds a NaN still gives NaN).
 *
 * Replaces at::native::xpu::_softmax_kernel / _log_softmax_kernel
 * (src/ATen/native/xpu/sycl/SoftMaxKernels.h:19-29) behind softmax_xpu_out / log_softmax_xpu_out
 * (src/ATen/native/xpu/SoftMax.cpp:22, :94); mode 2 replaces _safe_softmax_kernel
 * (SoftMaxKernels.h, host_softmax<false, true> in SoftMaxKernels.cpp:2125-2178) behind
 * _safe_softmax_xpu (SoftMax.cpp:102-126). */
int b2n_softmax_fwd(const void* x, void* y, int64_t outer, int64_t N, int64_t inner, int in_dtype,
                    int out_dtype, int is_log, void* stream);

/* Host-only query, no device needed: the shared-memory tile geometry the library uses for softmax over a dim
 * that is NOT the last ([outer, N, inner], inner > 1) on tensor-map TMA tiles, for a GPU with `sm_count` SMs and
 * `max_smem_bytes` of opt-in shared memory per CTA.  out[8] = {fits (0: another kernel family takes the shape),
 * box width W in elements, boxes per tile, rows per box, stages, threads per line, forward-in-registers flag,
 * dynamic shared memory in bytes}.  Invariants a caller (and the tests) can rely on when fits == 1:
 * W * elem_size is a multiple of 128 bytes and W <= 256; (W * boxes / columns-per-thread) * threads-per-line <= 512;
 * at least two stages; the shared memory fits.  The reference has no counterpart: its spatial kernels
 * (sycl/SoftMaxKernels.cpp:735-950) pick their work-group shape inside the launcher. */
int b2n_softmax_tile_plan(int64_t outer, int64_t N, int64_t inner, int elem_size, int backward, int sm_count,
                          int64_t max_smem_bytes, int* out);

/* dy: grad_dtype; y (forward output): grad_dtype; dx: dx_dtype (== grad_dtype, or a 16-bit type
 * with grad_dtype == B2N_F32 for the half_to_float backward).
 * softmax: dx = y*(dy - sum(y*dy)); log-softmax: dx = dy - exp(y)*sum(dy).
 *
 * Replaces _softmax_backward_kernel / _log_softmax_backward_kernel (sycl/SoftMaxKernels.h:31-43)
 * behind softmax_backward_xpu_out / log_softmax_backward_xpu_out (SoftMax.cpp:30, :61). */
int b2n_softmax_bwd(const void* dy, const void* y, void* dx, int64_t outer, int64_t N,
                    int64_t inner, int grad_dtype, int dx_dtype, int is_log, void* stream);

/* ---- masked softmax (last dim) -----------------------------------------------------------------
 * x, y: [M, N] of dtype; mask: bytes (a bool tensor), non-zero = masked out.  The mask row of
 * input row r is (r / mask_row_div) % mask_row_mod: (1, M) for a mask of the input's shape, (1, T)
 * for a [T, T] mask shared by every batch and head of a [B, H, T, T] input, (H*T, B) for a [B, T]
 * key-padding mask.  Masked elements give 0; a row with nothing left unmasked gives NaN.
 * Backward: mask of the gradient's shape; dx = y * (dy - sum over unmasked of y*dy), 0 where masked.
 *
 * Replaces masked_softmax_kernel / masked_softmax_backward_kernel
 * (src/ATen/native/xpu/sycl/SoftMaxKernels.cpp:2301-2362, :2364-2407) behind masked_softmax_xpu /
 * masked_softmax_backward_xpu (src/ATen/native/xpu/SoftMax.cpp:112-126) for the last dim; the
 * binding composes other dims from masked_fill and the plain softmax entry points. */
int b2n_masked_softmax_fwd(const void* x, const void* mask, void* y, int64_t M, int64_t N,
                           int64_t mask_row_div, int64_t mask_row_mod, int dtype, void* stream);
int b2n_masked_softmax_bwd(const void* dy, const void* y, const void* mask, void* dx, int64_t M,
                           int64_t N, int dtype, void* stream);

/* ---- nll_loss ---------------------------------------------------------------------------------
 * logp: [M, C] of dtype; target: [M] int64 (target_is_u8 == 0) or uint8; weight: [C] of dtype or
 * NULL.  reduction none: out[M]; mean/sum: out[1].  total_weight[1] of dtype.
 * sums_f32: optional device float[2] that receives {sum_i -w[t_i]*logp[i,t_i], sum_i w[t_i]} before
 * the mean division (what a row-sharded caller all-reduces); may be NULL.
 * workspace: >= b2n_nll_loss_workspace_bytes(M) bytes.
 * A target outside [0, C) other than ignore_index contributes nothing and records
 * B2N_ERR_TARGET_RANGE in the device status word (the reference asserts on the device instead).
 *
 * Replaces at::native::xpu::nll_loss_forward_kernel (src/ATen/native/xpu/sycl/LossNLLKernel.h)
 * behind nll_loss_forward_out_xpu (src/ATen/native/xpu/LossNLL.cpp:22). */
size_t b2n_nll_loss_workspace_bytes(int64_t M);
int b2n_nll_loss_fwd(const void* logp, const void* target, const void* weight, void* out,
                     void* total_weight, float* sums_f32, void* workspace, size_t workspace_bytes,
                     int64_t M, int64_t C, int reduction, int64_t ignore_index, int dtype,
                     int target_is_u8, void* stream);

/* grad_input [M, C] is zero-filled, then grad_input[i, t_i] = -w[t_i] * g (/ total_weight for
 * mean), g = grad_out[i] (none) or grad_out[0].
 *
 * Replaces at::native::xpu::nll_loss_backward_kernel (sycl/LossNLLKernel.h) behind
 * nll_loss_backward_out_xpu (LossNLL.cpp:35), including its grad_input.zero_(). */
int b2n_nll_loss_bwd(const void* grad_out, const void* target, const void* weight,
                     const void* total_weight, void* grad_input, int64_t M, int64_t C,
                     int reduction, int64_t ignore_index, int dtype, int target_is_u8,
                     void* stream);

/* ---- fused cross-entropy tail -------------------------------------------------------------------
 * b2n_nll_loss_bwd followed by b2n_softmax_bwd(is_log = 1) in one pass, without the dense [M, C]
 * gradient between them:
 *   dx[i, j] = s_i * (exp(logp[i, j]) - [j == target_i]),
 *   s_i = w[t_i] * g (/ total_weight for mean), g = grad_out[i] (none) or grad_out[0];
 * rows whose target is ignore_index are zero.  logp is the output of b2n_softmax_fwd(is_log = 1);
 * dx may alias logp.  One read and one write per element instead of the pair's write + two reads +
 * write.  Out-of-range targets are treated like b2n_nll_loss_fwd treats them.
 *
 * The reference has no single entry point for this: it is the composition its callers reach
 * through autograd, nll_loss_backward_out_xpu (src/ATen/native/xpu/LossNLL.cpp:35-56, kernel
 * sycl/LossNLLKernel.cpp:325-380) then log_softmax_backward_xpu_out (SoftMax.cpp:61-92); results
 * equal that composition evaluated in fp32. */
int b2n_cross_entropy_bwd(const void* logp, const void* target, const void* weight,
                          const void* grad_out, const void* total_weight, void* dx, int64_t M,
                          int64_t C, int reduction, int64_t ignore_index, int dtype,
                          int target_is_u8, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200NORM_H_ */
