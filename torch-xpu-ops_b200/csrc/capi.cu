// The C ABI declared in include/b200norm.h: argument validation, then the typed launchers.
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "launchers.h"
#include "plan.h"

namespace b2n {

namespace {
constexpr int kMaxDevices = 64;
__device__ int g_status_word = 0;  // one per device (each device that loads the module has its own)
// Tile-counter slots of the ring kernels: {next tile, CTAs finished} pairs, all zero between
// launches (the last CTA of a launch zeroes its pair).  Launches take slots in rotation, so two
// launches share a pair only if kTileCounterSlots launches were in flight at once.
constexpr unsigned kTileCounterSlots = 4096;
__device__ unsigned g_tile_counters[2 * kTileCounterSlots];
std::atomic<unsigned> g_next_counter_slot{0};

thread_local int tl_last_cuda_error = 0;
thread_local int tl_forced_path = B2N_PATH_AUTO;
thread_local bool tl_softmax_safe = false;
thread_local const char* tl_last_path = "none";
thread_local unsigned long long tl_launches = 0;

struct ProfileRecord { const char* name; cudaEvent_t start, stop; };
thread_local bool tl_profiling = false;
thread_local std::vector<ProfileRecord> tl_records;
constexpr size_t kMaxProfileRecords = 1 << 16;

struct PerDevice {
  std::mutex mu;
  std::atomic<bool> ready{false};
  DeviceInfo info{};
  int* status_ptr = nullptr;
  unsigned* counters = nullptr;
  // deferred status probe (b2n_status_post / b2n_status_poll): a pinned host word the status is copied
  // to behind the caller's work, and the event that says the copy has happened
  int* probe_host = nullptr;
  cudaEvent_t probe_event = nullptr;
  cudaStream_t probe_stream = nullptr;
  bool probe_pending = false;
};
PerDevice g_devices[kMaxDevices];

// Per-device set-up: attributes and the device addresses of the library's own words.  Only a
// complete set-up is remembered; a failed lookup (a sticky error pending, a stream capture under
// way) is tried again on the next call instead of leaving null pointers behind for good.
PerDevice& current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  PerDevice& pd = g_devices[dev % kMaxDevices];
  if (pd.ready.load(std::memory_order_acquire)) return pd;
  std::lock_guard<std::mutex> lock(pd.mu);
  if (pd.ready.load(std::memory_order_relaxed)) return pd;
  bool ok = cudaDeviceGetAttribute(&pd.info.sm_count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
  ok = ok && cudaDeviceGetAttribute(&pd.info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess;
  void* p = nullptr;
  if (ok && cudaGetSymbolAddress(&p, g_status_word) == cudaSuccess) pd.status_ptr = static_cast<int*>(p);
  if (ok && cudaGetSymbolAddress(&p, g_tile_counters) == cudaSuccess) pd.counters = static_cast<unsigned*>(p);
  if (ok && pd.status_ptr != nullptr && pd.counters != nullptr) pd.ready.store(true, std::memory_order_release);
  else cudaGetLastError();  // the failure is reported by the launch that needed the pointers
  return pd;
}
}  // namespace

const DeviceInfo& device_info() { return current_device().info; }
bool device_ready() { return current_device().ready.load(std::memory_order_acquire); }
int* device_status_ptr() { return current_device().status_ptr; }
bool softmax_safe_mode() { return tl_softmax_safe; }
unsigned* next_tile_counter() {
  unsigned* base = current_device().counters;
  if (base == nullptr) return nullptr;
  return base + 2 * (g_next_counter_slot.fetch_add(1, std::memory_order_relaxed) % kTileCounterSlots);
}
int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return B2N_OK;
  tl_last_cuda_error = static_cast<int>(e);
  return B2N_ERR_CUDA;
}
int launched() {
  ++tl_launches;
  return check_cuda(cudaGetLastError());
}

ProfileScope::ProfileScope(const char* kernel_name, cudaStream_t st) : slot(-1), stream(st) {
  if (!tl_profiling || tl_records.size() >= kMaxProfileRecords) return;
  ProfileRecord r{kernel_name, nullptr, nullptr};
  if (cudaEventCreate(&r.start) != cudaSuccess) return;
  if (cudaEventCreate(&r.stop) != cudaSuccess) { cudaEventDestroy(r.start); return; }
  cudaEventRecord(r.start, st);
  slot = static_cast<int>(tl_records.size());
  tl_records.push_back(r);
}
ProfileScope::~ProfileScope() {
  if (slot >= 0) cudaEventRecord(tl_records[slot].stop, stream);
}

RingTuning& ring_tuning() {
  thread_local RingTuning t;
  return t;
}

int forced_path() { return tl_forced_path; }
void note_path(const char* name) { tl_last_path = name; }

static bool valid_dtype(int dt) { return dt >= B2N_F32 && dt <= B2N_F64; }

}  // namespace b2n

using namespace b2n;

extern "C" {

int b2n_abi_version(void) { return B2N_ABI_VERSION; }

const char* b2n_strerror(int status) {
  switch (status) {
    case B2N_OK: return "ok";
    case B2N_ERR_BAD_ARG: return "bad argument";
    case B2N_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype combination";
    case B2N_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case B2N_ERR_CUDA: return "CUDA runtime error";
    case B2N_ERR_TIMEOUT: return "bounded device-side wait gave up";
    case B2N_ERR_TARGET_RANGE: return "nll_loss target out of range";
    case B2N_ERR_TOO_LARGE: return "size beyond the entry point's limit";
    default: return "unknown status";
  }
}

int b2n_last_cuda_error(void) { return tl_last_cuda_error; }

int b2n_set_path(int path) {
  const int prev = tl_forced_path;
  if (path >= B2N_PATH_AUTO && path <= B2N_PATH_TWOPASS) tl_forced_path = path;
  return prev;
}

const char* b2n_last_path(void) { return tl_last_path; }

int b2n_set_trace_buffer(void* device_buffer, size_t bytes) {
  RingTuning& t = ring_tuning();
  if (device_buffer == nullptr || bytes < 80) {
    t.trace_buf = nullptr;
    t.trace_cap = 0;
    return B2N_OK;
  }
  t.trace_buf = static_cast<unsigned long long*>(device_buffer);
  t.trace_cap = static_cast<unsigned>((bytes - 16) / 32);  // two writers, 16 bytes per record
  return B2N_OK;
}

int b2n_set_tuning(int knob, int value) {
  RingTuning& t = ring_tuning();
  if (value < 0) return B2N_ERR_BAD_ARG;
  switch (knob) {
    case B2N_TUNE_ROWS_PER_GROUP: t.rpg = value; return B2N_OK;
    case B2N_TUNE_STAGES: t.stages = value; return B2N_OK;
    case B2N_TUNE_STORE_LAG: t.lag = value; return B2N_OK;
    case B2N_TUNE_CLUSTER_SIZE: t.cluster = value; return B2N_OK;
    case B2N_TUNE_SM_MARGIN: t.sm_margin = value; return B2N_OK;
    case B2N_TUNE_TILE_KB: t.tile_kb = value; return B2N_OK;
    default: return B2N_ERR_BAD_ARG;
  }
}

unsigned long long b2n_launch_count(void) { return tl_launches; }

int b2n_profile_begin(void) {
  for (auto& r : tl_records) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
  tl_records.clear();
  tl_profiling = true;
  return B2N_OK;
}

int b2n_profile_end(char* report, size_t cap) {
  tl_profiling = false;
  struct Agg { const char* name; int launches; double ms; };
  std::vector<Agg> aggs;
  int rc = B2N_OK;
  for (auto& r : tl_records) {
    float ms = 0.0f;
    if (check_cuda(cudaEventSynchronize(r.stop)) || check_cuda(cudaEventElapsedTime(&ms, r.start, r.stop))) rc = B2N_ERR_CUDA;
    size_t k = 0;
    for (; k < aggs.size(); ++k)
      if (std::string(aggs[k].name) == r.name) break;
    if (k == aggs.size()) aggs.push_back({r.name, 0, 0.0});
    aggs[k].launches += 1;
    aggs[k].ms += ms;
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  tl_records.clear();
  std::string out;
  for (auto& a : aggs) out += std::string(a.name) + " " + std::to_string(a.launches) + " " + std::to_string(a.ms) + "\n";
  if (report != nullptr && cap > 0) {
    const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
    out.copy(report, n);
    report[n] = 0;
  }
  return rc;
}

int b2n_device_status(void* stream) {
  int* p = device_status_ptr();
  if (p == nullptr) return B2N_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int v = 0;
  if (check_cuda(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, st))) return B2N_ERR_CUDA;
  if (check_cuda(cudaStreamSynchronize(st))) return B2N_ERR_CUDA;
  if (v != 0) {
    if (check_cuda(cudaMemsetAsync(p, 0, sizeof(int), st))) return B2N_ERR_CUDA;
    // A kernel that gave up on a wait may have left its {next tile, finished} pair non-zero; the slot would
    // be handed to another launch kTileCounterSlots launches later.  Nothing of this library is running on
    // `st` now, so put every pair back to zero.
    unsigned* ctrs = current_device().counters;
    if (v == B2N_ERR_TIMEOUT && ctrs != nullptr &&
        check_cuda(cudaMemsetAsync(ctrs, 0, 2 * kTileCounterSlots * sizeof(unsigned), st)))
      return B2N_ERR_CUDA;
    if (check_cuda(cudaStreamSynchronize(st))) return B2N_ERR_CUDA;
  }
  return v;
}

int b2n_status_post(void* stream) {
  PerDevice& pd = current_device();
  if (!pd.ready.load(std::memory_order_acquire)) return B2N_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  std::lock_guard<std::mutex> lock(pd.mu);
  if (pd.probe_host == nullptr) {
    if (check_cuda(cudaHostAlloc(reinterpret_cast<void**>(&pd.probe_host), sizeof(int), cudaHostAllocDefault))) return B2N_ERR_CUDA;
    *pd.probe_host = 0;
    if (check_cuda(cudaEventCreateWithFlags(&pd.probe_event, cudaEventDisableTiming))) return B2N_ERR_CUDA;
  }
  if (pd.probe_pending) return B2N_OK;  // one probe in flight is enough: it sees whatever is recorded before it runs ... or the next one does
  if (check_cuda(cudaMemcpyAsync(pd.probe_host, pd.status_ptr, sizeof(int), cudaMemcpyDeviceToHost, st))) return B2N_ERR_CUDA;
  if (check_cuda(cudaEventRecord(pd.probe_event, st))) return B2N_ERR_CUDA;
  pd.probe_stream = st;
  pd.probe_pending = true;
  return B2N_OK;
}

int b2n_status_poll(void) {
  PerDevice& pd = current_device();
  if (!pd.ready.load(std::memory_order_acquire)) return B2N_OK;
  std::lock_guard<std::mutex> lock(pd.mu);
  if (!pd.probe_pending) return B2N_OK;
  const cudaError_t q = cudaEventQuery(pd.probe_event);
  if (q == cudaErrorNotReady) return B2N_OK;
  pd.probe_pending = false;
  if (q != cudaSuccess) return check_cuda(q);
  const int v = *pd.probe_host;
  if (v != 0) {
    *pd.probe_host = 0;
    // clear the device word behind the work already queued on the probe's stream, so the same failure is
    // reported once
    cudaMemsetAsync(pd.status_ptr, 0, sizeof(int), pd.probe_stream);
  }
  return v;
}

int b2n_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, void* mean, void* rstd,
                       int64_t M, int64_t N, double eps, int x_dtype, int w_dtype, void* stream) {
  if (M < 0 || N < 0 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return B2N_ERR_BAD_ARG;
  if (M == 0) return B2N_OK;
  if (!x || !y || !mean || !rstd) return B2N_ERR_BAD_ARG;
  if (gamma == nullptr && beta == nullptr) w_dtype = x_dtype;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_norm_fwd(false, x, gamma, beta, y, mean, rstd, M, N, eps, x_dtype, w_dtype,
                         static_cast<cudaStream_t>(stream));
}

int b2n_rms_norm_fwd(const void* x, const void* gamma, void* y, void* rstd, int64_t M, int64_t N, double eps,
                     int x_dtype, int w_dtype, void* stream) {
  if (M < 0 || N < 0 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return B2N_ERR_BAD_ARG;
  if (M == 0) return B2N_OK;
  if (!x || !y || !rstd) return B2N_ERR_BAD_ARG;
  if (gamma == nullptr) w_dtype = x_dtype;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_norm_fwd(true, x, gamma, nullptr, y, nullptr, rstd, M, N, eps, x_dtype, w_dtype,
                         static_cast<cudaStream_t>(stream));
}

size_t b2n_norm_bwd_workspace_bytes(int64_t M, int64_t N, int x_dtype, int w_dtype, int want_wgrad) {
  if (!valid_dtype(x_dtype)) return 0;
  return norm_bwd_workspace_bytes(M, N, x_dtype, w_dtype, want_wgrad);
}

int b2n_layer_norm_bwd(const void* dy, const void* x, const void* mean, const void* rstd, const void* gamma,
                       void* dx, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes, int64_t M,
                       int64_t N, int x_dtype, int w_dtype, void* stream) {
  if (M < 0 || N < 0 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return B2N_ERR_BAD_ARG;
  if (M == 0 || N == 0) return B2N_OK;
  if (!dy || !x || !mean || !rstd) return B2N_ERR_BAD_ARG;
  if (!dx && !dgamma && !dbeta) return B2N_OK;
  if (gamma == nullptr && dgamma == nullptr && dbeta == nullptr) w_dtype = x_dtype;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_norm_bwd(false, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, workspace, workspace_bytes, M, N,
                         x_dtype, w_dtype, static_cast<cudaStream_t>(stream));
}

int b2n_rms_norm_bwd(const void* dy, const void* x, const void* rstd, const void* gamma, void* dx, void* dgamma,
                     void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int x_dtype, int w_dtype,
                     void* stream) {
  if (M < 0 || N < 0 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return B2N_ERR_BAD_ARG;
  if (M == 0 || N == 0) return B2N_OK;
  if (!dy || !x || !rstd) return B2N_ERR_BAD_ARG;
  if (!dx && !dgamma) return B2N_OK;
  if (gamma == nullptr && dgamma == nullptr) w_dtype = x_dtype;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_norm_bwd(true, dy, x, nullptr, rstd, gamma, dx, dgamma, nullptr, workspace, workspace_bytes, M, N,
                         x_dtype, w_dtype, static_cast<cudaStream_t>(stream));
}

int b2n_norm_bwd_partials(int rms, const void* dy, const void* x, const void* mean, const void* rstd, const void* gamma,
                          void* dx, void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int x_dtype,
                          int w_dtype, int64_t* partial_rows, void* stream) {
  if (M < 0 || N < 0 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype) || partial_rows == nullptr) return B2N_ERR_BAD_ARG;
  *partial_rows = 0;
  if (M == 0 || N == 0) return B2N_OK;
  if (!dy || !x || !rstd || (!rms && !mean)) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_norm_bwd(rms != 0, dy, x, rms ? nullptr : mean, rstd, gamma, dx, nullptr, nullptr, workspace,
                         workspace_bytes, M, N, x_dtype, w_dtype, static_cast<cudaStream_t>(stream), partial_rows);
}

int b2n_norm_wgrad_fold(const void* workspace, int64_t partial_rows, int64_t N, void* dgamma, void* dbeta, int x_dtype,
                        int w_dtype, void* stream) {
  if (partial_rows < 0 || N < 0 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return B2N_ERR_BAD_ARG;
  if (N == 0 || (!dgamma && !dbeta)) return B2N_OK;
  if (!workspace || !is_aligned(workspace, 16)) return B2N_ERR_WORKSPACE;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_norm_wgrad_fold(workspace, partial_rows, N, dgamma, dbeta, x_dtype, w_dtype,
                                static_cast<cudaStream_t>(stream));
}

int b2n_softmax_fwd(const void* x, void* y, int64_t outer, int64_t N, int64_t inner, int in_dtype, int out_dtype,
                    int is_log, void* stream) {
  if (outer < 0 || N < 0 || inner < 0 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype)) return B2N_ERR_BAD_ARG;
  if (outer == 0 || N == 0 || inner == 0) return B2N_OK;
  if (!x || !y) return B2N_ERR_BAD_ARG;
  if (is_log < 0 || is_log > 2) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  tl_softmax_safe = is_log == 2;
  const int rc = launch_softmax_fwd(x, y, outer, N, inner, in_dtype, out_dtype, is_log == 1,
                                    static_cast<cudaStream_t>(stream));
  tl_softmax_safe = false;
  return rc;
}

int b2n_softmax_bwd(const void* dy, const void* y, void* dx, int64_t outer, int64_t N, int64_t inner,
                    int grad_dtype, int dx_dtype, int is_log, void* stream) {
  if (outer < 0 || N < 0 || inner < 0 || !valid_dtype(grad_dtype) || !valid_dtype(dx_dtype)) return B2N_ERR_BAD_ARG;
  if (outer == 0 || N == 0 || inner == 0) return B2N_OK;
  if (!dy || !y || !dx) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_softmax_bwd(dy, y, dx, outer, N, inner, grad_dtype, dx_dtype, is_log != 0,
                            static_cast<cudaStream_t>(stream));
}

size_t b2n_nll_loss_workspace_bytes(int64_t M) { return nll_loss_workspace_bytes(M); }

int b2n_nll_loss_fwd(const void* logp, const void* target, const void* weight, void* out, void* total_weight,
                     float* sums_f32, void* workspace, size_t workspace_bytes, int64_t M, int64_t C,
                     int reduction, int64_t ignore_index, int dtype, int target_is_u8, void* stream) {
  if (M < 0 || C < 0 || !valid_dtype(dtype) || reduction < B2N_REDUCE_NONE || reduction > B2N_REDUCE_SUM)
    return B2N_ERR_BAD_ARG;
  if (M > 0 && (!logp || !target)) return B2N_ERR_BAD_ARG;
  if (!out && !(reduction == B2N_REDUCE_NONE && M == 0)) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_nll_loss_fwd(logp, target, weight, out, total_weight, sums_f32, workspace, workspace_bytes, M, C,
                             reduction, ignore_index, dtype, target_is_u8 != 0, static_cast<cudaStream_t>(stream));
}

int b2n_nll_loss_bwd(const void* grad_out, const void* target, const void* weight, const void* total_weight,
                     void* grad_input, int64_t M, int64_t C, int reduction, int64_t ignore_index, int dtype,
                     int target_is_u8, void* stream) {
  if (M < 0 || C < 0 || !valid_dtype(dtype) || reduction < B2N_REDUCE_NONE || reduction > B2N_REDUCE_SUM)
    return B2N_ERR_BAD_ARG;
  if (M == 0 || C == 0) return B2N_OK;
  if (!grad_out || !target || !grad_input) return B2N_ERR_BAD_ARG;
  if (reduction == B2N_REDUCE_MEAN && !total_weight) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_nll_loss_bwd(grad_out, target, weight, total_weight, grad_input, M, C, reduction, ignore_index,
                             dtype, target_is_u8 != 0, static_cast<cudaStream_t>(stream));
}

int b2n_masked_softmax_fwd(const void* x, const void* mask, void* y, int64_t M, int64_t N, int64_t mask_row_div,
                           int64_t mask_row_mod, int dtype, void* stream) {
  if (M < 0 || N < 0 || mask_row_div < 1 || mask_row_mod < 1 || !valid_dtype(dtype)) return B2N_ERR_BAD_ARG;
  if (M == 0 || N == 0) return B2N_OK;
  if (!x || !mask || !y) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_masked_softmax_fwd(x, mask, y, M, N, mask_row_div, mask_row_mod, dtype,
                                   static_cast<cudaStream_t>(stream));
}

int b2n_masked_softmax_bwd(const void* dy, const void* y, const void* mask, void* dx, int64_t M, int64_t N,
                           int dtype, void* stream) {
  if (M < 0 || N < 0 || !valid_dtype(dtype)) return B2N_ERR_BAD_ARG;
  if (M == 0 || N == 0) return B2N_OK;
  if (!dy || !y || !mask || !dx) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_masked_softmax_bwd(dy, y, mask, dx, M, N, dtype, static_cast<cudaStream_t>(stream));
}

int b2n_cross_entropy_bwd(const void* logp, const void* target, const void* weight, const void* grad_out,
                          const void* total_weight, void* dx, int64_t M, int64_t C, int reduction,
                          int64_t ignore_index, int dtype, int target_is_u8, void* stream) {
  if (M < 0 || C < 0 || !valid_dtype(dtype) || reduction < B2N_REDUCE_NONE || reduction > B2N_REDUCE_SUM)
    return B2N_ERR_BAD_ARG;
  if (M == 0 || C == 0) return B2N_OK;
  if (!logp || !grad_out || !target || !dx) return B2N_ERR_BAD_ARG;
  if (reduction == B2N_REDUCE_MEAN && !total_weight) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  return launch_cross_entropy_bwd(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index,
                                  dtype, target_is_u8 != 0, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
