// b2n_layer_norm_bwd_noalloc: the layer-norm backward for callers that cannot provide scratch.
//
// Some hosts give an operator nothing but its tensors: an inference engine's plug-in `enqueue`
// callback, a serving loop whose memory pool was frozen at start-up, a process that has already
// handed the whole device-memory budget to another allocator.  They cannot call cudaMalloc (or an
// allocating library routine) on the call path, so they cannot supply the partial-sum workspace
// that b2n_layer_norm_bwd wants for dgamma/dbeta.  This entry point carries that workspace
// itself, as a fixed file-scope device array, and allocates nothing.
//
// What follows from that choice:
//  * the array is part of the loaded module: every GPU that loads the library holds its
//    kNoAllocScratchBytes until the process exits, whether or not this entry point is ever called;
//  * problems whose partial sums need more than that are refused (B2N_ERR_TOO_LARGE), never
//    truncated;
//  * all calls on one device share the one array.  Nothing in it has to start at zero — a call
//    overwrites every partial row it later folds — but two calls that overlap on the GPU
//    (different streams, or different host threads) write the same rows and race: serialise them;
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and caches it.  Make that first call before starting any stream capture.
#include <atomic>

#include "common.cuh"
#include "launchers.h"

namespace b2n {
namespace {

constexpr size_t kNoAllocScratchBytes = 16u << 20;  // 16 MiB: [148 partial rows][2][8192] fp32 is 9.25 MiB

// In host code this name is only a handle for the runtime's symbol table, not a device address;
// the kernels get the address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
// Only a successful lookup is remembered.  A first call that arrives while a stream capture is under way, or
// with a sticky error pending, fails — and the next call simply looks the address up again.
std::atomic<void*> g_scratch_address[kMaxDevices];

// Device address of the scratch array on the CURRENT device (looked up until it succeeds, then cached).
int scratch_for_current_device(void** out) {
  int dev = 0;
  if (int e = check_cuda(cudaGetDevice(&dev))) return e;
  if (dev < 0 || dev >= kMaxDevices) return B2N_ERR_BAD_ARG;
  void* p = g_scratch_address[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    const cudaError_t err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (err != cudaSuccess || p == nullptr) return check_cuda(err == cudaSuccess ? cudaErrorInvalidSymbol : err);
    g_scratch_address[dev].store(p, std::memory_order_release);  // concurrent first calls store the same address
  }
  *out = p;
  return B2N_OK;
}

}  // namespace
}  // namespace b2n

using namespace b2n;

extern "C" {

size_t b2n_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

int b2n_layer_norm_bwd_noalloc(const void* dy, const void* x, const void* mean, const void* rstd, const void* gamma,
                               void* dx, void* dgamma, void* dbeta, int64_t M, int64_t N, int x_dtype, int w_dtype,
                               void* stream) {
  if (M < 0 || N < 0 || x_dtype < B2N_F32 || x_dtype > B2N_F64 || w_dtype < B2N_F32 || w_dtype > B2N_F64)
    return B2N_ERR_BAD_ARG;
  if (M == 0 || N == 0) return B2N_OK;
  if (!dy || !x || !mean || !rstd) return B2N_ERR_BAD_ARG;
  if (!dx && !dgamma && !dbeta) return B2N_OK;
  if (gamma == nullptr && dgamma == nullptr && dbeta == nullptr) w_dtype = x_dtype;
  const bool want_wgrad = dgamma != nullptr || dbeta != nullptr;
  const size_t need = norm_bwd_workspace_bytes(M, N, x_dtype, w_dtype, want_wgrad ? 1 : 0);
  if (need > kNoAllocScratchBytes) return B2N_ERR_TOO_LARGE;  // the fixed array cannot hold this problem's partial sums
  if (!device_ready()) return B2N_ERR_CUDA;
  void* scratch = nullptr;
  if (want_wgrad) {
    if (int e = scratch_for_current_device(&scratch)) return e;
  }
  return launch_norm_bwd(false, dy, x, mean, rstd, gamma, dx, dgamma, dbeta, scratch, want_wgrad ? kNoAllocScratchBytes : 0,
                         M, N, x_dtype, w_dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
