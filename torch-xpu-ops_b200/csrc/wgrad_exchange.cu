// b2n_norm_wgrad_fold_allreduce: the weight-gradient fold of the norm backward and the all-reduce
// of its result over the ranks of one node, as ONE kernel over peer memory.
//
// A row-sharded layer-norm / RMS-norm backward leaves, on every rank, partial sums ws[P][2][N]; what
// the step needs is sum over ranks of (sum over partial rows) — 2N floats, 64 KiB for N = 8192.  A
// library all-reduce of a buffer that small is all latency (33 us measured for NCCL on two B200s, of
// which the wire needs two), and its kernel needs an SM of its own beside kernels that fill every
// SM.  Here each CTA owns a slice of the 2N columns and
//   1. folds its slice of the local partial rows (fixed order) into this rank's exchange buffer,
//   2. raises a flag in every peer's buffer (st.release.sys through the peer mapping),
//   3. waits for the same flag from every peer (bounded; B2N_ERR_TIMEOUT on expiry),
//   4. reads every rank's slice with plain peer loads — over NVLink / NVSwitch — adds them in RANK
//      order, so all ranks end with the same bits, and writes dgamma / dbeta.
// No multicast of any kind, no library call; the only traffic is (world - 1) x slice per CTA.
//
// Exchange buffer of one rank (device memory shared with the peers through CUDA IPC by the host):
//   data  [2][2 * n_max] float   two generations: a rank may be one call ahead of a peer
//   flags [2][kMaxRanks][kMaxCtas] uint32
//   epoch [kMaxCtas] uint32      generation counter, advanced by the kernel itself — nothing a CUDA
//                                graph replays has to change between replays
// Generation g uses half g & 1.  A rank cannot start generation g + 2 before every peer has raised
// its g + 1 flags, which a peer does only after it has finished reading generation g: two halves
// are enough.  All ranks must issue the same sequence of calls on a buffer (as with any collective),
// and a buffer serves ONE (N, CTA count) configuration: flags and generations are kept per CTA slice.
#include <cstring>

#include "common.cuh"
#include "launchers.h"

namespace b2n {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 256;
constexpr int kXThreads = 1024;

struct PeerTable { unsigned char* buf[kMaxRanks]; };

__host__ __device__ inline size_t exch_data_bytes(int64_t n_max) { return 2 * 2 * static_cast<size_t>(n_max) * sizeof(float); }
__host__ __device__ inline size_t exch_flags_bytes() { return 2 * kMaxRanks * kMaxCtas * sizeof(unsigned); }
__host__ __device__ inline size_t exch_total_bytes(int64_t n_max) {
  return exch_data_bytes(n_max) + exch_flags_bytes() + kMaxCtas * sizeof(unsigned);
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

template <typename WT>
__global__ void __launch_bounds__(kXThreads)
wgrad_fold_allreduce_kernel(const float* __restrict__ ws, int P, int N, int planes, PeerTable peers, int rank, int world,
                            int64_t n_max, WT* __restrict__ dgamma, WT* __restrict__ dbeta, int* status) {
  __shared__ float4 part[kXThreads];
  __shared__ unsigned s_epoch;
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the kernel before this one
  const int tid = threadIdx.x;
  const int total = planes * N;  // columns to reduce: dgamma, then dbeta
  const int per_cta = ((total / 4 + gridDim.x - 1) / gridDim.x) * 4;
  const int c0 = static_cast<int>(blockIdx.x) * per_cta;
  const int c1 = c0 + per_cta < total ? c0 + per_cta : total;
  unsigned char* mine = peers.buf[rank];
  unsigned* epochs = reinterpret_cast<unsigned*>(mine + exch_data_bytes(n_max) + exch_flags_bytes());
  if (tid == 0) {
    s_epoch = epochs[blockIdx.x] + 1u;  // only this CTA (of this launch, then of the next) touches the word
    s_ok = 1;
  }
  __syncthreads();
  const unsigned epoch = s_epoch;
  const unsigned half = epoch & 1u;
  float* my_data = reinterpret_cast<float*>(mine) + static_cast<size_t>(half) * 2 * n_max;

  // 1. fold: the slice's column quads side by side, `lanes` row lanes each (as many as the CTA's threads allow:
  //    a narrow slice gets many lanes and few rows per lane), the lanes' sums combined in lane order
  int lanes = 1;
  while (lanes < 32 && (per_cta / 4) * lanes * 2 <= kXThreads) lanes *= 2;
  const int quads = kXThreads / lanes;  // column quads per pass
  const int q = tid % quads, lane = tid / quads;
  for (int base = c0; base < c1; base += quads * 4) {  // uniform over the CTA
    const int c = base + q * 4;
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (c < c1) {
      const int plane = c >= N ? 1 : 0;
      const float* src = ws + static_cast<size_t>(plane) * N + (c - plane * N);
#pragma unroll 8
      for (int p = lane; p < P; p += lanes) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(p) * 2 * N));
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
    }
    part[lane * quads + q] = a;
    __syncthreads();
    if (lane == 0 && c < c1) {
      for (int l = 1; l < lanes; ++l) {
        const float4 v = part[l * quads + q];
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      *reinterpret_cast<float4*>(my_data + c) = a;  // [2][N] planes packed as plane * N + col: total <= 2 * n_max
    }
    __syncthreads();
  }

  // 2. + 3. tell every peer this slice is there; wait until theirs are
  if (world > 1) {
    __syncthreads();
    if (tid == 0) __threadfence_system();
    __syncthreads();
    if (tid < world && tid != rank) {
      unsigned* theirs = reinterpret_cast<unsigned*>(peers.buf[tid] + exch_data_bytes(n_max)) +
                         (static_cast<size_t>(half) * kMaxRanks + rank) * kMaxCtas + blockIdx.x;
      st_release_sys(theirs, epoch);
      const unsigned* here = reinterpret_cast<const unsigned*>(mine + exch_data_bytes(n_max)) +
                             (static_cast<size_t>(half) * kMaxRanks + tid) * kMaxCtas + blockIdx.x;
      const unsigned long long t0 = globaltimer_ns();
      for (uint32_t it = 1; ld_acquire_sys(here) != epoch; ++it) {
        if ((it & 0xffu) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
          record_status(status, B2N_ERR_TIMEOUT);
          s_ok = 0;
          break;
        }
      }
    }
    __syncthreads();
  }

  // 4. sum the ranks' slices in rank order (this rank's own included, read back from its buffer, so that every
  //    rank adds the same numbers in the same order)
  if (s_ok) {
    for (int c = c0 + tid * 4; c < c1; c += kXThreads * 4) {
      float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int r = 0; r < world; ++r) {
        const float* data = reinterpret_cast<const float*>(peers.buf[r]) + static_cast<size_t>(half) * 2 * n_max;
        const float4 v = r == rank ? *reinterpret_cast<const float4*>(my_data + c) : ld_peer_f4(data + c);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      const int plane = c >= N ? 1 : 0;
      WT* out = plane == 0 ? dgamma : dbeta;
      if (out != nullptr) {
        const int col = c - plane * N;
        out[col] = from_acc<WT>(a.x);
        out[col + 1] = from_acc<WT>(a.y);
        out[col + 2] = from_acc<WT>(a.z);
        out[col + 3] = from_acc<WT>(a.w);
      }
    }
  }
  __syncthreads();
  if (tid == 0) epochs[blockIdx.x] = epoch;
}

}  // namespace
}  // namespace b2n

using namespace b2n;

extern "C" {

// ---- exchange buffers -------------------------------------------------------------------------------
// The buffers are the library's own cudaMalloc allocations, exported and opened with the CUDA IPC calls
// directly.  Each rank opens its peers' handles WITH ITS OWN DEVICE CURRENT and cudaIpcMemLazyEnablePeerAccess:
// the mapping then belongs to the context whose kernels will use it, and peer access is switched on for exactly
// that pair (a mapping opened under the exporter's device index — what a framework's tensor sharing does —
// is not reachable from this device's kernels).
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the ABI carries IPC handles as 64 bytes");

int b2n_wgrad_exchange_alloc(int64_t n_max, void** local, unsigned char* handle64) {
  if (n_max <= 0 || local == nullptr || handle64 == nullptr) return B2N_ERR_BAD_ARG;
  void* p = nullptr;
  const size_t bytes = exch_total_bytes(n_max);
  if (int e = check_cuda(cudaMalloc(&p, bytes))) return e;
  if (int e = check_cuda(cudaMemset(p, 0, bytes))) { cudaFree(p); return e; }
  cudaIpcMemHandle_t h;
  if (int e = check_cuda(cudaIpcGetMemHandle(&h, p))) { cudaFree(p); return e; }
  if (int e = check_cuda(cudaDeviceSynchronize())) { cudaFree(p); return e; }
  memcpy(handle64, &h, sizeof(h));
  *local = p;
  return B2N_OK;
}

int b2n_wgrad_exchange_open(const unsigned char* handle64, void** mapped) {
  if (handle64 == nullptr || mapped == nullptr) return B2N_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (int e = check_cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess))) return e;
  *mapped = p;
  return B2N_OK;
}

int b2n_wgrad_exchange_close(void* mapped) { return mapped ? check_cuda(cudaIpcCloseMemHandle(mapped)) : B2N_OK; }
int b2n_wgrad_exchange_free(void* local) { return local ? check_cuda(cudaFree(local)) : B2N_OK; }

size_t b2n_wgrad_exchange_bytes(int64_t n_max) { return n_max > 0 ? exch_total_bytes(n_max) : 0; }

int b2n_norm_wgrad_fold_allreduce(const void* workspace, int64_t partial_rows, int64_t N, void* const* peer_buffers,
                                  int64_t n_max, int rank, int world, void* dgamma, void* dbeta, int w_dtype, int ctas,
                                  void* stream) {
  if (partial_rows < 0 || N <= 0 || n_max < N || world < 1 || world > kMaxRanks || rank < 0 || rank >= world ||
      peer_buffers == nullptr || ctas < 1 || ctas > kMaxCtas || N % 4 != 0)
    return B2N_ERR_BAD_ARG;
  if (!workspace || !is_aligned(workspace, 16)) return B2N_ERR_WORKSPACE;
  if (!dgamma && !dbeta) return B2N_ERR_BAD_ARG;
  if (!device_ready()) return B2N_ERR_CUDA;
  PeerTable t{};
  for (int r = 0; r < world; ++r) {
    if (peer_buffers[r] == nullptr || !is_aligned(peer_buffers[r], 16)) return B2N_ERR_BAD_ARG;
    t.buf[r] = static_cast<unsigned char*>(peer_buffers[r]);
  }
  const int planes = dbeta != nullptr ? 2 : 1;  // RMS norm leaves plane 1 of its partial rows unwritten
  const int p = static_cast<int>(partial_rows), n = static_cast<int>(N);
  const float* ws = static_cast<const float*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ProfileScope prof("wgrad_fold_allreduce", st);
  switch (w_dtype) {
    case B2N_F32:
      return launch_pdl(wgrad_fold_allreduce_kernel<float>, dim3(ctas), dim3(kXThreads), 0, st, ws, p, n, planes, t, rank,
                        world, n_max, static_cast<float*>(dgamma), static_cast<float*>(dbeta), device_status_ptr());
    case B2N_BF16:
      return launch_pdl(wgrad_fold_allreduce_kernel<bf16>, dim3(ctas), dim3(kXThreads), 0, st, ws, p, n, planes, t, rank,
                        world, n_max, static_cast<bf16*>(dgamma), static_cast<bf16*>(dbeta), device_status_ptr());
    case B2N_F16:
      return launch_pdl(wgrad_fold_allreduce_kernel<f16>, dim3(ctas), dim3(kXThreads), 0, st, ws, p, n, planes, t, rank,
                        world, n_max, static_cast<f16*>(dgamma), static_cast<f16*>(dbeta), device_status_ptr());
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

}  // extern "C"
