// Typed host launchers for layer norm / RMS norm.  Instantiated per (T, WT) pair in the norm_*.cu
// files so the instantiations compile in parallel.
#pragma once
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "launchers.h"
#include "norm_generic.cuh"
#include "norm_ring.cuh"
#include "norm_ring2w.cuh"
#include "norm_slab.cuh"
#include "plan.h"

namespace b2n {

// Elements per thread in the ring kernels.  The forward keeps x, gamma and beta in registers
// (with 32 elements the compiler re-loads the weights from global memory every row instead of
// holding 96 values); the backward keeps gamma, dgamma, dbeta and two working arrays.
constexpr int kNormFwdEpt = 16;
constexpr int kNormBwdEpt = 16;

// Opt the kernel into its dynamic shared memory, once per device.
template <typename K> int set_smem_once(K kernel, size_t bytes, std::atomic<uint64_t>& mask) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda(cudaGetLastError());
  const uint64_t bit = 1ull << (dev & 63);
  if (mask.load(std::memory_order_acquire) & bit) return B2N_OK;
  (void)bytes;
  const int st = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 device_info().max_smem_optin));
  if (st == B2N_OK) mask.fetch_or(bit, std::memory_order_release);
  return st;
}

inline int generic_grid(int64_t rows, int rows_per_block) {
  const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = static_cast<int64_t>(device_info().sm_count) * 16;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

template <typename T, typename WT>
bool norm_vectorizable(int64_t N, const void* a, const void* b, const void* c) {
  constexpr int V = 16 / sizeof(T);
  return N % V == 0 && is_aligned(a, 16) && (b == nullptr || is_aligned(b, 16)) &&
         (c == nullptr || is_aligned(c, 16));
}

// ---- rows longer than the ring takes: column slabs over a thread-block cluster (norm_slab.cuh) --------------
struct SlabPlan {
  bool ok = false;
  int c = 0;          // CTAs per cluster = slabs per row
  int slab_vecs = 0;  // 16-byte vectors per slab
  int tr = 0;         // rows per tile
  int depth = 1;      // tiles between a tile's phase A and its phase B (1 or 2)
  int stages = 0;
  size_t smem = 0;
};
// nin: tensors staged per tile (1 forward, 2 backward).  Not ok when the row does not split into at most 8 slabs of
// at most 512 threads x 16 elements, or fewer than three stages fit (a tile is held from its phase A to its phase B).
inline SlabPlan plan_slab(int64_t M, int64_t N, int esize, int nin, int max_smem) {
  SlabPlan p;
  const int vec = 16 / esize;
  if (M <= 0 || N <= 0 || N % vec != 0) return p;
  const int64_t nvec = N / vec;
  const int64_t cap = static_cast<int64_t>(kNsConsumers) * (kNsEpt / vec);  // vectors one CTA's threads hold
  const int forced_c = ring_tuning().cluster;
  for (int c = 2; c <= kNsMaxCluster; c *= 2) {
    if (forced_c >= 2 && c != forced_c) continue;
    const int64_t sv = (nvec + c - 1) / c;
    if (sv > cap) continue;
    for (int tr = 2; tr >= 1; --tr) {
      if (ring_tuning().rpg >= 1 && ring_tuning().rpg <= 2 && tr != ring_tuning().rpg) continue;
      const int64_t stage = static_cast<int64_t>(nin) * tr * sv * 16;
      int64_t s = (static_cast<int64_t>(max_smem) - kNsHeaderBytes) / stage;
      if (s > kNsMaxStages) s = kNsMaxStages;
      const int tuned = ring_tuning().stages;
      if (tuned >= 3 && tuned < s) s = tuned;
      const bool pinned_tr = ring_tuning().rpg >= 1 && ring_tuning().rpg <= 2;
      if (s < 3 || (tr == 2 && s < 4 && !pinned_tr)) continue;  // two-row tiles only when at least four of them fit
      p.ok = true;
      p.c = c;
      p.slab_vecs = static_cast<int>(sv);
      p.tr = tr;
      p.stages = static_cast<int>(s);
      // a tile occupies its stage for depth + 1 iterations: deeper only with stages to spare, and only in the forward
      // (measured on bf16 [16384, 16384]: forward 236 us at depth 2 / 241 at 1, backward 359 / 343)
      p.depth = (s >= 5 && nin == 1) ? 2 : 1;
      if (ring_tuning().lag >= 1 && ring_tuning().lag <= 2 && ring_tuning().lag + 2 <= s) p.depth = ring_tuning().lag;
      p.smem = static_cast<size_t>(kNsHeaderBytes + s * stage);
      return p;
    }
  }
  return p;
}

constexpr int kSlabNoFit = 1;  // (not a b2n_status) slab_launch: no cluster of this shape fits the device

// Launches `kernel` as clusters of p.c CTAs, as many clusters as the device holds at once (or as there are
// tiles), with the dependent-launch attribute.  *clusters_out: the number of clusters (= partial rows of the backward).
template <typename... KArgs, typename... Args>
int slab_launch(void (*kernel)(KArgs...), const SlabPlan& p, int64_t M, std::atomic<uint64_t>& smem_done, cudaStream_t st,
                int64_t* clusters_out, Args... args) {
  if (int e = set_smem_once(kernel, p.smem, smem_done)) return e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.c;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;  // the occupancy query wants the cluster shape only
  cfg.blockDim = dim3(kNsThreads);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = st;
  const int sms = persistent_ctas(device_info().sm_count);
  const int by_count = sms / p.c > 0 ? sms / p.c : 1;
  cfg.gridDim = dim3(static_cast<unsigned>(p.c) * static_cast<unsigned>(by_count));
  int max_clusters = 0;
  if (int e = check_cuda(cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg))) return e;
  if (max_clusters < 1) return kSlabNoFit;  // the device cannot hold even one such cluster: the caller takes another family
  if (max_clusters > by_count) max_clusters = by_count;
  const int64_t ntiles = (M + p.tr - 1) / p.tr;
  int64_t nclusters = ntiles < max_clusters ? ntiles : max_clusters;
  const int64_t waves = (ntiles + nclusters - 1) / nclusters;  // no cluster finishes before the busiest one
  nclusters = (ntiles + waves - 1) / waves;
  if (clusters_out != nullptr) *clusters_out = nclusters;
  if (getenv("B2N_DEBUG") != nullptr)
    fprintf(stderr, "[b200norm] slab launch: C=%d slab_vecs=%d rows/tile=%d depth=%d stages=%d smem=%zu max_clusters=%d clusters=%lld\n",
            p.c, p.slab_vecs, p.tr, p.depth, p.stages, p.smem, max_clusters, static_cast<long long>(nclusters));
  cfg.gridDim = dim3(static_cast<unsigned>(nclusters * p.c));
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return check_cuda(e);
  return launched();
}

template <typename T, typename WT, bool RMS>
int norm_fwd_slab_launch(const SlabPlan& p, const T* x, const WT* gamma, const WT* beta, T* y, float* mean, float* rstd,
                         int64_t M, int64_t N, double eps, cudaStream_t st) {
  ProfileScope prof(RMS ? "rms_norm_fwd_slab" : "layer_norm_fwd_slab", st);
  static std::atomic<uint64_t> done[6];
  int* status = device_status_ptr();
  auto go = [&](auto kernel, std::atomic<uint64_t>& d) {
    return slab_launch(kernel, p, M, d, st, nullptr, x, gamma, beta, y, mean, rstd, M, N, static_cast<float>(eps), p.slab_vecs,
                       p.stages, status);
  };
  // the usual case — whole slabs, two-row tiles — has its own instantiations; anything else takes the general ones
  const bool full = N == static_cast<int64_t>(p.c) * kNsConsumers * kNsEpt;
  if (full && p.tr == 2)
    return p.depth == 2 ? go(norm_fwd_slab_kernel<T, WT, RMS, 2, 2, true>, done[4]) : go(norm_fwd_slab_kernel<T, WT, RMS, 2, 1, true>, done[5]);
  if (p.tr == 2) return p.depth == 2 ? go(norm_fwd_slab_kernel<T, WT, RMS, 2, 2, false>, done[0]) : go(norm_fwd_slab_kernel<T, WT, RMS, 2, 1, false>, done[1]);
  return p.depth == 2 ? go(norm_fwd_slab_kernel<T, WT, RMS, 1, 2, false>, done[2]) : go(norm_fwd_slab_kernel<T, WT, RMS, 1, 1, false>, done[3]);
}

template <typename T, typename WT, bool RMS>
int norm_bwd_slab_launch(const SlabPlan& p, bool wgrad, const T* dy, const T* x, const float* mean, const float* rstd,
                         const WT* gamma, T* dx, float* ws, int64_t M, int64_t N, cudaStream_t st, int64_t* clusters) {
  ProfileScope prof(RMS ? "rms_norm_bwd_slab" : "layer_norm_bwd_slab", st);
  static std::atomic<uint64_t> done[10];
  int* status = device_status_ptr();
  auto go = [&](auto kernel, std::atomic<uint64_t>& d) {
    return slab_launch(kernel, p, M, d, st, clusters, dy, x, mean, rstd, gamma, dx, ws, M, N, p.slab_vecs, p.stages, status);
  };
  const bool full = N == static_cast<int64_t>(p.c) * kNsConsumers * kNsEpt;
  if (wgrad) {
    if (full && p.tr == 2 && p.depth == 1) return go(norm_bwd_slab_kernel<T, WT, RMS, true, 2, 1, true>, done[8]);
    if (full && p.tr == 1 && p.depth == 1) return go(norm_bwd_slab_kernel<T, WT, RMS, true, 1, 1, true>, done[9]);
    if (p.tr == 2) return p.depth == 2 ? go(norm_bwd_slab_kernel<T, WT, RMS, true, 2, 2, false>, done[0]) : go(norm_bwd_slab_kernel<T, WT, RMS, true, 2, 1, false>, done[1]);
    return p.depth == 2 ? go(norm_bwd_slab_kernel<T, WT, RMS, true, 1, 2, false>, done[2]) : go(norm_bwd_slab_kernel<T, WT, RMS, true, 1, 1, false>, done[3]);
  }
  if (p.tr == 2) return p.depth == 2 ? go(norm_bwd_slab_kernel<T, WT, RMS, false, 2, 2, false>, done[4]) : go(norm_bwd_slab_kernel<T, WT, RMS, false, 2, 1, false>, done[5]);
  return p.depth == 2 ? go(norm_bwd_slab_kernel<T, WT, RMS, false, 1, 2, false>, done[6]) : go(norm_bwd_slab_kernel<T, WT, RMS, false, 1, 1, false>, done[7]);
}

// ---- forward ------------------------------------------------------------------------------------
template <typename T, typename WT, bool RMS, int GROUP>
int norm_fwd_ring_launch(const RingPlan& p, const T* x, const WT* gamma, const WT* beta, T* y, float* mean,
                         float* rstd, int64_t M, int64_t N, double eps, cudaStream_t st) {
  constexpr int VPT = kNormFwdEpt / Pack16<T>::VEC;
  ProfileScope prof(RMS ? "rms_norm_fwd_ring" : "layer_norm_fwd_ring", st);
  auto go = [&](auto kernel, std::atomic<uint64_t>& done) -> int {
    if (int e = set_smem_once(kernel, p.smem, done)) return e;
    return launch_pdl(kernel, dim3(p.grid), dim3(kRingBlock), p.smem, st, x, gamma, beta, y, mean, rstd, M,
                      static_cast<int>(N), static_cast<float>(eps), p.stages | (p.lag << 8), p.rpg,
                      device_status_ptr(), next_tile_counter(), ring_tuning().trace_buf, ring_tuning().trace_cap);
  };
  static std::atomic<uint64_t> done[3];
  // rows that fill every thread's vectors exactly take the instantiation without range checks
  // ... and, when the planner chose the usual four rows per group per tile, with that count compiled in
  if (N == static_cast<int64_t>(GROUP) * VPT * Pack16<T>::VEC) {
    if (p.rpg == 4) return go(norm_fwd_ring_kernel<T, WT, RMS, GROUP, VPT, true, 4>, done[2]);
    return go(norm_fwd_ring_kernel<T, WT, RMS, GROUP, VPT, true, 0>, done[0]);
  }
  return go(norm_fwd_ring_kernel<T, WT, RMS, GROUP, VPT, false, 0>, done[1]);
}

template <typename T, typename WT, bool RMS>
int norm_fwd_typed(const void* x_, const void* gamma_, const void* beta_, void* y_, void* mean_, void* rstd_,
                   int64_t M, int64_t N, double eps, cudaStream_t st) {
  using A = acc_t<T>;
  const T* x = static_cast<const T*>(x_);
  const WT* gamma = static_cast<const WT*>(gamma_);
  const WT* beta = static_cast<const WT*>(beta_);
  T* y = static_cast<T*>(y_);
  A* mean = static_cast<A*>(mean_);
  A* rstd = static_cast<A*>(rstd_);
  const int forced = forced_path();

  if constexpr (sizeof(T) <= 4 && !std::is_same<T, double>::value) {
    if (forced != B2N_PATH_GENERIC && is_aligned(x, 16) && is_aligned(y, 16) && N <= (1 << 20)) {
      const DeviceInfo& di = device_info();
      // one tensor per stage: 64 KB tiles (half as many tile hand-overs) still leave three stages in rotation
      const RingPlan p = plan_ring(M, N, sizeof(T), 1, kNormFwdEpt, persistent_ctas(di.sm_count), di.max_smem_optin, 65536);
      if (p.ok && forced != B2N_PATH_CLUSTER) {
        note_path("ring");
        switch (p.group) {
          case 32: return norm_fwd_ring_launch<T, WT, RMS, 32>(p, x, gamma, beta, y, mean, rstd, M, N, eps, st);
          case 64: return norm_fwd_ring_launch<T, WT, RMS, 64>(p, x, gamma, beta, y, mean, rstd, M, N, eps, st);
          case 128: return norm_fwd_ring_launch<T, WT, RMS, 128>(p, x, gamma, beta, y, mean, rstd, M, N, eps, st);
          case 256: return norm_fwd_ring_launch<T, WT, RMS, 256>(p, x, gamma, beta, y, mean, rstd, M, N, eps, st);
          default: return norm_fwd_ring_launch<T, WT, RMS, 512>(p, x, gamma, beta, y, mean, rstd, M, N, eps, st);
        }
      }
      if (forced != B2N_PATH_CLUSTER && !p.ok && N > 8192 && N <= 16384) {
        // rows of up to twice what a ring CTA's registers hold: weights in registers, the row walked twice in shared memory
        const RingPlan p2 = plan_ring(M, N, sizeof(T), 1, kNorm2wEpt, persistent_ctas(di.sm_count), di.max_smem_optin, 65536);
        if (p2.ok && p2.group == kRingThreads && p2.stages >= 3) {
          note_path("ring2w");
          ProfileScope prof(RMS ? "rms_norm_fwd_ring2w" : "layer_norm_fwd_ring2w", st);
          auto go = [&](auto kernel, std::atomic<uint64_t>& done) -> int {
            if (int e = set_smem_once(kernel, p2.smem, done)) return e;
            return launch_pdl(kernel, dim3(p2.grid), dim3(kRingBlock), p2.smem, st, x, gamma, beta, y, mean, rstd, M,
                              static_cast<int>(N), static_cast<float>(eps), p2.stages | (p2.lag << 8), p2.rpg,
                              device_status_ptr(), next_tile_counter());
          };
          static std::atomic<uint64_t> done2w[2];
          if (N == static_cast<int64_t>(kRingThreads) * kNorm2wEpt) return go(norm_fwd_ring2w_kernel<T, WT, RMS, true>, done2w[0]);
          return go(norm_fwd_ring2w_kernel<T, WT, RMS, false>, done2w[1]);
        }
      }
      if (forced == B2N_PATH_AUTO || forced == B2N_PATH_CLUSTER) {
        // rows beyond the ring (or any row the slabs can take, when that family is pinned): column slabs over a cluster
        const SlabPlan sp = plan_slab(M, N, sizeof(T), 1, di.max_smem_optin);
        if (sp.ok) {
          const int e = norm_fwd_slab_launch<T, WT, RMS>(sp, x, gamma, beta, y, mean, rstd, M, N, eps, st);
          if (e != kSlabNoFit) {
            note_path("slab");
            return e;
          }
        }
      }
    }
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;

  note_path("generic");
  ProfileScope prof(RMS ? "rms_norm_fwd_generic" : "layer_norm_fwd_generic", st);
  constexpr int V = 16 / sizeof(T);
  const bool vec = norm_vectorizable<T, WT>(N, x, y, nullptr);
  const A eps_a = static_cast<A>(eps);
  if (N <= 1024) {
    const int grid = generic_grid(M, 8);
    if (vec) norm_fwd_generic_kernel<T, WT, RMS, 32, V><<<grid, 256, 0, st>>>(x, gamma, beta, y, mean, rstd, M, N, eps_a);
    else norm_fwd_generic_kernel<T, WT, RMS, 32, 1><<<grid, 256, 0, st>>>(x, gamma, beta, y, mean, rstd, M, N, eps_a);
  } else {
    const int grid = generic_grid(M, 1);
    const int threads = N <= 8192 ? 256 : 1024;
    if (vec) norm_fwd_generic_kernel<T, WT, RMS, 0, V><<<grid, threads, 0, st>>>(x, gamma, beta, y, mean, rstd, M, N, eps_a);
    else norm_fwd_generic_kernel<T, WT, RMS, 0, 1><<<grid, threads, 0, st>>>(x, gamma, beta, y, mean, rstd, M, N, eps_a);
  }
  return launched();
}

// ---- backward -----------------------------------------------------------------------------------
// full = true plans for every SM whatever margin is set: what the workspace must be large enough for.
template <typename T> RingPlan plan_norm_bwd(int64_t M, int64_t N, const DeviceInfo& di, bool full = false) {
  return plan_ring(M, N, sizeof(T), 2, kNormBwdEpt, full ? di.sm_count : persistent_ctas(di.sm_count),
                   di.max_smem_optin);
}
// The two-walk RMS backward: rows of 8192 < N <= 16384 whose two input rows leave three stages in shared memory.
template <typename T> RingPlan plan_norm_bwd_2w(int64_t M, int64_t N, const DeviceInfo& di, bool full = false) {
  RingPlan p;
  if (N <= 8192 || N > 16384) return p;
  p = plan_ring(M, N, sizeof(T), 2, kNorm2wEpt, full ? di.sm_count : persistent_ctas(di.sm_count), di.max_smem_optin);
  if (p.ok && (p.group != kRingThreads || p.stages < 3)) p.ok = false;
  return p;
}
// Number of partial rows ([2][N] accumulate-type values each) the weight-gradient reduction writes.
inline int64_t wgrad_generic_chunks(int64_t M) {
  int64_t c = (M + 63) / 64;
  return c < 1 ? 1 : (c > 256 ? 256 : c);
}
template <typename T> int64_t wgrad_partial_rows(int64_t M, int64_t N) {
  int64_t rows = wgrad_generic_chunks(M);
  if constexpr (sizeof(T) <= 4 && !std::is_same<T, double>::value) {
    const DeviceInfo& di = device_info();
    const RingPlan p = plan_norm_bwd<T>(M, N, di, true);
    if (p.ok && static_cast<int64_t>(p.grid) * p.ng > rows) rows = static_cast<int64_t>(p.grid) * p.ng;
    // the slab kernels write one partial row per cluster: at most one cluster per two SMs
    const SlabPlan sp = plan_slab(M, N, sizeof(T), 2, di.max_smem_optin);
    if (sp.ok && di.sm_count / 2 > rows) rows = di.sm_count / 2;
    // the two-walk RMS backward (rows of 8192 < N <= 16384) writes one per CTA
    const RingPlan p2 = plan_norm_bwd_2w<T>(M, N, di, true);
    if (p2.ok && p2.grid > rows) rows = p2.grid;
  }
  return rows;
}
template <typename T> size_t norm_bwd_ws_bytes_typed(int64_t M, int64_t N) {
  return static_cast<size_t>(wgrad_partial_rows<T>(M, N)) * 2 * static_cast<size_t>(N) * sizeof(acc_t<T>);
}

template <typename T, typename WT, bool RMS, int GROUP>
int norm_bwd_ring_launch(const RingPlan& p, bool wgrad, const T* dy, const T* x, const float* mean,
                         const float* rstd, const WT* gamma, T* dx, float* ws, int64_t M, int64_t N,
                         cudaStream_t st) {
  constexpr int VPT = kNormBwdEpt / Pack16<T>::VEC;
  ProfileScope prof(RMS ? "rms_norm_bwd_ring" : "layer_norm_bwd_ring", st);
  const bool full = N == static_cast<int64_t>(GROUP) * VPT * Pack16<T>::VEC;
  const int s_lag = p.stages | (p.lag << 8);
  const int n = static_cast<int>(N);
  // fixed tile assignment (no counter) with weight gradients: the partial sums a CTA forms, and with them
  // dgamma/dbeta, are then the same bits on every run
  unsigned* ctr = wgrad ? nullptr : next_tile_counter();
  auto go = [&](auto kernel, std::atomic<uint64_t>& done) -> int {
    if (int e = set_smem_once(kernel, p.smem, done)) return e;
    return launch_pdl(kernel, dim3(p.grid), dim3(kRingBlock), p.smem, st, dy, x, mean, rstd, gamma, dx, ws, M, n, s_lag,
                      p.rpg, device_status_ptr(), ctr);
  };
  static std::atomic<uint64_t> done[6];
  if (wgrad) {
    if (full && p.rpg == 2) return go(norm_bwd_ring_kernel<T, WT, RMS, GROUP, VPT, true, true, 2>, done[4]);
    if (full) return go(norm_bwd_ring_kernel<T, WT, RMS, GROUP, VPT, true, true, 0>, done[0]);
    return go(norm_bwd_ring_kernel<T, WT, RMS, GROUP, VPT, true, false, 0>, done[1]);
  }
  if (full && p.rpg == 2) return go(norm_bwd_ring_kernel<T, WT, RMS, GROUP, VPT, false, true, 2>, done[5]);
  if (full) return go(norm_bwd_ring_kernel<T, WT, RMS, GROUP, VPT, false, true, 0>, done[2]);
  return go(norm_bwd_ring_kernel<T, WT, RMS, GROUP, VPT, false, false, 0>, done[3]);
}

template <typename T, typename WT, bool RMS>
int norm_bwd_typed(const void* dy_, const void* x_, const void* mean_, const void* rstd_, const void* gamma_,
                   void* dx_, void* dgamma_, void* dbeta_, void* workspace, size_t workspace_bytes, int64_t M,
                   int64_t N, cudaStream_t st, int64_t* partials_out) {
  using A = acc_t<T>;
  const T* dy = static_cast<const T*>(dy_);
  const T* x = static_cast<const T*>(x_);
  const A* mean = static_cast<const A*>(mean_);
  const A* rstd = static_cast<const A*>(rstd_);
  const WT* gamma = static_cast<const WT*>(gamma_);
  T* dx = static_cast<T*>(dx_);
  WT* dgamma = static_cast<WT*>(dgamma_);
  WT* dbeta = RMS ? nullptr : static_cast<WT*>(dbeta_);
  // partials_out: the caller folds the partial sums itself (norm_wgrad_fold_typed), possibly on another stream;
  // the row kernels then only leave ws[*partials_out][2][N] behind.
  const bool wgrad = dgamma != nullptr || dbeta != nullptr || partials_out != nullptr;
  const int forced = forced_path();
  if (wgrad) {
    if (workspace == nullptr || !is_aligned(workspace, 16) || workspace_bytes < norm_bwd_ws_bytes_typed<T>(M, N))
      return B2N_ERR_WORKSPACE;
  }
  A* ws = static_cast<A*>(workspace);
  const dim3 fold_block(32, kFoldLanes);
  const dim3 fold_grid(static_cast<unsigned>((N + 31) / 32), 2);

  if constexpr (sizeof(T) <= 4 && !std::is_same<T, double>::value) {
    if (forced != B2N_PATH_GENERIC && dx != nullptr && is_aligned(dy, 16) && is_aligned(x, 16) &&
        is_aligned(dx, 16) && N <= (1 << 20)) {
      const DeviceInfo& di = device_info();
      const RingPlan p = plan_norm_bwd<T>(M, N, di);
      if constexpr (RMS) {
        if (!p.ok && forced == B2N_PATH_AUTO) {
          // rows of up to twice what a ring CTA's registers hold, RMS norm: gamma and dgamma in registers, two walks
          const RingPlan p2 = plan_norm_bwd_2w<T>(M, N, di);
          if (p2.ok) {
            note_path("ring2w");
            int e;
            {
              ProfileScope prof("rms_norm_bwd_ring2w", st);
              auto go = [&](auto kernel, std::atomic<uint64_t>& done) -> int {
                if (int e2 = set_smem_once(kernel, p2.smem, done)) return e2;
                return launch_pdl(kernel, dim3(p2.grid), dim3(kRingBlock), p2.smem, st, dy, x, rstd, gamma, dx, ws, M,
                                  static_cast<int>(N), p2.stages | (p2.lag << 8), p2.rpg, device_status_ptr());
              };
              static std::atomic<uint64_t> done2w[4];
              const bool full = N == static_cast<int64_t>(kRingThreads) * kNorm2wEpt;
              if (wgrad) e = full ? go(rms_norm_bwd_ring2w_kernel<T, WT, true, true>, done2w[0])
                                  : go(rms_norm_bwd_ring2w_kernel<T, WT, true, false>, done2w[1]);
              else e = full ? go(rms_norm_bwd_ring2w_kernel<T, WT, false, true>, done2w[2])
                            : go(rms_norm_bwd_ring2w_kernel<T, WT, false, false>, done2w[3]);
            }
            if (partials_out != nullptr) *partials_out = p2.grid;
            if (e != B2N_OK || !wgrad || partials_out != nullptr) return e;
            return launch_pdl(norm_bwd_wgrad_fold_kernel<float, WT>, fold_grid, fold_block, 0, st,
                              static_cast<const float*>(ws), dgamma, dbeta, static_cast<int64_t>(p2.grid), N);
          }
        }
      }
      if (!(p.ok && forced != B2N_PATH_CLUSTER) && (forced == B2N_PATH_AUTO || forced == B2N_PATH_CLUSTER)) {
        const SlabPlan sp = plan_slab(M, N, sizeof(T), 2, di.max_smem_optin);
        if (sp.ok) {
          int64_t clusters = 0;
          const int e = norm_bwd_slab_launch<T, WT, RMS>(sp, wgrad, dy, x, mean, rstd, gamma, dx, ws, M, N, st, &clusters);
          if (e != kSlabNoFit) {
            note_path("slab");
            if (partials_out != nullptr) *partials_out = clusters;
            if (e != B2N_OK || !wgrad || partials_out != nullptr) return e;
            return launch_pdl(norm_bwd_wgrad_fold_kernel<float, WT>, fold_grid, fold_block, 0, st,
                              static_cast<const float*>(ws), dgamma, dbeta, clusters, N);
          }
        }
      }
      if (p.ok && forced != B2N_PATH_CLUSTER) {
        note_path("ring");
        int e;
        switch (p.group) {
          case 32: e = norm_bwd_ring_launch<T, WT, RMS, 32>(p, wgrad, dy, x, mean, rstd, gamma, dx, ws, M, N, st); break;
          case 64: e = norm_bwd_ring_launch<T, WT, RMS, 64>(p, wgrad, dy, x, mean, rstd, gamma, dx, ws, M, N, st); break;
          case 128: e = norm_bwd_ring_launch<T, WT, RMS, 128>(p, wgrad, dy, x, mean, rstd, gamma, dx, ws, M, N, st); break;
          case 256: e = norm_bwd_ring_launch<T, WT, RMS, 256>(p, wgrad, dy, x, mean, rstd, gamma, dx, ws, M, N, st); break;
          default: e = norm_bwd_ring_launch<T, WT, RMS, 512>(p, wgrad, dy, x, mean, rstd, gamma, dx, ws, M, N, st); break;
        }
        if (partials_out != nullptr) *partials_out = static_cast<int64_t>(p.grid) * p.ng;
        if (e != B2N_OK || !wgrad || partials_out != nullptr) return e;
        return launch_pdl(norm_bwd_wgrad_fold_kernel<float, WT>, fold_grid, fold_block, 0, st,
                          static_cast<const float*>(ws), dgamma, dbeta, static_cast<int64_t>(p.grid) * p.ng, N);
      }
    }
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;

  note_path("generic");
  if (dx != nullptr) {
    ProfileScope prof(RMS ? "rms_norm_bwd_dx_generic" : "layer_norm_bwd_dx_generic", st);
    constexpr int V = 16 / sizeof(T);
    const bool vec = norm_vectorizable<T, WT>(N, dy, x, dx);
    if (N <= 1024) {
      const int grid = generic_grid(M, 8);
      if (vec) norm_bwd_dx_generic_kernel<T, WT, RMS, 32, V><<<grid, 256, 0, st>>>(dy, x, mean, rstd, gamma, dx, M, N);
      else norm_bwd_dx_generic_kernel<T, WT, RMS, 32, 1><<<grid, 256, 0, st>>>(dy, x, mean, rstd, gamma, dx, M, N);
    } else {
      const int grid = generic_grid(M, 1);
      const int threads = N <= 8192 ? 256 : 1024;
      if (vec) norm_bwd_dx_generic_kernel<T, WT, RMS, 0, V><<<grid, threads, 0, st>>>(dy, x, mean, rstd, gamma, dx, M, N);
      else norm_bwd_dx_generic_kernel<T, WT, RMS, 0, 1><<<grid, threads, 0, st>>>(dy, x, mean, rstd, gamma, dx, M, N);
    }
    if (int e = launched()) return e;
  }
  if (wgrad) {
    const int64_t chunks = wgrad_generic_chunks(M);
    const int64_t rpc = (M + chunks - 1) / chunks;
    const dim3 block(32, 8);
    const dim3 grid(static_cast<unsigned>((N + 31) / 32), static_cast<unsigned>(chunks));
    {
      ProfileScope prof("norm_bwd_wgrad_generic", st);
      norm_bwd_wgrad_partial_kernel<T, RMS><<<grid, block, 0, st>>>(dy, x, mean, rstd, ws, M, N, rpc);
      if (int e = launched()) return e;
    }
    if (partials_out != nullptr) {
      *partials_out = chunks;
      return B2N_OK;
    }
    norm_bwd_wgrad_fold_kernel<A, WT><<<fold_grid, fold_block, 0, st>>>(ws, dgamma, dbeta, chunks, N);
    if (int e = launched()) return e;
  }
  return B2N_OK;
}

// The fold on its own: ws[P][2][N] (accumulate type of T) -> dgamma / dbeta of type WT, fixed order.
template <typename T, typename WT>
int norm_wgrad_fold_typed(const void* ws, int64_t P, int64_t N, void* dgamma, void* dbeta, cudaStream_t st) {
  using A = acc_t<T>;
  const dim3 fold_block(32, kFoldLanes);
  const dim3 fold_grid(static_cast<unsigned>((N + 31) / 32), 2);
  return launch_pdl(norm_bwd_wgrad_fold_kernel<A, WT>, fold_grid, fold_block, 0, st, static_cast<const A*>(ws),
                    static_cast<WT*>(dgamma), static_cast<WT*>(dbeta), P, N);
}

// Declares/defines the per-type entry points that norm_dispatch.cu switches over.
#define B2N_NORM_TYPED_DECL(NAME)                                                                               \
  int norm_fwd_##NAME(bool rms, const void* x, const void* gamma, const void* beta, void* y, void* mean,       \
                      void* rstd, int64_t M, int64_t N, double eps, cudaStream_t st);                           \
  int norm_bwd_##NAME(bool rms, const void* dy, const void* x, const void* mean, const void* rstd,              \
                      const void* gamma, void* dx, void* dgamma, void* dbeta, void* ws, size_t ws_bytes,        \
                      int64_t M, int64_t N, cudaStream_t st, int64_t* partials_out);                            \
  int norm_fold_##NAME(const void* ws, int64_t P, int64_t N, void* dgamma, void* dbeta, cudaStream_t st);       \
  size_t norm_bwd_ws_##NAME(int64_t M, int64_t N);

#define B2N_NORM_TYPED_DEFINE(NAME, T, WT)                                                                      \
  int norm_fwd_##NAME(bool rms, const void* x, const void* gamma, const void* beta, void* y, void* mean,       \
                      void* rstd, int64_t M, int64_t N, double eps, cudaStream_t st) {                          \
    return rms ? norm_fwd_typed<T, WT, true>(x, gamma, beta, y, mean, rstd, M, N, eps, st)                      \
               : norm_fwd_typed<T, WT, false>(x, gamma, beta, y, mean, rstd, M, N, eps, st);                    \
  }                                                                                                             \
  int norm_bwd_##NAME(bool rms, const void* dy, const void* x, const void* mean, const void* rstd,              \
                      const void* gamma, void* dx, void* dgamma, void* dbeta, void* ws, size_t ws_bytes,        \
                      int64_t M, int64_t N, cudaStream_t st, int64_t* partials_out) {                           \
    return rms ? norm_bwd_typed<T, WT, true>(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out) \
               : norm_bwd_typed<T, WT, false>(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, ws, ws_bytes, M, N, st, partials_out); \
  }                                                                                                             \
  int norm_fold_##NAME(const void* ws, int64_t P, int64_t N, void* dgamma, void* dbeta, cudaStream_t st) {      \
    return norm_wgrad_fold_typed<T, WT>(ws, P, N, dgamma, dbeta, st);                                           \
  }                                                                                                             \
  size_t norm_bwd_ws_##NAME(int64_t M, int64_t N) { return norm_bwd_ws_bytes_typed<T>(M, N); }

B2N_NORM_TYPED_DECL(f32)
B2N_NORM_TYPED_DECL(f16)
B2N_NORM_TYPED_DECL(f16_w32)
B2N_NORM_TYPED_DECL(bf16)
B2N_NORM_TYPED_DECL(bf16_w32)
B2N_NORM_TYPED_DECL(f64)

}  // namespace b2n
