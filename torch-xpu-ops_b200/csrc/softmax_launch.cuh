// Typed host launchers for softmax / log-softmax.  Instantiated per type pair in softmax_*.cu.
#pragma once
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "launchers.h"
#include "plan.h"
#include "softmax_generic.cuh"
#include "softmax_ring.cuh"
#include "softmax_cluster.cuh"
#include "softmax_twopass.cuh"
#include "softmax_tma.cuh"

namespace b2n {

constexpr int kSoftmaxEpt = 32;  // elements per thread in the ring kernels

template <typename K> int set_smem_once_sm(K kernel, std::atomic<uint64_t>& mask) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda(cudaGetLastError());
  const uint64_t bit = 1ull << (dev & 63);
  if (mask.load(std::memory_order_acquire) & bit) return B2N_OK;
  const int st = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 device_info().max_smem_optin));
  if (st == B2N_OK) mask.fetch_or(bit, std::memory_order_release);
  return st;
}

inline int softmax_generic_grid(int64_t rows, int rows_per_block) {
  const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = static_cast<int64_t>(device_info().sm_count) * 16;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

template <typename T, bool LOG, int GROUP>
int softmax_fwd_ring_launch(const RingPlan& p, const T* x, T* y, int64_t M, int64_t N, cudaStream_t st,
                            RowMask rmask = RowMask{nullptr, 1u, 1u}) {
  constexpr int VPT = kSoftmaxEpt / Pack16<T>::VEC;
  // rows that fill every thread's vectors exactly take the instantiations without range checks
  const bool full = N == static_cast<int64_t>(GROUP) * VPT * Pack16<T>::VEC;
  auto go = [&](auto kernel, std::atomic<uint64_t>& done, const char* name) -> int {
    if (int e = set_smem_once_sm(kernel, done)) return e;
    ProfileScope prof(name, st);
    return launch_pdl(kernel, dim3(p.grid), dim3(kRingBlock), p.smem, st, x, y, M, static_cast<int>(N),
                      p.stages | (p.lag << 8), p.rpg, device_status_ptr(), next_tile_counter(), rmask);
  };
  static std::atomic<uint64_t> done[6];
  if (rmask.base != nullptr) {
    if constexpr (!LOG) {  // only the plain softmax has a masked form
      if (full) return go(softmax_fwd_ring_kernel<T, false, GROUP, VPT, true, false, true>, done[0], "masked_softmax_fwd_ring");
      return go(softmax_fwd_ring_kernel<T, false, GROUP, VPT, true, false, false>, done[1], "masked_softmax_fwd_ring");
    } else {
      return B2N_ERR_BAD_ARG;
    }
  }
  if (softmax_safe_mode()) {
    if constexpr (!LOG) {  // ... and a safe form (rows of -inf give zeros)
      if (full) return go(softmax_fwd_ring_kernel<T, false, GROUP, VPT, false, true, true>, done[2], "safe_softmax_fwd_ring");
      return go(softmax_fwd_ring_kernel<T, false, GROUP, VPT, false, true, false>, done[3], "safe_softmax_fwd_ring");
    } else {
      return B2N_ERR_BAD_ARG;
    }
  }
  const char* name = LOG ? "log_softmax_fwd_ring" : "softmax_fwd_ring";
  if (full) return go(softmax_fwd_ring_kernel<T, LOG, GROUP, VPT, false, false, true>, done[4], name);
  return go(softmax_fwd_ring_kernel<T, LOG, GROUP, VPT, false, false, false>, done[5], name);
}

template <typename T, bool LOG, int GROUP>
int softmax_bwd_ring_launch(const RingPlan& p, const T* dy, const T* y, T* dx, int64_t M, int64_t N,
                            cudaStream_t st, RowMask rmask = RowMask{nullptr, 1u, 1u}) {
  constexpr int VPT = kSoftmaxEpt / Pack16<T>::VEC;
  const bool full = N == static_cast<int64_t>(GROUP) * VPT * Pack16<T>::VEC;
  auto go = [&](auto kernel, std::atomic<uint64_t>& done, const char* name) -> int {
    if (int e = set_smem_once_sm(kernel, done)) return e;
    ProfileScope prof(name, st);
    return launch_pdl(kernel, dim3(p.grid), dim3(kRingBlock), p.smem, st, dy, y, dx, M, static_cast<int>(N),
                      p.stages | (p.lag << 8), p.rpg, device_status_ptr(), next_tile_counter(), rmask);
  };
  static std::atomic<uint64_t> done[4];
  if (rmask.base != nullptr) {
    if constexpr (!LOG) {
      if (full) return go(softmax_bwd_ring_kernel<T, false, GROUP, VPT, true, true>, done[0], "masked_softmax_bwd_ring");
      return go(softmax_bwd_ring_kernel<T, false, GROUP, VPT, true, false>, done[1], "masked_softmax_bwd_ring");
    } else {
      return B2N_ERR_BAD_ARG;
    }
  }
  const char* name = LOG ? "log_softmax_bwd_ring" : "softmax_bwd_ring";
  if (full) return go(softmax_bwd_ring_kernel<T, LOG, GROUP, VPT, false, true>, done[2], name);
  return go(softmax_bwd_ring_kernel<T, LOG, GROUP, VPT, false, false>, done[3], name);
}

// Rows too long for the ring: a row is split over a cluster of C CTAs (C = 1, 2, 4 or 8, one CTA per
// SM), each keeping its slice resident in shared memory.  Not ok when the row does not fit even 8
// CTAs (the caller then falls back to the generic kernels).
struct ClusterPlan { bool ok = false; int c = 0; int slice_vecs = 0; size_t smem = 0; };
inline ClusterPlan plan_cluster(int64_t N, int esize, int nin, int max_smem) {
  ClusterPlan p;
  const int vec = 16 / esize;
  if (N % vec != 0) return p;
  const int64_t nvec = N / vec;
  const int64_t budget = (static_cast<int64_t>(max_smem) - kSlabHeaderBytes) / 16 * 16;
  const int forced_c = ring_tuning().cluster;
  for (int c = 1; c <= kSlabMaxCluster; c *= 2) {
    if (forced_c >= 1 && c != forced_c) continue;
    const int64_t sv = (nvec + c - 1) / c;
    if (sv * 16 * nin <= budget && sv <= static_cast<int64_t>(kSlabChunkVecs) * kSlabMaxChunks) {
      p.ok = true;
      p.c = c;
      p.slice_vecs = static_cast<int>(sv);
      p.smem = static_cast<size_t>(kSlabHeaderBytes + sv * 16 * nin);
      break;
    }
  }
  return p;
}

template <typename T, bool LOG, bool BWD>
int softmax_cluster_launch(const ClusterPlan& p, const T* in0, const T* in1, T* out, int64_t M, int64_t N,
                           cudaStream_t st) {
  auto kernel = softmax_slab_kernel<T, LOG, BWD>;
  static std::atomic<uint64_t> mask{0};
  if (int e = set_smem_once_sm(kernel, mask)) return e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.c;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(kSlabThreads);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = st;
  // persistent clusters: as many as the device holds at once
  cfg.gridDim = dim3(static_cast<unsigned>(p.c) * device_info().sm_count);
  int max_clusters = 0;
  if (int e = check_cuda(cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg))) return e;
  if (max_clusters < 1) return B2N_ERR_BAD_ARG;
  const int64_t nclusters = M < max_clusters ? M : max_clusters;
  if (getenv("B2N_DEBUG") != nullptr)
    fprintf(stderr, "[b200norm] cluster launch: C=%d slice_vecs=%d smem=%zu max_clusters=%d clusters=%lld\n", p.c,
            p.slice_vecs, p.smem, max_clusters, static_cast<long long>(nclusters));
  cfg.gridDim = dim3(static_cast<unsigned>(nclusters * p.c));
  ProfileScope prof(BWD ? (LOG ? "log_softmax_bwd_cluster" : "softmax_bwd_cluster")
                        : (LOG ? "log_softmax_fwd_cluster" : "softmax_fwd_cluster"), st);
  int* status = device_status_ptr();
  const int slice_vecs = p.slice_vecs;
  if (int e = check_cuda(cudaLaunchKernelEx(&cfg, kernel, in0, in1, out, M, N, slice_vecs, status))) return e;
  return launched();
}

// The two-pass kernels move whole 16-byte vectors: a row must be a multiple of 16 bytes (rows of
// any other length — 50257 or 40001 elements, say — go to the generic kernels; a pinned two-pass
// path then reports B2N_ERR_BAD_ARG like every pinned family that cannot take the shape).
template <typename T> inline bool twopass_takes(int64_t N) { return N % static_cast<int64_t>(16 / sizeof(T)) == 0; }

// Rows of any length: two passes through the ring per row, the second served from L2.
template <typename T, bool LOG, bool BWD, bool SAFE>
int softmax_twopass_launch_as(const T* in0, const T* in1, T* out, int64_t M, int64_t N, cudaStream_t st) {
  auto kernel = softmax_twopass_kernel<T, LOG, BWD, SAFE>;
  static std::atomic<uint64_t> mask{0};
  if (int e = set_smem_once_sm(kernel, mask)) return e;
  const DeviceInfo& di = device_info();
  const int64_t stage = static_cast<int64_t>(kTwoPassChunkVecs) * 16 * (BWD ? 2 : 1);
  int64_t stages = (static_cast<int64_t>(di.max_smem_optin) - kRingHeaderBytes) / stage;
  if (stages > kMaxStages) stages = kMaxStages;
  const int tuned = ring_tuning().stages;
  if (tuned > 0 && tuned < stages) stages = tuned;
  if (stages < 3) return B2N_ERR_BAD_ARG;
  const size_t smem = static_cast<size_t>(kRingHeaderBytes + stages * stage);
  const int ctas = persistent_ctas(di.sm_count);
  const int grid = static_cast<int>(M < ctas ? M : ctas);
  ProfileScope prof(BWD ? (LOG ? "log_softmax_bwd_twopass" : "softmax_bwd_twopass")
                        : (LOG ? "log_softmax_fwd_twopass" : (SAFE ? "safe_softmax_fwd_twopass" : "softmax_fwd_twopass")),
                    st);
  return launch_pdl(kernel, dim3(grid), dim3(kRingBlock), smem, st, in0, in1, out, M, N, static_cast<int>(stages),
                    device_status_ptr(), next_tile_counter());
}
template <typename T, bool LOG, bool BWD>
int softmax_twopass_launch(const T* in0, const T* in1, T* out, int64_t M, int64_t N, cudaStream_t st) {
  if constexpr (!LOG && !BWD) {  // only the plain forward has a safe form
    if (softmax_safe_mode()) return softmax_twopass_launch_as<T, false, false, true>(in0, in1, out, M, N, st);
  }
  return softmax_twopass_launch_as<T, LOG, BWD, false>(in0, in1, out, M, N, st);
}

// Tile width (elements) for the shared-memory tile kernels of the non-last-dim softmax: 1 KB runs when at
// least two CTAs then fit an SM, halved down to 256-byte runs otherwise; 0 when not even that fits.
inline int spatial_tile_elems(int64_t N, int esize, int ntensors, int64_t inner, int max_smem) {
  int tile = 1024 / esize;
  const int min_tile = 256 / esize;
  const int64_t budget = (ring_tuning().tile_kb > 0 ? ring_tuning().tile_kb : 110) * 1024;
  while (tile > min_tile && (N * tile * esize * ntensors > budget || tile / 2 >= inner)) tile /= 2;
  if (N * tile * esize * ntensors > max_smem - kTileScratchBytes) return 0;  // the kernels keep a scratch area in front of the tile
  return tile;
}

// ---- non-last-dim softmax on tensor-map TMA tiles (softmax_tma.cuh) ----------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// cuTensorMapEncodeTiled, found through the runtime (the library does not link against the driver library)
inline EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

template <typename T> constexpr CUtensorMapDataType tensor_map_dtype() {
  if constexpr (std::is_same<T, float>::value) return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  else if constexpr (std::is_same<T, f16>::value) return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  else return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
}

constexpr int kTmaNoFit = 1;  // (not a b2n_status) the shape is not for the TMA tile kernel: the caller takes another one

// [outer, N, inner] of T as a rank-3 tensor map (inner fastest) with boxes of W x NB x 1 elements.
template <typename T>
bool encode_spatial_map(CUtensorMap* tm, const T* ptr, int64_t outer, int64_t N, int64_t inner, int W, int NB) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(inner) * sizeof(T), static_cast<cuuint64_t>(N) * inner * sizeof(T)};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(W), static_cast<cuuint32_t>(NB), 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(tm, tensor_map_dtype<T>(), 3, const_cast<T*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The tile geometry of softmax_spatial_tma_kernel for lines of N elements `inner` apart.
struct TmaTilePlan {
  bool ok = false;
  bool reg = false;  // forward with the thread's share of a line in registers
  int W = 0;         // box width (elements), a multiple of 16 bytes, at most 256 elements
  int NX = 0;        // boxes per tile along `inner`
  int NB = 0;        // rows per box
  int S = 0;         // stages
  int segs = 0;      // threads per line
};

// Widest tile first: every thread busy (512 column groups x segments), two stages (backward) or three (forward, two
// when nothing narrower than 128-byte runs would give three) in shared memory, not wider than the tensor, and
// narrower while there are fewer tiles than two per SM.
inline TmaTilePlan plan_tma_tile(int64_t outer, int64_t N, int64_t inner, int es, int nin, bool bwd, int64_t avail, int sms) {
  TmaTilePlan p;
  const int vec = 16 / es, cpt = es == 2 ? 2 : 1, line = 128 / es;  // elements per 16 bytes / per thread / per 128-byte line
  const int64_t nboxes = (N + 255) / 256;                 // boxes of at most 256 rows ...
  p.NB = static_cast<int>((N + nboxes - 1) / nboxes);     // ... of equal height: at most nboxes - 1 padding rows in all
  const int64_t npad = (N + p.NB - 1) / p.NB * p.NB;
  p.reg = !bwd && N <= 16 * kTmaRegRows;  // up to 16 threads per line (one warp of column groups left): 128-byte runs
  int segs = p.reg ? static_cast<int>((N + kTmaRegRows - 1) / kTmaRegRows) : 1;
  if (p.reg) {
    // Column groups come in whole warps (32), so several segment counts can give the same tile width; among those,
    // take the one that leaves the fewest threads and row slots (blocks of four) idle — the forward in registers is
    // bound by instruction issue.  Never a narrower tile for it: measured, width and long segments matter more
    // (N = 200: 7 segments x 64 groups = 448 threads -> 8 x 64 = 512, +6 %; N = 150 narrowed from 96 to 64 groups: -16 %).
    const int smin = segs, grp0 = kTmaConsumers / smin / 32 * 32;
    double best = -1.0;
    for (int sg = smin; sg <= 16 && kTmaConsumers / sg / 32 * 32 == grp0 && grp0 > 0; ++sg) {
      const int rows = static_cast<int>((N + sg - 1) / sg), slots = (rows + 3) / 4 * 4;
      const double util = (static_cast<double>(N) / (sg * slots)) * (static_cast<double>(grp0) * sg / kTmaConsumers);
      if (util > best + 1e-9) {
        best = util;
        segs = sg;
      }
    }
  }
  int64_t wt = static_cast<int64_t>(kTmaConsumers / segs) * cpt;
  const int64_t row_bytes = npad * es * nin;  // shared memory per column of a tile
  // Width first, stages second: the backward (two input tiles per stage) is sized for TWO stages — runs twice as wide
  // measured 4 to 18 % faster than a third stage of narrow ones (128-byte runs half a megabyte apart are what DRAM
  // likes least).  The forward keeps three stages where they leave at least one line per run.
  int64_t fit = avail / (bwd ? 2 : 3) / row_bytes;
  if (fit < line) fit = avail / 2 / row_bytes;
  if (wt > fit) wt = fit;
  if (wt > inner) wt = inner;
  while (wt > 2 * line && outer * ((inner + wt - 1) / wt) < 2ll * sms) wt /= 2;
  // Runs are whole 128-byte lines: every box then starts on a 128-byte boundary of shared memory, which the
  // bulk-tensor copy requires of its shared-memory address, whatever N is.
  wt = wt / line * line;
  // boxes: the fewest that are at most 256 elements wide and whole lines
  for (; wt >= line; wt -= line) {
    const int nx = static_cast<int>((wt + 255) / 256);
    if (wt % (static_cast<int64_t>(nx) * line) == 0) {
      p.NX = nx;
      p.W = static_cast<int>(wt / nx);
      break;
    }
  }
  if (p.W == 0) return p;  // runs below 128 bytes: the plain-load kernels take it
  const int groups = p.W * p.NX / cpt;
  if (!p.reg) {
    segs = kTmaConsumers / groups;
    if (segs > N) segs = static_cast<int>(N);
    if (segs > 32) segs = 32;
  }
  p.segs = segs;
  const int64_t s = avail / (row_bytes * p.W * p.NX);
  if (s < 2) return p;
  p.S = static_cast<int>(s > kTmaMaxStages ? kTmaMaxStages : s);
  // the kernel's teams: 32 adjacent column groups x segs warps on one named barrier each (ids 1..15)
  p.ok = groups * segs <= kTmaConsumers && segs >= 1 && groups % 32 == 0 && (segs == 1 || groups / 32 <= 15);
  return p;
}

struct TmaLaunchArgs {
  const CUtensorMap *tm0, *tm1, *tmo;
  int64_t outer;
  int N;
  int64_t inner;
  const TmaTilePlan* p;
  int safe;
  unsigned grid;
  size_t smem;
  cudaStream_t st;
};
// One function per kernel instantiation: each carries its own "shared-memory limit raised" record.
template <typename T, bool LOG, bool BWD, bool REG> int tma_tile_go(const TmaLaunchArgs& a) {
  auto kernel = softmax_spatial_tma_kernel<T, LOG, BWD, REG>;
  static std::atomic<uint64_t> done{0};
  if (int e = set_smem_once_sm(kernel, done)) return e;
  return launch_pdl(kernel, dim3(a.grid), dim3(kTmaThreads), a.smem, a.st, *a.tm0, *a.tm1, *a.tmo, a.outer, a.N, a.inner,
                    a.p->W, a.p->NX, a.p->NB, a.p->S, a.p->segs, a.safe, device_status_ptr());
}

// in0 / in1 / out as in softmax_spatial_tma_kernel.  Returns kTmaNoFit when the shape does not suit the kernel
// (rows or strides the tensor map cannot express, a tile that leaves no room for two stages, no encoder).
template <typename T, bool LOG, bool BWD>
int softmax_spatial_tma_launch(const T* in0, const T* in1, T* out, int64_t outer, int64_t N, int64_t inner, int safe,
                               cudaStream_t st) {
  constexpr int NIN = BWD ? 2 : 1;
  constexpr int es = sizeof(T);
  if (N < 2 || N > 65536 || outer > 0x7fffffffLL || inner > 0x7fffffffLL || (inner * es) % 16 != 0) return kTmaNoFit;
  if ((N * inner * es) >= (1ll << 40)) return kTmaNoFit;  // the tensor map's stride limit
  const DeviceInfo& di = device_info();
  const int64_t avail = static_cast<int64_t>(di.max_smem_optin) - kTmaHeaderBytes;
  const TmaTilePlan p = plan_tma_tile(outer, N, inner, es, NIN, BWD, avail, di.sm_count);
  if (!p.ok || (static_cast<int64_t>(p.W) * es) % 128 != 0) return kTmaNoFit;
  const int64_t npad = (N + p.NB - 1) / p.NB * p.NB;
  const int WT = p.W * p.NX;
  CUtensorMap tm0, tm1, tmo;
  if (!encode_spatial_map(&tm0, in0, outer, N, inner, p.W, p.NB)) return kTmaNoFit;
  if (!encode_spatial_map(&tm1, BWD ? in1 : in0, outer, N, inner, p.W, p.NB)) return kTmaNoFit;
  if (!encode_spatial_map(&tmo, out, outer, N, inner, p.W, p.NB)) return kTmaNoFit;
  const size_t smem = static_cast<size_t>(kTmaHeaderBytes) + static_cast<size_t>(p.S) * npad * WT * es * NIN;
  const int64_t tiles = outer * ((inner + WT - 1) / WT);
  const int ctas = persistent_ctas(di.sm_count);
  int64_t grid = tiles < ctas ? tiles : ctas;
  const int64_t waves = (tiles + grid - 1) / grid;
  grid = (tiles + waves - 1) / waves;
  if (getenv("B2N_DEBUG") != nullptr)
    fprintf(stderr, "b2n: tma tile W=%d NX=%d NB=%d S=%d segs=%d reg=%d tiles=%lld grid=%lld smem=%zu\n", p.W, p.NX, p.NB, p.S,
            p.segs, p.reg ? 1 : 0, static_cast<long long>(tiles), static_cast<long long>(grid), smem);
  ProfileScope prof(BWD ? (LOG ? "log_softmax_bwd_tma" : "softmax_bwd_tma") : (LOG ? "log_softmax_fwd_tma" : "softmax_fwd_tma"), st);
  note_path("tma");
  const TmaLaunchArgs a{&tm0, &tm1, &tmo, outer, static_cast<int>(N), inner, &p, safe, static_cast<unsigned>(grid), smem, st};
  if constexpr (!BWD) {
    if (p.reg) return tma_tile_go<T, LOG, false, true>(a);
  }
  return tma_tile_go<T, LOG, BWD, false>(a);
}

template <typename TI, typename TO, bool LOG>
int softmax_fwd_typed(const void* x_, void* y_, int64_t outer, int64_t N, int64_t inner, cudaStream_t st) {
  const TI* x = static_cast<const TI*>(x_);
  TO* y = static_cast<TO*>(y_);
  const int forced = forced_path();
  const int safe = softmax_safe_mode() ? 1 : 0;  // rows of -inf give zeros (softmax only)
  if (inner == 1) {
    const int64_t M = outer;
    if constexpr (std::is_same<TI, TO>::value && sizeof(TI) <= 4 && !std::is_same<TI, double>::value) {
      if (forced != B2N_PATH_GENERIC && is_aligned(x, 16) && is_aligned(y, 16) && N <= (1 << 20)) {
        const DeviceInfo& di = device_info();
        const RingPlan p = plan_ring(M, N, sizeof(TI), 1, kSoftmaxEpt, persistent_ctas(di.sm_count), di.max_smem_optin);
        if (p.ok && forced != B2N_PATH_CLUSTER && forced != B2N_PATH_TWOPASS) {
          note_path("ring");
          switch (p.group) {
            case 32: return softmax_fwd_ring_launch<TI, LOG, 32>(p, x, y, M, N, st);
            case 64: return softmax_fwd_ring_launch<TI, LOG, 64>(p, x, y, M, N, st);
            case 128: return softmax_fwd_ring_launch<TI, LOG, 128>(p, x, y, M, N, st);
            case 256: return softmax_fwd_ring_launch<TI, LOG, 256>(p, x, y, M, N, st);
            default: return softmax_fwd_ring_launch<TI, LOG, 512>(p, x, y, M, N, st);
          }
        }
        if (forced == B2N_PATH_CLUSTER) {
          const ClusterPlan cp = plan_cluster(N, sizeof(TI), 1, di.max_smem_optin);
          if (cp.ok) {
            note_path("cluster");
            return softmax_cluster_launch<TI, LOG, false>(cp, x, static_cast<const TI*>(nullptr), y, M, N, st);
          }
        } else if (twopass_takes<TI>(N) && (forced == B2N_PATH_TWOPASS || (forced == B2N_PATH_AUTO && N * sizeof(TI) >= 32768))) {
          note_path("twopass");
          return softmax_twopass_launch<TI, LOG, false>(x, static_cast<const TI*>(nullptr), y, M, N, st);
        }
      }
    }
    if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
    note_path("generic");
    ProfileScope prof(LOG ? "log_softmax_fwd_generic" : "softmax_fwd_generic", st);
    constexpr int V = 16 / sizeof(TI);  // vector width in elements, by the input type
    const bool vec = N % V == 0 && is_aligned(x, 16) && is_aligned(y, V * sizeof(TO));
    if (N <= 1024) {
      const int grid = softmax_generic_grid(M, 8);
      if (vec) softmax_fwd_generic_kernel<TI, TO, LOG, 32, V><<<grid, 256, 0, st>>>(x, y, M, N, safe);
      else softmax_fwd_generic_kernel<TI, TO, LOG, 32, 1><<<grid, 256, 0, st>>>(x, y, M, N, safe);
    } else {
      const int grid = softmax_generic_grid(M, 1);
      const int threads = N <= 8192 ? 256 : 1024;
      if (vec) softmax_fwd_generic_kernel<TI, TO, LOG, 0, V><<<grid, threads, 0, st>>>(x, y, M, N, safe);
      else softmax_fwd_generic_kernel<TI, TO, LOG, 0, 1><<<grid, threads, 0, st>>>(x, y, M, N, safe);
    }
    return launched();
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
  note_path("generic");
  if constexpr (std::is_same<TI, TO>::value && !std::is_same<TI, double>::value) {
    constexpr int VEC = 16 / sizeof(TI);
    const DeviceInfo& di = device_info();
    if (inner % VEC == 0 && inner >= 64 && is_aligned(x, 16) && is_aligned(y, 16) && ring_tuning().tile_kb == 0 &&
        forced == B2N_PATH_AUTO) {  // (a pinned generic path keeps to the plain-load tile kernels below)
      const int e = softmax_spatial_tma_launch<TI, LOG, false>(x, static_cast<const TI*>(nullptr), y, outer, N, inner, safe, st);
      if (e != kTmaNoFit) return e;
    }
    const int tile = spatial_tile_elems(N, sizeof(TI), 1, inner, di.max_smem_optin);
    if (tile > 0 && inner % VEC == 0 && inner >= 64 && is_aligned(x, 16) && is_aligned(y, 16) && N <= (1 << 20)) {
      auto kernel = softmax_fwd_tile_kernel<TI, LOG>;
      static std::atomic<uint64_t> done{0};
      if (int e = set_smem_once_sm(kernel, done)) return e;
      const size_t smem = kTileScratchBytes + static_cast<size_t>(N) * tile * sizeof(TI);
      const int64_t tiles = outer * ((inner + tile - 1) / tile);
      const int64_t cap = static_cast<int64_t>(di.sm_count) * 8;
      ProfileScope prof(LOG ? "log_softmax_fwd_tile" : "softmax_fwd_tile", st);
      kernel<<<static_cast<int>(tiles < cap ? tiles : cap), kTileThreads, smem, st>>>(x, y, outer, static_cast<int>(N), inner,
                                                                                        tile, safe);
      return launched();
    }
  }
  if (N <= 64) {
    // short lines: registers hold them, every element is touched once
    ProfileScope prof(LOG ? "log_softmax_fwd_spatial" : "softmax_fwd_spatial", st);
    const bool v2 = inner % 2 == 0 && is_aligned(x, 2 * sizeof(TI)) && is_aligned(y, 2 * sizeof(TO));
    const int grid = softmax_generic_grid(outer * (v2 ? inner / 2 : inner), 256);
    const int n = static_cast<int>(N);
#define B2N_SPATIAL_FWD(NMAX)                                                                                       \
  do {                                                                                                              \
    if (v2) softmax_fwd_spatial_reg_kernel<TI, TO, LOG, NMAX, 2><<<grid, 256, 0, st>>>(x, y, outer, n, inner, safe); \
    else softmax_fwd_spatial_reg_kernel<TI, TO, LOG, NMAX, 1><<<grid, 256, 0, st>>>(x, y, outer, n, inner, safe);    \
  } while (0)
    if (N <= 8) B2N_SPATIAL_FWD(8);
    else if (N <= 16) B2N_SPATIAL_FWD(16);
    else if (N <= 32) B2N_SPATIAL_FWD(32);
    else  // one line of 64 values per thread: two would halve the resident warps
      softmax_fwd_spatial_reg_kernel<TI, TO, LOG, 64, 1><<<softmax_generic_grid(outer * inner, 256), 256, 0, st>>>(
          x, y, outer, n, inner, safe);
#undef B2N_SPATIAL_FWD
    return launched();
  }
  const int grid = softmax_generic_grid(outer * inner, 256);
  softmax_fwd_spatial_kernel<TI, TO, LOG><<<grid, 256, 0, st>>>(x, y, outer, N, inner, safe);
  return launched();
}

template <typename TG, typename TO, bool LOG>
int softmax_bwd_typed(const void* dy_, const void* y_, void* dx_, int64_t outer, int64_t N, int64_t inner,
                      cudaStream_t st) {
  const TG* dy = static_cast<const TG*>(dy_);
  const TG* y = static_cast<const TG*>(y_);
  TO* dx = static_cast<TO*>(dx_);
  const int forced = forced_path();
  if (inner == 1) {
    const int64_t M = outer;
    if constexpr (std::is_same<TG, TO>::value && sizeof(TG) <= 4 && !std::is_same<TG, double>::value) {
      if (forced != B2N_PATH_GENERIC && is_aligned(dy, 16) && is_aligned(y, 16) && is_aligned(dx, 16) &&
          N <= (1 << 20)) {
        const DeviceInfo& di = device_info();
        const RingPlan p = plan_ring(M, N, sizeof(TG), 2, kSoftmaxEpt, persistent_ctas(di.sm_count), di.max_smem_optin);
        if (p.ok && forced != B2N_PATH_CLUSTER && forced != B2N_PATH_TWOPASS) {
          note_path("ring");
          switch (p.group) {
            case 32: return softmax_bwd_ring_launch<TG, LOG, 32>(p, dy, y, dx, M, N, st);
            case 64: return softmax_bwd_ring_launch<TG, LOG, 64>(p, dy, y, dx, M, N, st);
            case 128: return softmax_bwd_ring_launch<TG, LOG, 128>(p, dy, y, dx, M, N, st);
            case 256: return softmax_bwd_ring_launch<TG, LOG, 256>(p, dy, y, dx, M, N, st);
            default: return softmax_bwd_ring_launch<TG, LOG, 512>(p, dy, y, dx, M, N, st);
          }
        }
        if (forced == B2N_PATH_CLUSTER) {
          const ClusterPlan cp = plan_cluster(N, sizeof(TG), 2, di.max_smem_optin);
          if (cp.ok) {
            note_path("cluster");
            return softmax_cluster_launch<TG, LOG, true>(cp, dy, y, dx, M, N, st);
          }
        } else if (twopass_takes<TG>(N) && (forced == B2N_PATH_TWOPASS || (forced == B2N_PATH_AUTO && N * sizeof(TG) >= 32768))) {
          note_path("twopass");
          return softmax_twopass_launch<TG, LOG, true>(dy, y, dx, M, N, st);
        }
      }
    }
    if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
    note_path("generic");
    ProfileScope prof(LOG ? "log_softmax_bwd_generic" : "softmax_bwd_generic", st);
    constexpr int V = (16 / sizeof(TG)) < (16 / sizeof(TO)) ? (16 / sizeof(TG)) : (16 / sizeof(TO));
    const bool vec = N % V == 0 && is_aligned(dy, V * sizeof(TG)) && is_aligned(y, V * sizeof(TG)) &&
                     is_aligned(dx, V * sizeof(TO));
    if (N <= 1024) {
      const int grid = softmax_generic_grid(M, 8);
      if (vec) softmax_bwd_generic_kernel<TG, TO, LOG, 32, V><<<grid, 256, 0, st>>>(dy, y, dx, M, N);
      else softmax_bwd_generic_kernel<TG, TO, LOG, 32, 1><<<grid, 256, 0, st>>>(dy, y, dx, M, N);
    } else {
      const int grid = softmax_generic_grid(M, 1);
      const int threads = N <= 8192 ? 256 : 1024;
      if (vec) softmax_bwd_generic_kernel<TG, TO, LOG, 0, V><<<grid, threads, 0, st>>>(dy, y, dx, M, N);
      else softmax_bwd_generic_kernel<TG, TO, LOG, 0, 1><<<grid, threads, 0, st>>>(dy, y, dx, M, N);
    }
    return launched();
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
  note_path("generic");
  if constexpr (std::is_same<TG, TO>::value && !std::is_same<TG, double>::value) {
    constexpr int VEC = 16 / sizeof(TG);
    const DeviceInfo& di = device_info();
    if (inner % VEC == 0 && inner >= 64 && is_aligned(dy, 16) && is_aligned(y, 16) && is_aligned(dx, 16) &&
        ring_tuning().tile_kb == 0 && forced == B2N_PATH_AUTO) {
      const int e = softmax_spatial_tma_launch<TG, LOG, true>(dy, y, dx, outer, N, inner, 0, st);
      if (e != kTmaNoFit) return e;
    }
    const int tile = spatial_tile_elems(N, sizeof(TG), 2, inner, di.max_smem_optin);
    if (tile > 0 && inner % VEC == 0 && inner >= 64 && is_aligned(dy, 16) && is_aligned(y, 16) && is_aligned(dx, 16) &&
        N <= (1 << 20)) {
      auto kernel = softmax_bwd_tile_kernel<TG, LOG>;
      static std::atomic<uint64_t> done{0};
      if (int e = set_smem_once_sm(kernel, done)) return e;
      const size_t smem = kTileScratchBytes + static_cast<size_t>(N) * tile * sizeof(TG) * 2;
      const int64_t tiles = outer * ((inner + tile - 1) / tile);
      const int64_t cap = static_cast<int64_t>(di.sm_count) * 8;
      ProfileScope prof(LOG ? "log_softmax_bwd_tile" : "softmax_bwd_tile", st);
      kernel<<<static_cast<int>(tiles < cap ? tiles : cap), kTileThreads, smem, st>>>(dy, y, dx, outer, static_cast<int>(N), inner,
                                                                                        tile);
      return launched();
    }
  }
  if (N <= 64) {
    ProfileScope prof(LOG ? "log_softmax_bwd_spatial" : "softmax_bwd_spatial", st);
    const bool v2 = inner % 2 == 0 && is_aligned(dy, 2 * sizeof(TG)) && is_aligned(y, 2 * sizeof(TG)) &&
                    is_aligned(dx, 2 * sizeof(TO));
    const int grid = softmax_generic_grid(outer * (v2 ? inner / 2 : inner), 256);
    const int n = static_cast<int>(N);
#define B2N_SPATIAL_BWD(NMAX)                                                                                    \
  do {                                                                                                           \
    if (v2) softmax_bwd_spatial_reg_kernel<TG, TO, LOG, NMAX, 2><<<grid, 256, 0, st>>>(dy, y, dx, outer, n, inner); \
    else softmax_bwd_spatial_reg_kernel<TG, TO, LOG, NMAX, 1><<<grid, 256, 0, st>>>(dy, y, dx, outer, n, inner);    \
  } while (0)
    if (N <= 8) B2N_SPATIAL_BWD(8);
    else if (N <= 16) B2N_SPATIAL_BWD(16);
    else if (N <= 32) B2N_SPATIAL_BWD(32);
    else  // two lines of 64 values of dy and y each would not fit the register file: one line per thread
      softmax_bwd_spatial_reg_kernel<TG, TO, LOG, 64, 1><<<softmax_generic_grid(outer * inner, 256), 256, 0, st>>>(
          dy, y, dx, outer, n, inner);
#undef B2N_SPATIAL_BWD
    return launched();
  }
  const int grid = softmax_generic_grid(outer * inner, 256);
  softmax_bwd_spatial_kernel<TG, TO, LOG><<<grid, 256, 0, st>>>(dy, y, dx, outer, N, inner);
  return launched();
}

#define B2N_SOFTMAX_TYPED_DECL(NAME)                                                                         \
  int softmax_fwd_##NAME(bool is_log, const void* x, void* y, int64_t outer, int64_t N, int64_t inner,       \
                         cudaStream_t st);                                                                   \
  int softmax_bwd_##NAME(bool is_log, const void* dy, const void* y, void* dx, int64_t outer, int64_t N,     \
                         int64_t inner, cudaStream_t st);

// fwd: TI -> TO.  bwd: (dy, y) of type BG -> dx of type BO.
#define B2N_SOFTMAX_TYPED_DEFINE(NAME, TI, TO, BG, BO)                                                       \
  int softmax_fwd_##NAME(bool is_log, const void* x, void* y, int64_t outer, int64_t N, int64_t inner,       \
                         cudaStream_t st) {                                                                  \
    return is_log ? softmax_fwd_typed<TI, TO, true>(x, y, outer, N, inner, st)                               \
                  : softmax_fwd_typed<TI, TO, false>(x, y, outer, N, inner, st);                             \
  }                                                                                                          \
  int softmax_bwd_##NAME(bool is_log, const void* dy, const void* y, void* dx, int64_t outer, int64_t N,     \
                         int64_t inner, cudaStream_t st) {                                                   \
    return is_log ? softmax_bwd_typed<BG, BO, true>(dy, y, dx, outer, N, inner, st)                          \
                  : softmax_bwd_typed<BG, BO, false>(dy, y, dx, outer, N, inner, st);                        \
  }

B2N_SOFTMAX_TYPED_DECL(f32)
B2N_SOFTMAX_TYPED_DECL(f16)
B2N_SOFTMAX_TYPED_DECL(bf16)
B2N_SOFTMAX_TYPED_DECL(f64)
B2N_SOFTMAX_TYPED_DECL(f16_f32)   // half_to_float: fwd f16 -> f32, bwd f32 grads -> f16 dx
B2N_SOFTMAX_TYPED_DECL(bf16_f32)  // same with bf16

}  // namespace b2n
