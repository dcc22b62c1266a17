// Slab kernels for layer norm / RMS norm rows LONGER than one CTA's threads hold (N > 8192 elements):
// the reference's few-long-rows regime (RowwiseMomentsKernelFunctor / norm_global_reduce /
// NormUpdateKernelFunctor, src/ATen/native/xpu/sycl/Norm.h:620-696, :155-223, :789-812).
//
// A row is split into C column slabs (C = 2, 4 or 8), one per CTA of a thread-block cluster, one CTA
// per SM.  A CTA owns the SAME columns for the whole launch, exactly like a ring-kernel CTA, so its
// gamma/beta values — and, in the backward, its dgamma/dbeta accumulators — stay in registers: the
// weight gradients remain fused at any row length, and every element still crosses HBM once in each
// direction.  What a slab cannot know alone are the row's statistics (forward) or its two row sums
// (backward).  Those are exchanged through distributed shared memory, software-pipelined one tile
// deep so that the exchange latency hides behind arithmetic:
//
//   iteration i:   phase A of tile i      read the tile's rows from the stage, reduce the slab's partial
//                                         values over the CTA; one thread sends them to every CTA of the
//                                         cluster with st.async — a one-way remote store that counts its
//                                         bytes on the RECEIVER's exchange mbarrier (no fence, no separate
//                                         arrival, nothing comes back);
//                  phase B of tile i - D  wait for the C partials of that tile, combine them in rank
//                                         order (every CTA gets the same bits), read the rows again,
//                                         write the result in place, hand the stage to the producer.
//
// D (1 or 2) is the pipeline depth: how many tiles of arithmetic an exchange has to arrive.  Exchange
// slots rotate modulo 8: a peer can send the partials of tile t + Q only after it has seen this CTA's
// partials of tile t + Q - D - 1, which this CTA sends in iteration t + Q - D - 1; this CTA finishes
// reading those of tile t in iteration t + D; so Q >= 2 D + 2 slots never collide (6 for D = 2).
// Forward statistics are combined exactly (Chan et al.): slab c contributes its element count, its
// mean and its centred sum of squares M2; each slab's own moments use the shifted one-pass sums of the
// ring kernel, with the same exact second pass when the shift is far from the slab's mean.
//
// Tiles (TR consecutive rows; a slab of a row is one bulk copy) are assigned to clusters in a fixed
// round-robin, so the partial weight gradients — row `cluster index` of ws[P][2][N] — are the same
// bits on every run.  One producer thread owns all bulk copies; every wait is bounded.
#pragma once
#include <cooperative_groups.h>

#include "ring.cuh"
#include "softmax_cluster.cuh"  // distributed-shared-memory helpers (map_to_rank, mbar_arrive_remote, ...)

namespace b2n {

constexpr int kNsConsumers = 512;
constexpr int kNsThreads = kNsConsumers + 32;  // + one producer warp
constexpr int kNsMaxCluster = 8;
constexpr int kNsMaxStages = 8;
constexpr int kNsSlots = 8;
constexpr int kNsHeaderBytes = 2048;
constexpr int kNsEpt = 16;  // elements per thread, as in the ring kernels

struct NormSlabShared {
  uint64_t full[kNsMaxStages];
  uint64_t done[kNsMaxStages];
  uint64_t xbar[kNsSlots];                          // one arrival (the owner's, with the byte count) + C x 16 bytes per use
  alignas(16) float part[kNsSlots][kNsMaxCluster][2][2];  // [slot][source rank][row of the tile][value]: 16 bytes per source
  float red[kRingRedFloats];                        // CTA-level reduction scratch
  float slab_n[kNsMaxCluster];                      // elements of slab c (forward: weights of the combination)
};
static_assert(sizeof(NormSlabShared) <= kNsHeaderBytes, "slab header too large");

// 16 bytes into a peer's shared memory, counted on the peer's mbarrier when they land
__device__ __forceinline__ void st_async_f32x4(uint32_t cluster_addr, float a, float b, float c, float d, uint32_t cluster_mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(cluster_addr),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(cluster_mbar)
               : "memory");
}

struct NormSlabGeom {
  int64_t M;
  int64_t nvec;      // 16-byte vectors per full row
  int C, crank;
  int64_t cluster_id, nclusters;
  int slab_vecs;     // vectors per slab (the last slab may own fewer)
  int my_nv;         // vectors of this CTA's slab
  int64_t v0;        // first vector of this CTA's slab
  int S;             // stages
  uint32_t slab_stride;  // bytes between two row-slabs in a stage
  int64_t ntiles;
  int my_tiles;      // tiles this cluster processes (the launcher keeps it below 2^31)

  template <int TR> __device__ __forceinline__ void init(int64_t M_, int64_t N, int vec, int slab_vecs_, int S_) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    M = M_;
    nvec = N / vec;
    C = static_cast<int>(cluster.num_blocks());
    crank = static_cast<int>(cluster.block_rank());
    cluster_id = blockIdx.x / C;
    nclusters = gridDim.x / C;
    slab_vecs = slab_vecs_;
    v0 = static_cast<int64_t>(crank) * slab_vecs;
    const int64_t left = nvec - v0;
    my_nv = static_cast<int>(left < slab_vecs ? (left > 0 ? left : 0) : slab_vecs);
    S = S_;
    slab_stride = static_cast<uint32_t>(slab_vecs) * 16u;
    ntiles = (M + TR - 1) / TR;
    my_tiles = cluster_id < ntiles ? static_cast<int>((ntiles - cluster_id + nclusters - 1) / nclusters) : 0;
  }
  // elements of slab c (for the combination of the forward statistics)
  __device__ __forceinline__ float slab_elems(int c, int vec) const {
    const int64_t left = nvec - static_cast<int64_t>(c) * slab_vecs;
    const int64_t nv = left < slab_vecs ? (left > 0 ? left : 0) : slab_vecs;
    return static_cast<float>(nv * vec);
  }
};

// Where a tile lives — its stage, the parity of that stage's barriers for this use, its exchange slot and that
// slot's parity, its first row — carried from tile to tile by additions: no division or 64-bit multiply in the loops.
struct SlabCursor {
  int s;
  uint32_t phase;
  int slot;
  uint32_t xphase;
  int64_t row0;
  __device__ __forceinline__ void start(const NormSlabGeom& g, int tr) {
    s = 0; phase = 0; slot = 0; xphase = 0;
    row0 = g.cluster_id * tr;
  }
  __device__ __forceinline__ void advance(const NormSlabGeom& g, int64_t row_step) {
    if (++s == g.S) { s = 0; phase ^= 1u; }
    if (++slot == kNsSlots) { slot = 0; xphase ^= 1u; }
    row0 += row_step;
  }
};

// The producer loop (one thread): fill the stages, then per tile wait for the result, send it out and refill
// the stage whose store has finished reading.  NIN tensors per stage; the result overwrites tensor 0.
template <int NIN, int TR>
__device__ __forceinline__ void norm_slab_producer(NormSlabShared* sh, unsigned char* stages, const NormSlabGeom& g,
                                                   const unsigned char* in0, const unsigned char* in1, unsigned char* out,
                                                   int* status) {
  const uint32_t stage_bytes = static_cast<uint32_t>(NIN * TR) * g.slab_stride;
  const uint32_t slab_bytes = static_cast<uint32_t>(g.my_nv) * 16u;
  auto rows_of = [&](int64_t tile) {
    const int64_t left = g.M - tile * TR;
    return static_cast<int>(left < TR ? left : TR);
  };
  auto load = [&](int s, int64_t tile) {
    const int rows = rows_of(tile);
    unsigned char* dst = stages + static_cast<size_t>(s) * stage_bytes;
    if (slab_bytes == 0) {  // a slab without columns still takes part in every exchange
      mbar_arrive(&sh->full[s]);
      return;
    }
    mbar_arrive_expect_tx(&sh->full[s], slab_bytes * static_cast<uint32_t>(rows * NIN));
    for (int r = 0; r < rows; ++r) {
      const size_t goff = (static_cast<size_t>(tile * TR + r) * static_cast<size_t>(g.nvec) + static_cast<size_t>(g.v0)) * 16;
      bulk_g2s(dst + static_cast<size_t>(r) * g.slab_stride, in0 + goff, slab_bytes, &sh->full[s]);
      if (NIN == 2) bulk_g2s(dst + static_cast<size_t>(TR + r) * g.slab_stride, in1 + goff, slab_bytes, &sh->full[s]);
    }
  };
  // the load cursor runs S - 1 tiles ahead of the store cursor once the ring is full
  int issued = 0, ls = 0;
  int64_t ltile = g.cluster_id;
  for (; issued < g.S && issued < g.my_tiles; ++issued) {
    load(ls, ltile);
    if (++ls == g.S) ls = 0;
    ltile += g.nclusters;
  }
  int j = 0, s = 0;
  uint32_t parity = 0;
  int64_t tile = g.cluster_id;
  for (; j < g.my_tiles; ++j) {
    if (!mbar_wait(&sh->done[s], parity, status)) break;
    const int rows = rows_of(tile);
    const unsigned char* src = stages + static_cast<size_t>(s) * stage_bytes;
    if (slab_bytes != 0) {
      for (int r = 0; r < rows; ++r) {
        const size_t goff = (static_cast<size_t>(tile * TR + r) * static_cast<size_t>(g.nvec) + static_cast<size_t>(g.v0)) * 16;
        bulk_s2g(out + goff, src + static_cast<size_t>(r) * g.slab_stride, slab_bytes);
      }
    }
    bulk_commit();
    if (j >= 1 && issued < g.my_tiles) {  // the store of tile j - 1 has read its stage: that is where tile `issued` goes
      bulk_wait_read<1>();
      load(ls, ltile);                    // ls == (j - 1) % S here
      if (++ls == g.S) ls = 0;
      ltile += g.nclusters;
      ++issued;
    }
    if (++s == g.S) { s = 0; parity ^= 1u; }
    tile += g.nclusters;
  }
  // if a wait gave up, let the loads already issued land before the CTA's shared memory goes away
  for (int k = j; k < issued; ++k) {
    mbar_wait(&sh->full[s], parity, status);
    if (++s == g.S) { s = 0; parity ^= 1u; }
  }
  bulk_wait_read<0>();
}

// One thread of the CTA: arm this CTA's exchange barrier of the slot for the C x 16 bytes it is about to receive,
// then send the tile's partial values to every CTA of the cluster (its own included).  vals[r][k]: row r, value k.
template <int TR>
__device__ __forceinline__ void norm_slab_push(NormSlabShared* sh, const NormSlabGeom& g, int slot, const float (&vals)[TR][2]) {
  mbar_arrive_expect_tx(&sh->xbar[slot], static_cast<uint32_t>(g.C) * 16u);
  const float a = vals[0][0], b = vals[0][1], c2 = TR > 1 ? vals[TR - 1][0] : 0.0f, d = TR > 1 ? vals[TR - 1][1] : 0.0f;
  const uint32_t dst = smem_u32(&sh->part[slot][g.crank][0][0]), bar = smem_u32(&sh->xbar[slot]);
  for (int c = 0; c < g.C; ++c) st_async_f32x4(map_to_rank(dst, c), a, b, c2, d, map_to_rank(bar, c));
}

template <typename WT, int VPT, int VEC>
__device__ __forceinline__ void slab_load_weights(const WT* __restrict__ w, float fill, int64_t v0, int my_nv, int tid,
                                                  float2 (&out)[VPT * VEC / 2]) {
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tid + k * kNsConsumers;
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      const bool ok = w != nullptr && v < my_nv;
      const int64_t col = (v0 + v) * VEC + e;
      out[(k * VEC + e) / 2] = make_float2(ok ? to_acc<float>(w[col]) : fill, ok ? to_acc<float>(w[col + 1]) : fill);
    }
  }
}

// ---- forward -------------------------------------------------------------------------------------------
// FULL: every slab fills every thread's vectors exactly (N == C * 512 * 16): no column range checks.
template <typename T, typename WT, bool RMS, int TR, int D, bool FULL>
__global__ void __launch_bounds__(kNsThreads, 1)
norm_fwd_slab_kernel(const T* __restrict__ x, const WT* __restrict__ gamma, const WT* __restrict__ beta, T* __restrict__ y,
                     float* __restrict__ mean, float* __restrict__ rstd, int64_t M, int64_t N, float eps, int slab_vecs,
                     int S, int* status) {
  namespace cg = cooperative_groups;
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, VPT = kNsEpt / VEC, HP = kNsEpt / 2, VH = VEC / 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  NormSlabShared* sh = reinterpret_cast<NormSlabShared*>(smem_raw);
  unsigned char* stages = smem_raw + kNsHeaderBytes;
  cg::cluster_group cluster = cg::this_cluster();
  NormSlabGeom g;
  g.init<TR>(M, N, VEC, slab_vecs, S);
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->done[s], kNsConsumers / 32);
    }
    for (int s = 0; s < kNsSlots; ++s) mbar_init(&sh->xbar[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  cluster.sync();  // every CTA's barriers exist before a peer arrives on them
  pdl_launch_dependents();
  pdl_wait();

  if (tid >= kNsConsumers) {
    if (tid == kNsConsumers)
      norm_slab_producer<1, TR>(sh, stages, g, reinterpret_cast<const unsigned char*>(x), nullptr,
                                reinterpret_cast<unsigned char*>(y), status);
  } else {
    const uint32_t stage_bytes = static_cast<uint32_t>(TR) * g.slab_stride;
    const uint32_t stages_u32 = smem_u32(stages);
    const float inv_n = 1.0f / static_cast<float>(N);
    const float my_n = static_cast<float>(g.my_nv * VEC);
    const float inv_my_n = g.my_nv > 0 ? 1.0f / my_n : 0.0f;
    float2 gw[HP], gb[HP];
    slab_load_weights<WT, VPT, VEC>(gamma, 1.0f, g.v0, g.my_nv, tid, gw);
    if constexpr (!RMS) slab_load_weights<WT, VPT, VEC>(beta, 0.0f, g.v0, g.my_nv, tid, gb);
    int red_phase = 0;
    bool ok = true;
    if (tid < g.C) sh->slab_n[tid] = g.slab_elems(tid, VEC);  // read in phase B, behind several barriers
    const int64_t row_step = g.nclusters * TR;
    SlabCursor ca, cb;  // phase A's tile and phase B's (D tiles behind)
    ca.start(g, TR);
    cb.start(g, TR);
    for (int i = 0; i < g.my_tiles + D && ok; ++i) {
      if (i < g.my_tiles) {
        // ---- phase A of tile i: this slab's moments of each row --------------------------------------
        const int s = ca.s;
        if (!mbar_wait(&sh->full[s], ca.phase, status)) { ok = false; break; }
        const int64_t row0 = ca.row0;
        const uint32_t sbase = stages_u32 + static_cast<uint32_t>(s) * stage_bytes;
        float shift[TR];
        float red1[TR * (RMS ? 1 : 2)];
#pragma unroll
        for (int r = 0; r < TR; ++r) {
          const bool valid = row0 + r < M && g.my_nv > 0;
          const uint32_t rbase = sbase + static_cast<uint32_t>(r) * g.slab_stride;
          shift[r] = 0.0f;
          if (!RMS && valid) {
            float2 first[VH];
            P::unpack2(lds128(rbase), first);
            shift[r] = first[0].x;
          }
          const float2 nshift = bcast2(-shift[r]);
          float2 ps[2] = {bcast2(0.0f), bcast2(0.0f)}, pq[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * kNsConsumers;
            if (valid && (FULL || v < g.my_nv)) {
              float2 xv[VH];
              P::unpack2(lds128(rbase + v * 16), xv);
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                if constexpr (!RMS) {
                  xv[e] = add2(xv[e], nshift);
                  ps[e & 1] = add2(ps[e & 1], xv[e]);
                }
                pq[e & 1] = fma2(xv[e], xv[e], pq[e & 1]);
              }
            }
          }
          if constexpr (RMS) {
            red1[r] = hsum2(add2(pq[0], pq[1]));
          } else {
            red1[2 * r] = hsum2(add2(ps[0], ps[1]));
            red1[2 * r + 1] = hsum2(add2(pq[0], pq[1]));
          }
        }
        group_reduce<kNsConsumers, TR * (RMS ? 1 : 2)>(red1, sh->red, 0, tid, red_phase, SumOp());
        float vals[TR][2];  // what this slab contributes: {mean, M2} of its part of the row (RMS: {sum x^2, -})
        if constexpr (RMS) {
#pragma unroll
          for (int r = 0; r < TR; ++r) { vals[r][0] = red1[r]; vals[r][1] = 0.0f; }
        } else {
          // mean_c = shift + sum d / n_c,  M2_c = sum d^2 - (sum d)^2 / n_c; when the shift lies far from the
          // slab's mean the subtraction cancels, and the sums are taken again about the mean just found
          bool exact = true;
          float mu_d[TR], m2c[TR];
#pragma unroll
          for (int r = 0; r < TR; ++r) {
            mu_d[r] = red1[2 * r] * inv_my_n;
            m2c[r] = fmaf(-mu_d[r], red1[2 * r], red1[2 * r + 1]);
            exact = exact && (mu_d[r] * mu_d[r] * my_n <= 8.0f * m2c[r] || g.my_nv == 0);  // false for NaN and for a cancelled M2
          }
          if (!exact) {
            float red2[2 * TR];
#pragma unroll
            for (int r = 0; r < TR; ++r) {
              const bool valid = row0 + r < M && g.my_nv > 0;
              const uint32_t rbase = sbase + static_cast<uint32_t>(r) * g.slab_stride;
              shift[r] += mu_d[r];
              const float2 nshift = bcast2(-shift[r]);
              float2 q[2] = {bcast2(0.0f), bcast2(0.0f)}, c2[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
              for (int k = 0; k < VPT; ++k) {
                const int v = tid + k * kNsConsumers;
                if (valid && (FULL || v < g.my_nv)) {
                  float2 xv[VH];
                  P::unpack2(lds128(rbase + v * 16), xv);
#pragma unroll
                  for (int e = 0; e < VH; ++e) {
                    xv[e] = add2(xv[e], nshift);
                    c2[e & 1] = add2(c2[e & 1], xv[e]);
                    q[e & 1] = fma2(xv[e], xv[e], q[e & 1]);
                  }
                }
              }
              red2[2 * r] = hsum2(add2(c2[0], c2[1]));
              red2[2 * r + 1] = hsum2(add2(q[0], q[1]));
            }
            group_reduce<kNsConsumers, 2 * TR>(red2, sh->red, 0, tid, red_phase, SumOp());
#pragma unroll
            for (int r = 0; r < TR; ++r) {
              mu_d[r] = red2[2 * r] * inv_my_n;
              const float m2 = fmaf(-mu_d[r], red2[2 * r], red2[2 * r + 1]);
              m2c[r] = m2 < 0.0f ? 0.0f : m2;  // keeps NaN
            }
          }
#pragma unroll
          for (int r = 0; r < TR; ++r) { vals[r][0] = shift[r] + mu_d[r]; vals[r][1] = m2c[r]; }
        }
        if (tid == 0) norm_slab_push<TR>(sh, g, ca.slot, vals);
        ca.advance(g, row_step);
      }
      if (i >= D) {
        // ---- phase B of tile i - D: the row's statistics from the C slabs, then the output -------------
        const int slot = cb.slot;
        if (!mbar_wait(&sh->xbar[slot], cb.xphase, status)) { ok = false; break; }
        const int s = cb.s;
        const int64_t row0 = cb.row0;
        const uint32_t sbase = stages_u32 + static_cast<uint32_t>(s) * stage_bytes;
#pragma unroll
        for (int r = 0; r < TR; ++r) {
          if (row0 + r >= M) break;  // uniform over the cluster
          float mu = 0.0f, rsd;
          if constexpr (RMS) {
            float sum = 0.0f;
            for (int c = 0; c < g.C; ++c) sum += sh->part[slot][c][r][0];
            rsd = rsqrt_nr(sum * inv_n + eps);
          } else {
            for (int c = 0; c < g.C; ++c) mu = fmaf(sh->slab_n[c] * inv_n, sh->part[slot][c][r][0], mu);
            float m2 = 0.0f;
            for (int c = 0; c < g.C; ++c) {
              const float d = sh->part[slot][c][r][0] - mu;
              const float nc = sh->slab_n[c];
              m2 += nc > 0.0f ? fmaf(nc * d, d, sh->part[slot][c][r][1]) : 0.0f;
            }
            rsd = rsqrt_nr(m2 * inv_n + eps);
          }
          const uint32_t rbase = sbase + static_cast<uint32_t>(r) * g.slab_stride;
          const float2 rs2 = bcast2(rsd), c2 = bcast2(-mu * rsd);
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * kNsConsumers;
            if (FULL || v < g.my_nv) {
              float2 xv[VH], o[VH];
              P::unpack2(lds128(rbase + v * 16), xv);
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                const int j = k * VH + e;
                if constexpr (RMS) o[e] = mul2(mul2(xv[e], rs2), gw[j]);
                else o[e] = fma2(fma2(xv[e], rs2, c2), gw[j], gb[j]);
              }
              sts128(rbase + v * 16, P::pack2(o));
            }
          }
          if (g.crank == 0 && tid == 0) {
            if (!RMS && mean) mean[row0 + r] = mu;
            if (rstd) rstd[row0 + r] = rsd;
          }
        }
        fence_async_smem();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(&sh->done[s]);
        cb.advance(g, row_step);
      }
    }
  }
  cluster.sync();  // no CTA leaves while a peer may still write into its header
}

// ---- backward ------------------------------------------------------------------------------------------
// stage = [dy rows | x rows]; dx overwrites the dy rows.  ws: partial weight gradients, row `cluster index`.
template <typename T, typename WT, bool RMS, bool WGRAD, int TR, int D, bool FULL>
__global__ void __launch_bounds__(kNsThreads, 1)
norm_bwd_slab_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const WT* __restrict__ gamma, T* __restrict__ dx, float* __restrict__ ws,
                     int64_t M, int64_t N, int slab_vecs, int S, int* status) {
  namespace cg = cooperative_groups;
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, VPT = kNsEpt / VEC, HP = kNsEpt / 2, VH = VEC / 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  NormSlabShared* sh = reinterpret_cast<NormSlabShared*>(smem_raw);
  unsigned char* stages = smem_raw + kNsHeaderBytes;
  cg::cluster_group cluster = cg::this_cluster();
  NormSlabGeom g;
  g.init<TR>(M, N, VEC, slab_vecs, S);
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->done[s], kNsConsumers / 32);
    }
    for (int s = 0; s < kNsSlots; ++s) mbar_init(&sh->xbar[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  cluster.sync();
  pdl_launch_dependents();
  pdl_wait();

  if (tid >= kNsConsumers) {
    if (tid == kNsConsumers)
      norm_slab_producer<2, TR>(sh, stages, g, reinterpret_cast<const unsigned char*>(dy),
                                reinterpret_cast<const unsigned char*>(x), reinterpret_cast<unsigned char*>(dx), status);
  } else {
    const uint32_t stage_bytes = static_cast<uint32_t>(2 * TR) * g.slab_stride;
    const uint32_t xoff = static_cast<uint32_t>(TR) * g.slab_stride;  // the x rows follow the dy rows
    const uint32_t stages_u32 = smem_u32(stages);
    const float inv_n = 1.0f / static_cast<float>(N);
    float2 gw[HP], dg[HP], db[HP];
    slab_load_weights<WT, VPT, VEC>(gamma, 1.0f, g.v0, g.my_nv, tid, gw);
#pragma unroll
    for (int e = 0; e < HP; ++e) { dg[e] = bcast2(0.0f); db[e] = bcast2(0.0f); }
    int red_phase = 0;
    bool ok = true;
    // mean / rstd of a tile's rows are fetched one iteration before phase A needs them and kept until phase B:
    // hist[0] the tile fetched ahead, hist[1] phase A's, hist[1 + D] phase B's
    float mu_h[D + 2][TR], rs_h[D + 2][TR];
    auto fetch_stats = [&](int j, int64_t row0, float (&mu)[TR], float (&rs)[TR]) {
#pragma unroll
      for (int r = 0; r < TR; ++r) {
        const int64_t row = row0 + r;
        const bool in = j < g.my_tiles && row < M;
        mu[r] = (!RMS && in) ? __ldg(mean + row) : 0.0f;
        rs[r] = in ? __ldg(rstd + row) : 0.0f;
      }
    };
#pragma unroll
    for (int h = 0; h < D + 2; ++h)
#pragma unroll
      for (int r = 0; r < TR; ++r) { mu_h[h][r] = 0.0f; rs_h[h][r] = 0.0f; }
    const int64_t row_step = g.nclusters * TR;
    SlabCursor ca, cb;
    ca.start(g, TR);
    cb.start(g, TR);
    fetch_stats(0, ca.row0, mu_h[0], rs_h[0]);
    for (int i = 0; i < g.my_tiles + D && ok; ++i) {
#pragma unroll
      for (int h = D + 1; h >= 1; --h)
#pragma unroll
        for (int r = 0; r < TR; ++r) { mu_h[h][r] = mu_h[h - 1][r]; rs_h[h][r] = rs_h[h - 1][r]; }
      fetch_stats(i + 1, ca.row0 + row_step, mu_h[0], rs_h[0]);  // (ca still points at tile i here)
      float (&mu_a)[TR] = mu_h[1];
      float (&rs_a)[TR] = rs_h[1];
      float (&mu_b)[TR] = mu_h[1 + D];
      float (&rs_b)[TR] = rs_h[1 + D];
      if (i < g.my_tiles) {
        // ---- phase A of tile i: this slab's share of the two row sums ---------------------------------
        const int s = ca.s;
        if (!mbar_wait(&sh->full[s], ca.phase, status)) { ok = false; break; }
        const int64_t row0 = ca.row0;
        const uint32_t sbase = stages_u32 + static_cast<uint32_t>(s) * stage_bytes;
        float red1[TR * (RMS ? 1 : 2)];
#pragma unroll
        for (int r = 0; r < TR; ++r) {
          const bool valid = row0 + r < M;
          const uint32_t dbase = sbase + static_cast<uint32_t>(r) * g.slab_stride, xbase = dbase + xoff;
          const float2 nmu = bcast2(-mu_a[r]), rs2 = bcast2(rs_a[r]);
          float2 p1 = bcast2(0.0f), p2 = bcast2(0.0f);
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * kNsConsumers;
            if (valid && (FULL || v < g.my_nv)) {
              float2 dv[VH], xh[VH];
              P::unpack2(lds128(dbase + v * 16), dv);
              P::unpack2(lds128(xbase + v * 16), xh);
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                const int j = k * VH + e;
                const float2 gv = mul2(dv[e], gw[j]);
                p2 = fma2(gv, mul2(add2(xh[e], nmu), rs2), p2);
                if (!RMS) p1 = add2(p1, gv);
              }
            }
          }
          if constexpr (RMS) {
            red1[r] = hsum2(p2);
          } else {
            red1[2 * r] = hsum2(p1);
            red1[2 * r + 1] = hsum2(p2);
          }
        }
        group_reduce<kNsConsumers, TR * (RMS ? 1 : 2)>(red1, sh->red, 0, tid, red_phase, SumOp());
        if (tid == 0) {
          float vals[TR][2];  // {s1, s2} of this slab (RMS: {0, s2})
#pragma unroll
          for (int r = 0; r < TR; ++r) {
            vals[r][0] = RMS ? 0.0f : red1[2 * r];
            vals[r][1] = RMS ? red1[r] : red1[2 * r + 1];
          }
          norm_slab_push<TR>(sh, g, ca.slot, vals);
        }
      }
      // (the statistics fetched ahead at the top of the iteration used ca before this advance; past the last
      // tile the cursor simply runs on, its rows fail the range check)
      ca.advance(g, row_step);
      if (i >= D) {
        // ---- phase B of tile i - D: the row sums from the C slabs, dx, and the weight-gradient terms -----
        const int slot = cb.slot;
        if (!mbar_wait(&sh->xbar[slot], cb.xphase, status)) { ok = false; break; }
        const int s = cb.s;
        const int64_t row0 = cb.row0;
        const uint32_t sbase = stages_u32 + static_cast<uint32_t>(s) * stage_bytes;
#pragma unroll
        for (int r = 0; r < TR; ++r) {
          if (row0 + r >= M) break;  // uniform over the cluster
          float s1 = 0.0f, s2 = 0.0f;
          for (int c = 0; c < g.C; ++c) {
            s1 += sh->part[slot][c][r][0];
            s2 += sh->part[slot][c][r][1];
          }
          const float rsd = rs_b[r];
          const float2 nmu = bcast2(-mu_b[r]), rs2 = bcast2(rsd);
          const float2 nar = bcast2(-(s2 * inv_n * rsd)), nbr = bcast2(-(s1 * inv_n * rsd));
          const uint32_t dbase = sbase + static_cast<uint32_t>(r) * g.slab_stride, xbase = dbase + xoff;
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * kNsConsumers;
            if (FULL || v < g.my_nv) {
              float2 dv[VH], xh[VH], o[VH];
              P::unpack2(lds128(dbase + v * 16), dv);
              P::unpack2(lds128(xbase + v * 16), xh);
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                const int j = k * VH + e;
                xh[e] = mul2(add2(xh[e], nmu), rs2);
                const float2 gv = mul2(dv[e], gw[j]);
                o[e] = fma2(gv, rs2, fma2(xh[e], nar, nbr));  // rstd*gv - (xhat*s2 + s1)*rstd/N
                if (WGRAD) {
                  dg[j] = fma2(dv[e], xh[e], dg[j]);
                  if (!RMS) db[j] = add2(db[j], dv[e]);
                }
              }
              sts128(dbase + v * 16, P::pack2(o));
            }
          }
        }
        fence_async_smem();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(&sh->done[s]);
        cb.advance(g, row_step);
      }
    }
    if (WGRAD) {
      float* wg = ws + (static_cast<size_t>(g.cluster_id) * 2 + 0) * N;
      float* wb = ws + (static_cast<size_t>(g.cluster_id) * 2 + 1) * N;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tid + k * kNsConsumers;
        if (v < g.my_nv) {
          const int64_t col = (g.v0 + v) * VEC;
#pragma unroll
          for (int q = 0; q < VEC / 4; ++q) {
            const int j = (k * VEC + q * 4) / 2;
            *reinterpret_cast<float4*>(wg + col + q * 4) = make_float4(dg[j].x, dg[j].y, dg[j + 1].x, dg[j + 1].y);
            if (!RMS) *reinterpret_cast<float4*>(wb + col + q * 4) = make_float4(db[j].x, db[j].y, db[j + 1].x, db[j + 1].y);
          }
        }
      }
    }
  }
  cluster.sync();
}

}  // namespace b2n
