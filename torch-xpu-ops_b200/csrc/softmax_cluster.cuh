// Cluster kernels for softmax / log-softmax rows that do not fit one CTA's shared memory
// (BASELINE config 5: 128 256 bf16 = 250.5 KB per row).  A row is split over the C CTAs of a
// thread-block cluster; each CTA holds its slice in shared memory, so every element still crosses
// HBM once in each direction:
//
//   bulk-async (TMA) load of the slice -> local (max, sum) or sum -> exchange through distributed
//   shared memory (every CTA reads its peers' partials) -> result written in place -> bulk-async
//   store.
//
// Clusters are persistent (grid = what the device can hold at once); C is chosen so that three
// CTAs fit an SM, and the CTAs sharing an SM are in different phases, which overlaps one CTA's
// load with another's arithmetic and store.  No cluster multicast is used: every CTA loads only
// its own slice.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "softmax_generic.cuh"
#include "softmax_ring.cuh"

namespace b2n {

namespace cg = cooperative_groups;

constexpr int kClusterThreads = 256;
constexpr int kClusterHeaderBytes = 256;

// exp for a value already reduced by the row maximum: expf for fp32 storage, the hardware 2^x for
// 16-bit storage (see RowExp in softmax_ring.cuh)
template <typename T> __device__ __forceinline__ float row_exp(float d) {
  if constexpr (sizeof(T) == 4) return expf(d);
  else return ex2_approx(d * kLog2e);
}

struct ClusterShared {
  uint64_t full;     // slice landed
  float part[2][2];  // [row parity][{max, sum} or {sum, -}] of this CTA, read by its peers
  float red[32];     // CTA-level reduction scratch
};
static_assert(sizeof(ClusterShared) <= kClusterHeaderBytes, "cluster header too large");

// BWD == false: in0 = x, out = y (softmax or log-softmax forward).
// BWD == true:  in0 = dy, in1 = y (forward output), out = dx.
// slice_vecs: 16-byte vectors per CTA slice (the last CTA of a cluster may own fewer).
template <typename T, bool LOG, bool BWD>
__global__ void __launch_bounds__(kClusterThreads)
softmax_cluster_kernel(const T* __restrict__ in0, const T* __restrict__ in1, T* __restrict__ out, int64_t M,
                       int64_t N, int slice_vecs, int* status) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, VH = VEC / 2;
  constexpr int NIN = BWD ? 2 : 1;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  ClusterShared* cs = reinterpret_cast<ClusterShared*>(smem_raw);
  unsigned char* slot0 = smem_raw + kClusterHeaderBytes;

  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int crank = static_cast<int>(cluster.block_rank());
  const int64_t cluster_id = blockIdx.x / C, nclusters = gridDim.x / C;
  const int tid = threadIdx.x;

  const int64_t nvec = N / VEC;
  const int64_t v0 = static_cast<int64_t>(crank) * slice_vecs;
  const int my_nv = static_cast<int>(nvec - v0 < slice_vecs ? (nvec - v0 > 0 ? nvec - v0 : 0) : slice_vecs);
  const uint32_t my_bytes = static_cast<uint32_t>(my_nv) * 16u;
  const uint32_t slot_bytes = static_cast<uint32_t>(slice_vecs) * 16u;
  const uint32_t s0 = smem_u32(slot0), s1 = s0 + slot_bytes;
  const float ninf = acc_neg_inf<float>();

  if (tid == 0) {
    mbar_init(&cs->full, 1);
    mbar_init_fence();
  }
  __syncthreads();
  cluster.sync();  // every CTA's header exists before anyone reads it remotely

  bool ok = true;  // false after a bounded wait gave up: keep meeting the cluster barriers, do no work
  uint32_t it = 0;
  for (int64_t row = cluster_id; row < M; row += nclusters, ++it) {
    const size_t goff = (static_cast<size_t>(row) * static_cast<size_t>(nvec) + static_cast<size_t>(v0)) * 16;
    if (ok && my_bytes > 0) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&cs->full, my_bytes * NIN);
        bulk_g2s(slot0, reinterpret_cast<const unsigned char*>(in0) + goff, my_bytes, &cs->full);
        if (BWD) bulk_g2s(slot0 + slot_bytes, reinterpret_cast<const unsigned char*>(in1) + goff, my_bytes, &cs->full);
      }
      ok = mbar_wait(&cs->full, it & 1u, status);
    }

    // ---- pass 1 over the slice: this CTA's partial ------------------------------------------------
    float pa = BWD ? 0.0f : ninf, pb = 0.0f;  // forward: running (max, sum); backward: sum
    if (ok) {
      if constexpr (!BWD) {
        MaxSum<float> ms;
        ms.init();
        for (int v = tid; v < my_nv; v += kClusterThreads) {
          float2 f[VH];
          P::unpack2(lds128(s0 + v * 16), f);
          float vm = ninf;
#pragma unroll
          for (int e = 0; e < VH; ++e) vm = fmaxf(vm, fmaxf(f[e].x, f[e].y));
          // one rescale per vector instead of one per element
          const float nm = fmaxf(ms.m, vm);
          const float scale = (ms.m == ninf) ? 0.0f : row_exp<T>(ms.m - nm);
          const float base = (nm == ninf) ? 0.0f : nm;  // all -inf so far: exp(-inf - 0) = 0, NaN stays NaN
          float acc = 0.0f;
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            acc += row_exp<T>(f[e].x - base);
            acc += row_exp<T>(f[e].y - base);
          }
          ms.s = ms.s * scale + acc;
          ms.m = nm;
        }
        ms = warp_merge(ms);
        if ((tid & 31) == 0) { cs->red[2 * (tid >> 5)] = ms.m; cs->red[2 * (tid >> 5) + 1] = ms.s; }
        __syncthreads();
        MaxSum<float> tot;
        tot.m = cs->red[0]; tot.s = cs->red[1];
        for (int w = 1; w < kClusterThreads / 32; ++w) {
          MaxSum<float> t;
          t.m = cs->red[2 * w]; t.s = cs->red[2 * w + 1];
          tot.merge(t);
        }
        pa = tot.m; pb = tot.s;
      } else {
        float2 acc2[2] = {bcast2(0.0f), bcast2(0.0f)};
        for (int v = tid; v < my_nv; v += kClusterThreads) {
          float2 d[VH];
          P::unpack2(lds128(s0 + v * 16), d);
          if constexpr (LOG) {
#pragma unroll
            for (int e = 0; e < VH; ++e) acc2[e & 1] = add2(acc2[e & 1], d[e]);
          } else {
            float2 yv[VH];
            P::unpack2(lds128(s1 + v * 16), yv);
#pragma unroll
            for (int e = 0; e < VH; ++e) acc2[e & 1] = fma2(d[e], yv[e], acc2[e & 1]);
          }
        }
        float s = warp_reduce(hsum2(add2(acc2[0], acc2[1])), SumOp());
        if ((tid & 31) == 0) cs->red[tid >> 5] = s;
        __syncthreads();
        float tot = cs->red[0];
        for (int w = 1; w < kClusterThreads / 32; ++w) tot += cs->red[w];
        pa = tot;
      }
    }
    if (tid == 0) { cs->part[it & 1][0] = pa; cs->part[it & 1][1] = pb; }

    // ---- exchange: every CTA combines all C partials in rank order (same result everywhere) ------
    cluster.sync();
    float r0, r1 = 0.0f;
    if constexpr (!BWD) {
      MaxSum<float> tot;
      tot.init();
      for (int c = 0; c < C; ++c) {
        const float* rp = cluster.map_shared_rank(&cs->part[it & 1][0], c);
        MaxSum<float> t;
        t.m = rp[0]; t.s = rp[1];
        if (c == 0) tot = t; else tot.merge(t);
      }
      if (tot.m == -ninf) tot.s = acc_nan<float>();  // +inf in the row: exp(inf - inf)
      r0 = tot.m; r1 = tot.s;
    } else {
      float tot = 0.0f;
      for (int c = 0; c < C; ++c) tot += *cluster.map_shared_rank(&cs->part[it & 1][0], c);
      r0 = tot;
    }

    // ---- pass 2: result in place, then out ----------------------------------------------------------
    if (ok && my_bytes > 0) {
      if constexpr (!BWD) {
        const float lg = LOG ? logf(r1) : 0.0f;
        const float2 noff = bcast2(-(r0 + lg)), inv = bcast2(LOG ? 0.0f : 1.0f / r1);
        const float2 l2e = bcast2(kLog2e), c2 = bcast2(-r0 * kLog2e);
        for (int v = tid; v < my_nv; v += kClusterThreads) {
          float2 f[VH], o[VH];
          P::unpack2(lds128(s0 + v * 16), f);
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            if constexpr (LOG) {
              if constexpr (sizeof(T) == 4) o[e] = make_float2((f[e].x - r0) - lg, (f[e].y - r0) - lg);
              else o[e] = add2(f[e], noff);
            } else if constexpr (sizeof(T) == 4) {
              o[e] = make_float2(expf(f[e].x - r0) / r1, expf(f[e].y - r0) / r1);
            } else {
              const float2 t = fma2(f[e], l2e, c2);
              o[e] = mul2(make_float2(ex2_approx(t.x), ex2_approx(t.y)), inv);
            }
          }
          sts128(s0 + v * 16, P::pack2(o));
        }
      } else {
        const float2 ns = bcast2(-r0), l2e = bcast2(kLog2e);
        for (int v = tid; v < my_nv; v += kClusterThreads) {
          float2 d[VH], yv[VH], o[VH];
          P::unpack2(lds128(s0 + v * 16), d);
          P::unpack2(lds128(s1 + v * 16), yv);
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            if constexpr (LOG) {
              float2 ey;
              if constexpr (sizeof(T) == 4) {
                ey = make_float2(expf(yv[e].x), expf(yv[e].y));
              } else {
                const float2 t = mul2(yv[e], l2e);
                ey = make_float2(ex2_approx(t.x), ex2_approx(t.y));
              }
              o[e] = fma2(ey, ns, d[e]);
            } else {
              o[e] = mul2(yv[e], add2(d[e], ns));
            }
          }
          sts128(s0 + v * 16, P::pack2(o));
        }
      }
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        bulk_s2g(reinterpret_cast<unsigned char*>(out) + goff, slot0, my_bytes);
        bulk_commit();
        bulk_wait_read<0>();  // the slice is reloaded next (by this thread): its store must have read it
      }
    }
  }
  if (tid == 0) bulk_wait_all<0>();
  cluster.sync();  // no CTA leaves while a peer may still read its partials
}

}  // namespace b2n
