// Slab kernels for softmax / log-softmax rows too long for the ring (BASELINE config 5: 128 256
// bf16 = 250.5 KB per row, more than one CTA's shared memory).
//
// A row is split over the C CTAs of a thread-block cluster (C = 1, 2, 4 or 8; one CTA per SM).
// Each CTA keeps its slice of the row RESIDENT in shared memory between the two passes the math
// needs, so every element crosses HBM once in each direction:
//
//   pass 1  the slice arrives in 32 KB chunks (bulk-async / TMA, one mbarrier per chunk); the 16
//           consumer warps fold each chunk into per-thread running (max, sum exp) — or sum dy /
//           sum y*dy for the backward — as soon as it lands;
//   combine one CTA-wide reduction, then the C partials are exchanged through distributed shared
//           memory: every CTA writes its pair into every peer's header (st.shared::cluster) and
//           arrives on the peer's exchange mbarrier; each CTA waits on its own;
//   pass 2  chunk by chunk the result is written in place and handed to the producer, which
//           bulk-stores it and refills the chunk buffer with the NEXT row's data.
//
// So while pass 2 of row r drains, row r+1 is already streaming in behind it, and pass 1 of row
// r+1 finds most of its chunks present: loads and stores overlap the arithmetic of both passes.
// A producer warp (one thread) owns all bulk copies.  Every wait is an mbarrier wait with a time
// limit; no cluster multicast is used (every CTA loads only its own slice).
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "softmax_generic.cuh"
#include "softmax_ring.cuh"

namespace b2n {

namespace cg = cooperative_groups;

constexpr int kSlabConsumers = 512;                  // 16 consumer warps
constexpr int kSlabThreads = kSlabConsumers + 32;    // + one producer warp
constexpr int kSlabChunkVecs = 2048;                 // 32 KB chunks: 4 vectors per consumer thread
constexpr int kSlabMaxChunks = 8;
constexpr int kSlabMaxCluster = 8;
constexpr int kSlabHeaderBytes = 1024;

// exp for a value already reduced by the row maximum: expf for fp32 storage, the hardware 2^x for
// 16-bit storage (see RowExp in softmax_ring.cuh)
template <typename T> __device__ __forceinline__ float row_exp(float d) {
  if constexpr (sizeof(T) == 4) return expf(d);
  else return ex2_approx(d * kLog2e);
}

struct SlabShared {
  uint64_t full[kSlabMaxChunks];  // chunk landed (bulk-copy bytes counted); one phase per row
  uint64_t done[kSlabMaxChunks];  // every consumer warp wrote its part of the chunk's result
  uint64_t xchg;                  // all C partials of the current row are in `part`
  float part[2][kSlabMaxCluster][2];  // [row parity][rank][{max, sum} or {sum, -}], written by the peers
  float red[2][32];               // CTA-level reduction scratch, double-buffered by row parity
};
static_assert(sizeof(SlabShared) <= kSlabHeaderBytes, "slab header too large");

// remote shared-memory helpers (distributed shared memory of the cluster)
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_remote_f32x2(uint32_t cluster_addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(cluster_addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((it & 0x3ffu) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
      record_status(status, B2N_ERR_TIMEOUT);
      return false;
    }
  }
}

// BWD == false: in0 = x, out = y (softmax or log-softmax forward).
// BWD == true:  in0 = dy, in1 = y (forward output), out = dx.
// slice_vecs: 16-byte vectors per CTA slice (the last CTAs of a cluster may own fewer, or none).
template <typename T, bool LOG, bool BWD>
__global__ void __launch_bounds__(kSlabThreads, 1)
softmax_slab_kernel(const T* __restrict__ in0, const T* __restrict__ in1, T* __restrict__ out, int64_t M,
                    int64_t N, int slice_vecs, int* status) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, VH = VEC / 2;
  constexpr int NIN = BWD ? 2 : 1;
  constexpr int VPT = kSlabChunkVecs / kSlabConsumers;  // vectors per thread per chunk
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  SlabShared* sh = reinterpret_cast<SlabShared*>(smem_raw);
  unsigned char* slot0 = smem_raw + kSlabHeaderBytes;

  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int crank = static_cast<int>(cluster.block_rank());
  const int64_t cluster_id = blockIdx.x / C, nclusters = gridDim.x / C;
  const int tid = threadIdx.x;

  const int64_t nvec = N / VEC;
  const int64_t v0 = static_cast<int64_t>(crank) * slice_vecs;
  const int my_nv = static_cast<int>(nvec - v0 < slice_vecs ? (nvec - v0 > 0 ? nvec - v0 : 0) : slice_vecs);
  const int nch = (my_nv + kSlabChunkVecs - 1) / kSlabChunkVecs;
  const uint32_t slot_bytes = static_cast<uint32_t>(slice_vecs) * 16u;
  const float ninf = acc_neg_inf<float>();

  if (tid == 0) {
    for (int c = 0; c < kSlabMaxChunks; ++c) {
      mbar_init(&sh->full[c], 1);
      mbar_init(&sh->done[c], kSlabConsumers / 32);
    }
    mbar_init(&sh->xchg, C);
    mbar_init_fence();
  }
  __syncthreads();
  cluster.sync();  // every CTA's barriers exist before a peer arrives on them

  auto chunk_vecs = [&](int c) { return my_nv - c * kSlabChunkVecs < kSlabChunkVecs ? my_nv - c * kSlabChunkVecs : kSlabChunkVecs; };

  if (tid >= kSlabConsumers) {
    // ---------------- producer: all bulk copies of this CTA ----------------
    if (tid == kSlabConsumers) {
      auto load_chunk = [&](int64_t row, int c) {
        const uint32_t bytes = static_cast<uint32_t>(chunk_vecs(c)) * 16u;
        const size_t goff = (static_cast<size_t>(row) * static_cast<size_t>(nvec) + static_cast<size_t>(v0) +
                             static_cast<size_t>(c) * kSlabChunkVecs) * 16;
        unsigned char* dst = slot0 + static_cast<size_t>(c) * kSlabChunkVecs * 16;
        mbar_arrive_expect_tx(&sh->full[c], bytes * NIN);
        bulk_g2s(dst, reinterpret_cast<const unsigned char*>(in0) + goff, bytes, &sh->full[c]);
        if (BWD) bulk_g2s(dst + slot_bytes, reinterpret_cast<const unsigned char*>(in1) + goff, bytes, &sh->full[c]);
      };
      if (cluster_id < M)
        for (int c = 0; c < nch; ++c) load_chunk(cluster_id, c);
      uint32_t it = 0;
      bool ok = true;
      for (int64_t row = cluster_id; row < M && ok; row += nclusters, ++it) {
        const int64_t next = row + nclusters;
        for (int c = 0; c < nch; ++c) {
          if (!mbar_wait(&sh->done[c], it & 1u, status)) { ok = false; break; }
          const size_t goff = (static_cast<size_t>(row) * static_cast<size_t>(nvec) + static_cast<size_t>(v0) +
                               static_cast<size_t>(c) * kSlabChunkVecs) * 16;
          bulk_s2g(reinterpret_cast<unsigned char*>(out) + goff, slot0 + static_cast<size_t>(c) * kSlabChunkVecs * 16,
                   static_cast<uint32_t>(chunk_vecs(c)) * 16u);
          bulk_commit();
          if (c >= 1 && next < M) {  // the previous chunk's store has read its buffer: refill it
            bulk_wait_read<1>();
            load_chunk(next, c - 1);
          }
        }
        if (ok && nch > 0 && next < M) {
          bulk_wait_read<0>();
          load_chunk(next, nch - 1);
        }
      }
      bulk_wait_all<0>();
    }
  } else {
    // ---------------- consumers ----------------
    const uint32_t s0 = smem_u32(slot0), s1 = s0 + slot_bytes;
    const uint32_t xchg_local = smem_u32(&sh->xchg);
    uint32_t it = 0;
    for (int64_t row = cluster_id; row < M; row += nclusters, ++it) {
      // ---- pass 1: fold the chunks as they land -----------------------------------------------------
      bool ok = true;
      float pa, pb = 0.0f;
      if constexpr (!BWD) {
        MaxSum<float> ms;
        ms.init();
        for (int c = 0; c < nch && ok; ++c) {
          ok = mbar_wait(&sh->full[c], it & 1u, status);
          if (!ok) break;
          const int cv = chunk_vecs(c);
          const uint32_t cb = s0 + static_cast<uint32_t>(c) * kSlabChunkVecs * 16;
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * kSlabConsumers;
            if (v < cv) {
              float2 f[VH];
              P::unpack2(lds128(cb + v * 16), f);
              float vm = ninf;
#pragma unroll
              for (int e = 0; e < VH; ++e) vm = fmaxf(vm, fmaxf(f[e].x, f[e].y));
              // one rescale per 16-byte vector instead of one per element
              const float nm = fmaxf(ms.m, vm);
              const float scale = (ms.m == ninf) ? 0.0f : row_exp<T>(ms.m - nm);
              const float base = (nm == ninf) ? 0.0f : nm;  // all -inf so far: exp(-inf - 0) = 0; NaN stays NaN
              float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                a0 += row_exp<T>(f[e].x - base);
                a1 += row_exp<T>(f[e].y - base);
              }
              ms.s = fmaf(ms.s, scale, a0 + a1);
              ms.m = nm;
            }
          }
        }
        if (!ok) break;  // uniform: every consumer thread waited on the same barrier
        ms = warp_merge(ms);
        float* red = sh->red[it & 1];
        if ((tid & 31) == 0) { red[2 * (tid >> 5)] = ms.m; red[2 * (tid >> 5) + 1] = ms.s; }
        named_bar_sync(1, kSlabConsumers);
        MaxSum<float> tot;
        tot.m = red[0]; tot.s = red[1];
#pragma unroll
        for (int w = 1; w < kSlabConsumers / 32; ++w) {
          MaxSum<float> t;
          t.m = red[2 * w]; t.s = red[2 * w + 1];
          tot.merge(t);
        }
        pa = tot.m; pb = tot.s;
      } else {
        float2 acc2[2] = {bcast2(0.0f), bcast2(0.0f)};
        for (int c = 0; c < nch && ok; ++c) {
          ok = mbar_wait(&sh->full[c], it & 1u, status);
          if (!ok) break;
          const int cv = chunk_vecs(c);
          const uint32_t cb = static_cast<uint32_t>(c) * kSlabChunkVecs * 16;
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * kSlabConsumers;
            if (v < cv) {
              float2 d[VH];
              P::unpack2(lds128(s0 + cb + v * 16), d);
              if constexpr (LOG) {
#pragma unroll
                for (int e = 0; e < VH; ++e) acc2[e & 1] = add2(acc2[e & 1], d[e]);
              } else {
                float2 yv[VH];
                P::unpack2(lds128(s1 + cb + v * 16), yv);
#pragma unroll
                for (int e = 0; e < VH; ++e) acc2[e & 1] = fma2(d[e], yv[e], acc2[e & 1]);
              }
            }
          }
        }
        if (!ok) break;
        const float s = warp_reduce(hsum2(add2(acc2[0], acc2[1])), SumOp());
        float* red = sh->red[it & 1];
        if ((tid & 31) == 0) red[tid >> 5] = s;
        named_bar_sync(1, kSlabConsumers);
        float tot = red[0];
#pragma unroll
        for (int w = 1; w < kSlabConsumers / 32; ++w) tot += red[w];
        pa = tot;
      }

      // ---- exchange: push this CTA's pair into every CTA's header, then wait for all C pairs ---------
      if (tid < C) {
        const uint32_t dst = map_to_rank(smem_u32(&sh->part[it & 1][crank][0]), tid);
        st_remote_f32x2(dst, pa, pb);
        mbar_arrive_remote(map_to_rank(xchg_local, tid));
      }
      if (!mbar_wait_cluster(&sh->xchg, it & 1u, status)) break;
      float r0, r1 = 0.0f;
      if constexpr (!BWD) {
        MaxSum<float> tot;
        tot.m = sh->part[it & 1][0][0]; tot.s = sh->part[it & 1][0][1];
        for (int c = 1; c < C; ++c) {  // rank order: the same result in every CTA
          MaxSum<float> t;
          t.m = sh->part[it & 1][c][0]; t.s = sh->part[it & 1][c][1];
          tot.merge(t);
        }
        if (tot.m == -ninf) tot.s = acc_nan<float>();  // +inf in the row: exp(inf - inf)
        r0 = tot.m; r1 = tot.s;
      } else {
        float tot = 0.0f;
        for (int c = 0; c < C; ++c) tot += sh->part[it & 1][c][0];
        r0 = tot;
      }

      // ---- pass 2: result in place, chunk by chunk, each handed to the producer when written ---------
      const float lg = (!BWD && LOG) ? logf(r1) : 0.0f;
      const float2 noff = bcast2(-(r0 + lg)), inv = bcast2((!BWD && !LOG) ? 1.0f / r1 : 0.0f);
      const float2 l2e = bcast2(kLog2e), c2 = bcast2(-r0 * kLog2e), ns = bcast2(-r0);
      for (int c = 0; c < nch; ++c) {
        const int cv = chunk_vecs(c);
        const uint32_t cb = static_cast<uint32_t>(c) * kSlabChunkVecs * 16;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * kSlabConsumers;
          if (v < cv) {
            float2 f[VH], o[VH];
            P::unpack2(lds128(s0 + cb + v * 16), f);
            if constexpr (!BWD) {
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
            } else {
              float2 yv[VH];
              P::unpack2(lds128(s1 + cb + v * 16), yv);
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
                  o[e] = fma2(ey, ns, f[e]);       // dy - exp(y) * sum
                } else {
                  o[e] = mul2(yv[e], add2(f[e], ns));  // y * (dy - sum)
                }
              }
            }
            sts128(s0 + cb + v * 16, P::pack2(o));
          }
        }
        fence_async_smem();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(&sh->done[c]);
      }
    }
  }
  cluster.sync();  // no CTA leaves while a peer may still write into its header
}

}  // namespace b2n
