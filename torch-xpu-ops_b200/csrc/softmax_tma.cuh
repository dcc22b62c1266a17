// Softmax / log-softmax over a dim that is NOT the last, on tensor-map TMA tiles.
//
// The tensor is [outer, N, inner]; a line runs over N with stride `inner`.  A tile is all N line elements
// x W adjacent inner positions: N runs of W elements, `inner` elements apart.  That is exactly what a
// tiled bulk-tensor copy moves with ONE instruction: the tensor is described to the TMA unit as a
// rank-3 tensor (inner, N, outer), a tile is a box of W x NB x 1 elements (NB = N, or 256 rows at a time
// for longer lines), and `cp.async.bulk.tensor.3d` brings the box into shared memory — densely packed,
// row pitch W — while completing a transaction count on an mbarrier; the mirror instruction sends the
// result back.  Coordinates past the tensor's edge are filled with zeros on the way in and dropped on
// the way out, so edge tiles need no special case.  Every tile starts at x = k * W with W * sizeof(T) a
// multiple of 16 bytes, as the bulk-tensor copy requires.
//
// A tile is NX boxes wide (W <= 256 elements each) so that short lines still make tiles of tens of KB, and a
// line is shared by `segs` threads.  In the forward, when a thread's share of a line is at most 32 elements
// (lines up to 256 long), the thread keeps it in REGISTERS: one shared-memory read and ONE exp per element
// (exp(x - max) serves the sum and the output) — with two exps per element the kernel is bound by the
// special-function unit, not by HBM.
//
// Persistent CTAs, one per SM: a producer thread keeps S tiles in flight (loads of the next tiles and
// the store of the previous one overlap the arithmetic); 512 consumer threads work on the tile in shared
// memory as the tile kernels of softmax_generic.cuh do — a line shared by `segs` threads, each walking
// every segs-th element, consecutive threads on consecutive addresses, partial results combined in
// segment order — and leave the result in place.  Every element crosses HBM once each way.
// No cluster multicast; every wait bounded.
#pragma once
#include <cuda.h>

#include "ring.cuh"
#include "softmax_generic.cuh"

namespace b2n {

constexpr int kTmaConsumers = 512;
constexpr int kTmaThreads = kTmaConsumers + 128;  // + one producer warpgroup, which hands its registers to the consumers
constexpr int kTmaMaxStages = 4;
constexpr int kTmaHeaderBytes = 1024 + kTmaConsumers * 16;  // barriers, then one float4 of partial results per consumer

struct TmaTileShared {
  uint64_t full[kTmaMaxStages];
  uint64_t done[kTmaMaxStages];
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* tm, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(tm), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tm, int x, int y, int z, const void* src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(tm), "r"(x),
               "r"(y), "r"(z), "r"(smem_u32(src))
               : "memory");
}

// One 32-bit word of shared memory by its 32-bit shared-space address (address arithmetic stays in 32 bits).
__device__ __forceinline__ uint32_t lds_b32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts_b32(uint32_t a, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
// A word as the thread's column pair: two 16-bit values, or one fp32 value (y = -inf, the identity of the maximum).
template <typename T> __device__ __forceinline__ float2 word_to_pair(uint32_t w) {
  if constexpr (std::is_same<T, bf16>::value) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  else if constexpr (std::is_same<T, f16>::value) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  else return make_float2(__uint_as_float(w), acc_neg_inf<float>());
}
template <typename T> __device__ __forceinline__ uint32_t pair_to_word(float2 v) {
  if constexpr (std::is_same<T, bf16>::value) {
    const __nv_bfloat162 h = __float22bfloat162_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else if constexpr (std::is_same<T, f16>::value) {
    const __half2 h = __float22half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    return __float_as_uint(v.x);
  }
}

// BWD == false: in0 = x, out = y.   BWD == true: in0 = dy, in1 = y (forward output), out = dx.
// Tiles go to CTAs round-robin.
// W: box width in elements; NX: boxes per tile along `inner`; NB: rows per box; S: stages; segs: threads per line.
// REG (forward only): a thread's share of a line, at most kTmaRegRows elements per column, lives in registers.
constexpr int kTmaRegRows = 32;
template <typename T, bool LOG, bool BWD, bool REG>
__global__ void __launch_bounds__(kTmaThreads, 1)
softmax_spatial_tma_kernel(const __grid_constant__ CUtensorMap tm_in0, const __grid_constant__ CUtensorMap tm_in1,
                           const __grid_constant__ CUtensorMap tm_out, int64_t outer, int N, int64_t inner, int W, int NX,
                           int NB, int S, int segs, int safe, int* status) {
  constexpr int NIN = BWD ? 2 : 1;
  constexpr int CPT = sizeof(T) == 2 ? 2 : 1;  // columns a thread handles with one shared-memory access
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  TmaTileShared* sh = reinterpret_cast<TmaTileShared*>(smem_raw);
  float4* part = reinterpret_cast<float4*>(smem_raw + 1024);
  unsigned char* stages = smem_raw + kTmaHeaderBytes;

  const int tid = threadIdx.x;
  const int nbox = (N + NB - 1) / NB;
  const uint32_t box_bytes = static_cast<uint32_t>(NB) * W * sizeof(T);
  const uint32_t xbox_bytes = box_bytes * nbox;     // one column of boxes: all N rows (padded to whole boxes) x W
  const uint32_t tile_bytes = xbox_bytes * NX;      // one tensor's tile
  const uint32_t stage_bytes = tile_bytes * NIN;
  const int WT = W * NX;                            // tile width
  const int64_t tpo = (inner + WT - 1) / WT, total = outer * tpo;
  const int64_t first = blockIdx.x;
  const int my_tiles = first < total ? static_cast<int>((total - first + gridDim.x - 1) / gridDim.x) : 0;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->done[s], kTmaConsumers / 32);
    }
    mbar_init_fence();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();

  if (tid >= kTmaConsumers) {
    // ---------------- producer: every bulk-tensor copy of this CTA ----------------
    ring_producer_regs();
    if (tid == kTmaConsumers && my_tiles > 0) {
      auto coords = [&](int64_t t, int& x0, int& o) {
        const int64_t oo = t / tpo;
        o = static_cast<int>(oo);
        x0 = static_cast<int>((t - oo * tpo) * WT);
      };
      auto load = [&](int s, int64_t t) {
        int x0, o;
        coords(t, x0, o);
        unsigned char* dst = stages + static_cast<size_t>(s) * stage_bytes;
        mbar_arrive_expect_tx(&sh->full[s], stage_bytes);
        for (int bx = 0; bx < NX; ++bx)
          for (int b = 0; b < nbox; ++b) {
            const size_t off = static_cast<size_t>(bx) * xbox_bytes + static_cast<size_t>(b) * box_bytes;
            // (a box that starts past the tensor's edge is all zeros: still counted on the barrier)
            tma_load_3d(dst + off, &tm_in0, x0 + bx * W, b * NB, o, &sh->full[s]);
            if (BWD) tma_load_3d(dst + tile_bytes + off, &tm_in1, x0 + bx * W, b * NB, o, &sh->full[s]);
          }
      };
      int issued = 0, ls = 0;
      int64_t lt = first;
      for (; issued < S && issued < my_tiles; ++issued) {
        load(ls, lt);
        if (++ls == S) ls = 0;
        lt += gridDim.x;
      }
      int j = 0, s = 0;
      uint32_t parity = 0;
      int64_t t = first;
      for (; j < my_tiles; ++j) {
        if (!mbar_wait(&sh->done[s], parity, status)) break;
        int x0, o;
        coords(t, x0, o);
        const unsigned char* src = stages + static_cast<size_t>(s) * stage_bytes;
        for (int bx = 0; bx < NX; ++bx)
          for (int b = 0; b < nbox; ++b)
            tma_store_3d(&tm_out, x0 + bx * W, b * NB, o, src + static_cast<size_t>(bx) * xbox_bytes + static_cast<size_t>(b) * box_bytes);
        bulk_commit();
        if (j >= 1 && issued < my_tiles) {  // the store of tile j - 1 has read its stage: the next load goes there
          bulk_wait_read<1>();
          load(ls, lt);
          if (++ls == S) ls = 0;
          lt += gridDim.x;
          ++issued;
        }
        if (++s == S) { s = 0; parity ^= 1u; }
        t += gridDim.x;
      }
      // if a wait gave up, let the loads already issued land before the CTA's shared memory goes away
      for (int k = j; k < issued; ++k) {
        mbar_wait(&sh->full[s], parity, status);
        if (++s == S) { s = 0; parity ^= 1u; }
      }
      bulk_wait_read<0>();
    }
    return;
  }

  // ---------------- consumers ----------------
  ring_consumer_regs();
  const float ninf = acc_neg_inf<float>();
  const int gpb = W / CPT;            // column groups per box
  const int groups = gpb * NX;        // column groups of a tile; groups * segs <= kTmaConsumers (the launcher's doing)
  const bool active = tid < groups * segs;
  const int gidx = tid % groups, sg = tid / groups;
  // where this thread's columns start inside a tensor's tile: box gidx / gpb, then column (gidx % gpb) * CPT of it
  const uint32_t col_off = static_cast<uint32_t>(gidx / gpb) * xbox_bytes + static_cast<uint32_t>(gidx % gpb) * CPT * sizeof(T);
  const uint32_t row_pitch = static_cast<uint32_t>(W) * sizeof(T), seg_pitch = row_pitch * segs;
  const int my_rows = sg < N ? (N - sg + segs - 1) / segs : 0;  // rows sg, sg + segs, ... below N
  int s = 0;
  uint32_t parity = 0;
  for (int k = 0; k < my_tiles; ++k) {
    if (!mbar_wait(&sh->full[s], parity, status)) break;
    unsigned char* t0 = stages + static_cast<size_t>(s) * stage_bytes;
    T* col = reinterpret_cast<T*>(t0 + col_off);
    if constexpr (!BWD && REG) {
      // ---- forward, the thread's share of the line in registers: rows sg, sg + segs, ... ----
      float2 v[kTmaRegRows];
      const uint32_t a0 = smem_u32(t0) + col_off + static_cast<uint32_t>(sg) * row_pitch;
      float2 mx = make_float2(ninf, ninf), sum = make_float2(0.0f, 0.0f);
      if (active) {
#pragma unroll
        for (int r = 0; r < kTmaRegRows; ++r) {
          if (r < my_rows) {
            v[r] = word_to_pair<T>(lds_b32(a0 + r * seg_pitch));
            mx.x = fmaxf(mx.x, v[r].x);
            mx.y = fmaxf(mx.y, v[r].y);
          }
        }
        if (segs > 1) part[tid] = make_float4(mx.x, mx.y, 0.0f, 0.0f);
      }
      if (segs > 1) {  // (segs is the same for every thread)
        named_bar_sync(1, kTmaConsumers);
        if (active)
          for (int q = 0; q < segs; ++q) {
            const float4 pk = part[q * groups + gidx];
            mx.x = fmaxf(mx.x, pk.x);
            mx.y = fmaxf(mx.y, pk.y);
          }
      }
      if (active) {
        // the line's maximum is known: ONE exp per element serves both the sum and the output
        const float base0 = (mx.x == ninf) ? 0.0f : mx.x, base1 = (mx.y == ninf) ? 0.0f : mx.y;  // all -inf: exp(-inf - 0) = 0
#pragma unroll
        for (int r = 0; r < kTmaRegRows; ++r) {
          if (r < my_rows) {
            const float2 e = make_float2(exp_for<T>(v[r].x - base0), CPT == 2 ? exp_for<T>(v[r].y - base1) : 0.0f);
            sum.x += e.x;  // a NaN entry makes the sum NaN (the maximum ignored it); +inf gives exp(inf - inf) = NaN
            sum.y += e.y;
            if (!LOG) v[r] = e;
          }
        }
      }
      if (segs > 1) {
        named_bar_sync(1, kTmaConsumers);  // everyone has read the maxima
        if (active) part[tid] = make_float4(sum.x, sum.y, 0.0f, 0.0f);
        named_bar_sync(1, kTmaConsumers);
        if (active) {
          sum = make_float2(0.0f, 0.0f);
          for (int q = 0; q < segs; ++q) {  // segment order: every thread of the line gets the same bits
            const float4 pk = part[q * groups + gidx];
            sum.x += pk.x;
            sum.y += pk.y;
          }
        }
      }
      if (active) {
        const float2 lg = make_float2(LOG ? logf(sum.x) : 0.0f, LOG ? logf(sum.y) : 0.0f);
        const float2 inv = make_float2(LOG ? 0.0f : 1.0f / sum.x, LOG ? 0.0f : 1.0f / sum.y);
        const bool z0 = safe && mx.x == ninf && !(sum.x != sum.x), z1 = safe && mx.y == ninf && !(sum.y != sum.y);
#pragma unroll
        for (int r = 0; r < kTmaRegRows; ++r) {
          if (r < my_rows) {
            float2 e;
            if constexpr (LOG) e = make_float2((v[r].x - mx.x) - lg.x, (v[r].y - mx.y) - lg.y);  // as the row kernels round it
            else if constexpr (sizeof(T) == 4) e = make_float2(v[r].x / sum.x, 0.0f);
            else e = make_float2(v[r].x * inv.x, v[r].y * inv.y);
            if (z0) e.x = 0.0f;
            if (z1) e.y = 0.0f;
            sts_b32(a0 + r * seg_pitch, pair_to_word<T>(e));
          }
        }
      }
    } else if constexpr (!BWD) {
      OnlineMaxSum<T> a, b;  // b: the second column of a pair (16-bit storage)
      a.init();
      b.init();
      if (active) {
#pragma unroll 4
        for (int j = sg; j < N; j += segs) {
          if constexpr (CPT == 2) {
            const float2 v = ld_pair(col + static_cast<size_t>(j) * W);
            a.m = fmaxf(a.m, v.x);
            b.m = fmaxf(b.m, v.y);
          } else {
            a.m = fmaxf(a.m, to_acc<float>(col[static_cast<size_t>(j) * W]));
          }
        }
        const float base0 = (a.m == ninf) ? 0.0f : a.m, base1 = (b.m == ninf) ? 0.0f : b.m;
#pragma unroll 4
        for (int j = sg; j < N; j += segs) {
          if constexpr (CPT == 2) {
            const float2 v = ld_pair(col + static_cast<size_t>(j) * W);
            a.s += exp_for<T>(v.x - base0);  // a NaN entry makes the sum NaN (the maximum ignored it)
            b.s += exp_for<T>(v.y - base1);
          } else {
            a.s += exp_for<T>(to_acc<float>(col[static_cast<size_t>(j) * W]) - base0);
          }
        }
        part[tid] = make_float4(a.m, a.s, b.m, b.s);
      }
      named_bar_sync(1, kTmaConsumers);
      if (active) {
        const float4 p0 = part[gidx];
        a.m = p0.x; a.s = p0.y; b.m = p0.z; b.s = p0.w;
        for (int q = 1; q < segs; ++q) {  // segment order: every thread of the line gets the same bits
          const float4 pk = part[q * groups + gidx];
          a.merge(pk.x, pk.y);
          if (CPT == 2) b.merge(pk.z, pk.w);
        }
        const float2 mx = make_float2(a.m, b.m), sum = make_float2(a.s, b.s);
        const float2 lg = make_float2(LOG ? logf(sum.x) : 0.0f, LOG ? logf(sum.y) : 0.0f);
        const float2 inv = make_float2(LOG ? 0.0f : 1.0f / sum.x, LOG ? 0.0f : 1.0f / sum.y);
        const bool z0 = safe && mx.x == ninf && !(sum.x != sum.x), z1 = safe && mx.y == ninf && !(sum.y != sum.y);
#pragma unroll 4
        for (int j = sg; j < N; j += segs) {
          if constexpr (CPT == 2) {
            const float2 v = ld_pair(col + static_cast<size_t>(j) * W);
            const float dx0 = v.x - mx.x, dx1 = v.y - mx.y;
            float2 e = LOG ? make_float2(dx0 - lg.x, dx1 - lg.y) : make_float2(exp_for<T>(dx0) * inv.x, exp_for<T>(dx1) * inv.y);
            if (z0) e.x = 0.0f;
            if (z1) e.y = 0.0f;
            st_pair(col + static_cast<size_t>(j) * W, e);
          } else {
            const float d = to_acc<float>(col[static_cast<size_t>(j) * W]) - mx.x;
            const float e = LOG ? d - lg.x : exp_for<T>(d) / sum.x;
            col[static_cast<size_t>(j) * W] = from_acc<T>(z0 ? 0.0f : e);
          }
        }
      }
    } else {
      const T* ycol = reinterpret_cast<const T*>(t0 + tile_bytes + col_off);
      float2 sum = make_float2(0.0f, 0.0f);
      if (active) {
#pragma unroll 4
        for (int j = sg; j < N; j += segs) {
          const size_t l = static_cast<size_t>(j) * W;
          if constexpr (CPT == 2) {
            const float2 d = ld_pair(col + l);
            if constexpr (LOG) {
              sum.x += d.x;
              sum.y += d.y;
            } else {
              const float2 yy = ld_pair(ycol + l);
              sum.x = fmaf(d.x, yy.x, sum.x);
              sum.y = fmaf(d.y, yy.y, sum.y);
            }
          } else {
            const float d = to_acc<float>(col[l]);
            sum.x += LOG ? d : d * to_acc<float>(ycol[l]);
          }
        }
        part[tid] = make_float4(sum.x, sum.y, 0.0f, 0.0f);
      }
      named_bar_sync(1, kTmaConsumers);
      if (active) {
        const float4 p0 = part[gidx];
        sum = make_float2(p0.x, p0.y);
        for (int q = 1; q < segs; ++q) {
          const float4 pk = part[q * groups + gidx];
          sum.x += pk.x;
          sum.y += pk.y;
        }
#pragma unroll 4
        for (int j = sg; j < N; j += segs) {
          const size_t l = static_cast<size_t>(j) * W;
          if constexpr (CPT == 2) {
            const float2 d = ld_pair(col + l), yy = ld_pair(ycol + l);
            const float2 r = LOG ? make_float2(d.x - exp_for<T>(yy.x) * sum.x, d.y - exp_for<T>(yy.y) * sum.y)
                                 : make_float2(yy.x * (d.x - sum.x), yy.y * (d.y - sum.y));
            st_pair(col + l, r);
          } else {
            const float d = to_acc<float>(col[l]), yy = to_acc<float>(ycol[l]);
            col[l] = from_acc<T>(LOG ? d - exp_for<T>(yy) * sum.x : yy * (d - sum.x));
          }
        }
      }
    }
    // the partial results of this tile have been read by everyone before the next tile overwrites them: the
    // barrier at the next tile's hand-over is one full tile of work away, but a thread may race ahead — meet again
    named_bar_sync(1, kTmaConsumers);
    fence_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&sh->done[s]);
    if (++s == S) { s = 0; parity ^= 1u; }
  }
}

}  // namespace b2n
