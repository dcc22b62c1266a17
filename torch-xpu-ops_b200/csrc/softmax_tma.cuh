// Softmax / log-softmax over a dim that is NOT the last, on tensor-map TMA tiles.
//
// The tensor is [outer, N, inner]; a line runs over N with stride `inner`.  A tile is all N line elements
// x W adjacent inner positions: N runs of W elements, `inner` elements apart.  That is exactly what a
// tiled bulk-tensor copy moves with ONE instruction: the tensor is described to the TMA unit as a
// rank-3 tensor (inner, N, outer), a tile is a box of W x NB x 1 elements (NB = N, or equal boxes of at most 256 rows
// for longer lines), and `cp.async.bulk.tensor.3d` brings the box into shared memory — densely packed,
// row pitch W — while completing a transaction count on an mbarrier; the mirror instruction sends the
// result back.  Coordinates past the tensor's edge are filled with zeros on the way in and dropped on
// the way out, so edge tiles need no special case.  Every box starts at x = k * W with W * sizeof(T) a
// whole number of 128-byte lines: the copy's start is then 16-byte aligned in global memory, as it must be, and
// every box lands on a 128-byte boundary of shared memory, whatever N is.
//
// A tile is NX boxes wide (W <= 256 elements each) so that short lines still make tiles of tens of KB, and a
// line is shared by `segs` threads.  In the forward, when a thread's share of a line is at most 32 elements
// (lines up to 512 long), the thread keeps it in REGISTERS: one shared-memory read and ONE exp per element
// (exp(x - max) serves the sum and the output) — with two exps per element the kernel is bound by the
// special-function unit, not by HBM.
//
// Persistent CTAs, one per SM: a producer thread keeps S tiles in flight (loads of the next tiles and
// the store of the previous one overlap the arithmetic; a stage is refilled as soon as its store has READ it);
// 512 consumer threads work on the tile in shared memory — a line shared by `segs` threads, each taking every
// segs-th element, consecutive threads on consecutive addresses, partial results combined in segment order —
// and leave the result in place.  The threads that share lines (32 adjacent column groups x segs warps) form a
// team with a named barrier of its own; the teams never meet, so their phases overlap.  Every element crosses
// HBM once each way.  No cluster multicast; every wait bounded.
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
  float4* part = reinterpret_cast<float4*>(smem_raw + 1024);  // one slot per consumer thread ...
  float2* part2 = reinterpret_cast<float2*>(part);            // ... as two halves
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
      int issued = 0;
      int64_t lt = first;
      for (; issued < S && issued < my_tiles; ++issued) {
        load(issued, lt);
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
        if (issued < my_tiles) {
          // The stage is free again as soon as the store has READ it (well before it has reached memory), and this
          // thread has nothing else to do until the consumers finish the next tile: wait for that and refill the
          // stage at once, so that S - 1 tiles are loaded or on their way while one is worked on.
          bulk_wait_read<0>();
          load(s, lt);
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
  // The threads that share lines — 32 adjacent column groups x segs segments: segs whole warps — are a TEAM with a
  // named barrier of its own.  Nothing ever makes all consumers meet, so the teams drift apart and one team's
  // exp phase (special-function unit) overlaps another's load or store phase (shared-memory pipe), also across tiles.
  const int team_bar = 1 + (gidx >> 5), team_threads = 32 * segs;  // groups is a multiple of 32; at most 8 teams when segs > 1
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
      // Rows go in blocks of four: a block past the thread's share is skipped by a branch the whole warp takes
      // (predicated-off instructions would still take issue slots); 16-bit storage uses packed f32x2 arithmetic.
      float2 v[kTmaRegRows];
      const uint32_t a0 = smem_u32(t0) + col_off + static_cast<uint32_t>(sg) * row_pitch;
      float2 mx = make_float2(ninf, ninf), sum = make_float2(0.0f, 0.0f);
      if (active) {
#pragma unroll
        for (int b4 = 0; b4 < kTmaRegRows; b4 += 4) {
          if (b4 < my_rows) {
#pragma unroll
            for (int r = b4; r < b4 + 4; ++r) {
              if (r < my_rows) {
                v[r] = word_to_pair<T>(lds_b32(a0 + r * seg_pitch));
                mx.x = fmaxf(mx.x, v[r].x);
                mx.y = fmaxf(mx.y, v[r].y);
              }
            }
          }
        }
      }
      // Two barriers per tile, both the team's own.  A thread's slot holds its maxima in one half and its sums in
      // the other: the maxima of the next tile are written after this tile's second barrier, which every team
      // member reaches after reading this tile's maxima, and the sums after the next tile's first barrier.
      if (active && segs > 1) {  // (whole warps are active or not)
        part2[2 * tid] = mx;
        named_bar_sync(team_bar, team_threads);
        for (int q = 0; q < segs; ++q) {
          const float2 pk = part2[2 * (q * groups + gidx)];
          mx.x = fmaxf(mx.x, pk.x);
          mx.y = fmaxf(mx.y, pk.y);
        }
      }
      if (active) {
        // the line's maximum is known: ONE exp per element serves both the sum and the output
        const float base0 = (mx.x == ninf) ? 0.0f : mx.x, base1 = (mx.y == ninf) ? 0.0f : mx.y;  // all -inf: exp(-inf - 0) = 0
        const float2 nbase = make_float2(-base0, -base1), l2e = make_float2(kLog2e, kLog2e);
#pragma unroll
        for (int b4 = 0; b4 < kTmaRegRows; b4 += 4) {
          if (b4 < my_rows) {
#pragma unroll
            for (int r = b4; r < b4 + 4; ++r) {
              if (r < my_rows) {
                // a NaN entry makes the sum NaN (the maximum ignored it); +inf gives exp(inf - inf) = NaN
                float2 e;
                if constexpr (CPT == 2) {
                  const float2 t = mul2(add2(v[r], nbase), l2e);  // exp_for<T> on both columns ...
                  e = make_float2(ex2_approx(t.x), ex2_approx(t.y));
                  sum = add2(sum, e);
                } else {
                  e = make_float2(exp_for<T>(v[r].x - base0), 0.0f);
                  sum.x += e.x;
                }
                if (!LOG) v[r] = e;
              }
            }
          }
        }
      }
      if (active && segs > 1) {
        part2[2 * tid + 1] = sum;
        named_bar_sync(team_bar, team_threads);
        sum = make_float2(0.0f, 0.0f);
        for (int q = 0; q < segs; ++q) {  // segment order: every thread of the line gets the same bits
          const float2 pk = part2[2 * (q * groups + gidx) + 1];
          sum.x += pk.x;
          sum.y += pk.y;
        }
      }
      if (active) {
        const float2 nlg = make_float2(LOG ? -logf(sum.x) : 0.0f, LOG ? -logf(sum.y) : 0.0f), nmx = make_float2(-mx.x, -mx.y);
        // safe softmax: a line of -inf (and no NaN) gives zeros — exp(x - max) is 0 there, so a factor of 0 does it
        const bool z0 = !LOG && safe && mx.x == ninf && !(sum.x != sum.x), z1 = !LOG && safe && mx.y == ninf && !(sum.y != sum.y);
        const float2 inv = make_float2(LOG || z0 ? 0.0f : 1.0f / sum.x, LOG || z1 ? 0.0f : 1.0f / sum.y);
#pragma unroll
        for (int b4 = 0; b4 < kTmaRegRows; b4 += 4) {
          if (b4 < my_rows) {
#pragma unroll
            for (int r = b4; r < b4 + 4; ++r) {
              if (r < my_rows) {
                float2 e;
                if constexpr (LOG) e = add2(add2(v[r], nmx), nlg);  // (x - max) - log(sum), as the row kernels round it
                else if constexpr (sizeof(T) == 4) e = make_float2(z0 ? 0.0f : v[r].x / sum.x, 0.0f);
                else e = mul2(v[r], inv);
                sts_b32(a0 + r * seg_pitch, pair_to_word<T>(e));
              }
            }
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
      if constexpr (!BWD && !REG) {
      if (active && segs > 1) named_bar_sync(team_bar, team_threads);
    }
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
      // rows sg, sg + segs, ... of the thread's column pair, dy at a0 and y one tile further
      const uint32_t a0 = smem_u32(t0) + col_off + static_cast<uint32_t>(sg) * row_pitch, y0 = a0 + tile_bytes;
      float2 sum = make_float2(0.0f, 0.0f);
      if (active) {
        uint32_t o = 0;
#pragma unroll 4
        for (int r = 0; r < my_rows; ++r, o += seg_pitch) {
          const float2 d = word_to_pair<T>(lds_b32(a0 + o));
          if constexpr (LOG) {
            sum.x += d.x;
            sum.y += d.y;
          } else {
            const float2 yy = word_to_pair<T>(lds_b32(y0 + o));
            if constexpr (CPT == 2) {
              sum = fma2(d, yy, sum);
            } else {
              sum.x = fmaf(d.x, yy.x, sum.x);
            }
          }
        }
      }
      // One barrier per tile, the team's own: the halves of a thread's slot alternate from tile to tile, and a half
      // is written again only after the barrier of the tile in between, which every team member reaches after it
      // has read that half.
      if (active && segs > 1) {  // (whole warps are active or not)
        part2[2 * tid + (k & 1)] = sum;
        named_bar_sync(team_bar, team_threads);
        sum = make_float2(0.0f, 0.0f);
        for (int q = 0; q < segs; ++q) {  // segment order: every thread of the line gets the same bits
          const float2 pk = part2[2 * (q * groups + gidx) + (k & 1)];
          sum.x += pk.x;
          sum.y += pk.y;
        }
      }
      if (active) {
        const float2 nsum = make_float2(-sum.x, -sum.y);
        uint32_t o = 0;
#pragma unroll 4
        for (int r = 0; r < my_rows; ++r, o += seg_pitch) {
          const float2 d = word_to_pair<T>(lds_b32(a0 + o)), yy = word_to_pair<T>(lds_b32(y0 + o));
          const float2 res = LOG ? make_float2(d.x - exp_for<T>(yy.x) * sum.x, d.y - exp_for<T>(yy.y) * sum.y)
                                 : mul2(yy, add2(d, nsum));  // y * (dy - sum)
          sts_b32(a0 + o, pair_to_word<T>(res));
        }
      }
    }
    // (the three-walk forward keeps all four partial results in one slot: its team meets once more before the next
    // tile overwrites them)
    if constexpr (!BWD && !REG) {
      if (active && segs > 1) named_bar_sync(team_bar, team_threads);
    }
    fence_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&sh->done[s]);
    if (++s == S) { s = 0; parity ^= 1u; }
  }
}

}  // namespace b2n
