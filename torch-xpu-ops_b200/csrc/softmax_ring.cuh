// Ring kernels for softmax / log-softmax over the last dim (input and output of the same type).
// A row is shared by GROUP threads, VPT 16-byte vectors each, held in registers: one HBM read and
// one HBM write per element.
#pragma once
#include "ring.cuh"

namespace b2n {

// exp(x - mx) for a row maximum mx.  For 16-bit storage the result is rounded to 8 or 11 bits of
// mantissa anyway, so one FMA plus the hardware 2^x (relative error about 2^-22 plus
// |x - mx| * 2^-24) is enough; fp32 storage uses expf.
template <typename T> struct RowExp {
  float mx, c;
  __device__ __forceinline__ explicit RowExp(float m) : mx(m), c(-m * kLog2e) {}
  __device__ __forceinline__ float operator()(float x) const {
    if constexpr (sizeof(T) == 4) return expf(x - mx);
    else return ex2_approx(fmaf(x, kLog2e, c));
  }
};

// ---- optional mask (aten::_masked_softmax on the ring) ------------------------------------------
// mask: one byte per element, non-zero = masked out; the mask row of input row r is
// (r / row_div) % row_mod (see b2n_masked_softmax_fwd).  A thread fetches the VEC mask bytes of each
// of its vectors with one read-only global load, issued before the row's shared-memory loads so
// that both are in flight together; masks shared by many rows stay in L2.
struct RowMask {
  const unsigned char* base;  // nullptr: no mask
  unsigned row_div, row_mod;
};
template <int VEC> struct MaskWord;
template <> struct MaskWord<8> {
  uint2 w;
  __device__ __forceinline__ void load(const unsigned char* p) { w = __ldg(reinterpret_cast<const uint2*>(p)); }
  __device__ __forceinline__ void clear() { w = make_uint2(0u, 0u); }
  __device__ __forceinline__ bool masked(int e) const { return (((e < 4 ? w.x : w.y) >> (8 * (e & 3))) & 0xffu) != 0u; }
  // the eight mask bytes widened to eight 16-bit fields, all ones where masked: what a 16-byte vector of
  // 16-bit values is combined with directly (three bitwise operations per pair instead of a test per element)
  __device__ __forceinline__ uint4 halfword_masks() const {
    const unsigned a = __vcmpne4(w.x, 0u), b = __vcmpne4(w.y, 0u);  // 0xff per non-zero byte
    return make_uint4(__byte_perm(a, a, 0x1100), __byte_perm(a, a, 0x3322), __byte_perm(b, b, 0x1100),
                      __byte_perm(b, b, 0x3322));
  }
};
// -inf twice in the 16-bit storage types
template <typename T> __device__ __forceinline__ constexpr unsigned neg_inf_pair() { return 0u; }
template <> __device__ __forceinline__ constexpr unsigned neg_inf_pair<bf16>() { return 0xff80ff80u; }
template <> __device__ __forceinline__ constexpr unsigned neg_inf_pair<f16>() { return 0xfc00fc00u; }
__device__ __forceinline__ uint4 mask_to(const uint4& v, const uint4& m, unsigned fill) {  // v where m == 0, fill where m == 1
  return make_uint4((v.x & ~m.x) | (fill & m.x), (v.y & ~m.y) | (fill & m.y), (v.z & ~m.z) | (fill & m.z),
                    (v.w & ~m.w) | (fill & m.w));
}
template <> struct MaskWord<4> {
  unsigned w;
  __device__ __forceinline__ void load(const unsigned char* p) { w = __ldg(reinterpret_cast<const unsigned*>(p)); }
  __device__ __forceinline__ void clear() { w = 0u; }
  __device__ __forceinline__ bool masked(int e) const { return ((w >> (8 * e)) & 0xffu) != 0u; }
};

// MASKED and SAFE (rows of -inf give zeros) are template arguments so that the plain kernels carry none of their
// registers or branches.
// FULL: the row fills every thread's vectors exactly (N == GROUP * VPT * VEC): no range checks.
template <typename T, bool LOG, int GROUP, int VPT, bool MASKED, bool SAFE, bool FULL>
__global__ void __launch_bounds__(kRingBlock, 1)
softmax_fwd_ring_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t M, int N, int S_lag, int RPG,
                        int* status, unsigned* tile_ctr, RowMask mask) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S_lag, 1, tile_ctr);
  ring_init(rs, g.S, kRingThreads / 32);
  const int tid = threadIdx.x;
  if (tid >= kRingThreads) {  // producer warpgroup: one thread moves the tiles, all four warps shed registers
    ring_producer_regs();
    if (tid == kRingThreads) {
      RingProducer<1> prod(rs, stages, g, status);
      prod.in[0] = reinterpret_cast<const unsigned char*>(x);
      prod.out = reinterpret_cast<unsigned char*>(y);
      prod.run();
    }
    return;
  }
  ring_consumer_regs();

  const int grp = tid / GROUP, tg = tid % GROUP;
  const int nvec = FULL ? GROUP * VPT : N / VEC;  // FULL rows have a compile-time length
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  int red_phase = 0;
  const float ninf = acc_neg_inf<float>();
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start();
  for (;; cur.advance(g)) {
    int tile;
    if (!ring_consumer_wait(rs, cur, status, tile) || tile < 0) break;
    const int64_t tile_row0 = g.first_row(tile);
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      if (tile_row0 + lr >= M) break;  // uniform over the group
      const uint32_t rbase = sbase + static_cast<uint32_t>(lr) * row_bytes;
      constexpr int HP = EPT / 2, VH = VEC / 2;  // float2 pairs per thread / per 16-byte vector
      MaskWord<VEC> mw[MASKED ? VPT : 1];
      if constexpr (MASKED) {
        const unsigned row = static_cast<unsigned>(tile_row0 + lr);
        const unsigned char* mr = mask.base + static_cast<size_t>((row / mask.row_div) % mask.row_mod) * N;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (FULL || v < nvec) mw[k].load(mr + v * VEC);
          else mw[k].clear();
        }
      }
      float2 xv[HP];
      float pm[4] = {ninf, ninf, ninf, ninf};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (FULL || v < nvec) {
          if constexpr (MASKED && sizeof(T) == 2) {  // masked elements take no part: -inf, which comes out as exactly 0
            P::unpack2(mask_to(lds128(rbase + v * 16), mw[k].halfword_masks(), neg_inf_pair<T>()), &xv[k * VH]);
          } else {
            P::unpack2(lds128(rbase + v * 16), &xv[k * VH]);
          }
          if constexpr (MASKED && sizeof(T) != 2) {
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              if (mw[k].masked(2 * e)) xv[k * VH + e].x = ninf;
              if (mw[k].masked(2 * e + 1)) xv[k * VH + e].y = ninf;
            }
          }
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            pm[(2 * e) & 3] = fmaxf(pm[(2 * e) & 3], xv[k * VH + e].x);
            pm[(2 * e + 1) & 3] = fmaxf(pm[(2 * e + 1) & 3], xv[k * VH + e].y);
          }
        } else {
#pragma unroll
          for (int e = 0; e < VH; ++e) xv[k * VH + e] = bcast2(ninf);
        }
      }
      float mx[1] = {fmaxf(fmaxf(pm[0], pm[1]), fmaxf(pm[2], pm[3]))};
      group_reduce<GROUP, 1>(mx, rs->red, grp, tg, red_phase, MaxOp());
      // exp(x - max): 16-bit storage uses 2^(x*log2e - max*log2e) (one packed FMA + the hardware
      // 2^x per element); fp32 storage uses expf
      const float2 l2e = bcast2(kLog2e), c2 = bcast2(-mx[0] * kLog2e);
      float2 ps[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        if (FULL || tg + k * GROUP < nvec) {
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            const int j = k * VH + e;
            float2 ex;
            if constexpr (sizeof(T) == 4) {
              ex = make_float2(expf(xv[j].x - mx[0]), expf(xv[j].y - mx[0]));
            } else {
              const float2 t = fma2(xv[j], l2e, c2);
              ex = make_float2(ex2_approx(t.x), ex2_approx(t.y));
            }
            ps[j & 1] = add2(ps[j & 1], ex);
            if (!LOG) xv[j] = ex;
          }
        }
      }
      float sum[1] = {hsum2(add2(ps[0], ps[1]))};
      group_reduce<GROUP, 1>(sum, rs->red, grp, tg, red_phase, SumOp());
      const float lg = LOG ? logf(sum[0]) : 0.0f;
      const float2 noff = bcast2(-(mx[0] + lg));  // 16-bit log-softmax: x - (max + log sum) in one add
      const float2 inv = bcast2(LOG ? 0.0f : 1.0f / sum[0]);
      if (SAFE && mx[0] == ninf) {
        // safe softmax: a row of -inf gives zeros, not NaN — unless the row holds a NaN, which the
        // maximum cannot see; the row is read again to find out (rare; the branch is uniform over
        // the group, so the reduction inside it is legal)
        float has_nan[1] = {0.0f};
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (FULL || v < nvec) {
            float2 f[VH];
            P::unpack2(lds128(rbase + v * 16), f);
#pragma unroll
            for (int e = 0; e < VH; ++e)
              if (f[e].x != f[e].x || f[e].y != f[e].y) has_nan[0] = 1.0f;
          }
        }
        group_reduce<GROUP, 1>(has_nan, rs->red, grp, tg, red_phase, MaxOp());
        if (has_nan[0] == 0.0f) {
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tg + k * GROUP;
            if (FULL || v < nvec) sts128(rbase + v * 16, make_uint4(0u, 0u, 0u, 0u));
          }
          continue;
        }
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (FULL || v < nvec) {
          float2 o[VH];
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            const float2 t = xv[k * VH + e];
            if constexpr (LOG) {
              if constexpr (sizeof(T) == 4) o[e] = make_float2((t.x - mx[0]) - lg, (t.y - mx[0]) - lg);
              else o[e] = add2(t, noff);
            } else if constexpr (sizeof(T) == 4) {
              o[e] = make_float2(t.x / sum[0], t.y / sum[0]);
            } else {
              o[e] = mul2(t, inv);
            }
          }
          sts128(rbase + v * 16, P::pack2(o));
        }
      }
    }
    ring_consumer_release(rs, cur);
  }
}

// stage = [dy tile | y tile]; dx overwrites the dy tile.
// softmax: dx = y*(dy - sum(y*dy)); log-softmax: dx = dy - exp(y)*sum(dy).
template <typename T, bool LOG, int GROUP, int VPT, bool MASKED, bool FULL>
__global__ void __launch_bounds__(kRingBlock, 1)
softmax_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t M,
                        int N, int S_lag, int RPG, int* status, unsigned* tile_ctr, RowMask mask) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S_lag, 2, tile_ctr);
  ring_init(rs, g.S, kRingThreads / 32);
  const int tid = threadIdx.x;
  if (tid >= kRingThreads) {  // producer warpgroup: one thread moves the tiles, all four warps shed registers
    ring_producer_regs();
    if (tid == kRingThreads) {
      RingProducer<2> prod(rs, stages, g, status);
      prod.in[0] = reinterpret_cast<const unsigned char*>(dy);
      prod.in[1] = reinterpret_cast<const unsigned char*>(y);
      prod.out = reinterpret_cast<unsigned char*>(dx);
      prod.run();
    }
    return;
  }
  ring_consumer_regs();

  const int grp = tid / GROUP, tg = tid % GROUP;
  const int nvec = FULL ? GROUP * VPT : N / VEC;  // FULL rows have a compile-time length
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start();
  for (;; cur.advance(g)) {
    int tile;
    if (!ring_consumer_wait(rs, cur, status, tile) || tile < 0) break;
    const int64_t tile_row0 = g.first_row(tile);
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      if (tile_row0 + lr >= M) break;  // uniform over the group
      const uint32_t dbase = sbase + static_cast<uint32_t>(lr) * row_bytes;
      const uint32_t ybase = dbase + g.slot_bytes;
      constexpr int HP = EPT / 2, VH = VEC / 2;  // float2 pairs per thread / per 16-byte vector
      MaskWord<VEC> mw[MASKED ? VPT : 1];
      if constexpr (MASKED) {
        const unsigned row = static_cast<unsigned>(tile_row0 + lr);
        const unsigned char* mr = mask.base + static_cast<size_t>((row / mask.row_div) % mask.row_mod) * N;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (FULL || v < nvec) mw[k].load(mr + v * VEC);
          else mw[k].clear();
        }
      }
      float2 dv[HP], yv[HP];
      float2 ps[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (FULL || v < nvec) {
          if constexpr (MASKED && sizeof(T) == 2) {  // masked elements take no part in the row sum: +0 in both
            const uint4 hm = mw[k].halfword_masks();
            P::unpack2(mask_to(lds128(dbase + v * 16), hm, 0u), &dv[k * VH]);
            P::unpack2(mask_to(lds128(ybase + v * 16), hm, 0u), &yv[k * VH]);
          } else {
            P::unpack2(lds128(dbase + v * 16), &dv[k * VH]);
            P::unpack2(lds128(ybase + v * 16), &yv[k * VH]);
          }
          if constexpr (MASKED && sizeof(T) != 2) {
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              if (mw[k].masked(2 * e)) { dv[k * VH + e].x = 0.0f; yv[k * VH + e].x = 0.0f; }
              if (mw[k].masked(2 * e + 1)) { dv[k * VH + e].y = 0.0f; yv[k * VH + e].y = 0.0f; }
            }
          }
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            const int j = k * VH + e;
            if constexpr (LOG) ps[j & 1] = add2(ps[j & 1], dv[j]);
            else ps[j & 1] = fma2(dv[j], yv[j], ps[j & 1]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < VH; ++e) { dv[k * VH + e] = bcast2(0.0f); yv[k * VH + e] = bcast2(0.0f); }
        }
      }
      float sum[1] = {hsum2(add2(ps[0], ps[1]))};
      group_reduce<GROUP, 1>(sum, rs->red, grp, tg, red_phase, SumOp());
      const float2 ns = bcast2(-sum[0]), l2e = bcast2(kLog2e);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (FULL || v < nvec) {
          float2 o[VH];
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            const float2 d = dv[k * VH + e], yy = yv[k * VH + e];
            if constexpr (LOG) {
              float2 ey;
              if constexpr (sizeof(T) == 4) {
                ey = make_float2(expf(yy.x), expf(yy.y));
              } else {
                const float2 t = mul2(yy, l2e);
                ey = make_float2(ex2_approx(t.x), ex2_approx(t.y));
              }
              o[e] = fma2(ey, ns, d);   // dy - exp(y)*sum
            } else {
              o[e] = mul2(yy, add2(d, ns));  // y*(dy - sum)
            }
          }
          if constexpr (MASKED && sizeof(T) == 2) {  // exactly zero where masked, whatever the row sum is
            sts128(dbase + v * 16, mask_to(P::pack2(o), mw[k].halfword_masks(), 0u));
          } else {
            if constexpr (MASKED) {
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                if (mw[k].masked(2 * e)) o[e].x = 0.0f;
                if (mw[k].masked(2 * e + 1)) o[e].y = 0.0f;
              }
            }
            sts128(dbase + v * 16, P::pack2(o));
          }
        }
      }
    }
    ring_consumer_release(rs, cur);
  }
}

}  // namespace b2n
