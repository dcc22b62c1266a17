// GroupNorm forward on the shared-memory ring: the layer-norm forward ring kernel (norm_ring.cuh) with a
// per-CHANNEL affine map.  A row of the [N * G, D * HxW] view is a layer-norm row; what differs is that the
// weights of a thread's columns depend on the row's group — element j of row (n, g) takes gamma[g * D + j / HxW] —
// so they are fetched per row (two or four scalars per thread, L1-resident, issued before the statistics pass and
// used after it) instead of living in registers for the whole launch.  Taken when a row fits the ring
// (D * HxW <= 8192 elements, a whole number of 16-byte vectors none of which straddles two channels).
#pragma once
#include "ring.cuh"

namespace b2n {

// FULL: a row fills every thread's vectors exactly (N == GROUP * VPT * VEC): no column range checks, row length and
// byte offsets compile-time — as in the layer-norm ring kernels.
template <typename T, typename WT, typename ST, int GROUP, int VPT, bool FULL>
__global__ void __launch_bounds__(kRingBlock, 1)
group_norm_fwd_ring_kernel(const T* __restrict__ x, const WT* __restrict__ gamma, const WT* __restrict__ beta, T* __restrict__ y,
                           ST* __restrict__ mean, ST* __restrict__ rstd, int64_t M, int N, int G, int D, int HxW, float eps,
                           int S_lag, int RPG, int* status, unsigned* tile_ctr) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  constexpr int RB = 2;  // rows a group works on at once
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S_lag, 1, tile_ctr);
  ring_init(rs, g.S, kRingThreads / 32);
  const int tid = threadIdx.x;
  if (tid >= kRingThreads) {
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
  const int nvec = FULL ? GROUP * VPT : N / VEC;
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  const float inv_n = 1.0f / static_cast<float>(N);
  constexpr int HP = EPT / 2, VH = VEC / 2;
  int chan[VPT];  // channel, within the group, of each of this thread's vectors
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tg + k * GROUP;
    chan[k] = (FULL || v < nvec) ? (v * VEC) / HxW : 0;
  }
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start();
  for (;; cur.advance(g)) {
    int i;
    if (!ring_consumer_wait(rs, cur, status, i) || i < 0) break;
    const int64_t tile_row0 = g.first_row(i);
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; r += RB) {
      const int lr0 = grp * RPG + r;
      const int64_t row_a = tile_row0 + lr0;
      if (row_a >= M) break;  // uniform over the group
      bool valid[RB];
      uint32_t rbase[RB];
      float shift[RB];
      float2 xv[RB][HP];
      float gam[RB][VPT], bet[RB][VPT];
      float red1[RB * 2];
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        valid[b] = (r + b < RPG) && (row_a + b < M);
        rbase[b] = sbase + static_cast<uint32_t>(lr0 + b) * row_bytes;
        // (the launcher takes this kernel only for fewer than 2^31 rows: a 32-bit remainder)
        const int c0 = valid[b] ? static_cast<int>(static_cast<unsigned>(row_a + b) % static_cast<unsigned>(G)) * D : 0;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          gam[b][k] = (gamma != nullptr && valid[b]) ? to_acc<float>(gamma[c0 + chan[k]]) : 1.0f;
          bet[b][k] = (beta != nullptr && valid[b]) ? to_acc<float>(beta[c0 + chan[k]]) : 0.0f;
        }
        shift[b] = 0.0f;
        if (valid[b]) {
          float2 first[VH];
          P::unpack2(lds128(rbase[b]), first);
          shift[b] = first[0].x;
        }
        const float2 nshift = bcast2(-shift[b]);
        float2 ps[2] = {bcast2(0.0f), bcast2(0.0f)}, pq[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (valid[b] && (FULL || v < nvec)) {
            P::unpack2(lds128(rbase[b] + v * 16), &xv[b][k * VH]);
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              const int j = k * VH + e;
              xv[b][j] = add2(xv[b][j], nshift);
              ps[j & 1] = add2(ps[j & 1], xv[b][j]);
              pq[j & 1] = fma2(xv[b][j], xv[b][j], pq[j & 1]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < VH; ++e) xv[b][k * VH + e] = bcast2(0.0f);
          }
        }
        red1[2 * b] = hsum2(add2(ps[0], ps[1]));
        red1[2 * b + 1] = hsum2(add2(pq[0], pq[1]));
      }
      group_reduce<GROUP, RB * 2>(red1, rs->red, grp, tg, red_phase, SumOp());
      float mu_d[RB], rsd[RB], var[RB];
      bool exact = true;
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        mu_d[b] = red1[2 * b] * inv_n;
        const float m2 = mu_d[b] * mu_d[b];
        var[b] = fmaf(red1[2 * b + 1], inv_n, -m2);
        exact = exact && (m2 <= 8.0f * var[b]);
      }
      if (!exact) {  // the shift lay far from the mean (or NaN): once more about the mean just found
        float red2[2 * RB];
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          shift[b] += mu_d[b];
          const float2 nshift = bcast2(-shift[b]);
          float2 q[2] = {bcast2(0.0f), bcast2(0.0f)}, c[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tg + k * GROUP;
            if (valid[b] && (FULL || v < nvec)) {
              P::unpack2(lds128(rbase[b] + v * 16), &xv[b][k * VH]);
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                const int j = k * VH + e;
                xv[b][j] = add2(xv[b][j], nshift);
                c[j & 1] = add2(c[j & 1], xv[b][j]);
                q[j & 1] = fma2(xv[b][j], xv[b][j], q[j & 1]);
              }
            }
          }
          red2[2 * b] = hsum2(add2(c[0], c[1]));
          red2[2 * b + 1] = hsum2(add2(q[0], q[1]));
        }
        group_reduce<GROUP, 2 * RB>(red2, rs->red, grp, tg, red_phase, SumOp());
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          mu_d[b] = red2[2 * b] * inv_n;
          const float vq = fmaf(-mu_d[b], red2[2 * b], red2[2 * b + 1]) * inv_n;
          var[b] = vq < 0.0f ? 0.0f : vq;
        }
      }
#pragma unroll
      for (int b = 0; b < RB; ++b) rsd[b] = rsqrt_nr(var[b] + eps);
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        if (!valid[b]) continue;
        const float2 rs2 = bcast2(rsd[b]);
        const float2 c2 = bcast2(-mu_d[b] * rsd[b]);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (FULL || v < nvec) {
            const float2 gm = bcast2(gam[b][k]), bt = bcast2(bet[b][k]);
            float2 o[VH];
#pragma unroll
            for (int e = 0; e < VH; ++e) o[e] = fma2(fma2(xv[b][k * VH + e], rs2, c2), gm, bt);
            sts128(rbase[b] + v * 16, P::pack2(o));
          }
        }
        if (tg == 0) {
          mean[row_a + b] = from_acc<ST>(shift[b] + mu_d[b]);
          rstd[row_a + b] = from_acc<ST>(rsd[b]);
        }
      }
    }
    ring_consumer_release(rs, cur);
  }
}

// GroupNorm backward, dX only, on the same ring with two input tiles per stage (dy, which dX overwrites, and x):
//   g = dy * gamma[channel],  xhat = (x - mean) * rstd,  dx = rstd * (g - (xhat * sum(g * xhat) + sum(g)) / L)
// per row of the [N * G, L] view, from the forward's saved statistics.  A thread keeps g and xhat of its columns in
// registers between the two row sums and the output; gamma is fetched per row as in the forward.
template <typename T, typename WT, typename ST, int GROUP, int VPT, bool FULL>
__global__ void __launch_bounds__(kRingBlock, 1)
group_norm_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x, const ST* __restrict__ mean,
                           const ST* __restrict__ rstd, const WT* __restrict__ gamma, T* __restrict__ dx, int64_t M, int N, int G,
                           int D, int HxW, int S_lag, int RPG, int* status, unsigned* tile_ctr) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  constexpr int RB = 2;  // rows a group works on at once
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S_lag, 2, tile_ctr);
  ring_init(rs, g.S, kRingThreads / 32);
  const int tid = threadIdx.x;
  if (tid >= kRingThreads) {
    ring_producer_regs();
    if (tid == kRingThreads) {
      RingProducer<2> prod(rs, stages, g, status);
      prod.in[0] = reinterpret_cast<const unsigned char*>(dy);
      prod.in[1] = reinterpret_cast<const unsigned char*>(x);
      prod.out = reinterpret_cast<unsigned char*>(dx);
      prod.run();
    }
    return;
  }
  ring_consumer_regs();

  const int grp = tid / GROUP, tg = tid % GROUP;
  const int nvec = FULL ? GROUP * VPT : N / VEC;
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  const float inv_n = 1.0f / static_cast<float>(N);
  constexpr int HP = EPT / 2, VH = VEC / 2;
  int chan[VPT];  // channel, within the group, of each of this thread's vectors
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tg + k * GROUP;
    chan[k] = (FULL || v < nvec) ? (v * VEC) / HxW : 0;
  }
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start();
  for (;; cur.advance(g)) {
    int i;
    if (!ring_consumer_wait(rs, cur, status, i) || i < 0) break;
    const int64_t tile_row0 = g.first_row(i);
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; r += RB) {
      const int lr0 = grp * RPG + r;
      const int64_t row_a = tile_row0 + lr0;
      if (row_a >= M) break;  // uniform over the group
      bool valid[RB];
      uint32_t dbase[RB];
      float mu[RB], rsd[RB];
      float2 gv[RB][HP], xh[RB][HP];
      float red[RB * 2];
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        valid[b] = (r + b < RPG) && (row_a + b < M);
        dbase[b] = sbase + static_cast<uint32_t>(lr0 + b) * row_bytes;
        mu[b] = valid[b] ? to_acc<float>(mean[row_a + b]) : 0.0f;
        rsd[b] = valid[b] ? to_acc<float>(rstd[row_a + b]) : 0.0f;
        // (the launcher takes this kernel only for fewer than 2^31 rows: a 32-bit remainder)
        const int c0 = valid[b] ? static_cast<int>(static_cast<unsigned>(row_a + b) % static_cast<unsigned>(G)) * D : 0;
        float gam[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) gam[k] = (gamma != nullptr && valid[b]) ? to_acc<float>(gamma[c0 + chan[k]]) : 1.0f;
        const float2 nmu = bcast2(-mu[b]), rs2 = bcast2(rsd[b]);
        float2 p1[2] = {bcast2(0.0f), bcast2(0.0f)}, p2[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (valid[b] && (FULL || v < nvec)) {
            P::unpack2(lds128(dbase[b] + v * 16), &gv[b][k * VH]);
            P::unpack2(lds128(dbase[b] + g.slot_bytes + v * 16), &xh[b][k * VH]);
            const float2 gm = bcast2(gam[k]);
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              const int j = k * VH + e;
              gv[b][j] = mul2(gv[b][j], gm);
              xh[b][j] = mul2(add2(xh[b][j], nmu), rs2);
              p1[j & 1] = add2(p1[j & 1], gv[b][j]);
              p2[j & 1] = fma2(gv[b][j], xh[b][j], p2[j & 1]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              gv[b][k * VH + e] = bcast2(0.0f);
              xh[b][k * VH + e] = bcast2(0.0f);
            }
          }
        }
        red[2 * b] = hsum2(add2(p1[0], p1[1]));
        red[2 * b + 1] = hsum2(add2(p2[0], p2[1]));
      }
      group_reduce<GROUP, RB * 2>(red, rs->red, grp, tg, red_phase, SumOp());
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        if (!valid[b]) continue;
        const float2 rs2 = bcast2(rsd[b]);
        const float2 nar = bcast2(-(red[2 * b + 1] * inv_n * rsd[b])), nbr = bcast2(-(red[2 * b] * inv_n * rsd[b]));
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (FULL || v < nvec) {
            float2 o[VH];
#pragma unroll
            for (int e = 0; e < VH; ++e) o[e] = fma2(gv[b][k * VH + e], rs2, fma2(xh[b][k * VH + e], nar, nbr));
            sts128(dbase[b] + v * 16, P::pack2(o));
          }
        }
      }
    }
    ring_consumer_release(rs, cur);
  }
}

}  // namespace b2n
