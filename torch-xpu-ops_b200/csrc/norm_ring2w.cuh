// Layer norm / RMS norm forward for rows of 8192 < N <= 16384 elements on the shared-memory ring, one CTA per row.
//
// The ring kernels of norm_ring.cuh keep a thread's 16 elements of a row in registers between the moments and the
// output; twice that does not fit beside gamma and beta.  Here the WEIGHTS stay in registers (32 columns per thread:
// fp32 gamma / beta of 16384 columns are 128 KB, four times the bf16 row itself — fetching them per row would move
// more bytes through L2 than the data) and the row is walked twice in shared memory: once for the shifted moments,
// once for the output.  No cluster, no exchange: a row never leaves its CTA.  Everything else — persistent CTAs,
// bulk-async tiles on mbarriers, dynamic tile hand-out, two rows per reduction round, the exact second pass when the
// shift lies far from the mean — is the ring kernel's.  Rows longer than 16384 elements take the slab kernels
// (norm_slab.cuh), which split a row over a cluster.
#pragma once
#include "norm_ring.cuh"

namespace b2n {

constexpr int kNorm2wEpt = 32;  // elements of a row per thread

template <typename T, typename WT, bool RMS, bool FULL>
__global__ void __launch_bounds__(kRingBlock, 1)
norm_fwd_ring2w_kernel(const T* __restrict__ x, const WT* __restrict__ gamma, const WT* __restrict__ beta, T* __restrict__ y,
                       float* __restrict__ mean, float* __restrict__ rstd, int64_t M, int N, float eps, int S_lag, int RPG,
                       int* status, unsigned* tile_ctr) {
  using P = Pack16<T>;
  constexpr int GROUP = kRingThreads;  // the whole CTA on a row
  constexpr int VEC = P::VEC, VPT = kNorm2wEpt / VEC, HP = kNorm2wEpt / 2, VH = VEC / 2;
  constexpr int RB = 2;  // rows per reduction round
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), RPG, S_lag, 1, tile_ctr);
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

  const int nvec = FULL ? GROUP * VPT : N / VEC;
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  const float inv_n = 1.0f / static_cast<float>(N);
  float2 gw[HP], gb[HP];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tid + k * GROUP;
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      const bool ok = FULL || v < nvec;
      const int col = v * VEC + e;
      gw[(k * VEC + e) / 2] = (ok && gamma != nullptr) ? make_float2(to_acc<float>(gamma[col]), to_acc<float>(gamma[col + 1]))
                                                       : bcast2(1.0f);
      if constexpr (!RMS)
        gb[(k * VEC + e) / 2] = (ok && beta != nullptr) ? make_float2(to_acc<float>(beta[col]), to_acc<float>(beta[col + 1]))
                                                        : bcast2(0.0f);
    }
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
      const int64_t row_a = tile_row0 + r;
      if (row_a >= M) break;  // uniform over the CTA
      bool valid[RB];
      uint32_t rbase[RB];
      float shift[RB], mu_d[RB], var[RB], rsd[RB];
      // ---- walk 1: sums of d = x - shift and of d^2 (shift: the row's first element; RMS: zero) ----
      auto moments = [&](float (&red)[RB * 2]) {
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          const float2 nshift = bcast2(-shift[b]);
          float2 ps[2] = {bcast2(0.0f), bcast2(0.0f)}, pq[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            const int v = tid + k * GROUP;
            if (valid[b] && (FULL || v < nvec)) {
              float2 xv[VH];
              P::unpack2(lds128(rbase[b] + v * 16), xv);
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
          red[2 * b] = hsum2(add2(ps[0], ps[1]));
          red[2 * b + 1] = hsum2(add2(pq[0], pq[1]));
        }
        group_reduce<GROUP, RB * 2>(red, rs->red, 0, tid, red_phase, SumOp());
      };
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        valid[b] = (r + b < RPG) && (row_a + b < M);
        rbase[b] = sbase + static_cast<uint32_t>(r + b) * row_bytes;
        shift[b] = 0.0f;
        if (!RMS && valid[b]) {
          float2 first[VH];
          P::unpack2(lds128(rbase[b]), first);  // the same address for every thread: a broadcast
          shift[b] = first[0].x;
        }
      }
      float red1[RB * 2];
      moments(red1);
      if constexpr (RMS) {
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          mu_d[b] = 0.0f;
          var[b] = red1[2 * b + 1] * inv_n;
        }
      } else {
        bool exact = true;
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          mu_d[b] = red1[2 * b] * inv_n;
          const float m2 = mu_d[b] * mu_d[b];
          var[b] = fmaf(red1[2 * b + 1], inv_n, -m2);
          exact = exact && (!valid[b] || m2 <= 8.0f * var[b]);
        }
        if (!exact) {  // the shift lay far from the mean (or NaN): once more about the mean just found
#pragma unroll
          for (int b = 0; b < RB; ++b) shift[b] += mu_d[b];
          float red2[RB * 2];
          moments(red2);
#pragma unroll
          for (int b = 0; b < RB; ++b) {
            mu_d[b] = red2[2 * b] * inv_n;
            const float vq = fmaf(-mu_d[b], red2[2 * b], red2[2 * b + 1]) * inv_n;
            var[b] = vq < 0.0f ? 0.0f : vq;  // keeps NaN
          }
        }
      }
#pragma unroll
      for (int b = 0; b < RB; ++b) rsd[b] = rsqrt_nr(var[b] + eps);
      // ---- walk 2: y = ((d - mu_d) * rstd) * gamma + beta as two FMAs on d = x - shift ----
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        if (!valid[b]) continue;
        const float2 nshift = bcast2(-shift[b]), rs2 = bcast2(rsd[b]), c2 = bcast2(-mu_d[b] * rsd[b]);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * GROUP;
          if (FULL || v < nvec) {
            float2 xv[VH], o[VH];
            P::unpack2(lds128(rbase[b] + v * 16), xv);
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              const int j = k * VH + e;
              if constexpr (RMS) o[e] = mul2(mul2(xv[e], rs2), gw[j]);
              else o[e] = fma2(fma2(add2(xv[e], nshift), rs2, c2), gw[j], gb[j]);
            }
            sts128(rbase[b] + v * 16, P::pack2(o));
          }
        }
        if (tid == 0) {
          if (!RMS && mean) mean[row_a + b] = shift[b] + mu_d[b];
          if (rstd) rstd[row_a + b] = rsd[b];
        }
      }
    }
    ring_consumer_release(rs, cur);
  }
}

// RMS norm backward for the same rows, one CTA per row, stage = [dy row | x row], dx overwrites dy:
//   g = dy * gamma,  xhat = x * rstd,  s2 = sum(g * xhat),  dx = rstd * (g - xhat * s2 / N),  dgamma += dy * xhat.
// gamma and the dgamma accumulators of the thread's 32 columns live in registers (64 of them) — which is why this
// exists for RMS norm only: layer norm adds 32 dbeta accumulators, and 96 registers of persistent state do not fit
// (its rows of this length stay with the slab kernels).  The row is walked twice in shared memory: for s2, then
// for dx and dgamma.  Tiles are assigned to CTAs in the fixed pattern (no counter), so a CTA's partial weight
// gradient — row blockIdx.x of ws[P][2][N] — is the same bits on every run; rstd of the next tile's rows is
// fetched a tile ahead.
template <typename T, typename WT, bool WGRAD, bool FULL>
__global__ void __launch_bounds__(kRingBlock, 1)
rms_norm_bwd_ring2w_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ rstd,
                           const WT* __restrict__ gamma, T* __restrict__ dx, float* __restrict__ ws, int64_t M, int N,
                           int S_lag, int RPG, int* status) {
  using P = Pack16<T>;
  constexpr int GROUP = kRingThreads;
  constexpr int VEC = P::VEC, VPT = kNorm2wEpt / VEC, HP = kNorm2wEpt / 2, VH = VEC / 2;
  constexpr int RB = 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), RPG, S_lag, 2, nullptr);  // no tile counter: the fixed assignment
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

  const int nvec = FULL ? GROUP * VPT : N / VEC;
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  const float inv_n = 1.0f / static_cast<float>(N);
  float2 gw[HP], dg[HP];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tid + k * GROUP;
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      const bool ok = (FULL || v < nvec) && gamma != nullptr;
      const int col = v * VEC + e;
      gw[(k * VEC + e) / 2] = ok ? make_float2(to_acc<float>(gamma[col]), to_acc<float>(gamma[col + 1])) : bcast2(1.0f);
      dg[(k * VEC + e) / 2] = bcast2(0.0f);
    }
  }
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);
  auto load_rstd = [&](unsigned tile, float (&out)[RB]) {
#pragma unroll
    for (int b = 0; b < RB; ++b) {
      const int64_t row = tile < g.ntiles ? g.first_row(static_cast<int>(tile)) + b : M;
      out[b] = (b < RPG && row < M) ? __ldg(rstd + row) : 0.0f;
    }
  };
  float rs_c[RB], rs_n[RB];
  load_rstd(blockIdx.x, rs_c);

  RingCursor cur;
  cur.start();
  unsigned k_tile = 0;
  for (;; cur.advance(g), ++k_tile) {
    load_rstd(blockIdx.x + (k_tile + 1) * gridDim.x, rs_n);  // the next tile's, used a whole tile from now
    int i;
    if (!ring_consumer_wait(rs, cur, status, i) || i < 0) break;
    const int64_t tile_row0 = g.first_row(i);
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; r += RB) {
      const int64_t row_a = tile_row0 + r;
      if (row_a >= M) break;  // uniform over the CTA
      bool valid[RB];
      uint32_t dbase[RB];
      float rsd[RB];
      float red[RB];
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        valid[b] = (r + b < RPG) && (row_a + b < M);
        dbase[b] = sbase + static_cast<uint32_t>(r + b) * row_bytes;
        rsd[b] = r == 0 ? rs_c[b] : (valid[b] ? __ldg(rstd + row_a + b) : 0.0f);  // (tiles of more than two rows: in place)
        // ---- walk 1: s2 = sum (dy * gamma) * (x * rstd) ----
        const float2 rs2 = bcast2(rsd[b]);
        float2 p2[2] = {bcast2(0.0f), bcast2(0.0f)};
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * GROUP;
          if (valid[b] && (FULL || v < nvec)) {
            float2 dv[VH], xv[VH];
            P::unpack2(lds128(dbase[b] + v * 16), dv);
            P::unpack2(lds128(dbase[b] + g.slot_bytes + v * 16), xv);
#pragma unroll
            for (int e = 0; e < VH; ++e) p2[e & 1] = fma2(mul2(dv[e], gw[k * VH + e]), mul2(xv[e], rs2), p2[e & 1]);
          }
        }
        red[b] = hsum2(add2(p2[0], p2[1]));
      }
      group_reduce<GROUP, RB>(red, rs->red, 0, tid, red_phase, SumOp());
      // ---- walk 2: dx = rstd * g - xhat * (s2 / N) * rstd, dgamma += dy * xhat ----
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        if (!valid[b]) continue;
        const float2 rs2 = bcast2(rsd[b]), nar = bcast2(-(red[b] * inv_n * rsd[b]));
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * GROUP;
          if (FULL || v < nvec) {
            float2 dv[VH], xv[VH], o[VH];
            P::unpack2(lds128(dbase[b] + v * 16), dv);
            P::unpack2(lds128(dbase[b] + g.slot_bytes + v * 16), xv);
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              const int j = k * VH + e;
              const float2 xh = mul2(xv[e], rs2);
              o[e] = fma2(mul2(dv[e], gw[j]), rs2, mul2(xh, nar));
              if (WGRAD) dg[j] = fma2(dv[e], xh, dg[j]);
            }
            sts128(dbase[b] + v * 16, P::pack2(o));
          }
        }
      }
    }
    ring_consumer_release(rs, cur);
#pragma unroll
    for (int b = 0; b < RB; ++b) rs_c[b] = rs_n[b];
  }

  if (WGRAD) {
    float* wg = ws + static_cast<int64_t>(blockIdx.x) * 2 * N;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = tid + k * GROUP;
      if (FULL || v < nvec) {
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          const int j = (k * VEC + q * 4) / 2;
          *reinterpret_cast<float4*>(wg + v * VEC + q * 4) = make_float4(dg[j].x, dg[j].y, dg[j + 1].x, dg[j + 1].y);
        }
      }
    }
  }
}

}  // namespace b2n
