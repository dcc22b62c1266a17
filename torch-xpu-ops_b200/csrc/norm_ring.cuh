// Ring kernels for layer norm / RMS norm (forward, and backward with the weight gradients fused).
// Rows are 16-byte aligned multiples of 16 bytes; a row is shared by GROUP threads, each holding
// VPT 16-byte vectors of it in registers, so every element is read from HBM once and written once.
// Accumulation is fp32; mean/rstd are fp32.
//
// Instruction budget: at HBM speed an SM has roughly 20 thread-instructions per element, of which
// per-row overhead (barrier waits, the cross-thread reductions) takes a large share when a thread
// holds only 16 elements of a row.  Hence: independent partial accumulators (no 16-long dependent
// add chains), FMA forms for the output expressions, and no integer division in the row loop.
#pragma once
#include "ring.cuh"

namespace b2n {

// thread tg of a group owns vectors tg + k*GROUP (k < VPT) of every row its group processes, so its
// gamma/beta values — and, in the backward, its dgamma/dbeta accumulators — stay in registers for
// the whole launch.
// Values are kept as float2 pairs of neighbouring columns: the element-wise math runs on the
// packed fp32 instructions of sm_100 (fma2 / add2 / mul2 in common.cuh).
template <typename WT, int GROUP, int VPT, int VEC>
__device__ __forceinline__ void load_weights(const WT* __restrict__ w, float fill, int nvec, int tg,
                                             float2 (&out)[VPT * VEC / 2]) {
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tg + k * GROUP;
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      const bool ok = w != nullptr && v < nvec;
      out[(k * VEC + e) / 2] = make_float2(ok ? to_acc<float>(w[v * VEC + e]) : fill,
                                           ok ? to_acc<float>(w[v * VEC + e + 1]) : fill);
    }
  }
}

constexpr int kTraceTid = 160;  // the consumer thread that writes trace records (lane 0 of warp 5)

// FULL: the row fills every thread's vectors exactly (N == GROUP * VPT * VEC), so no access needs a range check.
// RPGT: rows per group per tile as a compile-time constant (0: taken from the launch argument).
template <typename T, typename WT, bool RMS, int GROUP, int VPT, bool FULL, int RPGT>
__global__ void __launch_bounds__(kRingBlock, 1)
norm_fwd_ring_kernel(const T* __restrict__ x, const WT* __restrict__ gamma, const WT* __restrict__ beta,
                     T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t M,
                     int N, float eps, int S_lag, int rpg_arg, int* status, unsigned* tile_ctr,
                     unsigned long long* trace_buf, unsigned trace_cap) {
  using P = Pack16<T>;
  const int RPG = RPGT > 0 ? RPGT : rpg_arg;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  constexpr int RB = 2;  // rows a group works on at once
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S_lag, 1, tile_ctr, trace_buf, trace_cap);
  unsigned tk = 0;  // trace record counter (diagnostic)
  if (threadIdx.x == kTraceTid) g.trace.put(0, tk, EV_C_STEP + 8, 0);  // kernel entry
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
  // FULL rows have a compile-time length, and with it compile-time byte offsets
  const int nvec = FULL ? GROUP * VPT : N / VEC;
  const float inv_n = 1.0f / static_cast<float>(FULL ? GROUP * VPT * VEC : N);
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  const uint32_t stage_bytes = (FULL && RPGT > 0) ? static_cast<uint32_t>(NG * RPGT) * row_bytes : g.stage_bytes;
  constexpr int HP = EPT / 2, VH = VEC / 2;  // float2 pairs per thread / per 16-byte vector
  float2 gw[HP], gb[HP];
  load_weights<WT, GROUP, VPT, VEC>(gamma, 1.0f, nvec, tg, gw);
  if constexpr (!RMS) load_weights<WT, GROUP, VPT, VEC>(beta, 0.0f, nvec, tg, gb);
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start();
  for (;; cur.advance(g)) {
    if (tid == kTraceTid) g.trace.put(0, tk, EV_C_WAIT_BEGIN, 0);
    int i;  // the tile in this stage
    if (!ring_consumer_wait(rs, cur, status, i) || i < 0) break;
    const int64_t tile_row0 = g.first_row(i);
    if (tid == kTraceTid) g.trace.put(0, tk, EV_C_WAIT_END, i);
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * stage_bytes;
    // A group takes its rows of the tile RB at a time: the partial sums of RB rows go through ONE
    // group reduction (one barrier, RB values), which halves the time the group's warps spend
    // waiting on each other when a single group spans the whole CTA.
#pragma unroll(RPGT > 0 ? RPGT : 1)
    for (int r = 0; r < RPG; r += RB) {
      const int lr0 = grp * RPG + r;
      const int64_t row_a = tile_row0 + lr0;
      if (row_a >= M) break;  // uniform over the group
      bool valid[RB];
      uint32_t rbase[RB];
      float shift[RB];
      float2 xv[RB][HP];
      float red1[RB * (RMS ? 1 : 2)];  // RMS: sum x^2;  layer norm: sum d and sum d^2 per row
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        valid[b] = (r + b < RPG) && (row_a + b < M);
        rbase[b] = sbase + static_cast<uint32_t>(lr0 + b) * row_bytes;
        // Layer norm works on d = x - shift, shift = the row's first element (a shared-memory
        // broadcast read): a large common offset then cancels exactly instead of being rounded
        // away in the row sums.  RMS norm needs the raw values (shift = 0).
        shift[b] = 0.0f;
        if (!RMS && valid[b]) {
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
              if constexpr (!RMS) {
                xv[b][j] = add2(xv[b][j], nshift);
                ps[j & 1] = add2(ps[j & 1], xv[b][j]);
              }
              pq[j & 1] = fma2(xv[b][j], xv[b][j], pq[j & 1]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < VH; ++e) xv[b][k * VH + e] = bcast2(0.0f);
          }
        }
        if constexpr (RMS) {
          red1[b] = hsum2(add2(pq[0], pq[1]));
        } else {
          red1[2 * b] = hsum2(add2(ps[0], ps[1]));
          red1[2 * b + 1] = hsum2(add2(pq[0], pq[1]));
        }
      }
      if (tid == kTraceTid) g.trace.put(0, tk, EV_C_STEP + 0, i);
      group_reduce<GROUP, RB * (RMS ? 1 : 2)>(red1, rs->red, grp, tg, red_phase, SumOp());
      if (tid == kTraceTid) g.trace.put(0, tk, EV_C_STEP + 1, i);
      float mu_d[RB], rsd[RB];  // mu_d: mean of (x - shift)
      if constexpr (RMS) {
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          mu_d[b] = 0.0f;
          rsd[b] = rsqrt_nr(red1[b] * inv_n + eps);
        }
      } else {
        // One reduction gives both moments of d.  var = E[d^2] - E[d]^2 loses (1 + 3 E[d]^2/var)
        // ulps to cancellation, which is harmless while the row's first element lies within a few
        // standard deviations of its mean (the usual case: |z| < 2.8 for 99.5 % of Gaussian rows).
        // Otherwise — decided on the reduced values, so identically by every thread of the group —
        // the variance is taken again about the mean with a second pass over the registers.
        float var[RB];
        bool exact = true;
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          mu_d[b] = red1[2 * b] * inv_n;
          const float m2 = mu_d[b] * mu_d[b];
          var[b] = fmaf(red1[2 * b + 1], inv_n, -m2);
          exact = exact && (m2 <= 8.0f * var[b]);  // false for NaN and for a variance that cancelled below zero
        }
        if (!exact) {
          // Second pass, from the tile still in shared memory, with the mean just found as the new
          // shift (an outlying first element also costs every d the low bits of x, so the registers
          // are rebuilt, not reused): c = sum d and q = sum d^2 about a shift that is now within
          // rounding of the mean give mean = shift + c/N and var = (q - c^2/N)/N without cancellation.
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
            var[b] = vq < 0.0f ? 0.0f : vq;  // keeps NaN
          }
        }
#pragma unroll
        for (int b = 0; b < RB; ++b) rsd[b] = rsqrt_nr(var[b] + eps);
      }
      if (tid == kTraceTid) g.trace.put(0, tk, EV_C_STEP + 5, i);
#pragma unroll
      for (int b = 0; b < RB; ++b) {
        if (!valid[b]) continue;
        // y = ((d - mu_d) * rstd) * gamma + beta as two FMAs: fma(fma(d, rstd, -mu_d*rstd), gamma, beta)
        const float2 rs2 = bcast2(rsd[b]);
        const float2 c2 = bcast2(-mu_d[b] * rsd[b]);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tg + k * GROUP;
          if (FULL || v < nvec) {
            float2 o[VH];
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              const int j = k * VH + e;
              if constexpr (RMS) o[e] = mul2(mul2(xv[b][j], rs2), gw[j]);
              else o[e] = fma2(fma2(xv[b][j], rs2, c2), gw[j], gb[j]);
            }
            sts128(rbase[b] + v * 16, P::pack2(o));
          }
        }
        if (tid == kTraceTid) g.trace.put(0, tk, EV_C_STEP + 6 + b, i);
        if (tg == 0) {
          if (!RMS && mean) mean[row_a + b] = shift[b] + mu_d[b];
          if (rstd) rstd[row_a + b] = rsd[b];
        }
      }
    }
    if (tid == kTraceTid) g.trace.put(0, tk, EV_C_STEP + 4, i);
    ring_consumer_release(rs, cur);
    if (tid == kTraceTid) g.trace.put(0, tk, EV_C_RELEASED, i);
  }
}

// Backward: stage = [dy tile | x tile]; dx overwrites the dy tile.  Every thread also accumulates
// dgamma/dbeta for its own columns over all rows its group sees and writes them, at the end, as
// partial row (blockIdx.x * NG + group) of ws ([P][2][N] fp32).  WGRAD = false skips that.
// dx must not be null (a backward without dx goes through the generic weight-gradient kernels).
//
// Per row: s1 = sum(gamma*dy), s2 = sum(gamma*dy*xhat), xhat = (x - mean) * rstd,
// dx = rstd * (gamma*dy - (xhat*s2 + s1)/N)   (RMS: mean = 0, s1 = 0).
// FULL: the row fills every thread's vectors exactly (N == GROUP * VPT * VEC), so no access needs a range check.
// RPGT: rows per group per tile as a compile-time constant (0: taken from the launch argument).
template <typename T, typename WT, bool RMS, int GROUP, int VPT, bool WGRAD, bool FULL, int RPGT>
__global__ void __launch_bounds__(kRingBlock, 1)
norm_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const WT* __restrict__ gamma, T* __restrict__ dx,
                     float* __restrict__ ws, int64_t M, int N, int S_lag, int rpg_arg, int* status,
                     unsigned* tile_ctr) {
  using P = Pack16<T>;
  const int RPG = RPGT > 0 ? RPGT : rpg_arg;
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
      prod.in[1] = reinterpret_cast<const unsigned char*>(x);
      prod.out = reinterpret_cast<unsigned char*>(dx);
      prod.run();
    }
    return;
  }
  ring_consumer_regs();

  const int grp = tid / GROUP, tg = tid % GROUP;
  // FULL rows have a compile-time length, and with it compile-time byte offsets
  const int nvec = FULL ? GROUP * VPT : N / VEC;
  const float inv_n = 1.0f / static_cast<float>(FULL ? GROUP * VPT * VEC : N);
  const uint32_t row_bytes = FULL ? static_cast<uint32_t>(GROUP * VPT * 16) : g.row_bytes;
  const uint32_t slot_bytes = (FULL && RPGT > 0) ? static_cast<uint32_t>(NG * RPGT) * row_bytes : g.slot_bytes;
  const uint32_t stage_bytes = 2u * slot_bytes;
  constexpr int HP = EPT / 2, VH = VEC / 2;  // float2 pairs per thread / per 16-byte vector
  float2 gw[HP], dg[HP], db[HP];
  load_weights<WT, GROUP, VPT, VEC>(gamma, 1.0f, nvec, tg, gw);
#pragma unroll
  for (int e = 0; e < HP; ++e) { dg[e] = bcast2(0.0f); db[e] = bcast2(0.0f); }
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start();
  // mean/rstd of the group's first two rows of a tile are fetched one whole tile ahead: a global
  // load issued where the value is needed would add its full latency to every row (rows 2 and 3 of
  // a four-row tile — short rows, several groups per CTA to hide it — load theirs in place).
  // Which tile the next stage holds is read from its tile_id slot before that stage has been
  // waited for — a hint (the producer has normally written it long before); the id seen after the
  // wait decides, and a wrong guess reloads in place.
  // lane b (b < 2) of every warp holds the statistics of row b: two registers per tile instead of four
  float mu_c = 0.0f, rs_c = 0.0f;
  int id_c = -1;  // the tile mu_c / rs_c were loaded for
  auto load_stats = [&](int64_t row0, float& mu, float& rsd) {
    const int b = threadIdx.x & 31;
    const bool ok = b < 2 && b < RPG && row0 + b < M;
    mu = (!RMS && ok) ? __ldg(mean + row0 + b) : 0.0f;
    rsd = ok ? __ldg(rstd + row0 + b) : 0.0f;
  };
  // fixed assignment (this CTA's k-th tile is blockIdx.x + k * gridDim.x) exactly when weight gradients are
  // accumulated: the launcher passes no tile counter then.  A compile-time fact, so that each instantiation
  // carries only its own way of finding the next tile's statistics.
  constexpr bool fixed = WGRAD;
  unsigned k_tile = 0;
  for (;; cur.advance(g), ++k_tile) {
    float mu_n = 0.0f, rs_n = 0.0f;
    int id_n = -1;
    if constexpr (fixed) {  // the next tile is known: fetch its statistics a whole tile ahead
      const unsigned t = blockIdx.x + (k_tile + 1) * gridDim.x;
      id_n = t < g.ntiles ? static_cast<int>(t) : -1;
      if (id_n >= 0) load_stats(g.first_row(id_n) + grp * RPG, mu_n, rs_n);
    }
    int i;  // the tile in this stage
    if (!ring_consumer_wait(rs, cur, status, i) || i < 0) break;
    const int64_t row_first = g.first_row(i) + grp * RPG;
    if (i != id_c) load_stats(row_first, mu_c, rs_c);  // first tile, or the hint was stale (uniform over a warp)
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * stage_bytes;
#pragma unroll(RPGT > 0 ? RPGT : 1)
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      const int64_t row = row_first + r;
      if (row >= M) break;  // uniform over the group
      const uint32_t dbase = sbase + static_cast<uint32_t>(lr) * row_bytes;
      const uint32_t xbase = dbase + slot_bytes;
      float mu, rsd;
      if (r < 2) {
        mu = __shfl_sync(0xffffffffu, mu_c, r);
        rsd = __shfl_sync(0xffffffffu, rs_c, r);
      } else {
        mu = RMS ? 0.0f : __ldg(mean + row);
        rsd = __ldg(rstd + row);
      }
      const float2 nmu = bcast2(-mu), rs2 = bcast2(rsd);
      float2 gv[HP], xh[HP];  // gamma*dy and xhat
      float2 p2 = bcast2(0.0f), p1 = bcast2(0.0f);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (FULL || v < nvec) {
          float2 dv[VH];
          P::unpack2(lds128(dbase + v * 16), dv);
          P::unpack2(lds128(xbase + v * 16), &xh[k * VH]);
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            const int j = k * VH + e;
            xh[j] = mul2(add2(xh[j], nmu), rs2);
            gv[j] = mul2(dv[e], gw[j]);
            p2 = fma2(gv[j], xh[j], p2);
            if (!RMS) p1 = add2(p1, gv[j]);
            if (WGRAD) {
              dg[j] = fma2(dv[e], xh[j], dg[j]);
              if (!RMS) db[j] = add2(db[j], dv[e]);
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < VH; ++e) { gv[k * VH + e] = bcast2(0.0f); xh[k * VH + e] = bcast2(0.0f); }
        }
      }
      float2 nar, nbr;  // -(s2/N)*rstd and -(s1/N)*rstd
      if constexpr (RMS) {
        float red[1] = {hsum2(p2)};
        group_reduce<GROUP, 1>(red, rs->red, grp, tg, red_phase, SumOp());
        nar = bcast2(-(red[0] * inv_n * rsd));
        nbr = bcast2(0.0f);
      } else {
        float red[2] = {hsum2(p2), hsum2(p1)};
        group_reduce<GROUP, 2>(red, rs->red, grp, tg, red_phase, SumOp());
        nar = bcast2(-(red[0] * inv_n * rsd));
        nbr = bcast2(-(red[1] * inv_n * rsd));
      }
      // dx = rstd*gv - (xhat*(s2/N)*rstd + (s1/N)*rstd): two packed FMAs per pair
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (FULL || v < nvec) {
          float2 o[VH];
#pragma unroll
          for (int e = 0; e < VH; ++e) {
            const int j = k * VH + e;
            o[e] = fma2(gv[j], rs2, fma2(xh[j], nar, nbr));
          }
          sts128(dbase + v * 16, P::pack2(o));
        }
      }
      if (!fixed && r == 0) {  // (dynamic assignment only) by now the producer has normally named the next stage's tile
        id_n = ring_peek_tile(rs, cur.next_stage(g));
        if (id_n >= 0) load_stats(g.first_row(id_n) + grp * RPG, mu_n, rs_n);
      }
    }
    ring_consumer_release(rs, cur);
    mu_c = mu_n;
    rs_c = rs_n;
    id_c = id_n;
  }

  if (WGRAD) {
    const int64_t prow = static_cast<int64_t>(blockIdx.x) * NG + grp;
    float* wg = ws + (prow * 2 + 0) * N;
    float* wb = ws + (prow * 2 + 1) * N;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = tg + k * GROUP;
      if (FULL || v < nvec) {
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          const int j = (k * VEC + q * 4) / 2;
          *reinterpret_cast<float4*>(wg + v * VEC + q * 4) = make_float4(dg[j].x, dg[j].y, dg[j + 1].x, dg[j + 1].y);
          if (!RMS)
            *reinterpret_cast<float4*>(wb + v * VEC + q * 4) = make_float4(db[j].x, db[j].y, db[j + 1].x, db[j + 1].y);
        }
      }
    }
  }
}

}  // namespace b2n
