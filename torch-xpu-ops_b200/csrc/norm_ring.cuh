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
template <typename WT, int GROUP, int VPT, int VEC>
__device__ __forceinline__ void load_weights(const WT* __restrict__ w, float fill, int nvec, int tg,
                                             float (&out)[VPT * VEC]) {
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = tg + k * GROUP;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      out[k * VEC + e] = (w != nullptr && v < nvec) ? to_acc<float>(w[v * VEC + e]) : fill;
  }
}

template <typename T, typename WT, bool RMS, int GROUP, int VPT>
__global__ void __launch_bounds__(kRingThreads, 1)
norm_fwd_ring_kernel(const T* __restrict__ x, const WT* __restrict__ gamma, const WT* __restrict__ beta,
                     T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t M,
                     int N, float eps, int S, int RPG, int* status) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S, 1);
  ring_init(rs, S, kRingThreads / 32);
  const int tid = threadIdx.x;
  RingProducer<1> prod(rs, stages, g, status);
  prod.in[0] = reinterpret_cast<const unsigned char*>(x);
  prod.out = reinterpret_cast<unsigned char*>(y);
  if (tid == 0) prod.prologue();
  bool prod_ok = true;  // thread 0: a failed wait ends its producer duties, not its consumer loop

  const int grp = tid / GROUP, tg = tid % GROUP;
  const int nvec = N / VEC;
  const float inv_n = 1.0f / static_cast<float>(N);
  float gw[EPT], gb[EPT];
  load_weights<WT, GROUP, VPT, VEC>(gamma, 1.0f, nvec, tg, gw);
  if constexpr (!RMS) load_weights<WT, GROUP, VPT, VEC>(beta, 0.0f, nvec, tg, gb);
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start(g);
  int64_t i = 0;
  for (; i < g.my_tiles; ++i, cur.advance(g)) {
    if (!ring_consumer_wait(rs, cur, status)) break;
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      const int64_t row = cur.row0 + lr;
      if (row >= M) break;  // uniform over the group
      const uint32_t rbase = sbase + static_cast<uint32_t>(lr) * g.row_bytes;
      // Layer norm works on d = x - shift, shift = the row's first element (a shared-memory
      // broadcast read): a large common offset then cancels exactly instead of being rounded away
      // in the row sum.  RMS norm needs the raw values (shift = 0).
      float shift = 0.0f;
      if constexpr (!RMS) {
        float first[VEC];
        P::unpack(lds128(rbase), first);
        shift = first[0];
      }
      float xv[EPT];
      float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          P::unpack(lds128(rbase + v * 16), &xv[k * VEC]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const int j = k * VEC + e;
            if constexpr (RMS) {
              part[j & 3] = fmaf(xv[j], xv[j], part[j & 3]);
            } else {
              xv[j] -= shift;
              part[j & 3] += xv[j];
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) xv[k * VEC + e] = 0.0f;
        }
      }
      float red1[1] = {(part[0] + part[1]) + (part[2] + part[3])};
      group_reduce<GROUP, 1>(red1, rs->red, grp, tg, red_phase, SumOp());
      float mu_d = 0.0f, rsd;  // mu_d: mean of (x - shift)
      if constexpr (RMS) {
        rsd = acc_rsqrt(red1[0] * inv_n + eps);
      } else {
        mu_d = red1[0] * inv_n;
        float q[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          if (tg + k * GROUP < nvec) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              const int j = k * VEC + e;
              const float d = xv[j] - mu_d;
              q[j & 3] = fmaf(d, d, q[j & 3]);
            }
          }
        }
        float red2[1] = {(q[0] + q[1]) + (q[2] + q[3])};
        group_reduce<GROUP, 1>(red2, rs->red, grp, tg, red_phase, SumOp());
        rsd = acc_rsqrt(red2[0] * inv_n + eps);
      }
      // y = ((d - mu_d) * rstd) * gamma + beta as two FMAs: fma(fma(d, rstd, -mu_d*rstd), gamma, beta)
      const float c = -mu_d * rsd;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const int j = k * VEC + e;
            if constexpr (RMS) o[e] = (xv[j] * rsd) * gw[j];
            else o[e] = fmaf(fmaf(xv[j], rsd, c), gw[j], gb[j]);
          }
          sts128(rbase + v * 16, P::pack(o));
        }
      }
      if (tg == 0) {
        if (!RMS && mean) mean[row] = shift + mu_d;
        if (rstd) rstd[row] = rsd;
      }
    }
    ring_consumer_release(rs, cur);
    if (tid == 0 && prod_ok) prod_ok = prod.after_tile(cur);
  }
  if (tid == 0) prod.epilogue(cur, i);
}

// Backward: stage = [dy tile | x tile]; dx overwrites the dy tile.  Every thread also accumulates
// dgamma/dbeta for its own columns over all rows its group sees and writes them, at the end, as
// partial row (blockIdx.x * NG + group) of ws ([P][2][N] fp32).  WGRAD = false skips that.
// dx must not be null (a backward without dx goes through the generic weight-gradient kernels).
//
// Per row: s1 = sum(gamma*dy), s2 = sum(gamma*dy*xhat), xhat = (x - mean) * rstd,
// dx = rstd * (gamma*dy - (xhat*s2 + s1)/N)   (RMS: mean = 0, s1 = 0).
template <typename T, typename WT, bool RMS, int GROUP, int VPT, bool WGRAD>
__global__ void __launch_bounds__(kRingThreads, 1)
norm_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const WT* __restrict__ gamma, T* __restrict__ dx,
                     float* __restrict__ ws, int64_t M, int N, int S, int RPG, int* status) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingThreads / GROUP;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.init(M, N, sizeof(T), NG * RPG, S, 2);
  ring_init(rs, S, kRingThreads / 32);
  const int tid = threadIdx.x;
  RingProducer<2> prod(rs, stages, g, status);
  prod.in[0] = reinterpret_cast<const unsigned char*>(dy);
  prod.in[1] = reinterpret_cast<const unsigned char*>(x);
  prod.out = reinterpret_cast<unsigned char*>(dx);
  if (tid == 0) prod.prologue();
  bool prod_ok = true;  // thread 0: a failed wait ends its producer duties, not its consumer loop

  const int grp = tid / GROUP, tg = tid % GROUP;
  const int nvec = N / VEC;
  const float inv_n = 1.0f / static_cast<float>(N);
  float gw[EPT], dg[EPT], db[EPT];
  load_weights<WT, GROUP, VPT, VEC>(gamma, 1.0f, nvec, tg, gw);
#pragma unroll
  for (int e = 0; e < EPT; ++e) { dg[e] = 0.0f; db[e] = 0.0f; }
  int red_phase = 0;
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start(g);
  int64_t i = 0;
  for (; i < g.my_tiles; ++i, cur.advance(g)) {
    // statistics of this group's first row in the tile: issued before the wait, so the global-load
    // latency hides behind it (later rows of a multi-row tile load theirs in place)
    const int64_t row_first = cur.row0 + grp * RPG;
    float mu_p = 0.0f, rs_p = 0.0f;
    if (row_first < M) {
      if (!RMS) mu_p = __ldg(mean + row_first);
      rs_p = __ldg(rstd + row_first);
    }
    if (!ring_consumer_wait(rs, cur, status)) break;
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      const int64_t row = row_first + r;
      if (row >= M) break;  // uniform over the group
      const uint32_t dbase = sbase + static_cast<uint32_t>(lr) * g.row_bytes;
      const uint32_t xbase = dbase + g.slot_bytes;
      float mu = mu_p, rsd = rs_p;
      if (r > 0) {
        if (!RMS) mu = __ldg(mean + row);
        rsd = __ldg(rstd + row);
      }
      float gv[EPT], xh[EPT];  // gamma*dy and xhat
      float p2[2] = {0.0f, 0.0f}, p1[2] = {0.0f, 0.0f};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float dv[VEC];
          P::unpack(lds128(dbase + v * 16), dv);
          P::unpack(lds128(xbase + v * 16), &xh[k * VEC]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const int j = k * VEC + e;
            xh[j] = (xh[j] - mu) * rsd;
            gv[j] = dv[e] * gw[j];
            p2[j & 1] = fmaf(gv[j], xh[j], p2[j & 1]);
            if (!RMS) p1[j & 1] += gv[j];
            if (WGRAD) {
              dg[j] = fmaf(dv[e], xh[j], dg[j]);
              if (!RMS) db[j] += dv[e];
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) { gv[k * VEC + e] = 0.0f; xh[k * VEC + e] = 0.0f; }
        }
      }
      float ar, br;
      if constexpr (RMS) {
        float red[1] = {p2[0] + p2[1]};
        group_reduce<GROUP, 1>(red, rs->red, grp, tg, red_phase, SumOp());
        ar = red[0] * inv_n * rsd;
        br = 0.0f;
      } else {
        float red[2] = {p2[0] + p2[1], p1[0] + p1[1]};
        group_reduce<GROUP, 2>(red, rs->red, grp, tg, red_phase, SumOp());
        ar = red[0] * inv_n * rsd;
        br = red[1] * inv_n * rsd;
      }
      // dx = rstd*gv - (xhat*(s2/N)*rstd + (s1/N)*rstd): two FMAs per element
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const int j = k * VEC + e;
            o[e] = fmaf(gv[j], rsd, -fmaf(xh[j], ar, br));
          }
          sts128(dbase + v * 16, P::pack(o));
        }
      }
    }
    ring_consumer_release(rs, cur);
    if (tid == 0 && prod_ok) prod_ok = prod.after_tile(cur);
  }
  if (tid == 0) prod.epilogue(cur, i);

  if (WGRAD) {
    const int64_t prow = static_cast<int64_t>(blockIdx.x) * NG + grp;
    float* wg = ws + (prow * 2 + 0) * N;
    float* wb = ws + (prow * 2 + 1) * N;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = tg + k * GROUP;
      if (v < nvec) {
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          const int j = k * VEC + q * 4;
          *reinterpret_cast<float4*>(wg + v * VEC + q * 4) = make_float4(dg[j], dg[j + 1], dg[j + 2], dg[j + 3]);
          if (!RMS)
            *reinterpret_cast<float4*>(wb + v * VEC + q * 4) = make_float4(db[j], db[j + 1], db[j + 2], db[j + 3]);
        }
      }
    }
  }
}

}  // namespace b2n
