// Ring kernels for layer norm / RMS norm (forward, and backward with the weight gradients fused).
// Rows are 16-byte aligned multiples of 16 bytes; a row is shared by GROUP threads, each holding
// VPT 16-byte vectors of it in registers, so every element is read from HBM once and written once.
// Accumulation is fp32; mean/rstd are fp32.
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
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingConsumerThreads / GROUP;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.M = M;
  g.row_bytes = static_cast<uint32_t>(N) * sizeof(T);
  g.TR = NG * RPG;
  g.S = S;
  g.stage_bytes = static_cast<uint32_t>(g.TR) * g.row_bytes;
  g.ntiles = (M + g.TR - 1) / g.TR;

  ring_init(rs, S, kRingConsumerThreads / 32);
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
  int phase = 0;

  const int64_t n = g.my_tiles();
  int64_t i = 0;
  for (; i < n; ++i) {
    if (!ring_consumer_wait(rs, g, i, status)) break;
    const int64_t row0 = g.tile_row0(i);
    const uint32_t sbase = smem_u32(stages + static_cast<size_t>(i % S) * g.stage_bytes);
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      const int64_t row = row0 + lr;
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
      float red1[1] = {0.0f};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          P::unpack(lds128(rbase + v * 16), &xv[k * VEC]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            if constexpr (RMS) {
              red1[0] += xv[k * VEC + e] * xv[k * VEC + e];
            } else {
              xv[k * VEC + e] -= shift;
              red1[0] += xv[k * VEC + e];
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) xv[k * VEC + e] = 0.0f;
        }
      }
      group_reduce<GROUP, 1>(red1, rs->red, grp, tg, phase, SumOp());
      float mu_d = 0.0f, rsd;  // mu_d: mean of (x - shift)
      if constexpr (RMS) {
        rsd = acc_rsqrt(red1[0] * inv_n + eps);
      } else {
        mu_d = red1[0] * inv_n;
        float red2[1] = {0.0f};
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          if (tg + k * GROUP < nvec) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              const float d = xv[k * VEC + e] - mu_d;
              red2[0] += d * d;
            }
          }
        }
        group_reduce<GROUP, 1>(red2, rs->red, grp, tg, phase, SumOp());
        rsd = acc_rsqrt(red2[0] * inv_n + eps);
      }
      const float mu = shift + mu_d;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float t = (xv[k * VEC + e] - mu_d) * rsd * gw[k * VEC + e];
            o[e] = RMS ? t : t + gb[k * VEC + e];
          }
          sts128(rbase + v * 16, P::pack(o));
        }
      }
      if (tg == 0) {
        if (!RMS && mean) mean[row] = mu;
        if (rstd) rstd[row] = rsd;
      }
    }
    ring_consumer_release(rs, g, i);
    if (tid == 0 && prod_ok) prod_ok = prod.after_tile(i);
  }
  if (tid == 0) prod.epilogue(i);
}

// Backward: stage = [dy tile | x tile]; dx overwrites the dy tile.  Every thread also accumulates
// dgamma/dbeta for its own columns over all rows its group sees and writes them, at the end, as
// partial row (blockIdx.x * NG + group) of ws ([P][2][N] fp32).  WGRAD = false skips that.
// dx must not be null (a backward without dx goes through the generic weight-gradient kernels).
template <typename T, typename WT, bool RMS, int GROUP, int VPT, bool WGRAD>
__global__ void __launch_bounds__(kRingThreads, 1)
norm_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const WT* __restrict__ gamma, T* __restrict__ dx,
                     float* __restrict__ ws, int64_t M, int N, int S, int RPG, int* status) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, EPT = VPT * VEC, NG = kRingConsumerThreads / GROUP;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  RingGeom g;
  g.M = M;
  g.row_bytes = static_cast<uint32_t>(N) * sizeof(T);
  g.TR = NG * RPG;
  g.S = S;
  g.stage_bytes = 2u * static_cast<uint32_t>(g.TR) * g.row_bytes;
  g.ntiles = (M + g.TR - 1) / g.TR;
  const uint32_t slot = static_cast<uint32_t>(g.TR) * g.row_bytes;

  ring_init(rs, S, kRingConsumerThreads / 32);
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
  int phase = 0;

  const int64_t n = g.my_tiles();
  int64_t i = 0;
  for (; i < n; ++i) {
    const int64_t row0 = g.tile_row0(i);
    // row statistics of this tile: issued before the wait so their latency hides behind it
    float mu_r[4], rs_r[4];  // RPG <= 4
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t row = row0 + grp * RPG + r;
      const bool ok = r < RPG && row < M;
      mu_r[r] = (!RMS && ok) ? __ldg(mean + row) : 0.0f;
      rs_r[r] = ok ? __ldg(rstd + row) : 0.0f;
    }
    if (!ring_consumer_wait(rs, g, i, status)) break;
    const uint32_t sbase = smem_u32(stages + static_cast<size_t>(i % S) * g.stage_bytes);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r >= RPG) break;
      const int lr = grp * RPG + r;
      const int64_t row = row0 + lr;
      if (row >= M) break;  // uniform over the group
      const uint32_t dbase = sbase + static_cast<uint32_t>(lr) * g.row_bytes;
      const uint32_t xbase = dbase + slot;
      const float mu = mu_r[r], rsd = rs_r[r];
      float gv[EPT], xh[EPT];  // gamma*dy and xhat
      float red[2] = {0.0f, 0.0f};
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
            red[0] += gv[j] * xh[j];
            if (!RMS) red[1] += gv[j];
            if (WGRAD) {
              dg[j] += dv[e] * xh[j];
              if (!RMS) db[j] += dv[e];
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) { gv[k * VEC + e] = 0.0f; xh[k * VEC + e] = 0.0f; }
        }
      }
      group_reduce<GROUP, 2>(red, rs->red, grp, tg, phase, SumOp());
      const float a = red[0] * inv_n, b = RMS ? 0.0f : red[1] * inv_n;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = rsd * (gv[k * VEC + e] - (xh[k * VEC + e] * a + b));
          sts128(dbase + v * 16, P::pack(o));
        }
      }
    }
    ring_consumer_release(rs, g, i);
    if (tid == 0 && prod_ok) prod_ok = prod.after_tile(i);
  }
  if (tid == 0) prod.epilogue(i);

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
