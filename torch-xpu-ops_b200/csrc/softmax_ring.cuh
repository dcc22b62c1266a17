// Ring kernels for softmax / log-softmax over the last dim (input and output of the same type).
// A row is shared by GROUP threads, VPT 16-byte vectors each, held in registers: one HBM read and
// one HBM write per element.
#pragma once
#include "ring.cuh"

namespace b2n {

__device__ __forceinline__ float ex2_approx(float v) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(v));  // no .ftz: subnormal results are kept
  return r;
}
constexpr float kLog2e = 1.4426950408889634f;

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

template <typename T, bool LOG, int GROUP, int VPT>
__global__ void __launch_bounds__(kRingThreads, 1)
softmax_fwd_ring_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t M, int N, int S, int RPG,
                        int* status) {
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
  int red_phase = 0;
  const float ninf = acc_neg_inf<float>();
  const uint32_t stages_u32 = smem_u32(stages);

  RingCursor cur;
  cur.start(g);
  int64_t i = 0;
  for (; i < g.my_tiles; ++i, cur.advance(g)) {
    if (!ring_consumer_wait(rs, cur, status)) break;
    const uint32_t sbase = stages_u32 + static_cast<uint32_t>(cur.s) * g.stage_bytes;
    for (int r = 0; r < RPG; ++r) {
      const int lr = grp * RPG + r;
      if (cur.row0 + lr >= M) break;  // uniform over the group
      const uint32_t rbase = sbase + static_cast<uint32_t>(lr) * g.row_bytes;
      float xv[EPT];
      float pm[4] = {ninf, ninf, ninf, ninf};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          P::unpack(lds128(rbase + v * 16), &xv[k * VEC]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) pm[e & 3] = fmaxf(pm[e & 3], xv[k * VEC + e]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) xv[k * VEC + e] = ninf;
        }
      }
      float mx[1] = {fmaxf(fmaxf(pm[0], pm[1]), fmaxf(pm[2], pm[3]))};
      group_reduce<GROUP, 1>(mx, rs->red, grp, tg, red_phase, MaxOp());
      const RowExp<T> rexp(mx[0]);
      float ps[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        if (tg + k * GROUP < nvec) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float ex = rexp(xv[k * VEC + e]);
            ps[e & 3] += ex;
            if (!LOG) xv[k * VEC + e] = ex;
          }
        }
      }
      float sum[1] = {(ps[0] + ps[1]) + (ps[2] + ps[3])};
      group_reduce<GROUP, 1>(sum, rs->red, grp, tg, red_phase, SumOp());
      const float lg = LOG ? logf(sum[0]) : 0.0f;
      const float off = mx[0] + lg;  // 16-bit log-softmax: x - (max + log sum) in one subtraction
      const float inv = LOG ? 0.0f : 1.0f / sum[0];
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float t = xv[k * VEC + e];
            if constexpr (LOG) o[e] = sizeof(T) == 4 ? (t - mx[0]) - lg : t - off;
            else if constexpr (sizeof(T) == 4) o[e] = t / sum[0];
            else o[e] = t * inv;
          }
          sts128(rbase + v * 16, P::pack(o));
        }
      }
    }
    ring_consumer_release(rs, cur);
    if (tid == 0 && prod_ok) prod_ok = prod.after_tile(cur);
  }
  if (tid == 0) prod.epilogue(cur, i);
}

// stage = [dy tile | y tile]; dx overwrites the dy tile.
// softmax: dx = y*(dy - sum(y*dy)); log-softmax: dx = dy - exp(y)*sum(dy).
template <typename T, bool LOG, int GROUP, int VPT>
__global__ void __launch_bounds__(kRingThreads, 1)
softmax_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t M,
                        int N, int S, int RPG, int* status) {
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
  prod.in[1] = reinterpret_cast<const unsigned char*>(y);
  prod.out = reinterpret_cast<unsigned char*>(dx);
  if (tid == 0) prod.prologue();
  bool prod_ok = true;  // thread 0: a failed wait ends its producer duties, not its consumer loop

  const int grp = tid / GROUP, tg = tid % GROUP;
  const int nvec = N / VEC;
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
      if (cur.row0 + lr >= M) break;  // uniform over the group
      const uint32_t dbase = sbase + static_cast<uint32_t>(lr) * g.row_bytes;
      const uint32_t ybase = dbase + g.slot_bytes;
      float dv[EPT], yv[EPT];
      float ps[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          P::unpack(lds128(dbase + v * 16), &dv[k * VEC]);
          P::unpack(lds128(ybase + v * 16), &yv[k * VEC]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const int j = k * VEC + e;
            if constexpr (LOG) ps[e & 3] += dv[j];
            else ps[e & 3] = fmaf(dv[j], yv[j], ps[e & 3]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) { dv[k * VEC + e] = 0.0f; yv[k * VEC + e] = 0.0f; }
        }
      }
      float sum[1] = {(ps[0] + ps[1]) + (ps[2] + ps[3])};
      group_reduce<GROUP, 1>(sum, rs->red, grp, tg, red_phase, SumOp());
      const float s = sum[0];
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tg + k * GROUP;
        if (v < nvec) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float d = dv[k * VEC + e], yy = yv[k * VEC + e];
            if constexpr (LOG) {
              const float ey = sizeof(T) == 4 ? expf(yy) : ex2_approx(yy * kLog2e);
              o[e] = fmaf(-ey, s, d);
            } else {
              o[e] = yy * (d - s);
            }
          }
          sts128(dbase + v * 16, P::pack(o));
        }
      }
    }
    ring_consumer_release(rs, cur);
    if (tid == 0 && prod_ok) prod_ok = prod.after_tile(cur);
  }
  if (tid == 0) prod.epilogue(cur, i);
}

}  // namespace b2n
