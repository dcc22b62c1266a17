// Sibling norms that share the row-statistics machinery: GroupNorm forward and the BatchNorm
// statistics.
//
// GroupNorm over a contiguous [N, C, HxW] tensor is a row-wise normalisation of [N * G, D * HxW]
// (D = C / G channels per group) followed by a per-CHANNEL affine map, so a row is handled like a
// layer-norm row — shifted one-pass moments in fp32, the exact second pass when the shift lies far
// from the mean — and only the weights differ: element j of row (n, g) takes gamma[g * D + j / HxW].
// One CTA per row at a time, 16-byte accesses when the row is a whole number of aligned vectors; the
// row is read a second time for the output, from L1/L2 (a group's row is a few KB to a few MB).
//
// BatchNorm statistics reduce the other way: per channel c over all n and all spatial positions.  One
// CTA per channel walks the N runs of HxW contiguous elements (warps over n, lanes along the run);
// for HxW < 16 (an [N, C] input) 32 adjacent channels share a CTA so that the lanes still read
// adjacent addresses.  Shifted one-pass sums again, merged exactly.
//
// Replaces group_norm_kernel (src/ATen/native/xpu/sycl/GroupNormKernels.h:17-28; moments functors
// GroupNormKernels.cpp:73-136, driver :365-499), batch_norm_stats_kernel and
// batch_norm_update_stats_kernel (sycl/BatchNormKernels.h:19, :52; BatchNormKernels.cpp:992, :3864).
#include <atomic>

#include "common.cuh"
#include "group_norm_ring.cuh"
#include "launchers.h"
#include "plan.h"

namespace b2n {
namespace {

// sums of (a, b) over the CTA; every thread gets the totals (fixed order).  scratch: 64 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch) {
  a = warp_reduce(a, SumOp());
  b = warp_reduce(b, SumOp());
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) { scratch[w] = a; scratch[32 + w] = b; }
  __syncthreads();
  float ra = scratch[0], rb = scratch[32];
  for (int i = 1; i < nw; ++i) { ra += scratch[i]; rb += scratch[32 + i]; }
  a = ra;
  b = rb;
}

template <typename T, int V>
__device__ __forceinline__ void row_shifted_sums(const T* __restrict__ row, int64_t L, float shift, float& s, float& q) {
  s = 0.0f;
  q = 0.0f;
  if constexpr (V > 1) {
    const int64_t nv = L / V;
    for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
      const Vec<T, V> xv = ld_vec<T, V>(row + v * V);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float d = to_acc<float>(xv.v[e]) - shift;
        s += d;
        q = fmaf(d, d, q);
      }
    }
  } else {
    for (int64_t j = threadIdx.x; j < L; j += blockDim.x) {
      const float d = to_acc<float>(row[j]) - shift;
      s += d;
      q = fmaf(d, d, q);
    }
  }
}

// One CTA per row of [rows = N * G, L = D * HxW].  ST: type of the mean / rstd outputs.
template <typename T, typename WT, typename ST, int V>
__global__ void __launch_bounds__(512)
group_norm_fwd_kernel(const T* __restrict__ x, const WT* __restrict__ gamma, const WT* __restrict__ beta, T* __restrict__ y,
                      ST* __restrict__ mean, ST* __restrict__ rstd, int64_t rows, int G, int D, int HxW, float eps) {
  __shared__ float scratch[64];
  const int64_t L = static_cast<int64_t>(D) * HxW;
  const float inv_l = 1.0f / static_cast<float>(L);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * L;
    T* yr = y + row * L;
    float shift = to_acc<float>(xr[0]);  // the same address for every thread: one broadcast load
    float s, q;
    row_shifted_sums<T, V>(xr, L, shift, s, q);
    block_sum2(s, q, scratch);
    float mu_d = s * inv_l;
    float var = fmaf(q, inv_l, -mu_d * mu_d);
    if (!(mu_d * mu_d <= 8.0f * var)) {  // cancellation (or NaN): once more about the mean just found
      shift += mu_d;
      row_shifted_sums<T, V>(xr, L, shift, s, q);
      block_sum2(s, q, scratch);
      mu_d = s * inv_l;
      const float v2 = fmaf(-mu_d, s, q) * inv_l;
      var = v2 < 0.0f ? 0.0f : v2;  // keeps NaN
    }
    const float mu = shift + mu_d;
    const float rs = 1.0f / sqrtf(var + eps);
    const int c0 = static_cast<int>(row % G) * D;  // first channel of this row's group
    if constexpr (V > 1) {
      const int64_t nv = L / V;
      const bool one_channel = HxW % V == 0;  // then a vector never straddles two channels
      for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
        const Vec<T, V> xv = ld_vec<T, V>(xr + v * V);
        Vec<T, V> o;
        const int j0 = static_cast<int>(v) * V;
        int c = c0 + j0 / HxW;
        float gm = gamma ? to_acc<float>(gamma[c]) : 1.0f, bt = beta ? to_acc<float>(beta[c]) : 0.0f;
#pragma unroll
        for (int e = 0; e < V; ++e) {
          if (!one_channel && e > 0) {
            const int ce = c0 + (j0 + e) / HxW;
            if (ce != c) {
              c = ce;
              gm = gamma ? to_acc<float>(gamma[c]) : 1.0f;
              bt = beta ? to_acc<float>(beta[c]) : 0.0f;
            }
          }
          o.v[e] = from_acc<T>(fmaf((to_acc<float>(xv.v[e]) - mu) * rs, gm, bt));
        }
        st_vec<T, V>(yr + v * V, o);
      }
    } else {
      for (int64_t j = threadIdx.x; j < L; j += blockDim.x) {
        const int c = c0 + static_cast<int>(j / HxW);
        const float gm = gamma ? to_acc<float>(gamma[c]) : 1.0f, bt = beta ? to_acc<float>(beta[c]) : 0.0f;
        yr[j] = from_acc<T>(fmaf((to_acc<float>(xr[j]) - mu) * rs, gm, bt));
      }
    }
    if (threadIdx.x == 0) {
      mean[row] = from_acc<ST>(mu);
      rstd[row] = from_acc<ST>(rs);
    }
    __syncthreads();  // scratch is reused by the next row
  }
}

// ---- group norm backward ------------------------------------------------------------------------------------
// Row (n, g) of [N * G, L = D * HxW] with xhat = (x - mean) * rstd and g_j = dy_j * gamma[c(j)]:
//   dx_j = rstd * (g_j - (xhat_j * s2 + s1) / L),  s1 = sum g,  s2 = sum g * xhat          (one CTA per row, two walks,
//   the second served by L1/L2);
//   dgamma[c] = sum over n and the channel's HxW elements of dy * xhat,  dbeta[c] = sum dy   (one CTA per channel).
// The formulas of the reference's backward (GroupNormKernels.cpp, ComputeInternalGradients / GroupNormBackward /
// GammaBetaBackward), evaluated in fp32 from the saved statistics.
template <typename T, typename WT, typename ST, int V>
__global__ void __launch_bounds__(512)
group_norm_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x, const ST* __restrict__ mean,
                         const ST* __restrict__ rstd, const WT* __restrict__ gamma, T* __restrict__ dx, int64_t rows, int G,
                         int D, int HxW) {
  __shared__ float scratch[64];
  const int64_t L = static_cast<int64_t>(D) * HxW;
  const float inv_l = 1.0f / static_cast<float>(L);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * L;
    const T* gr = dy + row * L;
    T* dr = dx + row * L;
    const float mu = to_acc<float>(mean[row]), rs = to_acc<float>(rstd[row]);
    const int c0 = static_cast<int>(row % G) * D;
    // V > 1 is taken only when HxW % V == 0: a vector then lies in one channel
    auto walk = [&](auto&& body) {
      if constexpr (V > 1) {
        const int64_t nv = L / V;
        for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
          const Vec<T, V> xv = ld_vec<T, V>(xr + v * V), gv = ld_vec<T, V>(gr + v * V);
          const float gm = gamma ? to_acc<float>(gamma[c0 + static_cast<int>((v * V) / HxW)]) : 1.0f;
          Vec<T, V> o;
#pragma unroll
          for (int e = 0; e < V; ++e) o.v[e] = body(to_acc<float>(xv.v[e]), to_acc<float>(gv.v[e]) * gm);
          if (body.stores) st_vec<T, V>(dr + v * V, o);
        }
      } else {
        for (int64_t j = threadIdx.x; j < L; j += blockDim.x) {
          const float gm = gamma ? to_acc<float>(gamma[c0 + static_cast<int>(j / HxW)]) : 1.0f;
          const T o = body(to_acc<float>(xr[j]), to_acc<float>(gr[j]) * gm);
          if (body.stores) dr[j] = o;
        }
      }
    };
    float s1 = 0.0f, s2 = 0.0f;
    struct Sums {
      float &s1, &s2, mu, rs;
      bool stores;
      __device__ T operator()(float xv, float g) const {
        s1 += g;
        s2 = fmaf(g, (xv - mu) * rs, s2);
        return T();
      }
    } sums{s1, s2, mu, rs, false};
    walk(sums);
    block_sum2(s1, s2, scratch);
    struct Out {
      float a, b, mu, rs;
      bool stores;
      __device__ T operator()(float xv, float g) const { return from_acc<T>(rs * (g - fmaf((xv - mu) * rs, a, b))); }
    } out{s2 * inv_l, s1 * inv_l, mu, rs, true};
    walk(out);
    __syncthreads();  // scratch is reused by the next row
  }
}

template <typename T, typename WT, typename ST, int V>
__global__ void __launch_bounds__(512)
group_norm_bwd_wgrad_kernel(const T* __restrict__ dy, const T* __restrict__ x, const ST* __restrict__ mean,
                            const ST* __restrict__ rstd, WT* __restrict__ dgamma, WT* __restrict__ dbeta, int64_t N, int C,
                            int G, int HxW) {
  __shared__ float scratch[64];
  const int c = blockIdx.x, D = C / G, g = c / D;
  float sg = 0.0f, sb = 0.0f;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  // warps over samples, lanes along the run: each sample's statistics are read once per warp
  for (int64_t n = w; n < N; n += nw) {
    const float mu = to_acc<float>(mean[n * G + g]), rs = to_acc<float>(rstd[n * G + g]);
    const T* xr = x + (n * C + c) * static_cast<int64_t>(HxW);
    const T* gr = dy + (n * C + c) * static_cast<int64_t>(HxW);
    float a = 0.0f, b = 0.0f;  // sum dy * (x - mu), sum dy of this run
    if constexpr (V > 1) {
      const int nv = HxW / V;
      auto add_pair = [&](const Vec<T, V>& xv, const Vec<T, V>& gv) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float d = to_acc<float>(gv.v[e]);
          a = fmaf(d, to_acc<float>(xv.v[e]) - mu, a);
          b += d;
        }
      };
      int v = l;
      for (; v + 96 < nv; v += 128) {  // four vector pairs in flight per lane
        Vec<T, V> xv[4], gv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          xv[u] = ld_vec<T, V>(xr + (v + 32 * u) * V);
          gv[u] = ld_vec<T, V>(gr + (v + 32 * u) * V);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) add_pair(xv[u], gv[u]);
      }
      for (; v < nv; v += 32) add_pair(ld_vec<T, V>(xr + v * V), ld_vec<T, V>(gr + v * V));
    } else {
      for (int j = l; j < HxW; j += 32) {
        const float d = to_acc<float>(gr[j]);
        a = fmaf(d, to_acc<float>(xr[j]) - mu, a);
        b += d;
      }
    }
    sg = fmaf(a, rs, sg);
    sb += b;
  }
  block_sum2(sg, sb, scratch);
  if (threadIdx.x == 0) {
    if (dgamma) dgamma[c] = from_acc<WT>(sg);
    if (dbeta) dbeta[c] = from_acc<WT>(sb);
  }
}

// ---- batch norm statistics ------------------------------------------------------------------------------
// x: [N, C, HxW].  Channel c's elements: N runs of HxW at (n * C + c) * HxW.  Results in fp32:
// mean[c]; second[c] = 1 / sqrt(var + eps) (MODE 0, batch_norm_stats) or the biased variance (MODE 1,
// batch_norm_update_stats, which also folds the batch statistics into running_mean / running_var with `momentum`,
// the variance unbiased by n / (n - 1)).  RT: type of the running statistics.
template <typename RT>
__device__ __forceinline__ void bn_finish(int mode, float mu, float var, float count, float eps, float momentum, int c,
                                          float* mean, float* second, RT* running_mean, RT* running_var) {
  mean[c] = mu;
  if (mode == 0) {
    second[c] = 1.0f / sqrtf(var + eps);
  } else {
    second[c] = var;
    if (running_mean != nullptr)
      running_mean[c] = from_acc<RT>((1.0f - momentum) * to_acc<float>(running_mean[c]) + momentum * mu);
    if (running_var != nullptr) {
      const float unbiased = var * (count / (count - 1.0f));
      running_var[c] = from_acc<RT>((1.0f - momentum) * to_acc<float>(running_var[c]) + momentum * unbiased);
    }
  }
}

// HxW >= 16: one CTA per channel, warps over n, lanes along the run.
template <typename T, typename RT>
__global__ void __launch_bounds__(512)
batch_norm_stats_spatial_kernel(const T* __restrict__ x, float* __restrict__ mean, float* __restrict__ second,
                                RT* __restrict__ running_mean, RT* __restrict__ running_var, int64_t N, int C, int64_t HxW,
                                float eps, float momentum, int mode) {
  __shared__ float scratch[64];
  const int c = blockIdx.x;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float count = static_cast<float>(N) * static_cast<float>(HxW);
  float shift = to_acc<float>(x[static_cast<int64_t>(c) * HxW]);
  float mu_d = 0.0f, var = 0.0f;
  for (int pass = 0; pass < 2; ++pass) {
    float s = 0.0f, q = 0.0f;
    for (int64_t n = w; n < N; n += nw) {
      const T* run = x + (n * C + c) * HxW;
      for (int64_t j = l; j < HxW; j += 32) {
        const float d = to_acc<float>(run[j]) - shift;
        s += d;
        q = fmaf(d, d, q);
      }
    }
    block_sum2(s, q, scratch);
    mu_d = s / count;
    if (pass == 0) {
      var = q / count - mu_d * mu_d;
      if (mu_d * mu_d <= 8.0f * var) break;  // well conditioned: done in one pass
      shift += mu_d;
    } else {
      const float v2 = (q - mu_d * s) / count;
      var = v2 < 0.0f ? 0.0f : v2;
    }
  }
  if (threadIdx.x == 0) bn_finish<RT>(mode, shift + mu_d, var, count, eps, momentum, c, mean, second, running_mean, running_var);
}

// HxW < 16: 32 adjacent channels per CTA (lanes along c when HxW == 1), row lanes over (n, position).
template <typename T, typename RT>
__global__ void __launch_bounds__(1024)
batch_norm_stats_flat_kernel(const T* __restrict__ x, float* __restrict__ mean, float* __restrict__ second,
                             RT* __restrict__ running_mean, RT* __restrict__ running_var, int64_t N, int C, int64_t HxW,
                             float eps, float momentum, int mode) {
  __shared__ float ss[32][33], sq[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 32
  const int c = blockIdx.x * 32 + tx;
  const int64_t per_c = N * HxW;
  const float count = static_cast<float>(per_c);
  float shift = c < C ? to_acc<float>(x[static_cast<int64_t>(c) * HxW]) : 0.0f;
  float mu_d = 0.0f, var = 0.0f;
  for (int pass = 0; pass < 2; ++pass) {
    float s = 0.0f, q = 0.0f;
    if (c < C) {
      for (int64_t i = ty; i < per_c; i += 32) {
        const int64_t n = i / HxW, j = i - n * HxW;
        const float d = to_acc<float>(x[(n * C + c) * HxW + j]) - shift;
        s += d;
        q = fmaf(d, d, q);
      }
    }
    __syncthreads();
    ss[ty][tx] = s;
    sq[ty][tx] = q;
    __syncthreads();
    s = 0.0f;
    q = 0.0f;
    for (int k = 0; k < 32; ++k) { s += ss[k][tx]; q += sq[k][tx]; }
    mu_d = s / count;
    bool redo = false;
    if (pass == 0) {
      var = q / count - mu_d * mu_d;
      redo = !(mu_d * mu_d <= 8.0f * var);
    } else {
      const float v2 = (q - mu_d * s) / count;
      var = v2 < 0.0f ? 0.0f : v2;
    }
    // the second pass is taken by the whole CTA if any of its channels needs it (the barriers above are CTA-wide)
    if (pass == 1 || !__syncthreads_or(redo ? 1 : 0)) break;
    if (redo) shift += mu_d;
    else { /* channels that were fine repeat the pass about the same shift: same result */ }
  }
  if (ty == 0 && c < C) bn_finish<RT>(mode, shift + mu_d, var, count, eps, momentum, c, mean, second, running_mean, running_var);
}

// ---- vector path: HxW a whole number of 16-byte vectors, x 16-byte aligned ---------------------------------
// Sums of d = x - sh and d^2 over vectors [begin, end) of one channel (xc: the channel's first element; vector idx
// is vector idx % HV of sample idx / HV).  16-byte loads, four in flight per thread — addresses first, then the
// loads back to back, then the arithmetic (packed f32x2); a thread's position advances by additions.
template <typename T>
__device__ __forceinline__ void bn_channel_sums(const T* __restrict__ xc, int64_t sample_stride, int64_t HV, int64_t begin,
                                                int64_t end, float sh, float& s_out, float& q_out) {
  using P = Pack16<T>;
  constexpr int V = P::VEC, VH = V / 2;
  const float2 nsh = make_float2(-sh, -sh);
  float2 s2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)}, q2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
  auto add_vec = [&](const uint4& w) {
    float2 xv[VH];
    P::unpack2(w, xv);
#pragma unroll
    for (int e = 0; e < VH; ++e) {
      const float2 d = add2(xv[e], nsh);
      s2[e & 1] = add2(s2[e & 1], d);
      q2[e & 1] = fma2(d, d, q2[e & 1]);
    }
  };
  // One stride of the CTA as (samples, vectors): j + step_j < 2 * HV, so one wrap suffices.  The thread carries a
  // POINTER and its vector index inside the run: a stride adds a constant to the pointer, a wrap into the next
  // sample's run another constant — no 64-bit multiply per vector.
  const int64_t stride = blockDim.x;
  const int64_t step_n = stride / HV;
  const int hv = static_cast<int>(HV), step_j = static_cast<int>(stride % HV);  // (a run has fewer than 2^31 vectors)
  const int64_t d_stride = step_n * sample_stride + static_cast<int64_t>(step_j) * V;  // elements
  const int64_t d_wrap = sample_stride - HV * V;
  int64_t idx = begin + threadIdx.x;
  const int64_t n0 = idx / HV;
  int j = static_cast<int>(idx - n0 * HV);
  const T* p = xc + n0 * sample_stride + static_cast<int64_t>(j) * V;
  auto advance = [&]() {
    j += step_j;
    p += d_stride;
    if (j >= hv) { j -= hv; p += d_wrap; }
  };
  for (; idx + 3 * stride < end; idx += 4 * stride) {
    const uint4* q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      q[u] = reinterpret_cast<const uint4*>(p);
      advance();
    }
    uint4 w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) w[u] = __ldg(q[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u) add_vec(w[u]);
  }
  if (idx < end) {
    // the last one to three strides, still loaded together: a stride past the end reads this thread's first vector
    // of the group again (a valid address) and is left out of the sums
    const uint4* q0 = reinterpret_cast<const uint4*>(p);
    const uint4* q[3];
    bool have[3];
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      have[u] = idx + u * stride < end;
      q[u] = have[u] ? reinterpret_cast<const uint4*>(p) : q0;
      advance();
    }
    uint4 w[3];
#pragma unroll
    for (int u = 0; u < 3; ++u) w[u] = __ldg(q[u]);
#pragma unroll
    for (int u = 0; u < 3; ++u)
      if (have[u]) add_vec(w[u]);
  }
  s_out = (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
  q_out = (q2[0].x + q2[0].y) + (q2[1].x + q2[1].y);
}

// The value the sums of a channel are taken about: the mean of the first element of up to eight samples.  Any
// value near the channel's mean will do (the result does not depend on it beyond rounding); ONE element is within
// 2.8 standard deviations of the mean only 99.5 % of the time, and every miss costs a second pass over the channel.
// Every CTA that touches a channel computes the same value.
template <typename T>
__device__ __forceinline__ float bn_channel_shift(const T* __restrict__ xc, int64_t sample_stride, int64_t N) {
  const int k = N < 8 ? static_cast<int>(N) : 8;
  float a = 0.0f;
  for (int n = 0; n < k; ++n) a += to_acc<float>(xc[n * sample_stride]);
  return a / static_cast<float>(k);
}

// Mean and variance of a channel from its sums about `shift`; when |mean - shift| is large against the spread
// (or the sums are NaN) the subtraction cancels and the whole CTA sums the channel once more about the mean found.
template <typename T, typename RT>
__device__ __forceinline__ void bn_channel_finish(const T* __restrict__ xc, int64_t sample_stride, int64_t HV, int64_t TV,
                                                  float shift, float s, float q, float count, int mode, float eps, float momentum,
                                                  int c, float* mean, float* second, RT* running_mean, RT* running_var,
                                                  float* scratch) {
  float mu_d = s / count;
  float var = q / count - mu_d * mu_d;
  if (!(mu_d * mu_d <= 8.0f * var)) {  // (uniform over the CTA: every thread holds the same s and q)
    shift += mu_d;
    bn_channel_sums<T>(xc, sample_stride, HV, 0, TV, shift, s, q);
    block_sum2(s, q, scratch);
    mu_d = s / count;
    const float v2 = (q - mu_d * s) / count;
    var = v2 < 0.0f ? 0.0f : v2;  // keeps NaN
  }
  if (threadIdx.x == 0) bn_finish<RT>(mode, shift + mu_d, var, count, eps, momentum, c, mean, second, running_mean, running_var);
}

// One CTA per channel (no scratch memory needed): fine when there are at least a few hundred channels.
template <typename T, typename RT>
__global__ void __launch_bounds__(512, 2)
batch_norm_stats_channel_kernel(const T* __restrict__ x, float* __restrict__ mean, float* __restrict__ second,
                                RT* __restrict__ running_mean, RT* __restrict__ running_var, int64_t N, int C, int64_t HxW,
                                float eps, float momentum, int mode) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float scratch[64];
  const int c = blockIdx.x;
  const int64_t HV = HxW / V, TV = N * HV, sample_stride = static_cast<int64_t>(C) * HxW;
  const T* xc = x + static_cast<int64_t>(c) * HxW;
  const float shift = bn_channel_shift<T>(xc, sample_stride, N);
  float s, q;
  bn_channel_sums<T>(xc, sample_stride, HV, 0, TV, shift, s, q);
  block_sum2(s, q, scratch);
  bn_channel_finish<T, RT>(xc, sample_stride, HV, TV, shift, s, q, static_cast<float>(N) * static_cast<float>(HxW), mode, eps,
                           momentum, c, mean, second, running_mean, running_var, scratch);
}

// Two kernels with scratch memory, for any number of channels.  The C * TV vectors of the tensor's channels, laid
// end to end, are cut into gridDim.x equal ranges of G vectors — ONE balanced wave of CTAs, whatever C is.  A range
// covers parts of one or more channels; for each, the CTA sums about the channel's shift value (bn_channel_shift: every
// CTA that touches a channel computes the same one, so the sums simply add) and leaves {sum d, sum d^2} in
// partial[c][slot], slot = this CTA's index among the CTAs that touch channel c.
template <typename T>
__global__ void __launch_bounds__(512, 2)
batch_norm_stats_range_kernel(const T* __restrict__ x, int64_t N, int C, int64_t HxW, int64_t G, int max_slots,
                              float2* __restrict__ partial) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float scratch[64];
  pdl_launch_dependents();  // the finish kernel may take its place on the SMs; it waits for this grid to complete
  const int64_t HV = HxW / V, TV = N * HV, sample_stride = static_cast<int64_t>(C) * HxW;
  const int64_t total = static_cast<int64_t>(C) * TV;
  int64_t g0 = static_cast<int64_t>(blockIdx.x) * G;
  const int64_t g1 = g0 + G < total ? g0 + G : total;
  int64_t c = g0 / TV;
  while (g0 < g1) {
    const int64_t cbase = c * TV, cend = cbase + TV;
    const int64_t seg_end = g1 < cend ? g1 : cend;
    const T* xc = x + c * HxW;
    const float shift = bn_channel_shift<T>(xc, sample_stride, N);
    float s, q;
    bn_channel_sums<T>(xc, sample_stride, HV, g0 - cbase, seg_end - cbase, shift, s, q);
    block_sum2(s, q, scratch);
    if (threadIdx.x == 0) partial[c * max_slots + (static_cast<int64_t>(blockIdx.x) - cbase / G)] = make_float2(s, q);
    g0 = seg_end;
    ++c;
  }
}
// One CTA per channel: add the channel's partial sums in slot order (the same bits on every run) and finish.
template <typename T, typename RT>
__global__ void __launch_bounds__(512, 2)
batch_norm_stats_finish_kernel(const T* __restrict__ x, float* __restrict__ mean, float* __restrict__ second,
                               RT* __restrict__ running_mean, RT* __restrict__ running_var, int64_t N, int C, int64_t HxW,
                               float eps, float momentum, int mode, int64_t G, int max_slots, const float2* __restrict__ partial) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float scratch[64];
  const int c = blockIdx.x;
  const int64_t HV = HxW / V, TV = N * HV, sample_stride = static_cast<int64_t>(C) * HxW;
  const int64_t cbase = static_cast<int64_t>(c) * TV;
  const int nslots = static_cast<int>((cbase + TV - 1) / G - cbase / G) + 1;  // CTAs of the range kernel that touched channel c
  pdl_wait();  // launched as a programmatic dependent of the range kernel: its partial sums are complete from here on
  float s = 0.0f, q = 0.0f;
  for (int k = 0; k < nslots; ++k) {
    const float2 pk = partial[static_cast<int64_t>(c) * max_slots + k];
    s += pk.x;
    q += pk.y;
  }
  const T* xc = x + static_cast<int64_t>(c) * HxW;
  bn_channel_finish<T, RT>(xc, sample_stride, HV, TV, bn_channel_shift<T>(xc, sample_stride, N), s, q, static_cast<float>(N) * static_cast<float>(HxW),
                           mode, eps, momentum, c, mean, second, running_mean, running_var, scratch);
}

// The range kernel's grid: two CTAs per SM, each with at least 4096 vectors; 0: the tensor is too small to be worth it.
struct BnStatsPlan {
  int grid = 0;
  int64_t G = 0;
  int max_slots = 0;
  size_t bytes = 0;
};
inline BnStatsPlan bn_stats_plan(int64_t N, int64_t C, int64_t HxW, int vec, int sm_count) {
  BnStatsPlan p;
  const int64_t tv = N * (HxW / vec), total = C * tv;
  int64_t grid = 2ll * sm_count;
  if (grid > total / 4096) grid = total / 4096;
  if (grid < 2 || tv < 1) return p;
  p.G = (total + grid - 1) / grid;
  p.grid = static_cast<int>((total + p.G - 1) / p.G);
  p.max_slots = static_cast<int>((tv + p.G - 1) / p.G) + 1;
  p.bytes = static_cast<size_t>(C) * p.max_slots * sizeof(float2);
  return p;
}

// ---- group norm weight gradients over every SM (scratch memory) --------------------------------------------------
// The same cut as the BatchNorm statistics: the C * N * HxW / V vectors of all channels, laid end to end, in
// gridDim.x equal ranges.  For its part of a channel a CTA accumulates
//   sum over vectors of rstd[n, g] * sum_e dy_e * (x_e - mean[n, g])   and   sum dy
// (linear in the vectors, so parts simply add), statistics looked up per vector (a run's vectors share them: L1),
// and leaves the pair in partial[c][slot]; a second kernel adds a channel's parts in slot order.
template <typename T, typename ST>
__global__ void __launch_bounds__(512, 2)
group_norm_wgrad_range_kernel(const T* __restrict__ dy, const T* __restrict__ x, const ST* __restrict__ mean,
                              const ST* __restrict__ rstd, int64_t N, int C, int G, int64_t HxW, int64_t Gv, int max_slots,
                              float2* __restrict__ partial) {
  using P = Pack16<T>;
  constexpr int V = P::VEC, VH = V / 2;
  __shared__ float scratch[64];
  const int64_t HV = HxW / V, TV = N * HV, sample_stride = static_cast<int64_t>(C) * HxW;
  const int64_t total = static_cast<int64_t>(C) * TV;
  const int D = C / G;
  pdl_launch_dependents();
  int64_t g0 = static_cast<int64_t>(blockIdx.x) * Gv;
  const int64_t g1 = g0 + Gv < total ? g0 + Gv : total;
  int64_t c = g0 / TV;
  const int64_t stride = blockDim.x, step_n = stride / HV;
  const int hv = static_cast<int>(HV), step_j32 = static_cast<int>(stride % HV);  // (a run has fewer than 2^31 vectors)
  const int64_t d_stride = step_n * sample_stride + static_cast<int64_t>(step_j32) * V, d_wrap = sample_stride - HV * V;
  while (g0 < g1) {
    const int64_t cbase = c * TV, cend = cbase + TV;
    const int64_t seg_end = g1 < cend ? g1 : cend;
    const int64_t coff = c * HxW;
    const int grp = static_cast<int>(c) / D;
    float sg = 0.0f, sb = 0.0f;
    auto add_vec = [&](const uint4& wx, const uint4& wd, int64_t n) {
      const float mu = to_acc<float>(mean[n * G + grp]), rs = to_acc<float>(rstd[n * G + grp]);
      float2 xv[VH], dv[VH];
      P::unpack2(wx, xv);
      P::unpack2(wd, dv);
      const float2 nmu = make_float2(-mu, -mu);
      float2 a = make_float2(0.0f, 0.0f), b = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int e = 0; e < VH; ++e) {
        a = fma2(dv[e], add2(xv[e], nmu), a);
        b = add2(b, dv[e]);
      }
      sg = fmaf(a.x + a.y, rs, sg);
      sb += b.x + b.y;
    };
    // the thread carries its element offset, its sample and its vector index inside the run: a stride adds constants,
    // a wrap into the next sample's run another one — no 64-bit multiply per vector
    const int64_t end = seg_end - cbase;
    int64_t idx = g0 - cbase + threadIdx.x;
    int64_t n = idx / HV;
    int j = static_cast<int>(idx - n * HV);
    int64_t off = coff + n * sample_stride + static_cast<int64_t>(j) * V;
    auto advance = [&]() {
      n += step_n;
      j += step_j32;
      off += d_stride;
      if (j >= hv) { j -= hv; ++n; off += d_wrap; }
    };
    for (; idx + 3 * stride < end; idx += 4 * stride) {  // four vector pairs in flight per thread
      int64_t offs[4], ns[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        offs[u] = off;
        ns[u] = n;
        advance();
      }
      uint4 wx[4], wd[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        wx[u] = __ldg(reinterpret_cast<const uint4*>(x + offs[u]));
        wd[u] = __ldg(reinterpret_cast<const uint4*>(dy + offs[u]));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) add_vec(wx[u], wd[u], ns[u]);
    }
    for (; idx < end; idx += stride) {
      add_vec(__ldg(reinterpret_cast<const uint4*>(x + off)), __ldg(reinterpret_cast<const uint4*>(dy + off)), n);
      advance();
    }
    block_sum2(sg, sb, scratch);
    if (threadIdx.x == 0) partial[c * max_slots + (static_cast<int64_t>(blockIdx.x) - cbase / Gv)] = make_float2(sg, sb);
    g0 = seg_end;
    ++c;
  }
}
// One thread per channel: the channel's parts in slot order (the same bits on every run).
template <typename WT>
__global__ void group_norm_wgrad_finish_kernel(const float2* __restrict__ partial, WT* __restrict__ dgamma, WT* __restrict__ dbeta,
                                               int C, int64_t TV, int64_t Gv, int max_slots) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();  // a programmatic dependent of the range kernel
  if (c >= C) return;
  const int64_t cbase = static_cast<int64_t>(c) * TV;
  const int nslots = static_cast<int>((cbase + TV - 1) / Gv - cbase / Gv) + 1;
  float sg = 0.0f, sb = 0.0f;
  for (int k = 0; k < nslots; ++k) {
    const float2 pk = partial[static_cast<int64_t>(c) * max_slots + k];
    sg += pk.x;
    sb += pk.y;
  }
  if (dgamma) dgamma[c] = from_acc<WT>(sg);
  if (dbeta) dbeta[c] = from_acc<WT>(sb);
}

template <typename T, typename WT, typename ST, int GROUP, bool FULL = false>
int group_norm_ring_launch(const RingPlan& p, const T* x, const WT* gamma, const WT* beta, T* y, ST* mean, ST* rstd,
                           int64_t rows, int64_t L, int64_t G, int64_t D, int64_t HxW, double eps, cudaStream_t st) {
  constexpr int VPT = 16 / Pack16<T>::VEC;
  if constexpr (!FULL) {
    if (L == static_cast<int64_t>(GROUP) * 16)  // the row fills every thread's vectors: the instantiation without range checks
      return group_norm_ring_launch<T, WT, ST, GROUP, true>(p, x, gamma, beta, y, mean, rstd, rows, L, G, D, HxW, eps, st);
  }
  auto kernel = group_norm_fwd_ring_kernel<T, WT, ST, GROUP, VPT, FULL>;
  static std::atomic<uint64_t> done{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda(cudaGetLastError());
  const uint64_t bit = 1ull << (dev & 63);
  if (!(done.load(std::memory_order_acquire) & bit)) {
    if (int e = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, device_info().max_smem_optin)))
      return e;
    done.fetch_or(bit, std::memory_order_release);
  }
  ProfileScope prof("group_norm_fwd_ring", st);
  return launch_pdl(kernel, dim3(p.grid), dim3(kRingBlock), p.smem, st, x, gamma, beta, y, mean, rstd, rows, static_cast<int>(L),
                    static_cast<int>(G), static_cast<int>(D), static_cast<int>(HxW), static_cast<float>(eps),
                    p.stages | (p.lag << 8), p.rpg, device_status_ptr(), next_tile_counter());
}

template <typename T, typename WT, typename ST>
int group_norm_launch(const void* x, const void* gamma, const void* beta, void* y, void* mean, void* rstd, int64_t N, int64_t C,
                      int64_t HxW, int64_t G, double eps, cudaStream_t st) {
  const int64_t rows = N * G, D = C / G, L = D * HxW;
  constexpr int V = 16 / sizeof(T);
  if (forced_path() != B2N_PATH_GENERIC && is_aligned(x, 16) && is_aligned(y, 16) && HxW % V == 0 && rows < 0x7fffffffLL) {
    // a group's row on the shared-memory ring, like a layer-norm row of the same length
    const DeviceInfo& di = device_info();
    const RingPlan p = plan_ring(rows, L, sizeof(T), 1, 16, persistent_ctas(di.sm_count), di.max_smem_optin, 65536);
    if (p.ok) {
      note_path("ring");
      const T* xp = static_cast<const T*>(x);
      const WT* g = static_cast<const WT*>(gamma);
      const WT* b = static_cast<const WT*>(beta);
      T* yp = static_cast<T*>(y);
      ST* mp = static_cast<ST*>(mean);
      ST* rp = static_cast<ST*>(rstd);
      switch (p.group) {
        case 32: return group_norm_ring_launch<T, WT, ST, 32>(p, xp, g, b, yp, mp, rp, rows, L, G, D, HxW, eps, st);
        case 64: return group_norm_ring_launch<T, WT, ST, 64>(p, xp, g, b, yp, mp, rp, rows, L, G, D, HxW, eps, st);
        case 128: return group_norm_ring_launch<T, WT, ST, 128>(p, xp, g, b, yp, mp, rp, rows, L, G, D, HxW, eps, st);
        case 256: return group_norm_ring_launch<T, WT, ST, 256>(p, xp, g, b, yp, mp, rp, rows, L, G, D, HxW, eps, st);
        default: return group_norm_ring_launch<T, WT, ST, 512>(p, xp, g, b, yp, mp, rp, rows, L, G, D, HxW, eps, st);
      }
    }
  }
  if (forced_path() == B2N_PATH_RING) return B2N_ERR_BAD_ARG;
  note_path("generic");
  const bool vec = L % V == 0 && is_aligned(x, 16) && is_aligned(y, 16);
  const int threads = L >= 8192 ? 512 : (L >= 2048 ? 256 : 128);
  const int64_t cap = static_cast<int64_t>(device_info().sm_count) * (2048 / threads);
  const int grid = static_cast<int>(rows < cap ? rows : cap);
  ProfileScope prof("group_norm_fwd", st);
  const T* xp = static_cast<const T*>(x);
  const WT* g = static_cast<const WT*>(gamma);
  const WT* b = static_cast<const WT*>(beta);
  if (vec)
    group_norm_fwd_kernel<T, WT, ST, V><<<grid, threads, 0, st>>>(xp, g, b, static_cast<T*>(y), static_cast<ST*>(mean),
                                                                 static_cast<ST*>(rstd), rows, static_cast<int>(G),
                                                                 static_cast<int>(D), static_cast<int>(HxW), static_cast<float>(eps));
  else
    group_norm_fwd_kernel<T, WT, ST, 1><<<grid, threads, 0, st>>>(xp, g, b, static_cast<T*>(y), static_cast<ST*>(mean),
                                                                 static_cast<ST*>(rstd), rows, static_cast<int>(G),
                                                                 static_cast<int>(D), static_cast<int>(HxW), static_cast<float>(eps));
  return launched();
}

template <typename T, typename WT, typename ST, int GROUP, bool FULL = false>
int group_norm_bwd_ring_launch(const RingPlan& p, const T* dy, const T* x, const ST* mean, const ST* rstd, const WT* gamma, T* dx,
                               int64_t rows, int64_t L, int64_t G, int64_t D, int64_t HxW, cudaStream_t st) {
  constexpr int VPT = 16 / Pack16<T>::VEC;
  if constexpr (!FULL) {
    if (L == static_cast<int64_t>(GROUP) * 16)
      return group_norm_bwd_ring_launch<T, WT, ST, GROUP, true>(p, dy, x, mean, rstd, gamma, dx, rows, L, G, D, HxW, st);
  }
  auto kernel = group_norm_bwd_ring_kernel<T, WT, ST, GROUP, VPT, FULL>;
  static std::atomic<uint64_t> done{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda(cudaGetLastError());
  const uint64_t bit = 1ull << (dev & 63);
  if (!(done.load(std::memory_order_acquire) & bit)) {
    if (int e = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, device_info().max_smem_optin)))
      return e;
    done.fetch_or(bit, std::memory_order_release);
  }
  return launch_pdl(kernel, dim3(p.grid), dim3(kRingBlock), p.smem, st, dy, x, mean, rstd, gamma, dx, rows, static_cast<int>(L),
                    static_cast<int>(G), static_cast<int>(D), static_cast<int>(HxW), p.stages | (p.lag << 8), p.rpg,
                    device_status_ptr(), next_tile_counter());
}

template <typename T, typename WT, typename ST>
int group_norm_bwd_launch(const void* dy, const void* x, const void* mean, const void* rstd, const void* gamma, void* dx,
                          void* dgamma, void* dbeta, int64_t N, int64_t C, int64_t HxW, int64_t G, void* workspace,
                          size_t workspace_bytes, cudaStream_t st) {
  const int64_t rows = N * G, D = C / G, L = D * HxW;
  constexpr int V = 16 / sizeof(T);
  const bool vec = HxW % V == 0 && is_aligned(x, 16) && is_aligned(dy, 16) && (dx == nullptr || is_aligned(dx, 16));
  const T* gp = static_cast<const T*>(dy);
  const T* xp = static_cast<const T*>(x);
  const ST* mp = static_cast<const ST*>(mean);
  const ST* rp = static_cast<const ST*>(rstd);
  ProfileScope prof("group_norm_bwd", st);
  bool dx_done = dx == nullptr;
  if (!dx_done && forced_path() != B2N_PATH_GENERIC && vec && rows < 0x7fffffffLL) {
    // dX on the shared-memory ring, like a layer-norm backward row of the same length
    const DeviceInfo& di = device_info();
    const RingPlan p = plan_ring(rows, L, sizeof(T), 2, 16, persistent_ctas(di.sm_count), di.max_smem_optin);
    if (p.ok) {
      note_path("ring");
      const WT* wp = static_cast<const WT*>(gamma);
      T* dp = static_cast<T*>(dx);
      int e;
      switch (p.group) {
        case 32: e = group_norm_bwd_ring_launch<T, WT, ST, 32>(p, gp, xp, mp, rp, wp, dp, rows, L, G, D, HxW, st); break;
        case 64: e = group_norm_bwd_ring_launch<T, WT, ST, 64>(p, gp, xp, mp, rp, wp, dp, rows, L, G, D, HxW, st); break;
        case 128: e = group_norm_bwd_ring_launch<T, WT, ST, 128>(p, gp, xp, mp, rp, wp, dp, rows, L, G, D, HxW, st); break;
        case 256: e = group_norm_bwd_ring_launch<T, WT, ST, 256>(p, gp, xp, mp, rp, wp, dp, rows, L, G, D, HxW, st); break;
        default: e = group_norm_bwd_ring_launch<T, WT, ST, 512>(p, gp, xp, mp, rp, wp, dp, rows, L, G, D, HxW, st); break;
      }
      if (e) return e;
      dx_done = true;
    }
  }
  if (!dx_done && forced_path() == B2N_PATH_RING) return B2N_ERR_BAD_ARG;
  if (!dx_done) {
    note_path("generic");
    const int threads = L >= 8192 ? 512 : (L >= 2048 ? 256 : 128);
    const int64_t cap = static_cast<int64_t>(device_info().sm_count) * (2048 / threads);
    const int grid = static_cast<int>(rows < cap ? rows : cap);
    const WT* wp = static_cast<const WT*>(gamma);
    if (vec)
      group_norm_bwd_dx_kernel<T, WT, ST, V><<<grid, threads, 0, st>>>(gp, xp, mp, rp, wp, static_cast<T*>(dx), rows,
                                                                       static_cast<int>(G), static_cast<int>(D), static_cast<int>(HxW));
    else
      group_norm_bwd_dx_kernel<T, WT, ST, 1><<<grid, threads, 0, st>>>(gp, xp, mp, rp, wp, static_cast<T*>(dx), rows,
                                                                       static_cast<int>(G), static_cast<int>(D), static_cast<int>(HxW));
    if (int e = launched()) return e;
  }
  if ((dgamma != nullptr || dbeta != nullptr) && vec && forced_path() != B2N_PATH_GENERIC) {
    // with scratch memory: one balanced wave of CTAs over all channels, then a fixed-order finish
    const BnStatsPlan p = bn_stats_plan(N, C, HxW, V, device_info().sm_count);
    if (p.grid > 0 && workspace != nullptr && workspace_bytes >= p.bytes && is_aligned(workspace, 8)) {
      float2* partial = static_cast<float2*>(workspace);
      group_norm_wgrad_range_kernel<T, ST><<<static_cast<unsigned>(p.grid), 512, 0, st>>>(
          gp, xp, mp, rp, N, static_cast<int>(C), static_cast<int>(G), HxW, p.G, p.max_slots, partial);
      if (int e = launched()) return e;
      return launch_pdl(group_norm_wgrad_finish_kernel<WT>, dim3(static_cast<unsigned>((C + 255) / 256)), dim3(256), 0, st,
                        static_cast<const float2*>(partial), static_cast<WT*>(dgamma), static_cast<WT*>(dbeta), static_cast<int>(C),
                        N * (HxW / V), p.G, p.max_slots);
    }
  }
  if (dgamma != nullptr || dbeta != nullptr) {
    const int threads = N * HxW >= 16384 ? 512 : 128;
    if (vec)
      group_norm_bwd_wgrad_kernel<T, WT, ST, V><<<static_cast<unsigned>(C), threads, 0, st>>>(
          gp, xp, mp, rp, static_cast<WT*>(dgamma), static_cast<WT*>(dbeta), N, static_cast<int>(C), static_cast<int>(G),
          static_cast<int>(HxW));
    else
      group_norm_bwd_wgrad_kernel<T, WT, ST, 1><<<static_cast<unsigned>(C), threads, 0, st>>>(
          gp, xp, mp, rp, static_cast<WT*>(dgamma), static_cast<WT*>(dbeta), N, static_cast<int>(C), static_cast<int>(G),
          static_cast<int>(HxW));
    if (int e = launched()) return e;
  }
  return B2N_OK;
}

template <typename T, typename RT>
int batch_norm_stats_launch(const void* x, float* mean, float* second, void* running_mean, void* running_var, int64_t N,
                            int64_t C, int64_t HxW, double eps, double momentum, int mode, void* workspace,
                            size_t workspace_bytes, cudaStream_t st) {
  ProfileScope prof("batch_norm_stats", st);
  const T* xp = static_cast<const T*>(x);
  RT* rm = static_cast<RT*>(running_mean);
  RT* rv = static_cast<RT*>(running_var);
  constexpr int V = 16 / sizeof(T);
  if (HxW % V == 0 && is_aligned(x, 16) && C <= 0x7fffffffLL) {
    const BnStatsPlan p = bn_stats_plan(N, C, HxW, V, device_info().sm_count);
    // with fewer CTAs than one per channel would give, or without scratch, one CTA per channel
    if (p.grid > 0 && workspace != nullptr && workspace_bytes >= p.bytes && is_aligned(workspace, 8)) {
      float2* partial = static_cast<float2*>(workspace);
      batch_norm_stats_range_kernel<T><<<static_cast<unsigned>(p.grid), 512, 0, st>>>(xp, N, static_cast<int>(C), HxW, p.G,
                                                                                    p.max_slots, partial);
      if (int e = launched()) return e;
      return launch_pdl(batch_norm_stats_finish_kernel<T, RT>, dim3(static_cast<unsigned>(C)), dim3(512), 0, st, xp, mean, second,
                        rm, rv, N, static_cast<int>(C), HxW, static_cast<float>(eps), static_cast<float>(momentum), mode, p.G,
                        p.max_slots, static_cast<const float2*>(partial));
    }
    batch_norm_stats_channel_kernel<T, RT><<<static_cast<unsigned>(C), 512, 0, st>>>(
        xp, mean, second, rm, rv, N, static_cast<int>(C), HxW, static_cast<float>(eps), static_cast<float>(momentum), mode);
    return launched();
  }
  if (HxW >= 16) {
    const int threads = N * HxW >= 16384 ? 512 : 128;
    batch_norm_stats_spatial_kernel<T, RT><<<static_cast<unsigned>(C), threads, 0, st>>>(
        xp, mean, second, rm, rv, N, static_cast<int>(C), HxW, static_cast<float>(eps), static_cast<float>(momentum), mode);
  } else {
    batch_norm_stats_flat_kernel<T, RT><<<static_cast<unsigned>((C + 31) / 32), dim3(32, 32), 0, st>>>(
        xp, mean, second, rm, rv, N, static_cast<int>(C), HxW, static_cast<float>(eps), static_cast<float>(momentum), mode);
  }
  return launched();
}

}  // namespace
}  // namespace b2n

using namespace b2n;

extern "C" {

int b2n_group_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, void* mean, void* rstd, int64_t N,
                       int64_t C, int64_t HxW, int64_t G, double eps, int x_dtype, int w_dtype, int stat_dtype, void* stream) {
  if (N < 0 || C < 0 || HxW < 0 || G < 1 || C % G != 0) return B2N_ERR_BAD_ARG;
  if (N == 0 || C == 0 || HxW == 0) return B2N_OK;
  if (!x || !y || !mean || !rstd) return B2N_ERR_BAD_ARG;
  if ((C / G) * HxW > 0x7fffffffLL || C > 0x7fffffffLL) return B2N_ERR_TOO_LARGE;
  if (!device_ready()) return B2N_ERR_CUDA;
  if (gamma == nullptr && beta == nullptr) w_dtype = x_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define B2N_GN(T, WT, ST) return group_norm_launch<T, WT, ST>(x, gamma, beta, y, mean, rstd, N, C, HxW, G, eps, st)
  if (x_dtype == B2N_F32 && w_dtype == B2N_F32 && stat_dtype == B2N_F32) B2N_GN(float, float, float);
  if (x_dtype == B2N_BF16 && w_dtype == B2N_BF16 && stat_dtype == B2N_BF16) B2N_GN(bf16, bf16, bf16);
  if (x_dtype == B2N_BF16 && w_dtype == B2N_F32 && stat_dtype == B2N_F32) B2N_GN(bf16, float, float);
  if (x_dtype == B2N_F16 && w_dtype == B2N_F16 && stat_dtype == B2N_F16) B2N_GN(f16, f16, f16);
  if (x_dtype == B2N_F16 && w_dtype == B2N_F32 && stat_dtype == B2N_F32) B2N_GN(f16, float, float);
#undef B2N_GN
  return B2N_ERR_UNSUPPORTED_DTYPE;
}

size_t b2n_group_norm_bwd_workspace_bytes(int64_t N, int64_t C, int64_t HxW, int x_dtype) {
  return b2n_batch_norm_stats_workspace_bytes(N, C, HxW, x_dtype);  // the same cut of the same layout
}

int b2n_group_norm_bwd(const void* dy, const void* x, const void* mean, const void* rstd, const void* gamma, void* dx,
                       void* dgamma, void* dbeta, int64_t N, int64_t C, int64_t HxW, int64_t G, int x_dtype, int w_dtype,
                       int stat_dtype, void* stream) {
  return b2n_group_norm_bwd_ws(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, N, C, HxW, G, x_dtype, w_dtype, stat_dtype, nullptr, 0,
                               stream);
}

int b2n_group_norm_bwd_ws(const void* dy, const void* x, const void* mean, const void* rstd, const void* gamma, void* dx,
                          void* dgamma, void* dbeta, int64_t N, int64_t C, int64_t HxW, int64_t G, int x_dtype, int w_dtype,
                          int stat_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  if (N < 0 || C < 0 || HxW < 0 || G < 1 || C % G != 0) return B2N_ERR_BAD_ARG;
  if (C == 0) return B2N_OK;
  if (!dy || !x || !mean || !rstd) return (N == 0 || HxW == 0) && !dx ? B2N_OK : B2N_ERR_BAD_ARG;
  if ((C / G) * HxW > 0x7fffffffLL || C > 0x7fffffffLL || HxW > 0x7fffffffLL) return B2N_ERR_TOO_LARGE;
  if (!device_ready()) return B2N_ERR_CUDA;
  if (gamma == nullptr && dgamma == nullptr && dbeta == nullptr) w_dtype = x_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define B2N_GNB(T, WT, ST) \
  return group_norm_bwd_launch<T, WT, ST>(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, N, C, HxW, G, workspace, workspace_bytes, st)
  if (x_dtype == B2N_F32 && w_dtype == B2N_F32 && stat_dtype == B2N_F32) B2N_GNB(float, float, float);
  if (x_dtype == B2N_BF16 && w_dtype == B2N_BF16 && stat_dtype == B2N_BF16) B2N_GNB(bf16, bf16, bf16);
  if (x_dtype == B2N_BF16 && w_dtype == B2N_F32 && stat_dtype == B2N_F32) B2N_GNB(bf16, float, float);
  if (x_dtype == B2N_F16 && w_dtype == B2N_F16 && stat_dtype == B2N_F16) B2N_GNB(f16, f16, f16);
  if (x_dtype == B2N_F16 && w_dtype == B2N_F32 && stat_dtype == B2N_F32) B2N_GNB(f16, float, float);
#undef B2N_GNB
  return B2N_ERR_UNSUPPORTED_DTYPE;
}

size_t b2n_batch_norm_stats_workspace_bytes(int64_t N, int64_t C, int64_t HxW, int x_dtype) {
  const int es = x_dtype == B2N_F32 ? 4 : (x_dtype == B2N_BF16 || x_dtype == B2N_F16) ? 2 : 0;
  if (es == 0 || N < 1 || C < 1 || HxW < 1 || C > 0x7fffffffLL) return 0;
  const int vec = 16 / es;
  if (HxW % vec != 0 || !device_ready()) return 0;
  return bn_stats_plan(N, C, HxW, vec, device_info().sm_count).bytes;
}

int b2n_batch_norm_stats(const void* x, float* mean, float* second, void* running_mean, void* running_var, int64_t N,
                         int64_t C, int64_t HxW, double eps, double momentum, int mode, int x_dtype, int running_dtype,
                         void* stream) {
  return b2n_batch_norm_stats_ws(x, mean, second, running_mean, running_var, N, C, HxW, eps, momentum, mode, x_dtype,
                                 running_dtype, nullptr, 0, stream);
}

int b2n_batch_norm_stats_ws(const void* x, float* mean, float* second, void* running_mean, void* running_var, int64_t N,
                            int64_t C, int64_t HxW, double eps, double momentum, int mode, int x_dtype, int running_dtype,
                            void* workspace, size_t workspace_bytes, void* stream) {
  if (N < 0 || C < 0 || HxW < 0 || mode < 0 || mode > 1) return B2N_ERR_BAD_ARG;
  if (C == 0) return B2N_OK;
  if (N == 0 || HxW == 0) return B2N_ERR_BAD_ARG;  // statistics of nothing
  if (!x || !mean || !second) return B2N_ERR_BAD_ARG;
  if (C > 0x7fffffffLL) return B2N_ERR_TOO_LARGE;
  if (!device_ready()) return B2N_ERR_CUDA;
  if (running_mean == nullptr && running_var == nullptr) running_dtype = B2N_F32;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define B2N_BN(T, RT) \
  return batch_norm_stats_launch<T, RT>(x, mean, second, running_mean, running_var, N, C, HxW, eps, momentum, mode, workspace, \
                                        workspace_bytes, st)
  if (x_dtype == B2N_F32 && running_dtype == B2N_F32) B2N_BN(float, float);
  if (x_dtype == B2N_BF16 && running_dtype == B2N_F32) B2N_BN(bf16, float);
  if (x_dtype == B2N_BF16 && running_dtype == B2N_BF16) B2N_BN(bf16, bf16);
  if (x_dtype == B2N_F16 && running_dtype == B2N_F32) B2N_BN(f16, float);
  if (x_dtype == B2N_F16 && running_dtype == B2N_F16) B2N_BN(f16, f16);
#undef B2N_BN
  return B2N_ERR_UNSUPPORTED_DTYPE;
}

}  // extern "C"
