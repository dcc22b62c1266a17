// Generic layer-norm / RMS-norm kernels: any N, any alignment, fp32 / fp16 / bf16 / fp64.
// Rows are re-read from global memory (L1/L2) instead of being held on chip; these are the
// kernels behind shapes the ring kernels do not take.
//
// Arithmetic follows at::native::xpu::layer_norm_kernel_impl and layer_norm_backward_kernel_impl
// (src/ATen/native/xpu/sycl/LayerNormKernels.cpp:648-699, :1117-1416) with two deliberate
// differences: the variance is a two-pass sum of (x-mean)^2 in the accumulate type (taken relative
// to the row's first element) instead of Welford updates, and no intermediate product is rounded
// to the storage type.
#pragma once
#include "common.cuh"

namespace b2n {

// TPR: threads per row (32 = one warp per row, several rows per CTA; 0 = the whole CTA).
// V: elements per vector access (1, or 16 bytes / sizeof(T) when everything is aligned).
template <typename T, typename WT, bool RMS, int TPR, int V>
__global__ void norm_fwd_generic_kernel(const T* __restrict__ x, const WT* __restrict__ gamma,
                                        const WT* __restrict__ beta, T* __restrict__ y,
                                        acc_t<T>* __restrict__ mean, acc_t<T>* __restrict__ rstd,
                                        int64_t M, int64_t N, acc_t<T> eps) {
  using A = acc_t<T>;
  __shared__ A scratch[32];
  const int tpr = TPR == 32 ? 32 : static_cast<int>(blockDim.x);
  const int rpb = TPR == 32 ? static_cast<int>(blockDim.x) / 32 : 1;
  const int sub = TPR == 32 ? static_cast<int>(threadIdx.x) / 32 : 0;
  const int lane = TPR == 32 ? static_cast<int>(threadIdx.x) % 32 : static_cast<int>(threadIdx.x);
  const int64_t nv = N / V;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rpb; row0 < M; row0 += static_cast<int64_t>(gridDim.x) * rpb) {
    const int64_t row = row0 + sub;
    if (row >= M) continue;  // only possible with TPR == 32 (no CTA-wide barrier below in that case)
    const T* xr = x + row * N;
    T* yr = y + row * N;
    // Layer norm sums are taken relative to the row's first element: a large common offset
    // (say 1e15 + small) then cancels exactly instead of being rounded away in the row sum.
    const A shift = RMS ? A(0) : to_acc<A>(xr[0]);
    A s = 0;
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> p = ld_vec<T, V>(xr + v * V);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const A a = to_acc<A>(p.v[e]) - shift;
        s += RMS ? a * a : a;
      }
    }
    s = row_reduce<TPR>(s, scratch, SumOp());
    A mu = 0, mu_d = 0, rs;
    if constexpr (RMS) {
      rs = acc_rsqrt(s / static_cast<A>(N) + eps);
    } else {
      mu_d = s / static_cast<A>(N);  // mean of (x - shift)
      mu = shift + mu_d;
      A q = 0;
      for (int64_t v = lane; v < nv; v += tpr) {
        const Vec<T, V> p = ld_vec<T, V>(xr + v * V);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const A d = (to_acc<A>(p.v[e]) - shift) - mu_d;
          q += d * d;
        }
      }
      q = row_reduce<TPR>(q, scratch, SumOp());
      rs = acc_rsqrt(q / static_cast<A>(N) + eps);
    }
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> p = ld_vec<T, V>(xr + v * V);
      Vec<T, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const int64_t j = v * V + e;
        A t = ((to_acc<A>(p.v[e]) - shift) - mu_d) * rs;
        if (gamma) t *= to_acc<A>(gamma[j]);
        if (!RMS && beta) t += to_acc<A>(beta[j]);
        o.v[e] = from_acc<T>(t);
      }
      st_vec<T, V>(yr + v * V, o);
    }
    if (lane == 0) {
      if (!RMS && mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
  }
}

// dx = rstd * (gamma*dy - (xhat*s2 + s1)/N), s1 = sum(gamma*dy), s2 = sum(gamma*dy*xhat),
// xhat = (x-mean)*rstd.  RMS: mean = 0 and s1 = 0.
template <typename T, typename WT, bool RMS, int TPR, int V>
__global__ void norm_bwd_dx_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                           const acc_t<T>* __restrict__ mean,
                                           const acc_t<T>* __restrict__ rstd,
                                           const WT* __restrict__ gamma, T* __restrict__ dx, int64_t M,
                                           int64_t N) {
  using A = acc_t<T>;
  __shared__ A scratch[32];
  const int tpr = TPR == 32 ? 32 : static_cast<int>(blockDim.x);
  const int rpb = TPR == 32 ? static_cast<int>(blockDim.x) / 32 : 1;
  const int sub = TPR == 32 ? static_cast<int>(threadIdx.x) / 32 : 0;
  const int lane = TPR == 32 ? static_cast<int>(threadIdx.x) % 32 : static_cast<int>(threadIdx.x);
  const int64_t nv = N / V;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rpb; row0 < M; row0 += static_cast<int64_t>(gridDim.x) * rpb) {
    const int64_t row = row0 + sub;
    if (row >= M) continue;
    const T* dyr = dy + row * N;
    const T* xr = x + row * N;
    T* dxr = dx + row * N;
    const A mu = RMS ? A(0) : mean[row];
    const A rs = rstd[row];
    A s1 = 0, s2 = 0;
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> pd = ld_vec<T, V>(dyr + v * V);
      const Vec<T, V> px = ld_vec<T, V>(xr + v * V);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        A g = to_acc<A>(pd.v[e]);
        if (gamma) g *= to_acc<A>(gamma[v * V + e]);
        const A xh = (to_acc<A>(px.v[e]) - mu) * rs;
        s1 += g;
        s2 += g * xh;
      }
    }
    s2 = row_reduce<TPR>(s2, scratch, SumOp());
    if constexpr (!RMS) s1 = row_reduce<TPR>(s1, scratch, SumOp()); else s1 = 0;
    const A inv_n = A(1) / static_cast<A>(N);
    const A a = s2 * inv_n, b = s1 * inv_n;
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> pd = ld_vec<T, V>(dyr + v * V);
      const Vec<T, V> px = ld_vec<T, V>(xr + v * V);
      Vec<T, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        A g = to_acc<A>(pd.v[e]);
        if (gamma) g *= to_acc<A>(gamma[v * V + e]);
        const A xh = (to_acc<A>(px.v[e]) - mu) * rs;
        o.v[e] = from_acc<T>(rs * (g - (xh * a + b)));
      }
      st_vec<T, V>(dxr + v * V, o);
    }
  }
}

// Weight-gradient partial sums.  CTA = 32 columns x 8 row lanes; CTA (bx, by) owns columns
// [32*bx, 32*bx+32) and the rows of chunk by.  ws layout: [chunk][2][N] in the accumulate type,
// plane 0 = dgamma partial, plane 1 = dbeta partial.
template <typename T, bool RMS>
__global__ void norm_bwd_wgrad_partial_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                              const acc_t<T>* __restrict__ mean,
                                              const acc_t<T>* __restrict__ rstd,
                                              acc_t<T>* __restrict__ ws, int64_t M, int64_t N,
                                              int64_t rows_per_chunk) {
  using A = acc_t<T>;
  __shared__ A sg[8][33], sb[8][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * 32 + tx;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
  const int64_t r1 = (r0 + rows_per_chunk < M) ? r0 + rows_per_chunk : M;
  A dg = 0, db = 0;
  if (col < N) {
    for (int64_t r = r0 + ty; r < r1; r += 8) {
      const A d = to_acc<A>(dy[r * N + col]);
      const A mu = RMS ? A(0) : mean[r];
      const A xh = (to_acc<A>(x[r * N + col]) - mu) * rstd[r];
      dg += d * xh;
      db += d;
    }
  }
  sg[ty][tx] = dg;
  sb[ty][tx] = db;
  __syncthreads();
  if (ty == 0 && col < N) {
    A g = sg[0][tx], b = sb[0][tx];
#pragma unroll
    for (int k = 1; k < 8; ++k) { g += sg[k][tx]; b += sb[k][tx]; }
    ws[(static_cast<int64_t>(blockIdx.y) * 2 + 0) * N + col] = g;
    ws[(static_cast<int64_t>(blockIdx.y) * 2 + 1) * N + col] = b;
  }
}

// Folds P partial rows [P][2][N] into dgamma (plane 0) and dbeta (plane 1) in a fixed order, so
// the result does not depend on scheduling.  blockIdx.y selects the plane.  A CTA is 32 columns x
// kFoldLanes row lanes: lane ty sums rows ty, ty + kFoldLanes, ... (a few independent loads each, so
// the kernel is not a chain of dependent loads), then the lanes' sums are added in lane order.
constexpr int kFoldLanes = 32;
template <typename A, typename WT>
__global__ void __launch_bounds__(32 * kFoldLanes)
norm_bwd_wgrad_fold_kernel(const A* __restrict__ ws, WT* __restrict__ dgamma, WT* __restrict__ dbeta, int64_t P,
                           int64_t N) {
  __shared__ A sm[kFoldLanes][33];
  pdl_launch_dependents();  // see common.cuh: no-ops unless launched with launch_pdl
  pdl_wait();
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int plane = blockIdx.y;
  WT* out = plane == 0 ? dgamma : dbeta;
  if (out == nullptr) return;  // uniform for the CTA
  const int64_t col = static_cast<int64_t>(blockIdx.x) * 32 + tx;
  A s = 0;
  if (col < N) {
#pragma unroll 4
    for (int64_t p = ty; p < P; p += kFoldLanes) s += ws[(p * 2 + plane) * N + col];
  }
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < N) {
    A r = sm[0][tx];
#pragma unroll
    for (int k = 1; k < kFoldLanes; ++k) r += sm[k][tx];
    out[col] = from_acc<WT>(r);
  }
}

}  // namespace b2n
