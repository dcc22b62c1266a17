// Generic softmax / log-softmax kernels: any N, any alignment, any softmax dim, fp32 / fp16 / bf16 /
// fp64, optional 16-bit -> fp32 output ("half_to_float").
//
// Semantics follow at::native::xpu::host_softmax / host_softmax_backward
// (src/ATen/native/xpu/sycl/SoftMaxKernels.cpp:2125-2240) and the CPU ATen kernels they are tested
// against: -inf entries give exactly 0 (softmax) / -inf (log-softmax); a row that is all -inf, or
// that holds +inf or NaN, comes out as NaN.
#pragma once
#include "common.cuh"

namespace b2n {

template <typename A> __device__ __forceinline__ A acc_nan();
template <> __device__ __forceinline__ float acc_nan<float>() { return __int_as_float(0x7fc00000); }
template <> __device__ __forceinline__ double acc_nan<double>() { return __longlong_as_double(0x7ff8000000000000LL); }

// running (max, sum of exp(x - max)) pair
template <typename A> struct MaxSum {
  A m, s;
  __device__ __forceinline__ void init() { m = acc_neg_inf<A>(); s = 0; }
  __device__ __forceinline__ void add(A x) {
    if (x > m) {
      s = s * acc_exp(m - x) + A(1);  // m == -inf: exp(-inf) == 0 and s == 0
      m = x;
    } else if (!(x == acc_neg_inf<A>())) {
      s += acc_exp(x - m);  // NaN propagates through here
    }
  }
  __device__ __forceinline__ void merge(const MaxSum& o) {
    const A nm = acc_max(m, o.m);
    const A a = (m == acc_neg_inf<A>()) ? A(0) : s * acc_exp(m - nm);
    const A b = (o.m == acc_neg_inf<A>()) ? A(0) : o.s * acc_exp(o.m - nm);
    // NaN sums must survive a -inf max on the same side
    s = ((m == acc_neg_inf<A>() && s != s) || (o.m == acc_neg_inf<A>() && o.s != o.s)) ? acc_nan<A>() : a + b;
    m = nm;
  }
};

template <typename A> __device__ __forceinline__ MaxSum<A> warp_merge(MaxSum<A> v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum<A> t;
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v.merge(t);
  }
  return v;
}

template <int TPR, typename A> __device__ __forceinline__ MaxSum<A> row_merge(MaxSum<A> v, A* scratch /*64*/) {
  v = warp_merge(v);
  if constexpr (TPR == 32) {
    return v;
  } else {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) { scratch[2 * w] = v.m; scratch[2 * w + 1] = v.s; }
    __syncthreads();
    MaxSum<A> r;
    r.m = scratch[0]; r.s = scratch[1];
    for (int i = 1; i < nw; ++i) {
      MaxSum<A> t;
      t.m = scratch[2 * i]; t.s = scratch[2 * i + 1];
      r.merge(t);
    }
    return r;
  }
}

// Softmax over the last dim.  Pass 1 streams the row once keeping a running (max, sum); pass 2
// re-reads it (L1/L2) and writes the result: two reads and one write per element.
template <typename TI, typename TO, bool LOG, int TPR, int V>
__global__ void softmax_fwd_generic_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t M, int64_t N,
                                           int safe) {
  using A = acc_t<TI>;
  __shared__ A scratch[64];
  const int tpr = TPR == 32 ? 32 : static_cast<int>(blockDim.x);
  const int rpb = TPR == 32 ? static_cast<int>(blockDim.x) / 32 : 1;
  const int sub = TPR == 32 ? static_cast<int>(threadIdx.x) / 32 : 0;
  const int lane = TPR == 32 ? static_cast<int>(threadIdx.x) % 32 : static_cast<int>(threadIdx.x);
  const int64_t nv = N / V;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rpb; row0 < M; row0 += static_cast<int64_t>(gridDim.x) * rpb) {
    const int64_t row = row0 + sub;
    if (row >= M) continue;
    const TI* xr = x + row * N;
    TO* yr = y + row * N;
    MaxSum<A> ms;
    ms.init();
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<TI, V> p = ld_vec<TI, V>(xr + v * V);
#pragma unroll
      for (int e = 0; e < V; ++e) ms.add(to_acc<A>(p.v[e]));
    }
    ms = row_merge<TPR>(ms, scratch);
    if (ms.m == -acc_neg_inf<A>()) ms.s = acc_nan<A>();  // +inf in the row: exp(inf - inf)
    const A mx = ms.m;
    const A lg = LOG ? acc_log(ms.s) : A(0);
    // safe softmax: a row of -inf gives zeros, not NaN (a NaN in the row has made the sum NaN and still wins)
    const bool zero_row = safe && mx == acc_neg_inf<A>() && !(ms.s != ms.s);
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<TI, V> p = ld_vec<TI, V>(xr + v * V);
      Vec<TO, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const A d = to_acc<A>(p.v[e]) - mx;
        o.v[e] = from_acc<TO>(zero_row ? A(0) : (LOG ? d - lg : acc_exp(d) / ms.s));
      }
      st_vec<TO, V>(yr + v * V, o);
    }
  }
}

// softmax: dx = y*(dy - sum(y*dy)); log-softmax: dx = dy - exp(y)*sum(dy).
// TG: type of dy and y; TO: type of dx.
template <typename TG, typename TO, bool LOG, int TPR, int V>
__global__ void softmax_bwd_generic_kernel(const TG* __restrict__ dy, const TG* __restrict__ y,
                                           TO* __restrict__ dx, int64_t M, int64_t N) {
  using A = acc_t<TG>;
  __shared__ A scratch[32];
  const int tpr = TPR == 32 ? 32 : static_cast<int>(blockDim.x);
  const int rpb = TPR == 32 ? static_cast<int>(blockDim.x) / 32 : 1;
  const int sub = TPR == 32 ? static_cast<int>(threadIdx.x) / 32 : 0;
  const int lane = TPR == 32 ? static_cast<int>(threadIdx.x) % 32 : static_cast<int>(threadIdx.x);
  const int64_t nv = N / V;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rpb; row0 < M; row0 += static_cast<int64_t>(gridDim.x) * rpb) {
    const int64_t row = row0 + sub;
    if (row >= M) continue;
    const TG* dyr = dy + row * N;
    const TG* yr = y + row * N;
    TO* dxr = dx + row * N;
    A s = 0;
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<TG, V> pd = ld_vec<TG, V>(dyr + v * V);
      if constexpr (LOG) {
#pragma unroll
        for (int e = 0; e < V; ++e) s += to_acc<A>(pd.v[e]);
      } else {
        const Vec<TG, V> py = ld_vec<TG, V>(yr + v * V);
#pragma unroll
        for (int e = 0; e < V; ++e) s += to_acc<A>(pd.v[e]) * to_acc<A>(py.v[e]);
      }
    }
    s = row_reduce<TPR>(s, scratch, SumOp());
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<TG, V> pd = ld_vec<TG, V>(dyr + v * V);
      const Vec<TG, V> py = ld_vec<TG, V>(yr + v * V);
      Vec<TO, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const A d = to_acc<A>(pd.v[e]), yy = to_acc<A>(py.v[e]);
        o.v[e] = from_acc<TO>(LOG ? d - acc_exp(yy) * s : yy * (d - s));
      }
      st_vec<TO, V>(dxr + v * V, o);
    }
  }
}

// Two adjacent 16-bit values as one 32-bit shared-memory access (the tile kernels walk lines two columns at a time).
__device__ __forceinline__ float2 ld_pair(const bf16* p) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ float2 ld_pair(const f16* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
__device__ __forceinline__ void st_pair(bf16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v); }
__device__ __forceinline__ void st_pair(f16* p, float2 v) { *reinterpret_cast<__half2*>(p) = __float22half2_rn(v); }

// ---- softmax over a dim that is not the last: shared-memory tiles ----------------------------------
// The tensor is [outer, N, inner]; a line runs over N with stride `inner`.  Reading lines one element
// at a time touches memory in 128-byte pieces half a megabyte apart, which DRAM serves at a fifth of
// its bandwidth.  Here a CTA stages a tile of `tile` adjacent inner positions x all N line elements
// in shared memory with 16-byte accesses — N contiguous runs of `tile` elements (1 KB where shared
// memory allows) — one thread per inner position then walks its line in shared memory (consecutive
// threads, consecutive addresses: no bank conflicts), leaves the result in place, and the tile goes
// back the same way.  Every element crosses HBM once each way, for any N whose tile fits.
// Requires inner % VEC == 0 and 16-byte aligned pointers; TI == TO.
template <typename T, bool LOG>
__global__ void __launch_bounds__(256)
softmax_fwd_tile_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t outer, int N, int64_t inner, int tile,
                        int safe) {
  using A = acc_t<T>;
  constexpr int VEC = 16 / sizeof(T);
  extern __shared__ __align__(16) unsigned char tile_smem[];
  T* sm = reinterpret_cast<T*>(tile_smem);
  const int64_t tpo = (inner + tile - 1) / tile, total = outer * tpo;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t o = t / tpo, i0 = (t % tpo) * tile;
    const int w = static_cast<int>(inner - i0 < tile ? inner - i0 : tile);  // a multiple of VEC
    const int vpr = w / VEC;
    const T* xb = x + o * N * inner + i0;
    T* yb = y + o * N * inner + i0;
    for (int j = warp; j < N; j += nwarp)
      for (int c = lane; c < vpr; c += 32)
        *reinterpret_cast<uint4*>(sm + static_cast<size_t>(j) * tile + c * VEC) =
            *reinterpret_cast<const uint4*>(xb + static_cast<int64_t>(j) * inner + c * VEC);
    __syncthreads();
    if constexpr (sizeof(T) == 2) {
      // 16-bit storage: a thread walks two adjacent lines with one 32-bit access per step
      for (int c = 2 * threadIdx.x; c < w; c += 2 * blockDim.x) {
        T* col = sm + c;
        float2 mx = make_float2(acc_neg_inf<float>(), acc_neg_inf<float>());
        bool nan0 = false, nan1 = false;
        for (int j = 0; j < N; ++j) {
          const float2 v = ld_pair(col + static_cast<size_t>(j) * tile);
          nan0 |= (v.x != v.x);
          nan1 |= (v.y != v.y);
          mx.x = fmaxf(mx.x, v.x);
          mx.y = fmaxf(mx.y, v.y);
        }
        float2 sum = make_float2(0.0f, 0.0f);
        for (int j = 0; j < N; ++j) {
          const float2 v = ld_pair(col + static_cast<size_t>(j) * tile);
          sum.x += exp_for<T>(v.x - mx.x);
          sum.y += exp_for<T>(v.y - mx.y);
        }
        if (nan0) sum.x = acc_nan<float>();
        if (nan1) sum.y = acc_nan<float>();
        const float2 lg = make_float2(LOG ? logf(sum.x) : 0.0f, LOG ? logf(sum.y) : 0.0f);
        const float2 inv = make_float2(LOG ? 0.0f : 1.0f / sum.x, LOG ? 0.0f : 1.0f / sum.y);
        const bool z0 = safe && mx.x == acc_neg_inf<float>() && !nan0, z1 = safe && mx.y == acc_neg_inf<float>() && !nan1;
        for (int j = 0; j < N; ++j) {
          const float2 v = ld_pair(col + static_cast<size_t>(j) * tile);
          const float dx0 = v.x - mx.x, dx1 = v.y - mx.y;
          float2 e = LOG ? make_float2(dx0 - lg.x, dx1 - lg.y)
                         : make_float2(exp_for<T>(dx0) * inv.x, exp_for<T>(dx1) * inv.y);
          if (z0) e.x = 0.0f;
          if (z1) e.y = 0.0f;
          st_pair(col + static_cast<size_t>(j) * tile, e);
        }
      }
    } else
    for (int c = threadIdx.x; c < w; c += blockDim.x) {
      // three walks over the line in shared memory (max; sum of exp; result): reads there are cheap, and exp
      // of a 16-bit result is one hardware instruction
      A mx = acc_neg_inf<A>();
      bool has_nan = false;
      for (int j = 0; j < N; ++j) {
        const A v = to_acc<A>(sm[static_cast<size_t>(j) * tile + c]);
        has_nan |= (v != v);
        mx = acc_max(mx, v);
      }
      A s = 0;
      for (int j = 0; j < N; ++j) s += exp_for<T>(to_acc<A>(sm[static_cast<size_t>(j) * tile + c]) - mx);
      if (has_nan) s = acc_nan<A>();  // (+inf in the line: exp(inf - inf) has made the sum NaN already)
      const A lg = LOG ? acc_log(s) : A(0);
      const A inv = LOG ? A(0) : A(1) / s;
      const bool zero = safe && mx == acc_neg_inf<A>() && !has_nan;
      for (int j = 0; j < N; ++j) {
        const A d = to_acc<A>(sm[static_cast<size_t>(j) * tile + c]) - mx;
        const A e = LOG ? d - lg : (sizeof(T) <= 2 ? exp_for<T>(d) * inv : exp_for<T>(d) / s);
        sm[static_cast<size_t>(j) * tile + c] = from_acc<T>(zero ? A(0) : e);
      }
    }
    __syncthreads();
    for (int j = warp; j < N; j += nwarp)
      for (int c = lane; c < vpr; c += 32)
        *reinterpret_cast<uint4*>(yb + static_cast<int64_t>(j) * inner + c * VEC) =
            *reinterpret_cast<const uint4*>(sm + static_cast<size_t>(j) * tile + c * VEC);
    __syncthreads();  // the next tile's loads overwrite the staging area
  }
}

// dy tile at sm[0 .. N*tile), y tile behind it; dx overwrites the dy tile.
template <typename T, bool LOG>
__global__ void __launch_bounds__(256)
softmax_bwd_tile_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t outer, int N,
                        int64_t inner, int tile) {
  using A = acc_t<T>;
  constexpr int VEC = 16 / sizeof(T);
  extern __shared__ __align__(16) unsigned char tile_smem[];
  T* sd = reinterpret_cast<T*>(tile_smem);
  T* sy = sd + static_cast<size_t>(N) * tile;
  const int64_t tpo = (inner + tile - 1) / tile, total = outer * tpo;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t o = t / tpo, i0 = (t % tpo) * tile;
    const int w = static_cast<int>(inner - i0 < tile ? inner - i0 : tile);
    const int vpr = w / VEC;
    const int64_t base = o * N * inner + i0;
    for (int j = warp; j < N; j += nwarp)
      for (int c = lane; c < vpr; c += 32) {
        const int64_t g = base + static_cast<int64_t>(j) * inner + c * VEC;
        const size_t l = static_cast<size_t>(j) * tile + c * VEC;
        *reinterpret_cast<uint4*>(sd + l) = *reinterpret_cast<const uint4*>(dy + g);
        *reinterpret_cast<uint4*>(sy + l) = *reinterpret_cast<const uint4*>(y + g);
      }
    __syncthreads();
    if constexpr (sizeof(T) == 2) {
      for (int c = 2 * threadIdx.x; c < w; c += 2 * blockDim.x) {
        float2 sum = make_float2(0.0f, 0.0f);
        for (int j = 0; j < N; ++j) {
          const size_t l = static_cast<size_t>(j) * tile + c;
          const float2 d = ld_pair(sd + l);
          if constexpr (LOG) {
            sum.x += d.x;
            sum.y += d.y;
          } else {
            const float2 yy = ld_pair(sy + l);
            sum.x = fmaf(d.x, yy.x, sum.x);
            sum.y = fmaf(d.y, yy.y, sum.y);
          }
        }
        for (int j = 0; j < N; ++j) {
          const size_t l = static_cast<size_t>(j) * tile + c;
          const float2 d = ld_pair(sd + l), yy = ld_pair(sy + l);
          const float2 o = LOG ? make_float2(d.x - exp_for<T>(yy.x) * sum.x, d.y - exp_for<T>(yy.y) * sum.y)
                               : make_float2(yy.x * (d.x - sum.x), yy.y * (d.y - sum.y));
          st_pair(sd + l, o);
        }
      }
    } else
    for (int c = threadIdx.x; c < w; c += blockDim.x) {
      A s = 0;
      for (int j = 0; j < N; ++j) {
        const size_t l = static_cast<size_t>(j) * tile + c;
        const A d = to_acc<A>(sd[l]);
        s += LOG ? d : d * to_acc<A>(sy[l]);
      }
      for (int j = 0; j < N; ++j) {
        const size_t l = static_cast<size_t>(j) * tile + c;
        const A d = to_acc<A>(sd[l]), yy = to_acc<A>(sy[l]);
        sd[l] = from_acc<T>(LOG ? d - exp_for<T>(yy) * s : yy * (d - s));
      }
    }
    __syncthreads();
    for (int j = warp; j < N; j += nwarp)
      for (int c = lane; c < vpr; c += 32)
        *reinterpret_cast<uint4*>(dx + base + static_cast<int64_t>(j) * inner + c * VEC) =
            *reinterpret_cast<const uint4*>(sd + static_cast<size_t>(j) * tile + c * VEC);
    __syncthreads();
  }
}


// ---- softmax over a dim that is not the last, lines short enough for registers ---------------------
// The tensor is [outer, N, inner]; a line runs over N with stride `inner`.  A thread owns V adjacent
// inner positions (V = 2 when `inner` and the pointers allow one 4- or 8-byte access for both), keeps
// its V lines of up to NMAX values in registers and touches every element once: one read, one write
// (the general kernels below read a line two or three times).  Neighbouring threads own neighbouring
// inner positions, so every access of a warp is one contiguous run.
template <typename TI, typename TO, bool LOG, int NMAX, int V>
__global__ void __launch_bounds__(256) softmax_fwd_spatial_reg_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t outer, int N,
                                               int64_t inner, int safe) {
  using A = acc_t<TI>;
  const int64_t innerv = inner / V, total = outer * innerv;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t o = idx / innerv, in = (idx % innerv) * V;
    const int64_t base = o * N * inner + in;
    A v[NMAX][V];
    A mx[V];
    bool has_nan[V];
#pragma unroll
    for (int e = 0; e < V; ++e) { mx[e] = acc_neg_inf<A>(); has_nan[e] = false; }
#pragma unroll
    for (int j = 0; j < NMAX; ++j) {
      if (j < N) {
        const Vec<TI, V> p = ld_vec<TI, V>(x + base + j * inner);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          v[j][e] = to_acc<A>(p.v[e]);
          has_nan[e] |= (v[j][e] != v[j][e]);
          mx[e] = acc_max(mx[e], v[j][e]);
        }
      }
    }
    A s[V];
#pragma unroll
    for (int e = 0; e < V; ++e) s[e] = 0;
#pragma unroll
    for (int j = 0; j < NMAX; ++j) {
      if (j < N) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          v[j][e] = v[j][e] - mx[e];
          const A ex = exp_for<TO>(v[j][e]);
          s[e] += ex;
          if (!LOG) v[j][e] = ex;
        }
      }
    }
    A lg[V], inv[V];
    bool zero[V];
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (has_nan[e] || mx[e] == -acc_neg_inf<A>()) s[e] = acc_nan<A>();  // NaN, or +inf in the line
      lg[e] = LOG ? acc_log(s[e]) : A(0);
      inv[e] = LOG ? A(0) : A(1) / s[e];  // 16-bit storage multiplies by it; wider storage divides (exactly rounded)
      zero[e] = safe && mx[e] == acc_neg_inf<A>() && !has_nan[e];
    }
#pragma unroll
    for (int j = 0; j < NMAX; ++j) {
      if (j < N) {
        Vec<TO, V> o2;
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const A sm = sizeof(TO) <= 2 ? v[j][e] * inv[e] : v[j][e] / s[e];
          o2.v[e] = from_acc<TO>(zero[e] ? A(0) : (LOG ? v[j][e] - lg[e] : sm));
        }
        st_vec<TO, V>(y + base + j * inner, o2);
      }
    }
  }
}

template <typename TG, typename TO, bool LOG, int NMAX, int V>
__global__ void __launch_bounds__(256) softmax_bwd_spatial_reg_kernel(const TG* __restrict__ dy, const TG* __restrict__ y,
                                               TO* __restrict__ dx, int64_t outer, int N, int64_t inner) {
  using A = acc_t<TG>;
  const int64_t innerv = inner / V, total = outer * innerv;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t o = idx / innerv, in = (idx % innerv) * V;
    const int64_t base = o * N * inner + in;
    A d[NMAX][V], yy[NMAX][V];
    A s[V];
#pragma unroll
    for (int e = 0; e < V; ++e) s[e] = 0;
#pragma unroll
    for (int j = 0; j < NMAX; ++j) {
      if (j < N) {
        const Vec<TG, V> pd = ld_vec<TG, V>(dy + base + j * inner);
        const Vec<TG, V> py = ld_vec<TG, V>(y + base + j * inner);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          d[j][e] = to_acc<A>(pd.v[e]);
          yy[j][e] = to_acc<A>(py.v[e]);
          s[e] += LOG ? d[j][e] : d[j][e] * yy[j][e];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NMAX; ++j) {
      if (j < N) {
        Vec<TO, V> o2;
#pragma unroll
        for (int e = 0; e < V; ++e)
          o2.v[e] = from_acc<TO>(LOG ? d[j][e] - exp_for<TO>(yy[j][e]) * s[e] : yy[j][e] * (d[j][e] - s[e]));
        st_vec<TO, V>(dx + base + j * inner, o2);
      }
    }
  }
}


// Softmax along a dim that is not the last: the tensor is [outer, N, inner] and one thread walks
// one (outer, inner) line with stride `inner`, so neighbouring threads touch neighbouring
// addresses.  Two passes: running (max, sum), then write.  Lines of up to 64 values take the register
// kernels above instead.
template <typename TI, typename TO, bool LOG>
__global__ void softmax_fwd_spatial_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t outer,
                                           int64_t N, int64_t inner, int safe) {
  using A = acc_t<TI>;
  const int64_t total = outer * inner;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t o = idx / inner, in = idx % inner;
    const TI* xp = x + o * N * inner + in;
    TO* yp = y + o * N * inner + in;
    // one pass for both statistics: a running (max, sum of exp(x - max)) pair
    MaxSum<A> ms;
    ms.init();
    bool has_nan = false;
    for (int64_t j = 0; j < N; ++j) {
      const A v = to_acc<A>(xp[j * inner]);
      has_nan |= (v != v);
      ms.add(v);
    }
    const A mx = ms.m;
    A s = ms.s;
    if (has_nan || mx == -acc_neg_inf<A>()) s = acc_nan<A>();  // NaN, or +inf in the line: exp(inf - inf)
    const A lg = LOG ? acc_log(s) : A(0);
    const bool zero_row = safe && mx == acc_neg_inf<A>() && !has_nan;
    for (int64_t j = 0; j < N; ++j) {
      const A d = to_acc<A>(xp[j * inner]) - mx;
      yp[j * inner] = from_acc<TO>(zero_row ? A(0) : (LOG ? d - lg : acc_exp(d) / s));
    }
  }
}

template <typename TG, typename TO, bool LOG>
__global__ void softmax_bwd_spatial_kernel(const TG* __restrict__ dy, const TG* __restrict__ y,
                                           TO* __restrict__ dx, int64_t outer, int64_t N, int64_t inner) {
  using A = acc_t<TG>;
  const int64_t total = outer * inner;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t o = idx / inner, in = idx % inner;
    const int64_t base = o * N * inner + in;
    A s = 0;
    for (int64_t j = 0; j < N; ++j) {
      const A d = to_acc<A>(dy[base + j * inner]);
      s += LOG ? d : d * to_acc<A>(y[base + j * inner]);
    }
    for (int64_t j = 0; j < N; ++j) {
      const A d = to_acc<A>(dy[base + j * inner]), yy = to_acc<A>(y[base + j * inner]);
      dx[base + j * inner] = from_acc<TO>(LOG ? d - acc_exp(yy) * s : yy * (d - s));
    }
  }
}

}  // namespace b2n
