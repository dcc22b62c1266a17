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
// memory allows), four loads in flight per thread — works on the lines there and sends the tile
// back the same way: every element crosses HBM once each way, for any N whose tile fits.
//
// In shared memory a line is shared by `segs` threads (as many as the CTA's threads allow for the
// tile's width: a 256-column tile of 16-bit values is 128 column pairs x 2 segments), each walking
// every segs-th element, consecutive threads touching consecutive addresses (no bank conflicts).  The segments' partial
// results are combined in segment order through a small scratch array, then each thread writes the
// results for the elements it walked.
// Requires inner % VEC == 0 and 16-byte aligned pointers; TI == TO.
constexpr int kTileThreads = 256;
constexpr int kTileScratchBytes = 4096;  // the segments' partial results, in front of the staged tile

// (max, sum of exp(x - max)) of a segment of a line, with the semantics of the row kernels: -inf entries give 0,
// a NaN makes the sum NaN (the maximum ignores it), +inf makes exp(inf - inf) = NaN
template <typename T> struct OnlineMaxSum {
  float m, s;
  __device__ __forceinline__ void init() { m = acc_neg_inf<float>(); s = 0.0f; }
  __device__ __forceinline__ void merge(float om, float os) {
    const float ninf = acc_neg_inf<float>();
    const float nm = fmaxf(m, om);
    // a NaN partial sum must survive a partial maximum of -inf (0 * exp(...) would hide it otherwise)
    const float a = (m == ninf) ? ((s != s) ? s : 0.0f) : s * exp_for<T>(m - nm);
    const float b = (om == ninf) ? ((os != os) ? os : 0.0f) : os * exp_for<T>(om - nm);
    s = a + b;
    m = nm;
  }
};

// Tile <-> global copies: a warp takes whole lines (its lanes the line's 16-byte vectors: one contiguous run per
// access), four lines at a time so that several loads are in flight per thread.
template <typename T> __device__ __forceinline__ void tile_copy_in(T* sm, const T* gb, int N, int64_t inner, int tile, int vpr) {
  constexpr int VEC = 16 / sizeof(T);
  if (N >= 32) {
    // many lines: the tile's vectors as one flat index space over the CTA's threads, eight loads in flight each
    // (measured better from a few dozen lines on; below that the per-vector division costs more than it gains)
    const int total = N * vpr;
#pragma unroll 8
    for (int i = threadIdx.x; i < total; i += kTileThreads) {
      const int j = i / vpr, c = i - j * vpr;
      *reinterpret_cast<uint4*>(sm + static_cast<size_t>(j) * tile + c * VEC) =
          *reinterpret_cast<const uint4*>(gb + static_cast<int64_t>(j) * inner + c * VEC);
    }
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = kTileThreads >> 5;
  for (int c = lane; c < vpr; c += 32) {
    int j = warp;
    for (; j + 3 * nwarp < N; j += 4 * nwarp) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(gb + static_cast<int64_t>(j + u * nwarp) * inner + c * VEC);
#pragma unroll
      for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(sm + static_cast<size_t>(j + u * nwarp) * tile + c * VEC) = v[u];
    }
    for (; j < N; j += nwarp)
      *reinterpret_cast<uint4*>(sm + static_cast<size_t>(j) * tile + c * VEC) =
          *reinterpret_cast<const uint4*>(gb + static_cast<int64_t>(j) * inner + c * VEC);
  }
}
template <typename T> __device__ __forceinline__ void tile_copy_out(T* gb, const T* sm, int N, int64_t inner, int tile, int vpr) {
  constexpr int VEC = 16 / sizeof(T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = kTileThreads >> 5;
  for (int j = warp; j < N; j += nwarp)
    for (int c = lane; c < vpr; c += 32)
      *reinterpret_cast<uint4*>(gb + static_cast<int64_t>(j) * inner + c * VEC) =
          *reinterpret_cast<const uint4*>(sm + static_cast<size_t>(j) * tile + c * VEC);
}

template <typename T, bool LOG>
__global__ void __launch_bounds__(kTileThreads)
softmax_fwd_tile_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t outer, int N, int64_t inner, int tile,
                        int safe) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int CPT = sizeof(T) == 2 ? 2 : 1;  // columns a thread handles with one shared-memory access
  extern __shared__ __align__(16) unsigned char tile_smem[];
  float4* part = reinterpret_cast<float4*>(tile_smem);  // per (segment, column group): {max0, sum0, max1, sum1}
  T* sm = reinterpret_cast<T*>(tile_smem + kTileScratchBytes);
  const int64_t tpo = (inner + tile - 1) / tile, total = outer * tpo;
  const float ninf = acc_neg_inf<float>();
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t o = t / tpo, i0 = (t % tpo) * tile;
    const int w = static_cast<int>(inner - i0 < tile ? inner - i0 : tile);  // a multiple of VEC
    tile_copy_in(sm, x + o * N * inner + i0, N, inner, tile, w / VEC);
    __syncthreads();
    const int groups = w / CPT;                                  // column groups of the tile (<= kTileThreads)
    int segs = kTileThreads / groups;
    if (segs > N) segs = N;
    if (segs > 32) segs = 32;
    const bool active = static_cast<int>(threadIdx.x) < groups * segs;
    const int gidx = threadIdx.x % groups, sg = threadIdx.x / groups;
    T* col = sm + gidx * CPT;
    OnlineMaxSum<T> a, b;  // b: the second column of a pair (16-bit storage)
    a.init();
    b.init();
    if (active) {
      // two short walks (maximum; then sum of exp about it) rather than one with a running pair: a walk's iterations
      // are then independent but for one fmax or one add, which is what lets several loads be in flight
#pragma unroll 4
      for (int j = sg; j < N; j += segs) {
        if constexpr (CPT == 2) {
          const float2 v = ld_pair(col + static_cast<size_t>(j) * tile);
          a.m = fmaxf(a.m, v.x);
          b.m = fmaxf(b.m, v.y);
        } else {
          a.m = fmaxf(a.m, to_acc<float>(col[static_cast<size_t>(j) * tile]));
        }
      }
      const float base0 = (a.m == ninf) ? 0.0f : a.m, base1 = (b.m == ninf) ? 0.0f : b.m;  // all -inf: exp(-inf - 0) = 0
#pragma unroll 4
      for (int j = sg; j < N; j += segs) {
        if constexpr (CPT == 2) {
          const float2 v = ld_pair(col + static_cast<size_t>(j) * tile);
          a.s += exp_for<T>(v.x - base0);  // a NaN entry makes the sum NaN (the maximum ignored it)
          b.s += exp_for<T>(v.y - base1);
        } else {
          a.s += exp_for<T>(to_acc<float>(col[static_cast<size_t>(j) * tile]) - base0);
        }
      }
      part[threadIdx.x] = make_float4(a.m, a.s, b.m, b.s);
    }
    __syncthreads();
    if (active) {
      const float4 p0 = part[gidx];
      a.m = p0.x; a.s = p0.y; b.m = p0.z; b.s = p0.w;
      for (int k = 1; k < segs; ++k) {  // segment order: every thread of the line gets the same bits
        const float4 pk = part[k * groups + gidx];
        a.merge(pk.x, pk.y);
        if (CPT == 2) b.merge(pk.z, pk.w);
      }
      // (+inf in the line: exp(inf - inf) has made the sum NaN already; a NaN entry too)
      const float2 mx = make_float2(a.m, b.m), sum = make_float2(a.s, b.s);
      const float2 lg = make_float2(LOG ? logf(sum.x) : 0.0f, LOG ? logf(sum.y) : 0.0f);
      const float2 inv = make_float2(LOG ? 0.0f : 1.0f / sum.x, LOG ? 0.0f : 1.0f / sum.y);
      const bool z0 = safe && mx.x == ninf && !(sum.x != sum.x), z1 = safe && mx.y == ninf && !(sum.y != sum.y);
#pragma unroll 4
      for (int j = sg; j < N; j += segs) {
        if constexpr (CPT == 2) {
          const float2 v = ld_pair(col + static_cast<size_t>(j) * tile);
          const float dx0 = v.x - mx.x, dx1 = v.y - mx.y;
          float2 e = LOG ? make_float2(dx0 - lg.x, dx1 - lg.y)
                         : make_float2(exp_for<T>(dx0) * inv.x, exp_for<T>(dx1) * inv.y);
          if (z0) e.x = 0.0f;
          if (z1) e.y = 0.0f;
          st_pair(col + static_cast<size_t>(j) * tile, e);
        } else {
          const float d = to_acc<float>(col[static_cast<size_t>(j) * tile]) - mx.x;
          const float e = LOG ? d - lg.x : exp_for<T>(d) / sum.x;
          col[static_cast<size_t>(j) * tile] = from_acc<T>(z0 ? 0.0f : e);
        }
      }
    }
    __syncthreads();
    tile_copy_out(y + o * N * inner + i0, sm, N, inner, tile, w / VEC);
    __syncthreads();  // the next tile's loads overwrite the staging area
  }
}

// dy tile first (behind the scratch), y tile behind it; dx overwrites the dy tile.
template <typename T, bool LOG>
__global__ void __launch_bounds__(kTileThreads)
softmax_bwd_tile_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t outer, int N,
                        int64_t inner, int tile) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int CPT = sizeof(T) == 2 ? 2 : 1;
  extern __shared__ __align__(16) unsigned char tile_smem[];
  float2* part = reinterpret_cast<float2*>(tile_smem);
  T* sd = reinterpret_cast<T*>(tile_smem + kTileScratchBytes);
  T* sy = sd + static_cast<size_t>(N) * tile;
  const int64_t tpo = (inner + tile - 1) / tile, total = outer * tpo;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t o = t / tpo, i0 = (t % tpo) * tile;
    const int w = static_cast<int>(inner - i0 < tile ? inner - i0 : tile);
    const int64_t base = o * N * inner + i0;
    tile_copy_in(sd, dy + base, N, inner, tile, w / VEC);
    tile_copy_in(sy, y + base, N, inner, tile, w / VEC);
    __syncthreads();
    const int groups = w / CPT;
    int segs = kTileThreads / groups;
    if (segs > N) segs = N;
    if (segs > 32) segs = 32;
    const bool active = static_cast<int>(threadIdx.x) < groups * segs;
    const int gidx = threadIdx.x % groups, sg = threadIdx.x / groups;
    const size_t c = static_cast<size_t>(gidx) * CPT;
    float2 sum = make_float2(0.0f, 0.0f);
    if (active) {
#pragma unroll 4
      for (int j = sg; j < N; j += segs) {
        const size_t l = static_cast<size_t>(j) * tile + c;
        if constexpr (CPT == 2) {
          const float2 d = ld_pair(sd + l);
          if constexpr (LOG) {
            sum.x += d.x;
            sum.y += d.y;
          } else {
            const float2 yy = ld_pair(sy + l);
            sum.x = fmaf(d.x, yy.x, sum.x);
            sum.y = fmaf(d.y, yy.y, sum.y);
          }
        } else {
          const float d = to_acc<float>(sd[l]);
          sum.x += LOG ? d : d * to_acc<float>(sy[l]);
        }
      }
      part[threadIdx.x] = sum;
    }
    __syncthreads();
    if (active) {
      sum = part[gidx];
      for (int k = 1; k < segs; ++k) {
        const float2 pk = part[k * groups + gidx];
        sum.x += pk.x;
        sum.y += pk.y;
      }
#pragma unroll 4
      for (int j = sg; j < N; j += segs) {
        const size_t l = static_cast<size_t>(j) * tile + c;
        if constexpr (CPT == 2) {
          const float2 d = ld_pair(sd + l), yy = ld_pair(sy + l);
          const float2 r = LOG ? make_float2(d.x - exp_for<T>(yy.x) * sum.x, d.y - exp_for<T>(yy.y) * sum.y)
                               : make_float2(yy.x * (d.x - sum.x), yy.y * (d.y - sum.y));
          st_pair(sd + l, r);
        } else {
          const float d = to_acc<float>(sd[l]), yy = to_acc<float>(sy[l]);
          sd[l] = from_acc<T>(LOG ? d - exp_for<T>(yy) * sum.x : yy * (d - sum.x));
        }
      }
    }
    __syncthreads();
    tile_copy_out(dx + base, sd, N, inner, tile, w / VEC);
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
