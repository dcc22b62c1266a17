// Masked softmax over the last dim (aten::_masked_softmax / _masked_softmax_backward).
//
// Forward: y = softmax(x) with the elements whose mask byte is non-zero treated as -inf: they come
// out as exactly 0; a row with every element masked comes out as NaN, like the CPU ATen kernel.
// The mask row of input row r is (r / row_div) % row_mod, which covers the three layouts of
// masked_softmax_kernel (src/ATen/native/xpu/sycl/SoftMaxKernels.cpp:2301-2362): a mask of the
// input's shape (row_div 1, row_mod M), a [T, T] source mask shared by every batch and head
// (row_div 1, row_mod T) and a [B, T] key-padding mask (row_div H*T, row_mod B).
// Backward (mask of the gradient's shape, :2364-2407): dx = y * (dy - sum_unmasked(y * dy)), zero
// where masked.
//
// Rows the ring takes (16-byte aligned, 16-bit or fp32, N within the ring's reach) run on the softmax
// ring kernels with the mask applied in registers (softmax_ring.cuh: RowMask).  Everything else runs
// on the kernels below: one warp per row up to 1024 elements, one CTA per row beyond; 16-byte loads
// of x with 8- or 4-byte loads of the mask when everything is aligned, scalar accesses otherwise; the
// row is read twice (second time from L1/L2).
#include "launchers.h"
#include "softmax_launch.cuh"

namespace b2n {
namespace {

template <int V> struct MaskVec { unsigned char b[V]; };
template <int V> __device__ __forceinline__ MaskVec<V> ld_mask(const unsigned char* p) {
  MaskVec<V> m;
  if constexpr (V == 8) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    *reinterpret_cast<uint2*>(m.b) = w;
  } else if constexpr (V == 4) {
    *reinterpret_cast<unsigned*>(m.b) = *reinterpret_cast<const unsigned*>(p);
  } else if constexpr (V == 2) {
    *reinterpret_cast<unsigned short*>(m.b) = *reinterpret_cast<const unsigned short*>(p);
  } else {
    m.b[0] = p[0];
  }
  return m;
}

template <typename T, int TPR, int V>
__global__ void masked_softmax_fwd_kernel(const T* __restrict__ x, const unsigned char* __restrict__ mask,
                                          T* __restrict__ y, int64_t M, int64_t N, int64_t row_div,
                                          int64_t row_mod) {
  using A = acc_t<T>;
  __shared__ A scratch[64];
  const int tpr = TPR == 32 ? 32 : static_cast<int>(blockDim.x);
  const int rpb = TPR == 32 ? static_cast<int>(blockDim.x) / 32 : 1;
  const int sub = TPR == 32 ? static_cast<int>(threadIdx.x) / 32 : 0;
  const int lane = TPR == 32 ? static_cast<int>(threadIdx.x) % 32 : static_cast<int>(threadIdx.x);
  const int64_t nv = N / V;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rpb; row0 < M; row0 += static_cast<int64_t>(gridDim.x) * rpb) {
    const int64_t row = row0 + sub;
    if (row >= M) continue;  // only with one warp per row: the other warps of the CTA never meet a CTA barrier
    const T* xr = x + row * N;
    T* yr = y + row * N;
    const unsigned char* mr = mask + ((row / row_div) % row_mod) * N;
    MaxSum<A> ms;
    ms.init();
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> p = ld_vec<T, V>(xr + v * V);
      const MaskVec<V> k = ld_mask<V>(mr + v * V);
#pragma unroll
      for (int e = 0; e < V; ++e)
        if (!k.b[e]) ms.add(to_acc<A>(p.v[e]));
    }
    ms = row_merge<TPR>(ms, scratch);
    if (ms.m == -acc_neg_inf<A>()) ms.s = acc_nan<A>();  // +inf in the row: exp(inf - inf)
    // every element masked (or every unmasked one -inf): max -inf, sum 0 -> 0/0: the whole row is NaN
    const bool dead = ms.m == acc_neg_inf<A>();
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> p = ld_vec<T, V>(xr + v * V);
      const MaskVec<V> k = ld_mask<V>(mr + v * V);
      Vec<T, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const A r = acc_exp(to_acc<A>(p.v[e]) - ms.m) / ms.s;
        o.v[e] = from_acc<T>(dead ? acc_nan<A>() : (k.b[e] ? A(0) : r));
      }
      st_vec<T, V>(yr + v * V, o);
    }
  }
}

template <typename T, int TPR, int V>
__global__ void masked_softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                          const unsigned char* __restrict__ mask, T* __restrict__ dx, int64_t M,
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
    const T* yr = y + row * N;
    const unsigned char* mr = mask + row * N;
    T* dxr = dx + row * N;
    A s = 0;
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> pd = ld_vec<T, V>(dyr + v * V);
      const Vec<T, V> py = ld_vec<T, V>(yr + v * V);
      const MaskVec<V> k = ld_mask<V>(mr + v * V);
#pragma unroll
      for (int e = 0; e < V; ++e)
        if (!k.b[e]) s += to_acc<A>(pd.v[e]) * to_acc<A>(py.v[e]);
    }
    s = row_reduce<TPR>(s, scratch, SumOp());
    for (int64_t v = lane; v < nv; v += tpr) {
      const Vec<T, V> pd = ld_vec<T, V>(dyr + v * V);
      const Vec<T, V> py = ld_vec<T, V>(yr + v * V);
      const MaskVec<V> k = ld_mask<V>(mr + v * V);
      Vec<T, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const A d = to_acc<A>(pd.v[e]), yy = to_acc<A>(py.v[e]);
        o.v[e] = from_acc<T>(k.b[e] ? A(0) : yy * (d - s));
      }
      st_vec<T, V>(dxr + v * V, o);
    }
  }
}

inline int masked_grid(int64_t rows, int rows_per_block) {
  const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = static_cast<int64_t>(device_info().sm_count) * 16;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

template <typename T>
int masked_fwd_typed(const void* x_, const unsigned char* mask, void* y_, int64_t M, int64_t N, int64_t row_div,
                     int64_t row_mod, cudaStream_t st) {
  const T* x = static_cast<const T*>(x_);
  T* y = static_cast<T*>(y_);
  constexpr int V = 16 / sizeof(T) > 8 ? 8 : 16 / sizeof(T);  // elements per vector (mask bytes per load)
  const bool vec = N % V == 0 && is_aligned(x, V * sizeof(T)) && is_aligned(y, V * sizeof(T)) && is_aligned(mask, V);
  const int forced = forced_path();
  if constexpr (sizeof(T) <= 4 && !std::is_same<T, double>::value) {
    if (forced != B2N_PATH_GENERIC && vec && is_aligned(x, 16) && is_aligned(y, 16) && M < (1LL << 31) &&
        row_div < (1LL << 32) && row_mod < (1LL << 32)) {
      const DeviceInfo& di = device_info();
      const RingPlan p = plan_ring(M, N, sizeof(T), 1, kSoftmaxEpt, persistent_ctas(di.sm_count), di.max_smem_optin);
      if (p.ok) {
        note_path("ring");
        const RowMask rm{mask, static_cast<unsigned>(row_div), static_cast<unsigned>(row_mod)};
        switch (p.group) {
          case 32: return softmax_fwd_ring_launch<T, false, 32>(p, x, y, M, N, st, rm);
          case 64: return softmax_fwd_ring_launch<T, false, 64>(p, x, y, M, N, st, rm);
          case 128: return softmax_fwd_ring_launch<T, false, 128>(p, x, y, M, N, st, rm);
          case 256: return softmax_fwd_ring_launch<T, false, 256>(p, x, y, M, N, st, rm);
          default: return softmax_fwd_ring_launch<T, false, 512>(p, x, y, M, N, st, rm);
        }
      }
    }
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
  note_path("generic");
  ProfileScope prof("masked_softmax_fwd", st);
  if (N <= 1024) {
    const int grid = masked_grid(M, 8);
    if (vec) masked_softmax_fwd_kernel<T, 32, V><<<grid, 256, 0, st>>>(x, mask, y, M, N, row_div, row_mod);
    else masked_softmax_fwd_kernel<T, 32, 1><<<grid, 256, 0, st>>>(x, mask, y, M, N, row_div, row_mod);
  } else {
    const int grid = masked_grid(M, 1);
    const int threads = N <= 8192 ? 256 : 1024;
    if (vec) masked_softmax_fwd_kernel<T, 0, V><<<grid, threads, 0, st>>>(x, mask, y, M, N, row_div, row_mod);
    else masked_softmax_fwd_kernel<T, 0, 1><<<grid, threads, 0, st>>>(x, mask, y, M, N, row_div, row_mod);
  }
  return launched();
}

template <typename T>
int masked_bwd_typed(const void* dy_, const void* y_, const unsigned char* mask, void* dx_, int64_t M, int64_t N,
                     cudaStream_t st) {
  const T* dy = static_cast<const T*>(dy_);
  const T* y = static_cast<const T*>(y_);
  T* dx = static_cast<T*>(dx_);
  constexpr int V = 16 / sizeof(T) > 8 ? 8 : 16 / sizeof(T);
  const bool vec = N % V == 0 && is_aligned(dy, V * sizeof(T)) && is_aligned(y, V * sizeof(T)) &&
                   is_aligned(dx, V * sizeof(T)) && is_aligned(mask, V);
  const int forced = forced_path();
  if constexpr (sizeof(T) <= 4 && !std::is_same<T, double>::value) {
    if (forced != B2N_PATH_GENERIC && vec && is_aligned(dy, 16) && is_aligned(y, 16) && is_aligned(dx, 16) &&
        M < (1LL << 31)) {
      const DeviceInfo& di = device_info();
      const RingPlan p = plan_ring(M, N, sizeof(T), 2, kSoftmaxEpt, persistent_ctas(di.sm_count), di.max_smem_optin);
      if (p.ok) {
        note_path("ring");
        const RowMask rm{mask, 1u, static_cast<unsigned>(M)};  // a mask of the gradient's shape
        switch (p.group) {
          case 32: return softmax_bwd_ring_launch<T, false, 32>(p, dy, y, dx, M, N, st, rm);
          case 64: return softmax_bwd_ring_launch<T, false, 64>(p, dy, y, dx, M, N, st, rm);
          case 128: return softmax_bwd_ring_launch<T, false, 128>(p, dy, y, dx, M, N, st, rm);
          case 256: return softmax_bwd_ring_launch<T, false, 256>(p, dy, y, dx, M, N, st, rm);
          default: return softmax_bwd_ring_launch<T, false, 512>(p, dy, y, dx, M, N, st, rm);
        }
      }
    }
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
  note_path("generic");
  ProfileScope prof("masked_softmax_bwd", st);
  if (N <= 1024) {
    const int grid = masked_grid(M, 8);
    if (vec) masked_softmax_bwd_kernel<T, 32, V><<<grid, 256, 0, st>>>(dy, y, mask, dx, M, N);
    else masked_softmax_bwd_kernel<T, 32, 1><<<grid, 256, 0, st>>>(dy, y, mask, dx, M, N);
  } else {
    const int grid = masked_grid(M, 1);
    const int threads = N <= 8192 ? 256 : 1024;
    if (vec) masked_softmax_bwd_kernel<T, 0, V><<<grid, threads, 0, st>>>(dy, y, mask, dx, M, N);
    else masked_softmax_bwd_kernel<T, 0, 1><<<grid, threads, 0, st>>>(dy, y, mask, dx, M, N);
  }
  return launched();
}

}  // namespace

int launch_masked_softmax_fwd(const void* x, const void* mask, void* y, int64_t M, int64_t N, int64_t row_div,
                              int64_t row_mod, int dtype, cudaStream_t st) {
  const unsigned char* m = static_cast<const unsigned char*>(mask);
  switch (dtype) {
    case B2N_F32: return masked_fwd_typed<float>(x, m, y, M, N, row_div, row_mod, st);
    case B2N_F16: return masked_fwd_typed<f16>(x, m, y, M, N, row_div, row_mod, st);
    case B2N_BF16: return masked_fwd_typed<bf16>(x, m, y, M, N, row_div, row_mod, st);
    case B2N_F64: return masked_fwd_typed<double>(x, m, y, M, N, row_div, row_mod, st);
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

int launch_masked_softmax_bwd(const void* dy, const void* y, const void* mask, void* dx, int64_t M, int64_t N,
                              int dtype, cudaStream_t st) {
  const unsigned char* m = static_cast<const unsigned char*>(mask);
  switch (dtype) {
    case B2N_F32: return masked_bwd_typed<float>(dy, y, m, dx, M, N, st);
    case B2N_F16: return masked_bwd_typed<f16>(dy, y, m, dx, M, N, st);
    case B2N_BF16: return masked_bwd_typed<bf16>(dy, y, m, dx, M, N, st);
    case B2N_F64: return masked_bwd_typed<double>(dy, y, m, dx, M, N, st);
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

}  // namespace b2n
