// Shared device helpers: element-type traits, 16-byte vectors, warp/block reductions, and thin
// wrappers over the sm_100a PTX used by the ring kernels (mbarrier, bulk-async copies).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200norm.h"

namespace b2n {

// ---------------------------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------------------------
using bf16 = __nv_bfloat16;
using f16 = __half;

template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };
template <typename T> using acc_t = typename AccOf<T>::type;

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = B2N_F32; };
template <> struct DtypeOf<f16> { static constexpr int value = B2N_F16; };
template <> struct DtypeOf<bf16> { static constexpr int value = B2N_BF16; };
template <> struct DtypeOf<double> { static constexpr int value = B2N_F64; };

__host__ __device__ inline size_t dtype_size(int dt) {
  return dt == B2N_F64 ? 8 : (dt == B2N_F32 ? 4 : 2);
}

template <typename A, typename T> __device__ __forceinline__ A to_acc(T v) { return static_cast<A>(v); }
template <> __device__ __forceinline__ float to_acc<float, bf16>(bf16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<float, f16>(f16 v) { return __half2float(v); }
template <> __device__ __forceinline__ double to_acc<double, bf16>(bf16 v) { return (double)__bfloat162float(v); }
template <> __device__ __forceinline__ double to_acc<double, f16>(f16 v) { return (double)__half2float(v); }

template <typename T, typename A> __device__ __forceinline__ T from_acc(A v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ bf16 from_acc<bf16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ f16 from_acc<f16, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ bf16 from_acc<bf16, double>(double v) { return __float2bfloat16_rn((float)v); }
template <> __device__ __forceinline__ f16 from_acc<f16, double>(double v) { return __float2half_rn((float)v); }

// math in the accumulate type; no fast-math anywhere (precise division, sqrt, exp, log)
__device__ __forceinline__ float acc_exp(float v) { return expf(v); }
__device__ __forceinline__ double acc_exp(double v) { return exp(v); }
__device__ __forceinline__ float acc_log(float v) { return logf(v); }
__device__ __forceinline__ double acc_log(double v) { return log(v); }
__device__ __forceinline__ float acc_rsqrt(float v) { return 1.0f / sqrtf(v); }
__device__ __forceinline__ double acc_rsqrt(double v) { return 1.0 / sqrt(v); }
// 1/sqrt(v) to within 1 ulp: hardware estimate (2 ulp) plus one Newton step, five instructions
// instead of the ~30 of an IEEE sqrt followed by an IEEE division
__device__ __forceinline__ float rsqrt_nr(float v) {
  const float r = rsqrtf(v);
  return r * fmaf(-0.5f * v * r, r, 1.5f);
}
__device__ __forceinline__ float acc_max(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ double acc_max(double a, double b) { return fmax(a, b); }
template <typename A> __device__ __forceinline__ A acc_neg_inf();
template <> __device__ __forceinline__ float acc_neg_inf<float>() { return -__int_as_float(0x7f800000); }
template <> __device__ __forceinline__ double acc_neg_inf<double>() { return -__longlong_as_double(0x7ff0000000000000LL); }

// ---------------------------------------------------------------------------------------------
// vectors of V elements (V * sizeof(T) <= 16 bytes), naturally aligned
// ---------------------------------------------------------------------------------------------
template <typename T, int V> struct alignas(sizeof(T) * V) Vec { T v[V]; };

template <typename T, int V> __device__ __forceinline__ Vec<T, V> ld_vec(const T* p) {
  return *reinterpret_cast<const Vec<T, V>*>(p);
}
template <typename T, int V> __device__ __forceinline__ void st_vec(T* p, const Vec<T, V>& v) {
  *reinterpret_cast<Vec<T, V>*>(p) = v;
}

__host__ __device__ inline bool is_aligned(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

// ---------------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------------
struct SumOp { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return a + b; } };
struct MaxOp { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return acc_max(a, b); } };

template <typename A, typename Op> __device__ __forceinline__ A warp_reduce(A v, Op op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Whole-CTA reduction; every thread gets the same value (partials are combined in warp order).
// scratch: >= 32 elements of A in shared memory.
template <typename A, typename Op> __device__ __forceinline__ A block_reduce(A v, A* scratch, Op op) {
  v = warp_reduce(v, op);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  A r = scratch[0];
  for (int i = 1; i < nw; ++i) r = op(r, scratch[i]);
  return r;
}

// Reduction over the TPR threads that share a row in the generic kernels: TPR == 32 is a warp,
// TPR == 0 the whole CTA.
template <int TPR, typename A, typename Op> __device__ __forceinline__ A row_reduce(A v, A* scratch, Op op) {
  if constexpr (TPR == 32) return warp_reduce(v, op);
  else return block_reduce(v, scratch, op);
}

// ---------------------------------------------------------------------------------------------
// device status word: kernels record a b2n_status here instead of trapping
// ---------------------------------------------------------------------------------------------
// (one int per device, passed to the kernels as an argument: see device_status_ptr below)
__device__ __forceinline__ void record_status(int* status, int code) { atomicCAS(status, 0, code); }

// 2^v by the hardware approximation (relative error ~2^-22: invisible after rounding to 8 or 11 bits of
// mantissa, which is where the kernels for 16-bit storage use it).
// 2^v on the special-function unit, results below 2^-126 flushed to zero: ONE instruction.  (Without .ftz the
// compiler wraps it in a compare and two conditional multiplies to keep subnormal results — four issue slots per
// exp, which the softmax kernels spend per element.)  Only kernels with 16-bit storage use it, on arguments <= 0:
// what is flushed is below 1.2e-38, far under one unit in the last place of anything such a result is compared at.
__device__ __forceinline__ float ex2_approx(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
constexpr float kLog2e = 1.4426950408889634f;
// exp(d) for a result stored as TO: the approximation for 16-bit storage, the precise function otherwise
template <typename TO> __device__ __forceinline__ float exp_for(float d) {
  if constexpr (sizeof(TO) <= 2) return ex2_approx(d * kLog2e);
  else return expf(d);
}
template <typename TO> __device__ __forceinline__ double exp_for(double d) { return exp(d); }

// Programmatic dependent launch (sm_90+).  A kernel launched with launch_pdl() below may become
// resident while the kernel before it in the stream is still running: pdl_wait() holds it until
// that kernel has completed and its writes are visible, so everything before the call (barrier
// setup, register reallocation) overlaps the predecessor's tail and the launch latency disappears.
// No global memory may be touched before pdl_wait().  pdl_launch_dependents() tells the scheduler
// that the NEXT kernel in the stream may be made resident as soon as SMs free up.  Both are no-ops
// in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// ---------------------------------------------------------------------------------------------
// sm_100a PTX: mbarrier + bulk-async (TMA) copies between global and shared memory.
// No cluster multicast is used anywhere.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after ~2 s of wall time, records B2N_ERR_TIMEOUT and returns false; the
// caller then leaves its loop.  Threads that wait on the same barrier give up together (the
// barrier either completed for all of them or for none), which keeps the exit uniform across the
// threads that also meet at a named barrier.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0x3ffu) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
      record_status(status, B2N_ERR_TIMEOUT);
      return false;
    }
  }
}
// global -> shared bulk copy, completion counted in bytes on an mbarrier of this CTA.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// shared -> global bulk copy, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still have to READ their shared-memory source.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make this thread's generic-proxy shared-memory writes visible to the async proxy (bulk stores).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// 16-byte shared-memory accesses by 32-bit shared address
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Packed fp32 arithmetic (sm_100: one instruction works on two fp32 lanes, each rounded exactly as
// its scalar counterpart).  The row kernels are bound by instruction issue, not by the FMA pipe,
// so halving the instruction count of the element-wise math is a direct win.
__device__ __forceinline__ float2 bcast2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float hsum2(float2 a) { return a.x + a.y; }

// 16 bytes <-> VEC floats for each storage type (VEC = 16 / sizeof(T))
template <typename T> struct Pack16;
template <> struct Pack16<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void unpack(const uint4& p, float* f) {
    f[0] = __uint_as_float(p.x); f[1] = __uint_as_float(p.y); f[2] = __uint_as_float(p.z); f[3] = __uint_as_float(p.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ void unpack2(const uint4& p, float2* f) {
    f[0] = make_float2(__uint_as_float(p.x), __uint_as_float(p.y));
    f[1] = make_float2(__uint_as_float(p.z), __uint_as_float(p.w));
  }
  static __device__ __forceinline__ uint4 pack2(const float2* f) {
    return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x), __float_as_uint(f[1].y));
  }
};
template <> struct Pack16<bf16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void unpack(const uint4& p, float* f) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ void unpack2(const uint4& p, float2* f) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  }
  static __device__ __forceinline__ uint4 pack2(const float2* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __float22bfloat162_rn(f[i]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Pack16<f16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void unpack(const uint4& p, float* f) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ void unpack2(const uint4& p, float2* f) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
  }
  static __device__ __forceinline__ uint4 pack2(const float2* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __float22half2_rn(f[i]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ---------------------------------------------------------------------------------------------
// host-side helpers shared by the launchers
// ---------------------------------------------------------------------------------------------
struct DeviceInfo {
  int sm_count;
  int max_smem_optin;  // bytes of dynamic shared memory a CTA may opt into
};
const DeviceInfo& device_info();          // cached per device
bool device_ready();                      // the current device's attributes, status word and tile counters were found
int check_cuda(cudaError_t e);            // records e for b2n_last_cuda_error; returns B2N_OK / B2N_ERR_CUDA
int forced_path();                        // b2n_set_path value of this thread
void note_path(const char* name);         // records the family used by the last launch
int* device_status_ptr();                 // device address of the status word of the current device
bool softmax_safe_mode();                 // this thread's softmax forward is the 'safe' variant (set by the C ABI)
unsigned* next_tile_counter();            // a zeroed {next tile, CTAs finished} pair for one ring-kernel launch
int launched();                           // counts one kernel launch; returns check_cuda(cudaGetLastError())

// Launch with the programmatic-stream-serialization attribute (see pdl_wait above).  The kernel
// must call pdl_wait() before its first global-memory access.
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return check_cuda(e);
  return launched();
}

// Brackets one main-kernel launch with a pair of CUDA events on its stream while this thread has
// profiling switched on (b2n_profile_begin); otherwise does nothing.
struct ProfileScope {
  ProfileScope(const char* kernel_name, cudaStream_t st);
  ~ProfileScope();
  int slot;
  cudaStream_t stream;
};

}  // namespace b2n
