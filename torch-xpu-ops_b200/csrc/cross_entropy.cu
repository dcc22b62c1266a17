// Fused tail of cross-entropy: nll_loss_backward followed by _log_softmax_backward_data in one
// pass, without the dense [M, C] gradient in between.
//
// The reference (like PyTorch) forms that gradient in two steps: nll_loss_backward zero-fills
// grad[M, C] and scatters -w*g at (i, t_i) (LossNLLKernel.cpp:325-380, LossNLL.cpp:35-56), then
// _log_softmax_backward_data reads it back together with the log-probabilities:
// dx = grad - exp(logp) * sum_j grad  (SoftMaxKernels.cpp host_softmax_backward<Log>, :2180-2240).
// With only one non-zero per row the sum is that value, so
//
//     dx[i, j] = s_i * (exp(logp[i, j]) - [j == t_i]),   s_i = w[t_i] * g_i  (/ total_weight for mean)
//
// and rows whose target is ignore_index are zero.  One read of logp and one write of dx: 4 bytes
// per element instead of 8 (zero-fill + dense gradient read) on top of them.
//
// Kernel: the same shared-memory ring as the other row kernels (ring.cuh), one pass, chunks of
// 32 KB of a row per stage; a persistent CTA takes whole rows (handed out dynamically) so the
// per-row scalars (target, scale) are fetched once per row.  dx may alias logp.
#include <atomic>
#include <type_traits>

#include "launchers.h"
#include "plan.h"
#include "ring.cuh"
#include "softmax_ring.cuh"

namespace b2n {
namespace {

constexpr int kCeChunkVecs = 2048;  // 16-byte vectors per chunk: 4 per consumer thread

template <typename IdxT> __device__ __forceinline__ int64_t ce_load_target(const void* target, int64_t i) {
  return static_cast<int64_t>(static_cast<const IdxT*>(target)[i]);
}

// Per-row scalars: the scale s_i (0 for an ignored or out-of-range target) and the target column.
template <typename T, typename IdxT>
__device__ __forceinline__ void ce_row_params(int64_t row, const void* target, const T* weight, const T* grad_out,
                                              const T* total_weight, int64_t C, int reduction,
                                              int64_t ignore_index, int* status, float& s, int64_t& t) {
  using A = acc_t<T>;
  t = ce_load_target<IdxT>(target, row);
  s = 0.0f;
  if (t == ignore_index) { t = -1; return; }
  if (t < 0 || t >= C) {
    record_status(status, B2N_ERR_TARGET_RANGE);
    t = -1;
    return;
  }
  const A w = weight ? to_acc<A>(weight[t]) : A(1);
  A g = to_acc<A>(reduction == B2N_REDUCE_NONE ? grad_out[row] : grad_out[0]);
  if (reduction == B2N_REDUCE_MEAN) g = g / to_acc<A>(*total_weight);
  s = static_cast<float>(w * g);
}

template <typename T, typename IdxT>
__global__ void __launch_bounds__(kRingBlock, 1)
ce_bwd_ring_kernel(const T* __restrict__ logp, const void* __restrict__ target, const T* __restrict__ weight,
                   const T* __restrict__ grad_out, const T* __restrict__ total_weight, T* __restrict__ dx,
                   int64_t M, int64_t N, int reduction, int64_t ignore_index, int S, int* status,
                   unsigned* tile_ctr) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, VH = VEC / 2;
  constexpr int VPT = kCeChunkVecs / kRingThreads;
  constexpr uint32_t kStageBytes = kCeChunkVecs * 16u;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  const int tid = threadIdx.x;
  const int64_t nvec = N / VEC;
  const int nch = static_cast<int>((nvec + kCeChunkVecs - 1) / kCeChunkVecs);
  auto chunk_vecs = [&](int c) {
    const int64_t left = nvec - static_cast<int64_t>(c) * kCeChunkVecs;
    return static_cast<int>(left < kCeChunkVecs ? left : kCeChunkVecs);
  };

  ring_init(rs, S, kRingThreads / 32);

  if (tid >= kRingThreads) {
    // ---------------- producer ----------------
    ring_producer_regs();
    if (tid == kRingThreads) {
      // Rows are handed out dynamically: the CTA's first row is blockIdx.x, later ones come from the
      // global counter, fetched one row ahead.  The row of every tile is left in the stage's tile_id
      // slot — for the consumers (which row's target and scale apply), for this thread's own store
      // later, and as the end marker (-1).
      auto fetch_row = [&]() {
        const unsigned r = gridDim.x + atomicAdd(tile_ctr, 1u);
        return r < static_cast<unsigned>(M) ? static_cast<int>(r) : -1;
      };
      int next_row = static_cast<int>(blockIdx.x);
      int l_row = -1, l_chunk = 0, l_stage = 0;  // cursor of the next tile to load
      unsigned loads_issued = 0, retired = 0;
      bool ended = false;
      auto issue_next_load = [&]() {
        if (l_chunk == 0) {  // a new row
          l_row = next_row;
          if (l_row < 0) {
            rs->tile_id[l_stage] = -1;
            mbar_arrive(&rs->full[l_stage]);
            ended = true;
            retired = atomicAdd(tile_ctr + 1, 1u);
            return;
          }
          next_row = fetch_row();
        }
        const uint32_t bytes = static_cast<uint32_t>(chunk_vecs(l_chunk)) * 16u;
        const size_t goff = (static_cast<size_t>(l_row) * static_cast<size_t>(nvec) +
                             static_cast<size_t>(l_chunk) * kCeChunkVecs) * 16;
        rs->tile_id[l_stage] = l_row;
        mbar_arrive_expect_tx(&rs->full[l_stage], bytes);
        bulk_g2s(stages + static_cast<size_t>(l_stage) * kStageBytes,
                 reinterpret_cast<const unsigned char*>(logp) + goff, bytes, &rs->full[l_stage]);
        ++loads_issued;
        if (++l_chunk == nch) l_chunk = 0;
        if (++l_stage == S) l_stage = 0;
      };
      for (int k = 0; k < S && !ended; ++k) issue_next_load();

      int chunk = 0, stage = 0;  // cursor of the tile whose completion is awaited
      uint32_t phase = 0;
      unsigned t = 0;
      for (; t < loads_issued; ++t) {
        const int row = rs->tile_id[stage];  // this thread's own earlier store
        const size_t goff = (static_cast<size_t>(row) * static_cast<size_t>(nvec) +
                             static_cast<size_t>(chunk) * kCeChunkVecs) * 16;
        if (!mbar_wait(&rs->done[stage], phase, status)) break;
        bulk_s2g(reinterpret_cast<unsigned char*>(dx) + goff, stages + static_cast<size_t>(stage) * kStageBytes,
                 static_cast<uint32_t>(chunk_vecs(chunk)) * 16u);
        bulk_commit();
        // the store of tile t-1 has read its stage once at most one group is pending; that stage is
        // where load number t-1+S belongs
        if (t > 0 && !ended) {
          bulk_wait_read<1>();
          issue_next_load();
        }
        if (++chunk == nch) chunk = 0;
        if (++stage == S) { stage = 0; phase ^= 1u; }
      }
      // if a wait gave up, let the loads already issued land before the CTA's shared memory goes away
      for (unsigned j = t; j < loads_issued; ++j) {
        mbar_wait(&rs->full[stage], phase, status);
        if (++stage == S) { stage = 0; phase ^= 1u; }
      }
      bulk_wait_all<0>();
      // the last CTA to stop taking rows zeroes the counter pair for the slot's next launch
      if (!ended) retired = atomicAdd(tile_ctr + 1, 1u);
      if (retired == gridDim.x - 1) {
        tile_ctr[0] = 0;
        tile_ctr[1] = 0;
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  ring_consumer_regs();
  const uint32_t stages_u32 = smem_u32(stages);
  int stage = 0;
  uint32_t phase = 0;
  for (;;) {  // one iteration per row, until the producer's end marker
    // the row's first chunk names the row; its target and scale are fetched then (the stages already
    // filled behind it keep the memory pipe busy meanwhile)
    bool ok = mbar_wait(&rs->full[stage], phase, status);
    if (!ok) break;
    const int row = rs->tile_id[stage];
    if (row < 0) break;  // uniform: every consumer reads the same slot
    float s;
    int64_t t;
    ce_row_params<T, IdxT>(row, target, weight, grad_out, total_weight, N, reduction, ignore_index, status, s, t);
    const int64_t tv = t >= 0 ? t / VEC : -1;  // the vector and the lane of the target column
    const int te = t >= 0 ? static_cast<int>(t % VEC) : 0;
    const float2 s2 = bcast2(s), l2e = bcast2(kLog2e);
    for (int c = 0; c < nch; ++c) {
      if (c > 0) ok = mbar_wait(&rs->full[stage], phase, status);
      if (!ok) break;
      const int cv = chunk_vecs(c);
      const uint32_t s0 = stages_u32 + static_cast<uint32_t>(stage) * kStageBytes;
      const int64_t tv_local = tv - static_cast<int64_t>(c) * kCeChunkVecs;  // target vector within this chunk
      // chunks of the full size (all but a row's last) run the copy of the loop without range checks
      auto run_chunk = [&](auto full_chunk) {
        constexpr bool FC = decltype(full_chunk)::value;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * kRingThreads;
          if (FC || v < cv) {
            float2 f[VH], o[VH];
            P::unpack2(lds128(s0 + v * 16), f);
#pragma unroll
            for (int e = 0; e < VH; ++e) {
              float2 ey;
              if constexpr (sizeof(T) == 4) {
                ey = make_float2(expf(f[e].x), expf(f[e].y));
              } else {
                const float2 tt = mul2(f[e], l2e);
                ey = make_float2(ex2_approx(tt.x), ex2_approx(tt.y));
              }
              o[e] = mul2(ey, s2);
            }
            if (v == tv_local) {  // one vector per row: s * (exp(y) - 1) at the target column
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                const float yx = f[e].x, yy = f[e].y;
                if (2 * e == te) o[e].x = s * ((sizeof(T) == 4 ? expf(yx) : ex2_approx(yx * kLog2e)) - 1.0f);
                if (2 * e + 1 == te) o[e].y = s * ((sizeof(T) == 4 ? expf(yy) : ex2_approx(yy * kLog2e)) - 1.0f);
              }
            }
            sts128(s0 + v * 16, P::pack2(o));
          }
        }
      };
      if (cv == kCeChunkVecs) run_chunk(std::true_type{});
      else run_chunk(std::false_type{});
      fence_async_smem();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&rs->done[stage]);
      if (++stage == S) { stage = 0; phase ^= 1u; }
    }
    if (!ok) break;  // uniform: all consumers waited on the same barrier
  }
}

// Any N, any alignment, fp64: one CTA per row at a time, plain loads and stores.
template <typename T, typename IdxT>
__global__ void ce_bwd_generic_kernel(const T* __restrict__ logp, const void* __restrict__ target,
                                      const T* __restrict__ weight, const T* __restrict__ grad_out,
                                      const T* __restrict__ total_weight, T* __restrict__ dx, int64_t M, int64_t N,
                                      int reduction, int64_t ignore_index, int* status) {
  using A = acc_t<T>;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    int64_t t = ce_load_target<IdxT>(target, row);
    A s = A(0);
    if (t == ignore_index) {
      t = -1;
    } else if (t < 0 || t >= N) {
      if (threadIdx.x == 0) record_status(status, B2N_ERR_TARGET_RANGE);
      t = -1;
    } else {
      const A w = weight ? to_acc<A>(weight[t]) : A(1);
      A g = to_acc<A>(reduction == B2N_REDUCE_NONE ? grad_out[row] : grad_out[0]);
      if (reduction == B2N_REDUCE_MEAN) g = g / to_acc<A>(*total_weight);
      s = w * g;
    }
    const T* y = logp + row * N;
    T* o = dx + row * N;
    for (int64_t j = threadIdx.x; j < N; j += blockDim.x) {
      const A e = acc_exp(to_acc<A>(y[j]));
      o[j] = from_acc<T>(s * (j == t ? e - A(1) : e));
    }
  }
}

template <typename T, typename IdxT>
int ce_bwd_typed(const void* logp_, const void* target, const void* weight_, const void* grad_out_,
                 const void* total_weight_, void* dx_, int64_t M, int64_t N, int reduction, int64_t ignore_index,
                 cudaStream_t st) {
  const T* logp = static_cast<const T*>(logp_);
  const T* weight = static_cast<const T*>(weight_);
  const T* grad_out = static_cast<const T*>(grad_out_);
  const T* total_weight = static_cast<const T*>(total_weight_);
  T* dx = static_cast<T*>(dx_);
  if (M == 0 || N == 0) return B2N_OK;
  const int forced = forced_path();
  const DeviceInfo& di = device_info();
  if constexpr (sizeof(T) <= 4 && !std::is_same<T, double>::value) {
    constexpr int VEC = Pack16<T>::VEC;
    // rows shorter than a few chunks would leave most of each stage empty: they take the plain kernel
    if (forced != B2N_PATH_GENERIC && is_aligned(logp, 16) && is_aligned(dx, 16) && N % VEC == 0 &&
        (forced == B2N_PATH_RING || N * static_cast<int64_t>(sizeof(T)) >= 16384)) {
      auto kernel = ce_bwd_ring_kernel<T, IdxT>;
      static std::atomic<uint64_t> mask{0};
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda(cudaGetLastError());
      const uint64_t bit = 1ull << (dev & 63);
      if (!(mask.load(std::memory_order_acquire) & bit)) {
        if (int e = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    di.max_smem_optin)))
          return e;
        mask.fetch_or(bit, std::memory_order_release);
      }
      const int64_t stage = static_cast<int64_t>(kCeChunkVecs) * 16;
      int64_t stages = (static_cast<int64_t>(di.max_smem_optin) - kRingHeaderBytes) / stage;
      if (stages > kMaxStages) stages = kMaxStages;
      const int tuned = ring_tuning().stages;
      if (tuned > 0 && tuned < stages) stages = tuned;
      if (stages >= 3) {
        note_path("ring");
        const size_t smem = static_cast<size_t>(kRingHeaderBytes + stages * stage);
        const int ctas = persistent_ctas(di.sm_count);
        const int grid = static_cast<int>(M < ctas ? M : ctas);
        ProfileScope prof("cross_entropy_bwd_ring", st);
        return launch_pdl(kernel, dim3(grid), dim3(kRingBlock), smem, st, logp, target, weight, grad_out, total_weight,
                          dx, M, N, reduction, ignore_index, static_cast<int>(stages), device_status_ptr(), next_tile_counter());
      }
    }
  }
  if (forced == B2N_PATH_RING || forced == B2N_PATH_CLUSTER || forced == B2N_PATH_TWOPASS) return B2N_ERR_BAD_ARG;
  note_path("generic");
  ProfileScope prof("cross_entropy_bwd_generic", st);
  const int64_t cap = static_cast<int64_t>(di.sm_count) * 8;
  const int grid = static_cast<int>(M < cap ? M : cap);
  ce_bwd_generic_kernel<T, IdxT><<<grid, N <= 4096 ? 256 : 1024, 0, st>>>(
      logp, target, weight, grad_out, total_weight, dx, M, N, reduction, ignore_index, device_status_ptr());
  return launched();
}

}  // namespace

int launch_cross_entropy_bwd(const void* logp, const void* target, const void* weight, const void* grad_out,
                             const void* total_weight, void* dx, int64_t M, int64_t C, int reduction,
                             int64_t ignore_index, int dtype, bool u8, cudaStream_t st) {
  switch (dtype) {
    case B2N_F32:
      return u8 ? ce_bwd_typed<float, uint8_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st)
                : ce_bwd_typed<float, int64_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st);
    case B2N_F16:
      return u8 ? ce_bwd_typed<f16, uint8_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st)
                : ce_bwd_typed<f16, int64_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st);
    case B2N_BF16:
      return u8 ? ce_bwd_typed<bf16, uint8_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st)
                : ce_bwd_typed<bf16, int64_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st);
    case B2N_F64:
      return u8 ? ce_bwd_typed<double, uint8_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st)
                : ce_bwd_typed<double, int64_t>(logp, target, weight, grad_out, total_weight, dx, M, C, reduction, ignore_index, st);
    default: return B2N_ERR_UNSUPPORTED_DTYPE;
  }
}

}  // namespace b2n
