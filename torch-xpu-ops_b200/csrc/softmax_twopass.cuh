// Two-pass ring kernels for softmax / log-softmax rows of any length (BASELINE config 5:
// 128 256 bf16 per row).
//
// One persistent CTA per SM owns whole rows and streams each row through the shared-memory ring
// TWICE, in 32 KB chunks: pass 1 folds the chunks into per-thread running statistics (max and
// sum exp for the forward, sum dy or sum y*dy for the backward) and stores nothing; one
// CTA-wide reduction per row; pass 2 streams the same chunks again, writes the result in place
// and bulk-stores it.  The second read of a row follows its first by one row length (250 KB),
// and all 148 CTAs together keep ~37 MB of such rows in flight, far less than the 126 MB L2 — so
// pass 2 is served from L2 and HBM sees one read and one write per element; the ring keeps
// loads in flight continuously through both passes, the reduction and the stores.
//
// Same roles as the other ring kernels (ring.cuh): 16 consumer warps, one producer warpgroup that
// gives its registers to the consumers, every wait an mbarrier wait with a time limit.
#pragma once
#include <type_traits>

#include "ring.cuh"
#include "softmax_generic.cuh"
#include "softmax_ring.cuh"

namespace b2n {

constexpr int kTwoPassChunkVecs = 2048;  // 16-byte vectors per chunk: 4 per consumer thread

// exp for a value already reduced by the row maximum: expf for fp32 storage, the hardware 2^x for
// 16-bit storage (see RowExp in softmax_ring.cuh)
template <typename T> __device__ __forceinline__ float row_exp2p(float d) {
  if constexpr (sizeof(T) == 4) return expf(d);
  else return ex2_approx(d * kLog2e);
}

// BWD == false: in0 = x, out = y.   BWD == true: in0 = dy, in1 = y (forward output), out = dx.
template <typename T, bool LOG, bool BWD, bool SAFE>
__global__ void __launch_bounds__(kRingBlock, 1)
softmax_twopass_kernel(const T* __restrict__ in0, const T* __restrict__ in1, T* __restrict__ out, int64_t M,
                       int64_t N, int S, int* status, unsigned* tile_ctr) {
  using P = Pack16<T>;
  constexpr int VEC = P::VEC, VH = VEC / 2;
  constexpr int NIN2 = BWD ? 2 : 1;                 // tensors staged per chunk in pass 2
  constexpr int NIN1 = (BWD && !LOG) ? 2 : 1;       // ... in pass 1 (log-softmax backward needs only dy)
  constexpr int VPT = kTwoPassChunkVecs / kRingThreads;
  constexpr uint32_t kChunkBytes = kTwoPassChunkVecs * 16u;
  constexpr uint32_t kStageBytes = kChunkBytes * NIN2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  RingShared* rs = reinterpret_cast<RingShared*>(smem_raw);
  unsigned char* stages = smem_raw + kRingHeaderBytes;

  const int tid = threadIdx.x;
  const int64_t nvec = N / VEC;
  const int nch = static_cast<int>((nvec + kTwoPassChunkVecs - 1) / kTwoPassChunkVecs);
  auto chunk_vecs = [&](int c) {
    const int64_t left = nvec - static_cast<int64_t>(c) * kTwoPassChunkVecs;
    return static_cast<int>(left < kTwoPassChunkVecs ? left : kTwoPassChunkVecs);
  };

  ring_init(rs, S, kRingThreads / 32);

  if (tid >= kRingThreads) {
    // ---------------- producer ----------------
    ring_producer_regs();
    if (tid == kRingThreads) {
      // Rows are handed out dynamically (as the ring kernels hand out tiles): the CTA's first row is
      // blockIdx.x, later ones come from the global counter, fetched one row ahead.  The row of
      // every tile is left in the stage's tile_id slot — for this thread's own store later, and as
      // the end marker (-1) the consumers look for at the start of a row.
      auto fetch_row = [&]() {
        const unsigned r = gridDim.x + atomicAdd(tile_ctr, 1u);
        return r < static_cast<unsigned>(M) ? static_cast<int>(r) : -1;
      };
      int next_row = static_cast<int>(blockIdx.x);
      int l_row = -1, l_pass = 0, l_chunk = 0, l_stage = 0;  // cursor of the next tile to load
      unsigned loads_issued = 0, retired = 0;
      bool ended = false;
      auto issue_next_load = [&]() {
        if (l_pass == 0 && l_chunk == 0) {  // a new row
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
                             static_cast<size_t>(l_chunk) * kTwoPassChunkVecs) * 16;
        unsigned char* dst = stages + static_cast<size_t>(l_stage) * kStageBytes;
        const int nin = l_pass == 0 ? NIN1 : NIN2;
        rs->tile_id[l_stage] = l_row;
        mbar_arrive_expect_tx(&rs->full[l_stage], bytes * nin);
        bulk_g2s(dst, reinterpret_cast<const unsigned char*>(in0) + goff, bytes, &rs->full[l_stage]);
        if (nin == 2) bulk_g2s(dst + kChunkBytes, reinterpret_cast<const unsigned char*>(in1) + goff, bytes, &rs->full[l_stage]);
        ++loads_issued;
        if (++l_chunk == nch) {
          l_chunk = 0;
          if (++l_pass == 2) l_pass = 0;
        }
        if (++l_stage == S) l_stage = 0;
      };
      for (int k = 0; k < S && !ended; ++k) issue_next_load();

      // cursor of the tile whose completion is awaited
      int pass = 0, chunk = 0, stage = 0;
      uint32_t phase = 0;
      int pending = 0;                // bulk stores issued and not yet known to have drained (0..2)
      int64_t free_upto = -1;         // every tile <= free_upto has released its stage
      unsigned t = 0;
      for (; t < loads_issued; ++t) {
        const int row = rs->tile_id[stage];  // this thread's own earlier store
        if (!mbar_wait(&rs->done[stage], phase, status)) break;
        if (pass == 0) {
          // nothing to store; stages are recycled in tile order, so older stores must have drained
          if (pending > 0) { bulk_wait_read<0>(); pending = 0; }
          free_upto = t;
        } else {
          const size_t goff = (static_cast<size_t>(row) * static_cast<size_t>(nvec) +
                               static_cast<size_t>(chunk) * kTwoPassChunkVecs) * 16;
          bulk_s2g(reinterpret_cast<unsigned char*>(out) + goff, stages + static_cast<size_t>(stage) * kStageBytes,
                   static_cast<uint32_t>(chunk_vecs(chunk)) * 16u);
          bulk_commit();
          if (++pending > 1) { bulk_wait_read<1>(); pending = 1; }
          free_upto = static_cast<int64_t>(t) - pending;
        }
        while (!ended && static_cast<int64_t>(loads_issued) - S <= free_upto) issue_next_load();
        if (++chunk == nch) {
          chunk = 0;
          if (++pass == 2) pass = 0;
        }
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
  const float ninf = acc_neg_inf<float>();
  int red_phase = 0;
  int stage = 0;
  uint32_t phase = 0;
  auto next_stage = [&]() { if (++stage == S) { stage = 0; phase ^= 1u; } };
  auto release = [&]() {
    fence_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&rs->done[stage]);
  };

  for (;;) {  // one iteration per row, until the producer's end marker
    // ---- pass 1: running statistics over the row's chunks ------------------------------------------
    float pm = ninf, ps = 0.0f;          // forward: per-thread running max and sum of exp(x - pm)
    float2 acc2[2] = {bcast2(0.0f), bcast2(0.0f)};  // backward: sum dy or sum y*dy
    bool ok = true;
    for (int c = 0; c < nch; ++c) {
      ok = mbar_wait(&rs->full[stage], phase, status);
      if (ok && c == 0 && rs->tile_id[stage] < 0) ok = false;  // no rows left (uniform: every consumer reads the same slot)
      if (!ok) break;
      const int cv = chunk_vecs(c);
      const uint32_t s0 = stages_u32 + static_cast<uint32_t>(stage) * kStageBytes, s1 = s0 + kChunkBytes;
      // chunks of the full size (all but a row's last) run the copy of the loop without range checks
      auto run_chunk = [&](auto full_chunk) {
        constexpr bool FC = decltype(full_chunk)::value;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * kRingThreads;
          if (FC || v < cv) {
            float2 f[VH];
            P::unpack2(lds128(s0 + v * 16), f);
            if constexpr (!BWD) {
              float vm = ninf;
#pragma unroll
              for (int e = 0; e < VH; ++e) vm = fmaxf(vm, fmaxf(f[e].x, f[e].y));
              // one rescale per 16-byte vector instead of one per element
              const float nm = fmaxf(pm, vm);
              const float scale = (pm == ninf) ? 0.0f : row_exp2p<T>(pm - nm);
              const float base = (nm == ninf) ? 0.0f : nm;  // all -inf so far: exp(-inf - 0) = 0; NaN stays NaN
              float2 a = bcast2(0.0f);
              if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int e = 0; e < VH; ++e) a = add2(a, make_float2(expf(f[e].x - base), expf(f[e].y - base)));
              } else {
                // 2^(x*log2e - base*log2e): one packed FMA per pair, then the hardware 2^x
                const float2 l2e = bcast2(kLog2e), nb = bcast2(-base * kLog2e);
#pragma unroll
                for (int e = 0; e < VH; ++e) {
                  const float2 tt = fma2(f[e], l2e, nb);
                  a = add2(a, make_float2(ex2_approx(tt.x), ex2_approx(tt.y)));
                }
              }
              ps = fmaf(ps, scale, hsum2(a));
              pm = nm;
            } else if constexpr (LOG) {
#pragma unroll
              for (int e = 0; e < VH; ++e) acc2[e & 1] = add2(acc2[e & 1], f[e]);
            } else {
              float2 yv[VH];
              P::unpack2(lds128(s1 + v * 16), yv);
#pragma unroll
              for (int e = 0; e < VH; ++e) acc2[e & 1] = fma2(f[e], yv[e], acc2[e & 1]);
            }
          }
        }
      };
      if (cv == kTwoPassChunkVecs) run_chunk(std::true_type{});
      else run_chunk(std::false_type{});
      release();
      next_stage();
    }
    if (!ok) break;  // uniform: all consumers waited on the same barrier

    // ---- one reduction over the 512 consumer threads -----------------------------------------------
    float r0, r1 = 0.0f;
    if constexpr (!BWD) {
      float mx[1] = {pm};
      group_reduce<kRingThreads, 1>(mx, rs->red, 0, tid, red_phase, MaxOp());
      // a NaN running sum must survive a thread maximum of -inf (0 * exp(...) would hide it otherwise)
      float sc[1] = {(pm == ninf) ? ((ps != ps) ? ps : 0.0f) : ps * row_exp2p<T>(pm - mx[0])};
      group_reduce<kRingThreads, 1>(sc, rs->red, 0, tid, red_phase, SumOp());
      r0 = mx[0];
      r1 = (r0 == -ninf) ? acc_nan<float>() : sc[0];  // +inf in the row: exp(inf - inf)
    } else {
      float sm[1] = {hsum2(add2(acc2[0], acc2[1]))};
      group_reduce<kRingThreads, 1>(sm, rs->red, 0, tid, red_phase, SumOp());
      r0 = sm[0];
    }

    // ---- pass 2: the same chunks again (from L2), result in place, out through the producer ----------
    const float lg = (!BWD && LOG) ? logf(r1) : 0.0f;
    const float2 noff = bcast2(-(r0 + lg)), inv = bcast2((!BWD && !LOG) ? 1.0f / r1 : 0.0f);
    // safe softmax: a row of -inf gives zeros, not NaN (a NaN in the row has made the sum NaN and still wins)
    const bool zero_row = SAFE && !BWD && r0 == ninf && !(r1 != r1);
    const float2 l2e = bcast2(kLog2e), c2 = bcast2(-r0 * kLog2e), ns = bcast2(-r0);
    for (int c = 0; c < nch; ++c) {
      ok = mbar_wait(&rs->full[stage], phase, status);
      if (!ok) break;
      const int cv = chunk_vecs(c);
      const uint32_t s0 = stages_u32 + static_cast<uint32_t>(stage) * kStageBytes, s1 = s0 + kChunkBytes;
      // chunks of the full size (all but a row's last) run the copy of the loop without range checks
      auto run_chunk = [&](auto full_chunk) {
        constexpr bool FC = decltype(full_chunk)::value;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * kRingThreads;
          if (FC || v < cv) {
            float2 f[VH], o[VH];
            P::unpack2(lds128(s0 + v * 16), f);
            if constexpr (!BWD) {
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                if constexpr (LOG) {
                  if constexpr (sizeof(T) == 4) o[e] = make_float2((f[e].x - r0) - lg, (f[e].y - r0) - lg);
                  else o[e] = add2(f[e], noff);
                } else if constexpr (sizeof(T) == 4) {
                  o[e] = make_float2(expf(f[e].x - r0) / r1, expf(f[e].y - r0) / r1);
                } else {
                  const float2 tt = fma2(f[e], l2e, c2);
                  o[e] = mul2(make_float2(ex2_approx(tt.x), ex2_approx(tt.y)), inv);
                }
              }
            } else {
              float2 yv[VH];
              P::unpack2(lds128(s1 + v * 16), yv);
#pragma unroll
              for (int e = 0; e < VH; ++e) {
                if constexpr (LOG) {
                  float2 ey;
                  if constexpr (sizeof(T) == 4) {
                    ey = make_float2(expf(yv[e].x), expf(yv[e].y));
                  } else {
                    const float2 tt = mul2(yv[e], l2e);
                    ey = make_float2(ex2_approx(tt.x), ex2_approx(tt.y));
                  }
                  o[e] = fma2(ey, ns, f[e]);           // dy - exp(y) * sum
                } else {
                  o[e] = mul2(yv[e], add2(f[e], ns));  // y * (dy - sum)
                }
              }
            }
            if constexpr (SAFE) sts128(s0 + v * 16, zero_row ? make_uint4(0u, 0u, 0u, 0u) : P::pack2(o));
            else sts128(s0 + v * 16, P::pack2(o));
          }
        }
      };
      if (cv == kTwoPassChunkVecs) run_chunk(std::true_type{});
      else run_chunk(std::false_type{});
      release();
      next_stage();
    }
    if (!ok) break;
  }
}

}  // namespace b2n
