// Host-side launch planning for the ring kernels.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "ring.cuh"

namespace b2n {

struct RingPlan {
  bool ok = false;
  int group = 0;   // threads per row: 32, 64, 128, 256 or 512
  int ng = 0;      // row groups per CTA = 512 / group
  int rpg = 1;     // rows per group per tile
  int stages = 0;  // ring depth
  int lag = 1;     // stores left in flight before a stage is refilled (see RingProducer::after_tile)
  int grid = 0;    // persistent CTAs
  size_t smem = 0; // dynamic shared memory per CTA
};

// Per-thread overrides for tuning sweeps (0 = automatic); set through b2n_set_tuning.
struct RingTuning {
  int rpg = 0, stages = 0, lag = 0;
  int cluster = 0;  // CTAs per row in the cluster kernels (1, 2, 4 or 8)
  int sm_margin = 0;  // SMs the persistent kernels leave free (for a collective's kernel running beside them)
  int tile_kb = 0;    // non-last-dim softmax: shared memory one staged tile may take (0: automatic)
  unsigned long long* trace_buf = nullptr;  // device buffer for the event trace (diagnostic), or null
  unsigned trace_cap = 0;                   // records it can hold
};
RingTuning& ring_tuning();

// CTAs of a persistent kernel on a device with sm_count SMs: one per SM, less the margin the caller asked for.
inline int persistent_ctas(int sm_count) {
  const int n = sm_count - ring_tuning().sm_margin;
  return n < 1 ? 1 : n;
}

// N elements of `esize` bytes per row, `nin` tensors staged per tile, `ept` elements per thread.
// `target`: bytes per tensor per tile to aim for; `default_lag`: see RingPlan::lag; `reserve`: bytes of
// shared memory the kernel keeps between the ring header and the stages.
// Not ok when the row is not a multiple of 16 bytes, does not fit 512 threads x ept elements, or
// fewer than two stages fit in shared memory.
inline RingPlan plan_ring(int64_t M, int64_t N, int esize, int nin, int ept, int sm_count, int max_smem,
                          int64_t target = 32768, int default_lag = 1, int64_t reserve = 0) {
  RingPlan p;
  const int vec = 16 / esize;
  if (M <= 0 || N <= 0 || N % vec != 0) return p;
  const int64_t nvec = N / vec;
  const int vpt = ept / vec;
  int group = 32;
  while (group <= kRingThreads && static_cast<int64_t>(group) * vpt < nvec) group *= 2;
  if (group > kRingThreads) return p;
  p.group = group;
  p.ng = kRingThreads / group;
  const int64_t row_bytes = N * esize;
  int64_t rpg = target / (p.ng * row_bytes);
  // keep at least ~4 tiles per CTA when there are few rows
  while (rpg > 1 && (M + p.ng * rpg - 1) / (p.ng * rpg) < 4LL * sm_count) --rpg;
  p.rpg = static_cast<int>(rpg < 1 ? 1 : (rpg > 4 ? 4 : rpg));
  if (p.rpg == 3) p.rpg = 2;  // the kernels take a group's rows two at a time
  const RingTuning& tune = ring_tuning();
  if (tune.rpg > 0) p.rpg = tune.rpg > 4 ? 4 : tune.rpg;
  const int64_t stage = static_cast<int64_t>(nin) * p.ng * p.rpg * row_bytes;
  int64_t s = (static_cast<int64_t>(max_smem) - kRingHeaderBytes - reserve) / stage;
  if (s > kMaxStages) s = kMaxStages;
  if (tune.stages > 0 && tune.stages < s) s = tune.stages;
  if (s < 2) return p;
  p.stages = static_cast<int>(s);
  p.lag = default_lag;
  if (tune.lag > 0) p.lag = tune.lag;
  if (p.lag > s - 2) p.lag = static_cast<int>(s) - 2;
  if (p.lag < 1) p.lag = 1;
  if (p.lag > 3) p.lag = 3;
  p.smem = static_cast<size_t>(kRingHeaderBytes + reserve + s * stage);
  const int64_t ntiles = (M + p.ng * p.rpg - 1) / (p.ng * p.rpg);
  if (ntiles > 0x7fff0000LL) return p;  // tile indices are handed out through a 32-bit counter
  p.grid = static_cast<int>(ntiles < sm_count ? ntiles : sm_count);
  // No CTA can finish before the one with the most tiles: with w = ceil(ntiles / grid) tiles on the busiest CTA,
  // ceil(ntiles / w) CTAs do the same work in the same time.  The SMs this leaves out (one of 148 for 8192 rows of
  // 8192, none for 65536) are free for whatever runs beside the kernel — a collective's kernel on another stream.
  const int64_t waves = (ntiles + p.grid - 1) / p.grid;
  p.grid = static_cast<int>((ntiles + waves - 1) / waves);
  p.ok = true;
  return p;
}

}  // namespace b2n
