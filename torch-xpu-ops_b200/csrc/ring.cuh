// The shared-memory ring that the persistent "ring" kernels stream rows through.
//
// One CTA per SM runs for the whole launch.  Its rows come in tiles of TR consecutive rows (one
// contiguous byte range per tensor, because the tensors are row-major contiguous).  One thread
// moves tiles global -> shared with bulk-async (TMA) copies that complete on an mbarrier, the
// warps turn the tile into its result IN PLACE in shared memory, and the same thread sends the
// result shared -> global with a bulk-async store.  S stages are in rotation, so loads of the
// next tiles and the store of the previous one overlap the arithmetic, and the bytes in flight per
// SM do not depend on occupancy or register count.
//
// Stage layout: NIN input tiles back to back (tile k at k * TR * row_bytes); the result overwrites
// input tile 0.  Tile i of a CTA is global tile blockIdx.x + i * gridDim.x.
#pragma once
#include "common.cuh"

namespace b2n {

constexpr int kMaxStages = 16;
constexpr int kRingHeaderBytes = 1024;            // barriers + flags + reduction scratch
constexpr int kRingRedFloats = 128;               // reduction scratch inside the header
constexpr int kRingConsumerThreads = 512;
constexpr int kRingThreads = kRingConsumerThreads;  // thread 0 doubles as the producer

struct RingShared {
  uint64_t full[kMaxStages];  // tile landed in the stage (bulk-copy bytes counted)
  uint64_t done[kMaxStages];  // every consumer warp finished writing the stage's result
  int pad[4];
  float red[kRingRedFloats];  // per-group reduction scratch, double-buffered
};
static_assert(sizeof(RingShared) <= kRingHeaderBytes, "ring header too large");

struct RingGeom {
  int64_t M;           // rows
  uint32_t row_bytes;  // bytes per row of one tensor (multiple of 16)
  int TR;              // rows per tile
  int S;               // stages
  uint32_t stage_bytes;
  int64_t ntiles;
  __device__ __forceinline__ int64_t my_tiles() const {
    return ntiles > blockIdx.x ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  }
  __device__ __forceinline__ int64_t tile_row0(int64_t i) const {
    return (static_cast<int64_t>(blockIdx.x) + i * gridDim.x) * TR;
  }
  __device__ __forceinline__ uint32_t tile_bytes(int64_t row0) const {
    const int64_t rows = (M - row0 < TR) ? (M - row0) : TR;
    return static_cast<uint32_t>(rows) * row_bytes;
  }
};

__device__ __forceinline__ void ring_init(RingShared* rs, int S, int consumer_warps) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&rs->full[s], 1);
      mbar_init(&rs->done[s], consumer_warps);
    }
    mbar_init_fence();
  }
  __syncthreads();
}

// Producer duties, carried by thread 0 of the CTA between its own consumer work (a 17th warp would
// cap every thread at 96 registers, because a fifth warp on one SM sub-partition shrinks the
// per-thread share of its register file; 16 warps leave 128).
// in[k]: base of input tensor k; out: base of the result tensor.
template <int NIN> struct RingProducer {
  RingShared* rs;
  unsigned char* stages;
  const RingGeom& g;
  const unsigned char* in[NIN];
  unsigned char* out;
  int* status;
  int64_t n;             // tiles of this CTA
  int64_t loads_issued;  // tiles whose loads have been issued

  __device__ __forceinline__ RingProducer(RingShared* rs_, unsigned char* stages_, const RingGeom& g_, int* status_)
      : rs(rs_), stages(stages_), g(g_), out(nullptr), status(status_), n(g_.my_tiles()), loads_issued(0) {}

  __device__ __forceinline__ void issue_load(int64_t i) {
    const int s = static_cast<int>(i % g.S);
    const int64_t row0 = g.tile_row0(i);
    const uint32_t bytes = g.tile_bytes(row0);
    const uint32_t slot = static_cast<uint32_t>(g.TR) * g.row_bytes;
    unsigned char* dst = stages + static_cast<size_t>(s) * g.stage_bytes;
    mbar_arrive_expect_tx(&rs->full[s], bytes * NIN);
#pragma unroll
    for (int k = 0; k < NIN; ++k) bulk_g2s(dst + k * slot, in[k] + row0 * g.row_bytes, bytes, &rs->full[s]);
  }
  // Before the first tile: fill the ring.
  __device__ __forceinline__ void prologue() {
    const int64_t pre = n < g.S ? n : g.S;
    for (int64_t i = 0; i < pre; ++i) issue_load(i);
    loads_issued = pre;
  }
  // After this thread's own work on tile i: send the tile out once every warp has finished it, then
  // refill the stage of tile i-1, whose store (now the second newest group) has read its source.
  __device__ __forceinline__ bool after_tile(int64_t i) {
    const int s = static_cast<int>(i % g.S);
    if (!mbar_wait(&rs->done[s], static_cast<uint32_t>((i / g.S) & 1), status)) return false;
    const int64_t row0 = g.tile_row0(i);
    bulk_s2g(out + row0 * g.row_bytes, stages + static_cast<size_t>(s) * g.stage_bytes, g.tile_bytes(row0));
    bulk_commit();
    if (i >= 1 && loads_issued < n) {
      bulk_wait_read<1>();
      issue_load(loads_issued);  // == i - 1 + S
      ++loads_issued;
    }
    return true;
  }
  // After the last tile, or after a wait gave up at tile `reached`: nothing of this CTA may still be
  // in flight when its shared memory goes away.
  __device__ __forceinline__ void epilogue(int64_t reached) {
    for (int64_t j = reached; j < loads_issued; ++j)
      mbar_wait(&rs->full[j % g.S], static_cast<uint32_t>((j / g.S) & 1), status);
    bulk_wait_all<0>();
  }
};

// Consumer side of one tile: wait for it, and (after the caller's arithmetic) hand it back.
__device__ __forceinline__ bool ring_consumer_wait(RingShared* rs, const RingGeom& g, int64_t i, int* status) {
  return mbar_wait(&rs->full[i % g.S], static_cast<uint32_t>((i / g.S) & 1), status);
}
__device__ __forceinline__ void ring_consumer_release(RingShared* rs, const RingGeom& g, int64_t i) {
  fence_async_smem();
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(&rs->done[i % g.S]);
}

// ---- reductions over the GROUP threads that share a row ----------------------------------------
// GROUP == 32: shuffles only.  GROUP > 32: per-warp partials through the header scratch and a
// named barrier private to the group (id 1 + group).  `phase` alternates the scratch half so one
// barrier per reduction is enough.  K values are reduced together.
template <int GROUP, int K, typename Op>
__device__ __forceinline__ void group_reduce(float (&v)[K], float* red, int group, int tg, int& phase, Op op) {
#pragma unroll
  for (int k = 0; k < K; ++k) v[k] = warp_reduce(v[k], op);
  if constexpr (GROUP > 32) {
    constexpr int W = GROUP / 32;
    static_assert((kRingConsumerThreads / 32) * 2 * 2 <= kRingRedFloats, "scratch too small");
    static_assert(K <= 2, "scratch sized for two values");
    float* buf = red + ((group * 2 + phase) * W) * 2;
    phase ^= 1;
    if ((tg & 31) == 0) {
#pragma unroll
      for (int k = 0; k < K; ++k) buf[(tg >> 5) * 2 + k] = v[k];
    }
    named_bar_sync(1 + group, GROUP);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      float r = buf[k];
#pragma unroll
      for (int w = 1; w < W; ++w) r = op(r, buf[w * 2 + k]);
      v[k] = r;
    }
  }
}

}  // namespace b2n
