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
// Roles: 16 consumer warps (512 threads) and one producer warpgroup (4 warps, of which one thread
// works).  The producer's bulk-copy instructions and its wait for a store to drain block for about
// as long as HBM takes to move a tile, so they must not sit in a warp that also has a consumer's
// share of every row.  A 17th..20th warp would normally cap every thread at 96 registers; the
// producer warpgroup therefore gives its registers back (setmaxnreg.dec) and the consumers grow to
// 112 (setmaxnreg.inc; the CTA cannot hold more than its launch allocation of 640 x 96, and asking
// for more would wait forever), the warp-specialisation pattern of sm_90+.
//
// Stage layout: NIN input tiles back to back (tile k at k * TR * row_bytes); the result overwrites
// input tile 0.  Tile i of a CTA is global tile blockIdx.x + i * gridDim.x.
//
// All per-tile bookkeeping (stage index, barrier phase, first row) is carried incrementally in a
// RingCursor: with one or two rows per tile, a 64-bit division per tile would cost more
// instructions than the arithmetic on the row.
#pragma once
#include "common.cuh"

namespace b2n {

constexpr int kMaxStages = 16;
constexpr int kRingHeaderBytes = 1024;  // barriers + reduction scratch
constexpr int kRingRedFloats = 160;     // reduction scratch inside the header
constexpr int kRingThreads = 512;       // consumer threads (16 warps)
constexpr int kRingBlock = 640;         // + one producer warpgroup
constexpr int kConsumerRegs = 112;      // the CTA keeps its launch allocation (640 x 96): 512 x 112 + 128 x 24 <= 61440

__device__ __forceinline__ void ring_producer_regs() { asm volatile("setmaxnreg.dec.sync.aligned.u32 24;"); }
__device__ __forceinline__ void ring_consumer_regs() { asm volatile("setmaxnreg.inc.sync.aligned.u32 112;"); }

struct RingShared {
  uint64_t full[kMaxStages];  // tile landed in the stage (bulk-copy bytes counted)
  uint64_t done[kMaxStages];  // every warp finished writing the stage's result
  int pad[4];
  float red[kRingRedFloats];  // per-group reduction scratch, double-buffered
};
static_assert(sizeof(RingShared) <= kRingHeaderBytes, "ring header too large");

// Optional event trace (a diagnostic: see b2n_set_trace_buffer).  CTA 0 appends (event, tile,
// %globaltimer) records; buf[0] is the record count, records follow as pairs of 64-bit words.
enum RingEvent : unsigned {
  EV_C_WAIT_BEGIN = 1, EV_C_WAIT_END = 2, EV_C_RELEASED = 3,
  EV_P_DONE_SEEN = 4, EV_P_STORE_ISSUED = 5, EV_P_READ_WAITED = 6, EV_P_LOAD_ISSUED = 7,
  EV_C_STEP = 8  // + step number: points inside the consumer's arithmetic
};
struct RingTrace {
  unsigned long long* buf;
  unsigned cap;  // records per writer (two writers: consumer thread 0 and the producer thread)
  // Each writer appends to its own half with a private counter (no atomics: the stores are fire
  // and forget, so tracing barely perturbs the timing).  word 0 / word 1 = the writers' counts.
  __device__ __forceinline__ void put(unsigned writer, unsigned& k, unsigned ev, int64_t tile) const {
    if (buf == nullptr || blockIdx.x != 0 || k >= cap) return;
    unsigned long long* p = buf + 2 + 2 * (static_cast<size_t>(writer) * cap + k);
    p[0] = (static_cast<unsigned long long>(ev) << 48) | static_cast<unsigned long long>(tile);
    p[1] = globaltimer_ns();
    buf[writer] = ++k;
  }
};

struct RingGeom {
  RingTrace trace;
  int64_t M;            // rows
  int64_t tile_stride;  // rows between consecutive tiles of this CTA = gridDim.x * TR
  int64_t my_tiles;     // tiles this CTA processes
  int64_t first_row;    // first row of this CTA's tile 0
  uint32_t row_bytes;   // bytes per row of one tensor (multiple of 16)
  uint32_t slot_bytes;  // TR * row_bytes: one tensor's share of a stage
  uint32_t stage_bytes;
  int TR;               // rows per tile
  int S;                // stages
  int lag;              // bulk stores the producer leaves in flight before it refills a stage (1..3)

  // S_lag packs the two launch parameters: stages in the low 8 bits, lag above them.
  __device__ __forceinline__ void init(int64_t M_, int N, int esize, int TR_, int S_lag, int nin,
                                       unsigned long long* trace_buf = nullptr, unsigned trace_cap = 0) {
    trace.buf = trace_buf;
    trace.cap = trace_cap;
    M = M_;
    TR = TR_;
    S = S_lag & 0xff;
    lag = S_lag >> 8;
    row_bytes = static_cast<uint32_t>(N) * esize;
    slot_bytes = static_cast<uint32_t>(TR_) * row_bytes;
    stage_bytes = slot_bytes * nin;
    tile_stride = static_cast<int64_t>(gridDim.x) * TR_;
    first_row = static_cast<int64_t>(blockIdx.x) * TR_;
    const int64_t ntiles = (M_ + TR_ - 1) / TR_;
    my_tiles = ntiles > blockIdx.x ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  }
  __device__ __forceinline__ uint32_t tile_bytes(int64_t row0) const {
    const int64_t rows = (M - row0 < TR) ? (M - row0) : TR;
    return static_cast<uint32_t>(rows) * row_bytes;
  }
};

// Where one tile lives: its stage, the parity of that stage's barriers for this use, its first row.
struct RingCursor {
  int64_t row0;
  int s;
  uint32_t phase;
  __device__ __forceinline__ void start(const RingGeom& g) { row0 = g.first_row; s = 0; phase = 0; }
  __device__ __forceinline__ void advance(const RingGeom& g) {
    row0 += g.tile_stride;
    if (++s == g.S) { s = 0; phase ^= 1u; }
  }
};

__device__ __forceinline__ void ring_init(RingShared* rs, int S, int warps) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&rs->full[s], 1);
      mbar_init(&rs->done[s], warps);
    }
    mbar_init_fence();
  }
  __syncthreads();
}

// The producer loop, run by ONE thread of the producer warpgroup.
// in[k]: base of input tensor k; out: base of the result tensor.
template <int NIN> struct RingProducer {
  RingShared* rs;
  unsigned char* stages;
  const RingGeom& g;
  const unsigned char* in[NIN];
  unsigned char* out;
  int* status;
  int64_t loads_left;  // tiles whose loads have not been issued yet
  RingCursor next;     // the next tile to load

  __device__ __forceinline__ RingProducer(RingShared* rs_, unsigned char* stages_, const RingGeom& g_, int* status_)
      : rs(rs_), stages(stages_), g(g_), out(nullptr), status(status_), loads_left(g_.my_tiles) {
    next.start(g_);
  }
  __device__ __forceinline__ void issue_next_load() {
    const uint32_t bytes = g.tile_bytes(next.row0);
    unsigned char* dst = stages + static_cast<size_t>(next.s) * g.stage_bytes;
    const size_t goff = static_cast<size_t>(next.row0) * g.row_bytes;
    mbar_arrive_expect_tx(&rs->full[next.s], bytes * NIN);
#pragma unroll
    for (int k = 0; k < NIN; ++k) bulk_g2s(dst + k * g.slot_bytes, in[k] + goff, bytes, &rs->full[next.s]);
    next.advance(g);
    --loads_left;
  }
  // Fill the ring; then, tile by tile: wait until every consumer warp has finished the tile, send
  // it out, and refill the stage of the tile `lag` tiles back, whose store (now the lag-th newest
  // bulk group) has finished reading shared memory — with S stages in rotation that stage is
  // exactly where the next tile to load belongs.
  __device__ __forceinline__ void run() {
    for (int k = 0; k < g.S && loads_left > 0; ++k) issue_next_load();
    RingCursor cur;
    cur.start(g);
    int stores = 0;
    unsigned tk = 0;
    int64_t i = 0;
    for (; i < g.my_tiles; ++i, cur.advance(g)) {
      if (!mbar_wait(&rs->done[cur.s], cur.phase, status)) break;
      g.trace.put(1, tk, EV_P_DONE_SEEN, i);
      bulk_s2g(out + static_cast<size_t>(cur.row0) * g.row_bytes,
               stages + static_cast<size_t>(cur.s) * g.stage_bytes, g.tile_bytes(cur.row0));
      bulk_commit();
      g.trace.put(1, tk, EV_P_STORE_ISSUED, i);
      if (stores < 4) ++stores;
      if (stores > g.lag && loads_left > 0) {
        if (g.lag == 1) bulk_wait_read<1>();
        else if (g.lag == 2) bulk_wait_read<2>();
        else bulk_wait_read<3>();
        g.trace.put(1, tk, EV_P_READ_WAITED, i);
        issue_next_load();
        g.trace.put(1, tk, EV_P_LOAD_ISSUED, i);
      }
    }
    // Nothing of this CTA may still be in flight when its shared memory goes away: if a wait gave
    // up, let the loads that were issued but never consumed land first.
    const int64_t issued = g.my_tiles - loads_left;
    for (int64_t j = i; j < issued; ++j) {
      mbar_wait(&rs->full[cur.s], cur.phase, status);
      cur.advance(g);
    }
    bulk_wait_all<0>();
  }
};

// Consumer side of one tile: wait for it, and (after the caller's arithmetic) hand it back.
__device__ __forceinline__ bool ring_consumer_wait(RingShared* rs, const RingCursor& cur, int* status) {
  return mbar_wait(&rs->full[cur.s], cur.phase, status);
}
__device__ __forceinline__ void ring_consumer_release(RingShared* rs, const RingCursor& cur) {
  fence_async_smem();
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(&rs->done[cur.s]);
}

// ---- reductions over the GROUP threads that share a row ----------------------------------------
// K values (K = 1, 2 or 4) are reduced together, in a fixed order (bit-reproducible).
//
// Within a warp the K values share one butterfly: each of the first log2(K) exchanges halves the
// number of values a lane carries (lane ^ 16 leaves values {0,1} in lanes 0-15 and {2,3} in lanes
// 16-31; lane ^ 8 splits those again), so value k ends up, fully summed, in the lanes of segment k
// of the warp (32/K lanes each) after 2 + 1 + 3 shuffles for four values instead of 4 x 5.
// Across the W = GROUP/32 warps of a group: the first lane of each segment writes the warp's total
// of its value to the header scratch ([group][phase][K][W], double-buffered by `phase` so one named
// barrier per reduction is enough); after the barrier every warp reads the K*W partials one (or,
// for K*W = 64, two) per lane and finishes with a log2(W)-level butterfly inside W-lane segments —
// one shared-memory load and at most four shuffles per thread instead of W loads and W adds.
template <int GROUP, int K, typename Op>
__device__ __forceinline__ void group_reduce(float (&v)[K], float* red, int group, int tg, int& phase, Op op) {
  static_assert(K == 1 || K == 2 || K == 4, "one, two or four values");
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = tg & 31;
  float x;
  if constexpr (K == 1) {
    x = warp_reduce(v[0], op);
  } else if constexpr (K == 2) {
    const bool hi = (lane & 16) != 0;
    const float keep = hi ? v[1] : v[0];
    const float send = hi ? v[0] : v[1];
    x = op(keep, __shfl_xor_sync(kFull, send, 16));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) x = op(x, __shfl_xor_sync(kFull, x, o));
  } else {
    const bool hi = (lane & 16) != 0, hi8 = (lane & 8) != 0;
    const float a0 = op(hi ? v[2] : v[0], __shfl_xor_sync(kFull, hi ? v[0] : v[2], 16));
    const float a1 = op(hi ? v[3] : v[1], __shfl_xor_sync(kFull, hi ? v[1] : v[3], 16));
    x = op(hi8 ? a1 : a0, __shfl_xor_sync(kFull, hi8 ? a0 : a1, 8));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) x = op(x, __shfl_xor_sync(kFull, x, o));
  }
  constexpr int SEG = 32 / K;  // value k sits in lanes [k*SEG, (k+1)*SEG) of every warp
  if constexpr (GROUP == 32) {
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = __shfl_sync(kFull, x, k * SEG);
  } else {
    constexpr int W = GROUP / 32;
    static_assert((kRingThreads / 32) * 2 * 4 <= kRingRedFloats, "scratch too small");
    float* buf = red + (group * 2 + phase) * (4 * W);  // fixed stride: reductions of different K may alternate
    phase ^= 1;
    if ((lane & (SEG - 1)) == 0) buf[(lane / SEG) * W + (tg >> 5)] = x;
    named_bar_sync(1 + group, GROUP);
    if constexpr (W * K <= 32) {
      float y = buf[lane < W * K ? lane : 0];
#pragma unroll
      for (int o = W / 2; o > 0; o >>= 1) y = op(y, __shfl_xor_sync(kFull, y, o));
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = __shfl_sync(kFull, y, k * W);
    } else {
      // 64 partials (four values x 16 warps): lane l holds (value l/16, warp l%16) and
      // (value 2 + l/16, warp l%16); the first exchange folds the two into one
      static_assert(W == 16 && K == 4, "two partials per lane");
      const float y0 = buf[lane], y1 = buf[lane + 32];
      const bool hi8 = (lane & 8) != 0;
      float y = op(hi8 ? y1 : y0, __shfl_xor_sync(kFull, hi8 ? y0 : y1, 8));
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) y = op(y, __shfl_xor_sync(kFull, y, o));
      v[0] = __shfl_sync(kFull, y, 0);
      v[1] = __shfl_sync(kFull, y, 16);
      v[2] = __shfl_sync(kFull, y, 8);
      v[3] = __shfl_sync(kFull, y, 24);
    }
  }
}

}  // namespace b2n
