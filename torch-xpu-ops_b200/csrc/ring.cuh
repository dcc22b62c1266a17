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
// input tile 0.
//
// Tiles are handed out dynamically: the producer thread takes the next tile index from a global
// counter (one atomicAdd per tile, fetched one tile ahead so its latency never shows) and leaves
// it in the stage's tile_id slot for the consumers.  A CTA that starts late — because another
// kernel, say a collective on a second stream, still holds its SM — then simply takes fewer
// tiles, instead of making the whole launch wait for a fixed share it began late.  The counter
// lives in a library-owned slot {next tile, CTAs finished}; the last CTA to finish zeroes it.
// (The norm backward with weight gradients keeps a fixed assignment: see RingProducer::fetch.)
//
// Stage index and barrier phase are carried incrementally in a RingCursor; no division in the
// tile loop.
#pragma once
#include "common.cuh"

namespace b2n {

constexpr int kMaxStages = 16;
constexpr int kRingHeaderBytes = 1024;  // barriers + reduction scratch
constexpr int kRingRedFloats = 128;     // reduction scratch inside the header
constexpr int kRingThreads = 512;       // consumer threads (16 warps)
constexpr int kRingBlock = 640;         // + one producer warpgroup
constexpr int kConsumerRegs = 112;      // the CTA keeps its launch allocation (640 x 96): 512 x 112 + 128 x 32 == 61440

__device__ __forceinline__ void ring_producer_regs() { asm volatile("setmaxnreg.dec.sync.aligned.u32 32;"); }
__device__ __forceinline__ void ring_consumer_regs() { asm volatile("setmaxnreg.inc.sync.aligned.u32 112;"); }

struct RingShared {
  uint64_t full[kMaxStages];  // tile landed in the stage (bulk-copy bytes counted)
  uint64_t done[kMaxStages];  // every warp finished writing the stage's result
  int tile_id[kMaxStages];    // which tile the stage holds; -1: no tiles are left (written by the producer)
  int pad[4];
  float red[kRingRedFloats];  // per-group reduction scratch, double-buffered
};
static_assert(sizeof(RingShared) <= kRingHeaderBytes, "ring header too large");

// Optional event trace (a diagnostic: see b2n_set_trace_buffer).  CTA 0 appends (event, tile,
// %globaltimer) records; buf[0] is the record count, records follow as pairs of 64-bit words.
enum RingEvent : unsigned {
  EV_C_WAIT_BEGIN = 1, EV_C_WAIT_END = 2, EV_C_RELEASED = 3,
  EV_C_STEP = 8  // + step number: points inside the consumer's arithmetic
};
struct RingTrace {
  unsigned long long* buf;
  unsigned cap;  // records per writer slot (slot 0: one consumer thread; slot 1 is free)
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
  unsigned* ctr;        // global {next tile, CTAs finished} pair of this launch
  uint32_t ntiles;      // tiles in the launch
  uint32_t row_bytes;   // bytes per row of one tensor (multiple of 16)
  uint32_t slot_bytes;  // TR * row_bytes: one tensor's share of a stage
  uint32_t stage_bytes;
  uint32_t last_bytes;  // bytes per tensor of the last tile (fewer rows when TR does not divide M)
  int TR;               // rows per tile
  int S;                // stages
  int lag;              // bulk stores the producer leaves in flight before it refills a stage (1..3)

  // S_lag packs the two launch parameters: stages in the low 8 bits, lag above them.
  __device__ __forceinline__ void init(int64_t M_, int N, int esize, int TR_, int S_lag, int nin, unsigned* ctr_,
                                       unsigned long long* trace_buf = nullptr, unsigned trace_cap = 0) {
    trace.buf = trace_buf;
    trace.cap = trace_cap;
    M = M_;
    ctr = ctr_;
    TR = TR_;
    S = S_lag & 0xff;
    lag = S_lag >> 8;
    row_bytes = static_cast<uint32_t>(N) * esize;
    slot_bytes = static_cast<uint32_t>(TR_) * row_bytes;
    stage_bytes = slot_bytes * nin;
    ntiles = static_cast<uint32_t>((M_ + TR_ - 1) / TR_);
    last_bytes = static_cast<uint32_t>(M_ - static_cast<int64_t>(ntiles - 1) * TR_) * row_bytes;
  }
  __device__ __forceinline__ int64_t first_row(int tile) const { return static_cast<int64_t>(tile) * TR; }
  // per tensor: where a tile starts and how many bytes it has
  __device__ __forceinline__ size_t tile_offset(int tile) const { return static_cast<size_t>(tile) * slot_bytes; }
  __device__ __forceinline__ uint32_t tile_bytes(int tile) const {
    return static_cast<uint32_t>(tile) + 1u == ntiles ? last_bytes : slot_bytes;
  }
};

// Where the next tile of a CTA lives: its stage and the parity of that stage's barriers for this use.
struct RingCursor {
  int s;
  uint32_t phase;
  __device__ __forceinline__ void start() { s = 0; phase = 0; }
  __device__ __forceinline__ void advance(const RingGeom& g) {
    if (++s == g.S) { s = 0; phase ^= 1u; }
  }
  __device__ __forceinline__ int next_stage(const RingGeom& g) const { return s + 1 == g.S ? 0 : s + 1; }
};

__device__ __forceinline__ void ring_init(RingShared* rs, int S, int warps) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&rs->full[s], 1);
      mbar_init(&rs->done[s], warps);
    }
    for (int s = 0; s < kMaxStages; ++s) rs->tile_id[s] = -1;
    mbar_init_fence();
  }
  __syncthreads();
  // Up to here nothing outside the CTA has been touched.  Let the next kernel of the stream become
  // resident as SMs free up, and wait for the previous one to finish before the first global access.
  pdl_launch_dependents();
  pdl_wait();
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
  int next_id;     // the tile the next load will fetch, taken from the counter one tile ahead; -1: none left
  unsigned issued; // tiles whose loads have been issued
  bool ended;      // the end marker has been placed: nothing more to load
  RingCursor next; // where the next load goes
  unsigned fetched;  // tile indices taken so far
  unsigned retired;  // how many CTAs had finished taking tiles before this one

  __device__ __forceinline__ RingProducer(RingShared* rs_, unsigned char* stages_, const RingGeom& g_, int* status_)
      : rs(rs_), stages(stages_), g(g_), out(nullptr), status(status_), next_id(-1), issued(0), ended(false), fetched(0), retired(0) {
    next.start();
  }
  // A CTA's first S tiles are blockIdx.x + k * gridDim.x (no atomic in front of the loads that fill
  // the ring); tiles from S * gridDim.x on come from the counter.  Without a counter
  // (g.ctr == nullptr) the fixed pattern continues: the assignment a kernel asks for when what it
  // accumulates across tiles (the norm backward's weight gradients) must not depend on which CTA
  // happened to be early.
  __device__ __forceinline__ int fetch() {
    unsigned t;
    if (g.ctr == nullptr || fetched < static_cast<unsigned>(g.S)) t = blockIdx.x + fetched * gridDim.x;
    else t = static_cast<unsigned>(g.S) * gridDim.x + atomicAdd(g.ctr, 1u);
    ++fetched;
    return t < g.ntiles ? static_cast<int>(t) : -1;
  }
  // Loads the next tile into the next stage, or — when the tiles have run out — marks that stage
  // as the end: its `full` barrier completes without a copy and the consumers leave when they
  // reach it.  The tile_id store is ordered before the barrier operation that follows it.
  __device__ __forceinline__ void issue_next_load() {
    const int id = next_id;
    rs->tile_id[next.s] = id;
    if (id < 0) {
      mbar_arrive(&rs->full[next.s]);
      ended = true;
      // this CTA takes no more tiles: say so now, look at the answer when everything else is done
      if (g.ctr != nullptr) retired = atomicAdd(g.ctr + 1, 1u);
    } else {
      unsigned char* dst = stages + static_cast<size_t>(next.s) * g.stage_bytes;
      const size_t goff = g.tile_offset(id);
      const uint32_t bytes = g.tile_bytes(id);
      mbar_arrive_expect_tx(&rs->full[next.s], bytes * NIN);
#pragma unroll
      for (int k = 0; k < NIN; ++k) bulk_g2s(dst + k * g.slot_bytes, in[k] + goff, bytes, &rs->full[next.s]);
      ++issued;
      next_id = fetch();
    }
    next.advance(g);
  }
  // Fill the ring; then, tile by tile: wait until every consumer warp has finished the tile, send
  // it out, and refill the stage of the tile `lag` tiles back, whose store (now the lag-th newest
  // bulk group) has finished reading shared memory — with S stages in rotation that stage is
  // exactly where the next load belongs.
  __device__ __forceinline__ void run() {
    next_id = fetch();
    for (int k = 0; k < g.S && !ended; ++k) issue_next_load();
    RingCursor cur;
    cur.start();
    int stores = 0;
    unsigned done = 0;
    for (; done < issued; ++done, cur.advance(g)) {
      // what the store will need, worked out before the wait (the id is this thread's own earlier store)
      const int id = rs->tile_id[cur.s];
      unsigned char* gdst = out + g.tile_offset(id);
      const unsigned char* ssrc = stages + static_cast<size_t>(cur.s) * g.stage_bytes;
      const uint32_t bytes = g.tile_bytes(id);
      if (!mbar_wait(&rs->done[cur.s], cur.phase, status)) break;
      bulk_s2g(gdst, ssrc, bytes);
      bulk_commit();
      if (stores < 4) ++stores;
      if (stores > g.lag && !ended) {
        if (g.lag == 1) bulk_wait_read<1>();
        else if (g.lag == 2) bulk_wait_read<2>();
        else bulk_wait_read<3>();
        issue_next_load();
      }
    }
    // Nothing of this CTA may still be in flight when its shared memory goes away: if a wait gave
    // up, let the loads that were issued but never consumed land first.
    for (unsigned j = done; j < issued; ++j) {
      mbar_wait(&rs->full[cur.s], cur.phase, status);
      cur.advance(g);
    }
    // The stores must have READ their stage before the CTA's shared memory goes away; that they have been
    // WRITTEN is the business of the kernel boundary (and of griddepcontrol.wait in a dependent kernel), so the
    // CTA does not sit out the ~1 us write acknowledgement of its last tile.
    bulk_wait_read<0>();
    // The last CTA to finish taking tiles zeroes the counter pair for the slot's next launch (every
    // CTA's last fetch completed before it said so: its result is what ended the CTA's loads).
    if (g.ctr != nullptr && !ended) retired = atomicAdd(g.ctr + 1, 1u);  // a wait gave up before the end marker
    if (g.ctr != nullptr && retired == gridDim.x - 1) {
      g.ctr[0] = 0;
      g.ctr[1] = 0;
    }
  }
};

// Consumer side of one tile: wait for the stage, learn which tile it holds (tile < 0: none left;
// false: the wait gave up), and — after the caller's arithmetic — hand it back.
__device__ __forceinline__ bool ring_consumer_wait(RingShared* rs, const RingCursor& cur, int* status, int& tile) {
  if (!mbar_wait(&rs->full[cur.s], cur.phase, status)) return false;
  tile = rs->tile_id[cur.s];
  return true;
}
// The tile id the producer has left — or is yet to leave — in a stage the consumers have not waited
// for: a hint to prefetch by, to be checked against the real id after the wait.
__device__ __forceinline__ int ring_peek_tile(RingShared* rs, int stage) {
  return *reinterpret_cast<volatile int*>(&rs->tile_id[stage]);
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
