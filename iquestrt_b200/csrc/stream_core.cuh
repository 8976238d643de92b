// The weight-streaming engine every kernel of the path is built on.
//
// One persistent CTA per SM.  A dedicated producer warp streams e4m3 (or bf16) weight tiles
// from HBM into a shared-memory ring with TMA, ONE copy per ring stage (16-32 KB): a
// tiled `cp.async.bulk.tensor.2d` box of (rows x 1 KB) when a stage is a K-slice of its
// rows, an untiled `cp.async.bulk` when the stage's rows are whole and therefore
// contiguous.  Completion is counted in bytes on an mbarrier per ring slot.  (Measured on
// B200: one 16 KB copy per stage with six stages in flight streams at 7.0 TB/s; sixteen
// 1 KB copies per stage reach 3.9 TB/s.)
// The consumer warps (sixteen, or eight / six when two CTAs share an SM) read the ring with
// 16-byte shared loads and feed warp-level MMAs
// whose B operand carries the (at most eight) activation rows, so a byte of weight costs
// 1/512 of an MMA and no conversion instruction.  The K index inside an MMA is permuted
// so that every lane's A and B fragments are plain 16-byte runs (see `consume_stage`).
//
// Work is the list of (tile, k-stage) items in tile-major order.  Either every CTA takes
// whole tiles (contiguous ranges, or round robin), or CTA i owns the contiguous item range
// [i*T/G, (i+1)*T/G) ("stream-K"), so that every SM streams the same number of bytes to
// within one stage whatever the shape; `tile_aligned_split` picks by a small cost model.
// A tile whose stages fall in more than one CTA is finished by whichever contributor
// arrives last at the tile's counter: it sums the contributors' fp32 partials from scratch
// in CTA order, so the result does not depend on arrival order, and nothing waits on
// another CTA.
//
// The per-stage consumer path is kept to a few dozen instructions: everything that
// depends only on the tile or the weight group is hoisted out of the stage loop, and the
// weight scales of all the CTA's stages are gathered into shared memory once, before the
// first stage is consumed.
//
// After its last tile every CTA takes a ticket; the last one runs the kernel's global
// epilogue (all-reduce tail, or top-k selection) on the completed rows.
#pragma once

#include <cstddef>

#include "common.cuh"

namespace iqb {

constexpr int kMaxStages = 16;
constexpr int kMaxGroups = 72;                    // 8 rows x 8 routed + shared, with slack
constexpr int kMaxCols = 8;                       // MMA N
constexpr int kSmemLimit = 232448;                // 227 KiB per CTA on sm_100
// Two CTAs on an SM: 228 KiB per SM, 1 KiB reserved per resident CTA.  The hardware packs
// the CTAs of a launch onto as few SMs as their resources allow, so two kinds of half-SM
// CTA exist.  A "spread" CTA asks for a little more than half of the SM's shared memory:
// two of them never share an SM, so a launch of one CTA per SM really lands one per SM
// (a stream that needs every SM's bandwidth), yet a "small" CTA of the next or previous
// kernel of the chain still fits beside it.  A small CTA may pack two to an SM.
constexpr int kSmemSpread = 117 * 1024;           // exactly what a spread CTA requests
constexpr int kSmemLimitSmall = 233472 - 2 * 1024 - kSmemSpread;   // a small CTA: up to 108 KiB

// Ring geometry: a stage is (16*RT) weight rows x (KW*RUNS*64) bytes; warp (rs, kp) of the
// RT*KW consumer warps owns row sub-tile rs and the kp-th slice of RUNS 64-byte runs.  A
// CTA is the consumer warps plus one producer and one epilogue warp.
//
// Sixteen consumer warps with a 160 KB ring (one CTA per SM) get the most out of HBM on a
// long stream.  Eight (or six) consumer warps with a ring of about 96 KB leave room for a
// SECOND CTA on the SM: the CTAs of the next kernel of a programmatic-dependent-launch chain
// become resident while this kernel is still streaming, set themselves up and fill their
// own ring with weights before their dependency wait, so a short stream does not pay the
// launch, the set-up and the first-byte latency of its successor end to end.
// `SHARE_`: 0 = by warp count (up to eight consumer warps: a small half-SM CTA, else a
// whole SM), 1 = a whole SM whatever the warp count (a few-warp CTA with a much deeper
// ring), 2 = small half-SM CTA, 3 = spread half-SM CTA (see kSmemSpread).
template <int RT_, int KW_, int RUNS_, int SHARE_ = 0>
struct Geo {
  static constexpr int RT = RT_, KW = KW_, RUNS = RUNS_;
  static constexpr int WARPS = RT * KW;                 // consumer warps
  static_assert(WARPS == 6 || WARPS == 8 || WARPS == 16, "6, 8 or 16 consumer warps");
  static constexpr int CONSUMER_THREADS = WARPS * 32;
  // + the producer warp + the epilogue warp; never fewer than ten warps, so that every
  // half-SM kernel asks the register file for the same shape (see below)
  static constexpr int THREADS = CONSUMER_THREADS + 64 < 320 ? 320 : CONSUMER_THREADS + 64;
  static constexpr int PRODUCER_WARP = WARPS;
  static constexpr int EPILOGUE_WARP = WARPS + 1;
  static constexpr int CTAS_PER_SM = SHARE_ == 1 ? 1 : (SHARE_ >= 2 ? 2 : (WARPS <= 8 ? 2 : 1));
  // The thread count the kernels declare as their launch bound.  A half-SM CTA has to fit
  // beside a ten-warp CTA of 96 registers per thread of another kernel, and registers are
  // handed out per scheduler (16 K each): bound to 320 threads and two CTAs per SM a kernel
  // gets 96 registers and fits.  (A 256-thread CTA bound to two per SM may use 128 and then
  // does NOT fit: measured, its CTAs only started when the neighbours left.)
  static constexpr int BOUND_THREADS = THREADS;
  static constexpr bool SPREAD = SHARE_ == 3;
  static_assert(CTAS_PER_SM == 1 || WARPS <= 8, "two CTAs per SM need few warps");
  static constexpr int ROWS = 16 * RT;
  static constexpr int KC = KW * RUNS * 64;
  // A stage lands as NBOX dense boxes of (ROWS x BOXK bytes), one TMA copy each (a tensor
  // map box is at most 256 four-byte elements wide): row pitch = BOXK.  When BOXK is a
  // multiple of 128 the two rows a quarter-warp reads share banks (a 2-way conflict on
  // 16-byte loads), which costs nothing at the ~25 B/clk/SM a weight stream needs.
  static constexpr int BOXK = KC > 1024 ? 1024 : KC;
  static constexpr int NBOX = KC / BOXK;
  static_assert(KC % BOXK == 0 && (RUNS * 64 <= BOXK) && (BOXK % (RUNS * 64) == 0),
                "a warp's K slice lies inside one box");
  static constexpr int PITCH = BOXK;
  static constexpr int STAGE_BYTES = ROWS * KC;
  // One weight scale per (warp, run) of a stage, gathered into shared memory.
  static constexpr int SCALES_PER_STAGE = WARPS * RUNS;
};

// One weight matrix instance ("group"): an expert, the shared expert, or the only matrix.
struct GroupDesc {
  const uint8_t* w;        // first byte of the group's [rows, k_bytes] matrix
  const float* scale;      // its scale table (row-major [rows/rg, k/kg]); unused for bf16
  int row_base;            // the group's first row inside its tensor map
  int map_id;              // which of the launch's tensor maps covers the group
  int k_base;              // first byte of the group's K range inside its rows (tiled copies;
  int pad_;                //   the scale tables and the staged activations are not offset)
  float col_mul[kMaxCols]; // per MMA column multiplier (routing weight; 1 otherwise)
  int16_t col_row[kMaxCols];  // staged activation row per MMA column, -1 = column unused
  int16_t col_out[kMaxCols];  // output row per MMA column
};

static_assert(offsetof(GroupDesc, col_mul) % 8 == 0 && offsetof(GroupDesc, col_row) % 8 == 0 &&
                  offsetof(GroupDesc, col_out) % 8 == 0 && sizeof(GroupDesc) % 8 == 0,
              "the column arrays are cleared with 8-byte stores");

enum TileMode : int {
  kRowsPerGroup = 0,  // tiles = groups x row-tiles; every tile contracts over one group's K
  kConcatK = 1,       // tiles = row-tiles; every tile contracts over all groups' K in turn
};

// Uniform description of one launch's streaming work (same on every CTA).
struct StreamShape {
  int mode;
  int n_groups;
  int rows_per_group;  // weight rows per group
  int k_bytes;         // bytes of a weight row that a tile contracts over
  int row_bytes;       // bytes between weight rows in memory; 0 = k_bytes (rows are dense)
  int rg_shift;        // log2(weight rows per scale entry)
  int kg_shift;        // log2(weight bytes along K per scale entry)
  int pair_half;       // >0: a tile takes ROWS/2 rows at f and ROWS/2 rows at pair_half + f
  int x_rows;          // staged activation rows
  int x_pitch;         // bytes between staged activation rows in shared memory
  int x_blocks;        // activation scale entries per staged row (k / 128)
  int n_stages;        // ring depth
  int max_items;       // most stages one CTA can own (sizes the shared scale table)
  int whole_tiles;     // 1: never split a tile when there are no more tiles than CTAs; 2: never
  int round_robin;     // 1: when CTAs take whole tiles, CTA c takes tiles c, c+G, c+2G, ...
};

// Scratch owned by the caller (zero-filled once; every launch leaves it zeroed again).
struct StreamScratch {
  float* partials;        // [grid][2][ROWS*8]
  uint32_t* tile_counter; // [tiles]
  uint32_t* ticket;       // [1]
  int* status;            // [1] first error code of any launch using this scratch
  unsigned long long* trace;   // trace builds: this CTA's 16 stamps (else null)
};

// One %globaltimer stamp into slot `k` of the CTA's trace words (trace builds only).
__device__ __forceinline__ void trace_stamp(const StreamScratch& scr, int k) {
  if (scr.trace) scr.trace[k] = globaltimer_ns();
}
// One SM-clock stamp into fine slot `k` (words 16..31 of the CTA's trace words).
__device__ __forceinline__ void trace_clock(const StreamScratch& scr, int k) {
#ifdef IQ_TRACE
  if (scr.trace) scr.trace[16 + k] = static_cast<unsigned long long>(clock64());
#endif
}

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// Item range of CTA `cta` of `grid` over `total` items.
// (total < 2^31: floor(total * cta / grid) from 32-bit divisions only -- a 64-bit division
// is a subroutine of a few hundred instructions, and this runs at the head of every CTA)
__host__ __device__ __forceinline__ long long item_begin(long long total, int grid, int cta) {
  const uint32_t t = static_cast<uint32_t>(total), g = static_cast<uint32_t>(grid);
  const uint32_t q = t / g, r = t - q * g;
  return static_cast<long long>(q) * cta + (r * static_cast<uint32_t>(cta)) / g;
}
// The CTA that owns item q (inverse of item_begin; needs grid <= total).
__host__ __device__ __forceinline__ int item_owner(long long total, int grid, long long q) {
  return static_cast<int>(((q + 1) * grid + total - 1) / total - 1);
}

template <class G>
struct StreamSmem {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t red_full[2];   // the consumers' per-tile partials are in red[i]
  uint64_t red_empty[2];  // the epilogue warp has read red[i]
  volatile int abort_flag;
  int is_last_tile;   // broadcast: this CTA finishes the current split tile
  int is_last_cta;    // broadcast: this CTA runs the global epilogue
  int pad;
  GroupDesc groups[kMaxGroups];
  int route_ids[64 + kMaxGroups + 1 + 32];   // routed expert ids while the group table is built (+ stand-in ids)
  float red[2][G::WARPS][32][4];
};

// Weight row `r` of a tile -> row index inside the group.
__device__ __forceinline__ int tile_row(const StreamShape& sh, int rows, int tile_in_group, int r) {
  if (sh.pair_half > 0) {
    const int half = rows / 2;
    return r < half ? tile_in_group * half + r : sh.pair_half + tile_in_group * half + (r - half);
  }
  return tile_in_group * rows + r;
}

template <class G>
__host__ __device__ __forceinline__ int stream_tiles_per_group(const StreamShape& sh) {
  return sh.pair_half > 0 ? sh.pair_half / (G::ROWS / 2) : sh.rows_per_group / G::ROWS;
}
template <class G>
__host__ __device__ __forceinline__ int stream_num_tiles(const StreamShape& sh) {
  const int tpg = stream_tiles_per_group<G>(sh);
  return sh.mode == kRowsPerGroup ? sh.n_groups * tpg : tpg;
}
template <class G>
__host__ __device__ __forceinline__ int stream_stages_per_tile(const StreamShape& sh) {
  const int kstages = sh.k_bytes / G::KC;
  return sh.mode == kRowsPerGroup ? kstages : kstages * sh.n_groups;
}

// Exact a / d for 0 <= a < 65536 and 1 <= d < 65536 as one multiply-high: magic(d) =
// floor(2^32 / d) + 1 (0 stands for d == 1).  The per-entry index arithmetic of the scale
// gather runs on every CTA's critical path; a runtime integer division costs ~30
// instructions, this costs one.
__host__ __device__ __forceinline__ uint32_t div_magic(int d) {
  // (floor((2^32 - 1) / d) + 1: the same number unless d is a power of two, where it is
  // one less and still exact; a 32-bit division instead of a 64-bit one)
  return d <= 1 ? 0u : 0xffffffffu / static_cast<uint32_t>(d) + 1u;
}
__device__ __forceinline__ int fast_div(int a, uint32_t magic) {
  return magic ? static_cast<int>(__umulhi(static_cast<uint32_t>(a), magic)) : a;
}

// The CTA's share of the work, in 32-bit terms.
struct CtaWork {
  int tile0;      // first tile
  int tile_step;  // distance between the CTA's consecutive tiles (1 unless round robin)
  int stage0;     // first stage inside it
  int n_items;    // stages owned
  int spt;        // stages per tile
  int kstages;    // stages per group K
  int tpg;        // tiles per group
  uint32_t mg_spt, mg_kstages, mg_tpg;   // div_magic of the three
};

template <class G>
__device__ __forceinline__ CtaWork cta_work(const StreamShape& sh, long long it0, long long it1) {
  CtaWork w;
  w.kstages = sh.k_bytes / G::KC;
  w.tpg = stream_tiles_per_group<G>(sh);
  w.spt = sh.mode == kRowsPerGroup ? w.kstages : w.kstages * sh.n_groups;
  w.mg_spt = div_magic(w.spt);
  w.mg_kstages = div_magic(w.kstages);
  w.mg_tpg = div_magic(w.tpg);
  w.tile0 = static_cast<int>(static_cast<uint32_t>(it0) / static_cast<uint32_t>(w.spt));
  w.tile_step = 1;
  w.stage0 = static_cast<int>(it0 - static_cast<long long>(w.tile0) * w.spt);
  w.n_items = static_cast<int>(it1 - it0);
  return w;
}

// How the items are cut between CTAs.  Cutting the item range evenly (stream-K) keeps every
// SM streaming the same number of bytes, but a tile split between two CTAs has to be
// settled through global memory (publish, fence, count, sum: three or four round trips,
// about 3 us) and that is hidden only behind tiles long enough to stream meanwhile.  Giving
// every CTA whole tiles avoids the settlement at the price of imbalance.  The choice is
// made from a small cost model in nanoseconds: a stage of S bytes passes through one SM in
// about S/44 ns (148 SMs at 6.5 TB/s).
template <class G>
__host__ __device__ __forceinline__ bool tile_aligned_split(int n_tiles, int spt, int grid,
                                                            int whole_flag) {
  const int g = n_tiles < grid ? n_tiles : grid;        // CTAs that get work
  if (whole_flag >= 2 || (whole_flag && n_tiles <= grid)) return true;
  const int per = (n_tiles + g - 1) / g;                // most tiles any CTA takes
  if (n_tiles >= grid && g * 10 >= grid * 9 &&
      static_cast<long long>(per) * grid * 8 <= static_cast<long long>(n_tiles) * 9)
    return true;                                        // balanced to within an eighth
  const long long stage_ns = G::STAGE_BYTES / 44;
  const long long total = static_cast<long long>(n_tiles) * spt;
  const long long even_ns =
      static_cast<long long>((static_cast<uint32_t>(total) + grid - 1) / static_cast<uint32_t>(grid)) *
      stage_ns;
  const long long whole_ns = static_cast<long long>(per) * spt * stage_ns;
  const long long tile_ns = spt * stage_ns;
  const long long settle_ns = tile_ns < 4000 ? 3000 : 500;   // exposed unless tiles are long
  return whole_ns <= even_ns + settle_ns;
}

// The CTA's share; `grid` is the number of CTAs launched.  CTAs beyond the work get
// n_items == 0.  `split_grid` receives the CTA count the stream-K owner arithmetic uses.
template <class G>
__device__ __forceinline__ CtaWork cta_share(const StreamShape& sh, int grid, int cta,
                                             int& split_grid) {
  const int n_tiles = stream_num_tiles<G>(sh);
  const int spt = stream_stages_per_tile<G>(sh);
  const long long total = static_cast<long long>(n_tiles) * spt;
  // A stream of a few megabytes is bound by latency, not bandwidth: settling a split tile
  // costs more than streaming all of its stages through one SM.
  if (tile_aligned_split<G>(n_tiles, spt, grid, sh.whole_tiles)) {
    const int g = n_tiles < grid ? n_tiles : grid;
    split_grid = g;
    if (cta >= g) return cta_work<G>(sh, 0, 0);
    if (sh.round_robin) {
      // tiles cta, cta + grid, ...: the CTA's first tile does not depend on how many
      // tiles (groups) there turn out to be
      const int count = (n_tiles - cta + grid - 1) / grid;
      CtaWork w = cta_work<G>(sh, static_cast<long long>(cta) * spt,
                              static_cast<long long>(cta + count) * spt);
      w.tile_step = grid;
      return w;
    }
    const long long t0 = static_cast<uint32_t>(n_tiles * cta) / static_cast<uint32_t>(g);
    const long long t1 = static_cast<uint32_t>(n_tiles * (cta + 1)) / static_cast<uint32_t>(g);
    return cta_work<G>(sh, t0 * spt, t1 * spt);
  }
  const int g = total < grid ? static_cast<int>(total) : grid;
  split_grid = g;
  if (cta >= g) return cta_work<G>(sh, 0, 0);
  return cta_work<G>(sh, item_begin(total, g, cta), item_begin(total, g, cta + 1));
}

// A stage is a set of whole, dense rows: one untiled copy moves it.
template <class G>
__host__ __device__ __forceinline__ bool stream_whole_rows(const StreamShape& sh) {
  return sh.k_bytes == G::KC && G::NBOX == 1 && (sh.row_bytes == 0 || sh.row_bytes == sh.k_bytes);
}

// (group, tile-in-group, k-stage) of stage `s` of tile `tile`.
struct StagePos {
  int group, tig, kstage;
};
__device__ __forceinline__ StagePos stage_pos(const StreamShape& sh, const CtaWork& w, int tile,
                                              int s) {
  StagePos p;
  if (sh.mode == kRowsPerGroup) {
    p.group = tile / w.tpg;
    p.tig = tile - p.group * w.tpg;
    p.kstage = s;
  } else {
    p.group = s / w.kstages;
    p.tig = tile;
    p.kstage = s - p.group * w.kstages;
  }
  return p;
}

// The order in which a CTA visits the tiles of its item range.  A tile the CTA shares with
// its neighbour costs serial global round trips to finish (publish, count, sum), so the
// shared tile at the END of the range is visited FIRST: by the time the CTA reaches its
// last tiles, which are whole and are emitted directly, every shared tile has long been
// settled by both of its owners.  The producer, the consumers and the epilogue warp all
// walk the same sequence.
struct TileVisit {
  int tile;      // tile index
  int s_begin;   // stage range [s_begin, s_end) of the tile owned by this CTA
  int s_end;
  int local0;    // position of stage s_begin in the CTA's natural stage order
};

struct TileWalk {
  int n_tiles;       // tiles touched
  int n_first;       // stages owned in the first touched tile
  bool last_first;   // visit the last touched tile before the others
  __device__ __forceinline__ void init(const CtaWork& w) {
    if (w.n_items <= 0) { n_tiles = 0; n_first = 0; last_first = false; return; }
    n_first = w.spt - w.stage0 < w.n_items ? w.spt - w.stage0 : w.n_items;
    const int rest = w.n_items - n_first;
    n_tiles = 1 + (rest + w.spt - 1) / w.spt;
    last_first = n_tiles >= 2 && (rest % w.spt) != 0;
  }
  __device__ __forceinline__ TileVisit visit(const CtaWork& w, int k) const {
    const int i = last_first ? (k == 0 ? n_tiles - 1 : k - 1) : k;   // natural index
    TileVisit v;
    v.tile = w.tile0 + i * w.tile_step;
    v.s_begin = i == 0 ? w.stage0 : 0;
    v.local0 = i == 0 ? 0 : n_first + (i - 1) * w.spt;
    const int avail = w.n_items - v.local0;
    v.s_end = w.spt - v.s_begin < avail ? w.spt : v.s_begin + avail;
    return v;
  }
};

// Where a role stands in the ring (slot + mbarrier parity) and in the pair of per-tile
// reduction buffers.  A kernel that runs several streams back to back through one ring
// carries these from one stream to the next.
struct RingPos {
  int slot = 0;
  uint32_t phase = 0;
};
struct RedPos {
  int buf = 0;
  uint32_t phase = 0;
};

// ------------------------------------------------------------------------------------
// Producer: one elected lane of one warp, one or two copies per stage.  `dep_wait`: the
// consumers of this stream do not start before the kernel's dependency wait (pass false
// for a stream that is consumed ahead of that wait).  `map0/map1` are the
// launch's tensor maps (u32 elements, box = KC bytes x box rows), used when a stage is a
// K-slice of its rows; whole-row stages are contiguous and use the untiled copy.
template <class G, class S>
__device__ __forceinline__ void produce(const StreamShape& sh, S* sm, const GroupDesc* groups,
                                        uint8_t* ring, int slot_bytes, const CtaWork& w,
                                        int* status, const CUtensorMap* map0,
                                        const CUtensorMap* map1, RingPos& pos,
                                        bool dep_wait = true) {
  const int lane = threadIdx.x & 31;
  int slot = pos.slot;
  uint32_t phase = pos.phase;
  const bool whole_rows = stream_whole_rows<G>(sh);
  const int halves = sh.pair_half > 0 ? 2 : 1;
  constexpr int kHalfRows = G::ROWS / 2;
  const int copy_rows = halves == 2 ? kHalfRows : G::ROWS;
  // Weights pass through once: marked evict-first they do not push the lines that are
  // reused from launch to launch (activations, scale tables, the kernels' instructions)
  // out of L2.
  const uint64_t policy = policy_evict_first();
  TileWalk walk;
  walk.init(w);
  for (int k = 0; k < walk.n_tiles; ++k) {
    const TileVisit tv = walk.visit(w, k);
    StagePos p = stage_pos(sh, w, tv.tile, tv.s_begin);
    for (int s = tv.s_begin; s < tv.s_end; ++s) {
      if (!mbar_try_wait(&sm->empty[slot], phase ^ 1u)) {
        // The ring is full.  When the consumers may still be held at their dependency
        // wait, join that (untimed) wait first: only then does the pipeline budget apply.
        if (dep_wait) pdl_wait();
        if (!mbar_wait(&sm->empty[slot], phase ^ 1u, &sm->abort_flag)) {
          if (!sm->abort_flag) set_status(status, IQ_ERR_PIPE_TIMEOUT);
          sm->abort_flag = 1;
          return;
        }
      }
      if (lane == 0) {
        const GroupDesc& gd = groups[p.group];
        uint64_t* bar = &sm->full[slot];
        mbar_arrive_expect_tx(bar, G::ROWS * G::KC);
        uint8_t* dst = ring + slot * slot_bytes;
        for (int hf = 0; hf < halves; ++hf) {
          const int row = tile_row(sh, G::ROWS, p.tig, hf * kHalfRows);
          if (whole_rows) {
            bulk_g2s_evict_first(dst + hf * kHalfRows * G::PITCH,
                                 gd.w + static_cast<size_t>(row) * sh.k_bytes,
                                 copy_rows * G::KC, bar, policy);
          } else {
#pragma unroll
            for (int b = 0; b < G::NBOX; ++b)
              tma_2d_g2s_evict_first(dst + b * (G::ROWS * G::BOXK) + hf * kHalfRows * G::PITCH,
                                     gd.map_id ? map1 : map0,
                                     gd.k_base / 4 + p.kstage * (G::KC / 4) + b * (G::BOXK / 4),
                                     gd.row_base + row, bar, policy);
          }
        }
      }
      __syncwarp();
      if (++slot == sh.n_stages) { slot = 0; phase ^= 1u; }
      if (++p.kstage == w.kstages) {   // kConcatK: on to the next group's K
        p.kstage = 0;
        ++p.group;
      }
    }
  }
  pos.slot = slot;
  pos.phase = phase;
}
template <class G>
__device__ __forceinline__ void produce(const StreamShape& sh, StreamSmem<G>* sm, uint8_t* ring,
                                        const CtaWork& w, int* status, const CUtensorMap* map0,
                                        const CUtensorMap* map1, bool dep_wait = true) {
  RingPos pos;
  produce<G>(sh, sm, sm->groups, ring, G::STAGE_BYTES, w, status, map0, map1, pos, dep_wait);
}

// The element type of the streamed matrix decides the MMA; everything else is bytes.
struct ElemE4M3 {
  static constexpr bool kScaled = true;
  __device__ static __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    mma_e4m3(d, a0, a1, a2, a3, b0, b1);
  }
};
struct ElemBF16 {
  static constexpr bool kScaled = false;
  __device__ static __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    mma_bf16(d, a0, a1, a2, a3, b0, b1);
  }
};

// Gathers the weight scale of every (stage, warp, run) the CTA will consume into
// `sc[stage_local * SCALES_PER_STAGE + warp * RUNS + run]`: one global load per entry,
// issued by the consumer threads before the first stage.  Split in two so that the
// caller can put other loads (the activations) in flight between issue and use:
// `gather_scales_load` fills `held` with the thread's first kGatherHeld entries, and
// `gather_scales_store` writes them out and handles any entries beyond those.
constexpr int kGatherHeld = 4;

template <class G>
__device__ __forceinline__ float gather_one(const StreamShape& sh, const GroupDesc* groups,
                                            const CtaWork& w, int i) {
  const int krow = sh.k_bytes >> sh.kg_shift;
  const int st = i / G::SCALES_PER_STAGE, e = i - st * G::SCALES_PER_STAGE;
  const int warp = e / G::RUNS, run = e - warp * G::RUNS;
  const int rs = warp / G::KW, kp = warp - rs * G::KW;
  // (all operands are far below 65536: stages per CTA, tiles <= 16384, stages per tile)
  const int lin = w.stage0 + st;
  const int tq = fast_div(lin, w.mg_spt);
  const int tile = w.tile0 + tq * w.tile_step, s = lin - tq * w.spt;
  StagePos p;
  if (sh.mode == kRowsPerGroup) {
    p.group = fast_div(tile, w.mg_tpg);
    p.tig = tile - p.group * w.tpg;
    p.kstage = s;
  } else {
    p.group = fast_div(s, w.mg_kstages);
    p.tig = tile;
    p.kstage = s - p.group * w.kstages;
  }
  const int row0 = tile_row(sh, G::ROWS, p.tig, rs * 16);
  const int kb = p.kstage * G::KC + kp * (G::RUNS * 64) + run * 64;
  return __ldg(groups[p.group].scale + static_cast<size_t>(row0 >> sh.rg_shift) * krow +
               (kb >> sh.kg_shift));
}

template <class G, class E>
__device__ __forceinline__ void gather_scales_load(const StreamShape& sh, const GroupDesc* groups,
                                                   const CtaWork& w, int tid,
                                                   float (&held)[kGatherHeld]) {
  if (!E::kScaled) return;
  const int total = w.n_items * G::SCALES_PER_STAGE;
#pragma unroll
  for (int j = 0; j < kGatherHeld; ++j) {
    const int i = tid + j * G::CONSUMER_THREADS;
    held[j] = i < total ? gather_one<G>(sh, groups, w, i) : 0.f;
  }
}

template <class G, class E>
__device__ __forceinline__ void gather_scales_store(const StreamShape& sh, const GroupDesc* groups,
                                                    const CtaWork& w, float* sc, int tid,
                                                    const float (&held)[kGatherHeld]) {
  if (!E::kScaled) return;
  const int total = w.n_items * G::SCALES_PER_STAGE;
#pragma unroll
  for (int j = 0; j < kGatherHeld; ++j) {
    const int i = tid + j * G::CONSUMER_THREADS;
    if (i < total) sc[i] = held[j];
  }
  for (int i = tid + kGatherHeld * G::CONSUMER_THREADS; i < total; i += G::CONSUMER_THREADS)
    sc[i] = gather_one<G>(sh, groups, w, i);
}

template <class G, class E>
__device__ __forceinline__ void gather_scales_load(const StreamShape& sh, const StreamSmem<G>* sm,
                                                   const CtaWork& w, int tid,
                                                   float (&held)[kGatherHeld]) {
  gather_scales_load<G, E>(sh, sm->groups, w, tid, held);
}
template <class G, class E>
__device__ __forceinline__ void gather_scales_store(const StreamShape& sh, const StreamSmem<G>* sm,
                                                    const CtaWork& w, float* sc, int tid,
                                                    const float (&held)[kGatherHeld]) {
  gather_scales_store<G, E>(sh, sm->groups, w, sc, tid, held);
}

// Per-(tile, group) consumer state: everything the stage loop needs that does not change
// from stage to stage.  Addresses are 32-bit shared-space addresses.
struct GroupCtx {
  uint32_t xb;         // this lane's B-fragment bytes at k-stage 0 (row col_row[g]); 0 = none
  uint32_t xs0, xs1;   // activation scale rows of D columns 2t and 2t+1
  float m0, m1;        // their multipliers (0 for unused columns)
};

template <class G>
__device__ __forceinline__ GroupCtx group_ctx(const StreamShape& sh, const GroupDesc& gd,
                                              uint32_t xq, uint32_t xs, int warp, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const int kp = warp % G::KW;
  GroupCtx c;
  const int xrow = gd.col_row[g];
  c.xb = xrow < 0 ? 0u : xq + xrow * sh.x_pitch + kp * (G::RUNS * 64) + t * 16;
  const int xr0 = gd.col_row[2 * t], xr1 = gd.col_row[2 * t + 1];
  c.m0 = xr0 < 0 ? 0.f : gd.col_mul[2 * t];
  c.m1 = xr1 < 0 ? 0.f : gd.col_mul[2 * t + 1];
  c.xs0 = xs + (xr0 < 0 ? 0 : xr0) * sh.x_blocks * 4;
  c.xs1 = xs + (xr1 < 0 ? 0 : xr1) * sh.x_blocks * 4;
  return c;
}

// One stage on one consumer warp, in three steps so that a caller can interleave several
// stages (`StageRegs` holds what is in flight).  Lane = 4g + t reads bytes [16t, 16t+16) of
// each 64-byte run of rows g and g+8 of its sub-tile, and the same bytes of activation row
// col_row[g].  MMA k-slot 4t+j (resp. 16+4t+j) of the first MMA is byte 16t+j (resp.
// 16t+4+j) of the run, of the second MMA byte 16t+8+j (resp. 16t+12+j): A and B use the
// same permutation of K, which a dot product does not see.
template <class G>
struct StageRegs {
  uint4 wa[G::RUNS], wb[G::RUNS], xv[G::RUNS];
  float pa[G::RUNS][4], pb[G::RUNS][4];
};

template <class G>
__device__ __forceinline__ void stage_load(StageRegs<G>& r, uint32_t a_lo, const GroupCtx& gc,
                                           int kbyte0) {
  const uint32_t a_hi = a_lo + 8 * G::PITCH;
#pragma unroll
  for (int run = 0; run < G::RUNS; ++run) {
    r.wa[run] = lds128(a_lo + run * 64);
    r.wb[run] = lds128(a_hi + run * 64);
    r.xv[run] = make_uint4(0u, 0u, 0u, 0u);
    if (gc.xb) r.xv[run] = lds128(gc.xb + kbyte0 + run * 64);
  }
}

// Every MMA of the stage gets its own accumulator: the tensor pipe's latency is paid once
// per stage (or per batch of stages), not once per dependent MMA.
template <class G, class E>
__device__ __forceinline__ void stage_mma(StageRegs<G>& r) {
#pragma unroll
  for (int run = 0; run < G::RUNS; ++run) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { r.pa[run][i] = 0.f; r.pb[run][i] = 0.f; }
    E::mma(r.pa[run], r.wa[run].x, r.wb[run].x, r.wa[run].y, r.wb[run].y, r.xv[run].x, r.xv[run].y);
    E::mma(r.pb[run], r.wa[run].z, r.wb[run].z, r.wa[run].w, r.wb[run].w, r.xv[run].z, r.xv[run].w);
  }
}

template <class G, class E>
__device__ __forceinline__ void stage_fold(const StageRegs<G>& r, const GroupCtx& gc, int kbyte0,
                                           int kwarp0, uint32_t wsc, float (&acc)[4]) {
#pragma unroll
  for (int run = 0; run < G::RUNS; ++run) {
    float s0 = gc.m0, s1 = gc.m1;
    if (E::kScaled) {
      const int xblk = (kbyte0 + kwarp0 + run * 64) >> 7;
      const float ws = lds_f32(wsc + run * 4);
      s0 *= ws * lds_f32(gc.xs0 + xblk * 4);
      s1 *= ws * lds_f32(gc.xs1 + xblk * 4);
    }
    acc[0] = fmaf(r.pa[run][0] + r.pb[run][0], s0, acc[0]);
    acc[1] = fmaf(r.pa[run][1] + r.pb[run][1], s1, acc[1]);
    acc[2] = fmaf(r.pa[run][2] + r.pb[run][2], s0, acc[2]);
    acc[3] = fmaf(r.pa[run][3] + r.pb[run][3], s1, acc[3]);
  }
}

// Identity of a finished tile handed to `emit`.
struct TileId {
  int tile, group, tig;
};

// The walk through the CTA's share and the first tile's group context, worked out by
// `consume_head` beforehand.  A kernel whose activations come from its predecessor calls
// that BEFORE its dependency wait: the index arithmetic then runs while the predecessor is
// still finishing instead of between the wait and the first stage.
template <class G>
struct ConsumeHead {
  TileWalk walk;
  TileVisit tv;
  StagePos p;
  GroupCtx gc;
};
template <class G>
__device__ __forceinline__ ConsumeHead<G> consume_head(const StreamShape& sh,
                                                       const GroupDesc* groups,
                                                       const uint8_t* xq, const float* xs,
                                                       const CtaWork& w) {
  ConsumeHead<G> h;
  h.walk.init(w);
  h.tv = h.walk.visit(w, 0);
  h.p = stage_pos(sh, w, h.tv.tile, h.tv.s_begin);
  h.gc = GroupCtx{};
  if (h.walk.n_tiles > 0)
    h.gc = group_ctx<G>(sh, groups[h.p.group], smem_u32(xq), smem_u32(xs), threadIdx.x >> 5,
                        threadIdx.x & 31);
  return h;
}

// Consumers: up to sixteen warps per SM (four per scheduler: the per-stage path is a latency
// chain, so thread-level parallelism is what keeps the SM ahead of the stream).  At the end of a
// tile each warp drops its fragment into `red[i]` and moves on; the epilogue warp folds
// the fragments.  (Two stages in flight per warp were tried: at the 96 registers a
// half-SM CTA may use they spilled, and the layer ran half as fast.)
template <class G, class E, class S>
__device__ __forceinline__ void consume(const StreamShape& sh, S* sm, const GroupDesc* groups,
                                        const uint8_t* ring, int slot_bytes, const uint8_t* xq,
                                        const float* xs, const float* sc, const CtaWork& w,
                                        const StreamScratch& scr, RingPos& pos, RedPos& rpos,
                                        const ConsumeHead<G>* head = nullptr) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rs = warp / G::KW, kp = warp - rs * G::KW;
  const int kwarp0 = kp * (G::RUNS * 64);
  const int a_off = (kwarp0 / G::BOXK) * (G::ROWS * G::BOXK) + (rs * 16 + g) * G::PITCH +
                    kwarp0 % G::BOXK + t * 16;
  int slot = pos.slot;
  uint32_t phase = pos.phase;
  int red_buf = rpos.buf;
  uint32_t red_phase = rpos.phase;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t sc_s = smem_u32(sc) + warp * G::RUNS * 4;
  const uint32_t ring_s = smem_u32(ring), xq_s = smem_u32(xq), xs_s = smem_u32(xs);
  TileWalk walk;
  if (head) walk = head->walk;
  else walk.init(w);
  for (int k = 0; k < walk.n_tiles; ++k) {
    const bool from_head = head && k == 0;
    const TileVisit tv = from_head ? head->tv : walk.visit(w, k);
    uint32_t wsc = sc_s + tv.local0 * (G::SCALES_PER_STAGE * 4);
    int s = tv.s_begin;
    const int s_end = tv.s_end;
    StagePos p = from_head ? head->p : stage_pos(sh, w, tv.tile, s);
    bool first_group = true;
    // ---- stages [s_begin, s_end) of this tile, group by group
    while (s < s_end) {
      const GroupCtx gc = (from_head && first_group)
                              ? head->gc
                              : group_ctx<G>(sh, groups[p.group], xq_s, xs_s, warp, lane);
      first_group = false;
      int ks_end = w.kstages;
      if (s_end - s < ks_end - p.kstage) ks_end = p.kstage + (s_end - s);
      for (int ks = p.kstage; ks < ks_end; ++ks, ++s) {
        if (tid == 0 && k == 0 && s == tv.s_begin) trace_clock(scr, 0);
        if (tid == 0 && k == 0 && s == tv.s_begin + 1) trace_clock(scr, 3);
        if (!mbar_wait(&sm->full[slot], phase, &sm->abort_flag)) {
          if (!sm->abort_flag) set_status(scr.status, IQ_ERR_PIPE_TIMEOUT);
          sm->abort_flag = 1;
          return;
        }
        if (tid == 0 && k == 0 && s == tv.s_begin) { trace_stamp(scr, 6); trace_clock(scr, 1); }
        if (tid == 0 && k == 0 && s == tv.s_begin + 1) trace_clock(scr, 4);
        StageRegs<G> regs;
        stage_load<G>(regs, ring_s + slot * slot_bytes + a_off, gc, ks * G::KC);
        stage_mma<G, E>(regs);
        stage_fold<G, E>(regs, gc, ks * G::KC, kwarp0, wsc, acc);
        __syncwarp();
        if (tid == 0 && k == 0 && s == tv.s_begin) { trace_stamp(scr, 7); trace_clock(scr, 2); }
        if (tid == 0 && k == 0 && s == tv.s_begin + 1) trace_clock(scr, 5);
        if (lane == 0) mbar_arrive(&sm->empty[slot]);
        if (++slot == sh.n_stages) { slot = 0; phase ^= 1u; }
        wsc += G::SCALES_PER_STAGE * 4;
      }
      p.kstage = 0;
      ++p.group;        // kConcatK: next group's K; kRowsPerGroup: loop ends here
    }

    // ---- the CTA's share of this tile is complete: hand the warp's partial to the
    // epilogue warp and go straight on to the next tile.
    if (!mbar_wait(&sm->red_empty[red_buf], red_phase ^ 1u, &sm->abort_flag)) {
      if (!sm->abort_flag) set_status(scr.status, IQ_ERR_PIPE_TIMEOUT);
      sm->abort_flag = 1;
      return;
    }
    float(*red)[32][4] = sm->red[red_buf];
#pragma unroll
    for (int i = 0; i < 4; ++i) { red[warp][lane][i] = acc[i]; acc[i] = 0.f; }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->red_full[red_buf]);
    if (tid == 0 && k == 0) { trace_stamp(scr, 8); trace_clock(scr, 6); }
    if (++red_buf == 2) { red_buf = 0; red_phase ^= 1u; }
  }
  pos.slot = slot;
  pos.phase = phase;
  rpos.buf = red_buf;
  rpos.phase = red_phase;
}
template <class G, class E>
__device__ __forceinline__ void consume(const StreamShape& sh, StreamSmem<G>* sm,
                                        const uint8_t* ring, const uint8_t* xq, const float* xs,
                                        const float* sc, const CtaWork& w,
                                        const StreamScratch& scr,
                                        const ConsumeHead<G>* head = nullptr) {
  RingPos pos;
  RedPos rpos;
  consume<G, E>(sh, sm, sm->groups, ring, G::STAGE_BYTES, xq, xs, sc, w, scr, pos, rpos, head);
}

// The epilogue warp: for every tile of the CTA, in order, folds the consumers' fragments
// and hands the finished values to `emit`.  Two lane layouts:
//   kVec == false: `emit(tile_id, r, col, val)` is called four times per tile and lane,
//     with (r, col) = ((l + 32 j) >> 3, (l + 32 j) & 7) and val[sub] = the sum for weight
//     row 16*sub + r of the tile and MMA column col (a quarter-warp covers one row's eight
//     columns: the layout for kernels that combine columns or sub-tiles);
//   kVec == true: `emit(tile_id, r0, col, val)` is called once per tile and lane with
//     col = l >> 2, r0 = 4 * (l & 3) and val[j][sub] = the sum for weight row
//     16*sub + r0 + j: four consecutive output features of one activation row per lane,
//     so a row-major result leaves as 8- or 16-byte stores.
// A tile whose stages are split between CTAs goes through the scratch: every contributor
// publishes its fp32 partial, and the last one to arrive at the tile's counter sums them
// in CTA order and emits.  In kConcatK mode `tile_id.group` is 0.
template <bool kVec>
__device__ __forceinline__ int epilogue_index(int lane, int j) {
  return kVec ? (((lane & 3) * 4 + j) << 3) + (lane >> 2) : lane + 32 * j;   // r * 8 + col
}
template <class G, bool kVec, class Emit>
__device__ __forceinline__ void epilogue_emit(Emit& emit, const TileId& id, int lane,
                                              const float (&val)[4][G::RT]) {
  if constexpr (kVec) {
    emit(id, (lane & 3) * 4, lane >> 2, val);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) emit(id, (lane + 32 * j) >> 3, (lane + 32 * j) & 7, val[j]);
  }
}
template <class G, bool kVec, class S, class Emit>
__device__ __forceinline__ void epilogue(const StreamShape& sh, S* sm, const CtaWork& w,
                                         long long total, int grid, int cta,
                                         const StreamScratch& scr, RedPos& rpos, Emit emit) {
  const int lane = threadIdx.x & 31;
  const bool concat = sh.mode != kRowsPerGroup;
  int red_buf = rpos.buf;
  uint32_t red_phase = rpos.phase;
  TileWalk walk;
  walk.init(w);
  for (int k = 0; k < walk.n_tiles; ++k) {
    const TileVisit tv = walk.visit(w, k);
    const int tile = tv.tile;
    const bool whole = tv.s_begin == 0 && tv.s_end == w.spt;
    TileId id;
    id.tile = tile;
    id.group = concat ? 0 : tile / w.tpg;
    id.tig = concat ? tile : tile - id.group * w.tpg;
    if (!mbar_wait(&sm->red_full[red_buf], red_phase, &sm->abort_flag)) {
      if (!sm->abort_flag) set_status(scr.status, IQ_ERR_PIPE_TIMEOUT);
      sm->abort_flag = 1;
      return;
    }
    if (lane == 0 && k == 0) trace_stamp(scr, 13);
    const float(*red)[32][4] = sm->red[red_buf];
    float val[4][G::RT];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = epilogue_index<kVec>(lane, j), r = idx >> 3, col = idx & 7;
      const int fl = 4 * (r & 7) + (col >> 1), fi = (r >> 3) * 2 + (col & 1);
#pragma unroll
      for (int sub = 0; sub < G::RT; ++sub) {
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < G::KW; ++q) v += red[sub * G::KW + q][fl][fi];
        val[j][sub] = v;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->red_empty[red_buf]);   // the consumers may reuse red[i]
    if (++red_buf == 2) { red_buf = 0; red_phase ^= 1u; }
    if (whole) {
      epilogue_emit<G, kVec>(emit, id, lane, val);
      if (lane == 0 && k == 0) trace_stamp(scr, 14);
    } else {
      const int pslot = (tile == w.tile0) ? 0 : 1;
      float* mine = scr.partials + (static_cast<size_t>(cta) * 2 + pslot) * (G::ROWS * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub) mine[sub * 128 + lane + 32 * j] = val[j][sub];
      __threadfence();
      __syncwarp();
      const long long tile_first = static_cast<long long>(tile) * w.spt;
      const int c_first = item_owner(total, grid, tile_first);
      const int c_last = item_owner(total, grid, tile_first + w.spt - 1);
      int last = 0;
      if (lane == 0) {
        const uint32_t prev = atomicAdd(scr.tile_counter + tile, 1u);
        last = (prev == static_cast<uint32_t>(c_last - c_first));
        if (last) {
          scr.tile_counter[tile] = 0;     // leave the scratch ready for the next launch
          __threadfence();
        }
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int sub = 0; sub < G::RT; ++sub) val[j][sub] = 0.f;
        for (int cc = c_first; cc <= c_last; ++cc) {
          const int ft = static_cast<int>(item_begin(total, grid, cc) / w.spt);
          const float* pp =
              scr.partials + (static_cast<size_t>(cc) * 2 + (tile == ft ? 0 : 1)) * (G::ROWS * 8);
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int sub = 0; sub < G::RT; ++sub)
              val[j][sub] += __ldcg(pp + sub * 128 + lane + 32 * j);
        }
        epilogue_emit<G, kVec>(emit, id, lane, val);
      }
    }
  }
  rpos.buf = red_buf;
  rpos.phase = red_phase;
}
template <class G, bool kVec, class Emit>
__device__ __forceinline__ void epilogue(const StreamShape& sh, StreamSmem<G>* sm,
                                         const CtaWork& w, long long total, int grid, int cta,
                                         const StreamScratch& scr, Emit emit) {
  RedPos rpos;
  epilogue<G, kVec>(sh, sm, w, total, grid, cta, scr, rpos, emit);
}

// After the CTA's last emit: returns true on the one CTA that arrives last, on every one of
// its threads, with all other CTAs' global writes visible.  Call from all threads of the CTA.
template <class G>
__device__ __forceinline__ bool last_cta(StreamSmem<G>* sm, const StreamScratch& scr, int grid) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(scr.ticket, 1u);
    const int last = (prev == static_cast<uint32_t>(grid - 1));
    if (last) {
      *scr.ticket = 0;
      __threadfence();
    }
    sm->is_last_cta = last;
  }
  __syncthreads();
  return sm->is_last_cta != 0;
}

// Barrier set-up; call once from all threads before any produce/consume.
template <class G>
__device__ __forceinline__ void stream_init(const StreamShape& sh, StreamSmem<G>* sm) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < sh.n_stages; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], G::WARPS);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm->red_full[i], G::WARPS);
      mbar_init(&sm->red_empty[i], 1);
    }
    sm->abort_flag = 0;
    sm->is_last_tile = 0;
    sm->is_last_cta = 0;
    mbar_fence_init();
  }
}

// The producer's copies target this CTA's shared memory: before the CTA may exit every
// issued copy must have landed.  Consumers wait on every full barrier they consume, so on
// the normal path nothing is in flight here; on the abort path give stragglers a bounded
// grace period.
template <class G>
__device__ __forceinline__ void stream_drain_on_abort(StreamSmem<G>* sm) {
  if (sm->abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { }
  }
}

}  // namespace iqb
