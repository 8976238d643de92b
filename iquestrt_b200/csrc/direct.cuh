// The direct form of the expert Down for short streams.
//
// The streaming engine (stream_core.cuh) pays a fixed price per launch -- ring and barrier
// set-up, the hand-over between its roles, a few hundred cycles of bookkeeping per stage --
// that a stream of a few megabytes never earns back: measured on one rank's shard of eight
// (14 MB per launch), its Down took 14 us of which 4.4 us were nine stages through the
// consumer loop and 1 us the hand-over to the epilogue warp.  Here the same product is laid
// out for latency instead: many small CTAs, no ring, no roles.  A CTA owns 32 weight rows
// of every group (expert); warp (s, q) of its eight owns row sub-tile s (16 rows) and the
// units q, q+4, ... of the list of (group, K part) units.  A warp loads its 16 rows of a
// unit straight from global memory into MMA fragments with 16-byte loads -- the first unit
// BEFORE the dependency wait, while the later units' rows are prefetched into L2 (the
// routes were written two launches back, the weights never change); after the wait the
// CTA copies the Gate's activation rows into shared memory in one pass, and every warp
// folds unit after unit into one fp32 fragment, the next unit's loads in flight behind
// the current unit's MMAs; the four warps of a sub-tile are added in warp order through
// shared memory, and one warp of the sub-tile rounds and stores (and pushes the tagged
// words to the all-reduce's landing zone, like the engine's epilogue).  The launch's last
// CTAs are the all-reduce's tail CTAs, unchanged.
// Numerics: per 64-byte run `acc += (partial) * (weight scale * multiplier)` like the
// engine; groups are added per warp in ascending order and the warps in warp order (the
// engine adds all groups in ascending order), so a result may differ from the engine's in
// the last bit of the fp32 sum.
#pragma once

namespace iqb {

struct DownDirectParams {
  IQ_TRACE_FIELD
  MoeCommon mc;
  const void* act;           // [m * (top_k + n_shared), i_loc]: e4m3, or bf16 (quantised per
  int act_kind;              //   1x128 group while it is staged)
  __nv_bfloat16* out;
  void* scratch;
  int n_tail;
  int push;
  int per_round;
  int pdl_level;
  iq_tail_args tail;
  PushView pv;
};

// Weight rows per CTA: 32 (two sub-tiles of four warps, 256 threads), or 48 (three sub-tiles of
// three warps, 288 threads; an option, see the launches).
constexpr int kDirectRows = 32;

constexpr int kDirectMaxRows = 72;               // staged activation rows (pairs + shared rows)
constexpr int kDirectMaxWidth = 512;             // widest expert slice (bytes per activation row)

struct DirectSmem {
  GroupDesc groups[kMaxGroups];
  int route_ids[64 + kMaxGroups + 1];
  float red[9][32][4];
  float xs[kDirectMaxRows * (kDirectMaxWidth / 128)];   // activation scales: rows x (i_loc / 128)
  __align__(16) uint8_t xq[16];          // the staged rows start here: rows x (i_loc + 16) bytes
};
// Shared memory of a tile CTA for `rows` staged activation rows of `i_loc` bytes.
__host__ __device__ inline size_t down_direct_smem(int rows, int i_loc) {
  return offsetof(DirectSmem, xq) + static_cast<size_t>(rows) * (i_loc + 16);
}

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// One unit of work of a warp: RPU 64-byte runs (starting at run `run0`) of one group's 16
// rows.  For this lane: rows g and g+8 of the sub-tile, bytes [16t, 16t+16) of each run, and
// the runs' weight scales.
template <int RPU>
struct DirectW {
  uint4 wa[RPU], wb[RPU];
  float ws[RPU];
};
template <int RPU>
__device__ __forceinline__ void direct_load_w(DirectW<RPU>& w, const GroupDesc& gd, int i_loc,
                                              int row0, int run0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const uint8_t* a = gd.w + static_cast<size_t>(row0 + g) * i_loc + run0 * 64 + t * 16;
  const uint8_t* b = a + static_cast<size_t>(8) * i_loc;
  const float* sc = gd.scale + static_cast<size_t>(row0 >> 7) * (i_loc >> 6) + run0;
#pragma unroll
  for (int run = 0; run < RPU; ++run) {
    w.wa[run] = ldg_nc_u4(a + run * 64);
    w.wb[run] = ldg_nc_u4(b + run * 64);
    w.ws[run] = __ldg(sc + run);
  }
}

// RT: 64-byte runs per weight row (i_loc / 64); RPU: runs per unit (RT / RPU units per group).
// (Bound to 320 threads and two CTAs per SM like the half-SM streaming kernels: 96 registers,
// so that a CTA fits beside a ten-warp neighbour -- the register file is per scheduler.)
template <int RT, int RPU, int SUBS>
__global__ void __launch_bounds__(320, 2) down_direct_kernel(const __grid_constant__ DownDirectParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kParts = RT / RPU;
  constexpr int kQ = SUBS == 3 ? 3 : 4;            // warps per row sub-tile
  constexpr int kThreads = SUBS * kQ * 32;
  static_assert(RT % RPU == 0, "whole units");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const int tile_ctas = static_cast<int>(gridDim.x) - p.n_tail;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  if (cta >= tile_ctas) {
    PushView pv = p.pv;
#ifdef IQ_TRACE
    pv.trace = p.trace ? p.trace + blockIdx.x * kTraceWords : nullptr;
#endif
    tail_cta(p.tail, pv, p.per_round, cta - tile_ctas, p.n_tail, smem);
    if (tid == 0) { IQ_STAMP(p, 11); IQ_CLOCK(p, 10); }
    return;
  }
  DirectSmem* sm = reinterpret_cast<DirectSmem*>(smem);
  int* status = scratch_of(p.scratch).status;
  const bool early = p.pdl_level >= 2;
  if (!early) after_wait();
  const int n_groups = build_groups(sm->groups, p.mc, true, true, status, sm->route_ids);
  const int i_loc = p.mc.i_loc, m = p.mc.m, h = p.mc.h;
  const int sub = warp / kQ, q = warp - sub * kQ;
  const int row0 = cta * (SUBS * 16) + sub * 16;
  const int g8 = lane >> 2, t = lane & 3;
  const int n_units = n_groups * kParts;
  const int xpitch = i_loc + 16;

  // ---- ahead of the dependency wait: the first unit's weights into registers, the later
  // units' weight rows into L2 (one 128-byte line per lane covers 16 rows x 256 bytes)
  DirectW<RPU> cur, nxt;
  int unit = q;
  if (unit < n_units)
    direct_load_w<RPU>(cur, sm->groups[unit / kParts], i_loc, row0, (unit % kParts) * RPU, lane);
  for (int u = unit + kQ; u < n_units; u += kQ) {
    const GroupDesc& gd = sm->groups[u / kParts];
    const int line = lane;                       // 16 rows x (RPU * 64 bytes) in 128-byte lines
    const int lines_per_row = (RPU * 64 + 127) / 128;
    if (line < 16 * lines_per_row) {
      const int r = line / lines_per_row, c = line - r * lines_per_row;
      prefetch_l2(gd.w + static_cast<size_t>(row0 + r) * i_loc + (u % kParts) * RPU * 64 + c * 128);
    }
  }
  if (early) after_wait();
  if (tid == 0) IQ_STAMP(p, 1);

  // ---- the Gate's activations: one pass of 16-byte loads into shared memory
  const bool scaled = p.act_kind != IQ_ACT_E4M3;
  const int x_blocks = (i_loc + 127) >> 7;
  {
    const int rows = m * (p.mc.top_k + p.mc.n_shared);
    if (scaled) {
      StreamShape sh{};                   // (what the staging routine reads of it)
      sh.x_pitch = xpitch;
      sh.x_blocks = x_blocks;
      stage_rows_bf16_groupq(sm->xq, sm->xs, sh, static_cast<const __nv_bfloat16*>(p.act), i_loc,
                             rows, i_loc, false, tid, kThreads);
    } else {
      const int vec = i_loc >> 4;
      const uint8_t* act = static_cast<const uint8_t*>(p.act);
      for (int i = tid; i < rows * vec; i += kThreads) {
        const int r = i / vec, v = i - r * vec;
        *reinterpret_cast<uint4*>(sm->xq + r * xpitch + v * 16) =
            ldg_cg_u4(act + static_cast<size_t>(r) * i_loc + v * 16);
      }
    }
  }
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 2);

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t xq_s = smem_u32(sm->xq);
  while (unit < n_units) {
    if (unit + kQ < n_units)
      direct_load_w<RPU>(nxt, sm->groups[(unit + kQ) / kParts], i_loc, row0,
                         ((unit + kQ) % kParts) * RPU, lane);
    const GroupDesc& gd = sm->groups[unit / kParts];
    const int run0 = (unit % kParts) * RPU;
    const int xrow = gd.col_row[g8];
    const int xr0 = gd.col_row[2 * t], xr1 = gd.col_row[2 * t + 1];
    const float m0 = xr0 < 0 ? 0.f : gd.col_mul[2 * t];
    const float m1 = xr1 < 0 ? 0.f : gd.col_mul[2 * t + 1];
    float part[RPU][4];
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (xrow >= 0) xv = lds128(xq_s + xrow * xpitch + (run0 + run) * 64 + t * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) part[run][i] = 0.f;
      mma_e4m3(part[run], cur.wa[run].x, cur.wb[run].x, cur.wa[run].y, cur.wb[run].y, xv.x, xv.y);
      mma_e4m3(part[run], cur.wa[run].z, cur.wb[run].z, cur.wa[run].w, cur.wb[run].w, xv.z, xv.w);
    }
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      float s0 = m0 * cur.ws[run], s1 = m1 * cur.ws[run];
      if (scaled) {
        const int xblk = (run0 + run) >> 1;
        s0 *= sm->xs[(xr0 < 0 ? 0 : xr0) * x_blocks + xblk];
        s1 *= sm->xs[(xr1 < 0 ? 0 : xr1) * x_blocks + xblk];
      }
      acc[0] = fmaf(part[run][0], s0, acc[0]);
      acc[1] = fmaf(part[run][1], s1, acc[1]);
      acc[2] = fmaf(part[run][2], s0, acc[2]);
      acc[3] = fmaf(part[run][3], s1, acc[3]);
    }
    unit += kQ;
    cur = nxt;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) sm->red[warp][lane][i] = acc[i];
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 4);

  // ---- one warp per sub-tile adds its four warps in warp order, rounds and stores
  if (q == 0) {
    const int col = lane >> 2, r0 = (lane & 3) * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + j;
      const int fl = 4 * (r & 7) + (col >> 1), fi = (r >> 3) * 2 + (col & 1);
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kQ; ++w) s += sm->red[sub * kQ + w][fl][fi];
      v[j] = s;
    }
    if (col < m) {
      const bool push = p.push != 0;
      const uint32_t tag = push ? tag16_of(ld_volatile_u32(p.pv.epoch)) : 0u;
      const int feat = row0 + r0;
      store_row4(p.out, static_cast<size_t>(col) * h + feat, v, push, p.pv, tag, col, feat);
    }
    if (lane == 0 && sub == 0) IQ_STAMP(p, 5);
  }
}


// ------------------------------------------------------------------------------------
// The direct form of iq_linear for short streams (the row-parallel o_proj of a shard, the
// column-parallel QKV): the same layout as the Down's -- 32 weight rows per CTA, warp
// (s, q) owns row sub-tile s and the K units q, q+4, ... of 256 bytes -- with the
// activations staged (and quantised per 1x128 group, or split into two e4m3 terms) once per
// CTA after the wait, one weight scale per run and one activation scale per 128 bytes.
struct LinearDirectParams {
  IQ_TRACE_FIELD
  const void* x;
  const float* x_scale;
  int x_kind, m, k, n;
  int rg_shift, kg_shift;
  const uint8_t* w;
  const float* w_scale;
  __nv_bfloat16* out;
  float* out_f32;
  void* scratch;
  int n_tail;
  int push;
  int per_round;
  iq_tail_args tail;
  PushView pv;
};

constexpr int kDirectUnitRuns = 4;                       // 64-byte runs per K unit
constexpr int kDirectUnitBytes = kDirectUnitRuns * 64;

// Shared memory of a tile CTA: the reduction buffer, then the staged activation rows
// (x_rows x (k + 64) bytes) and their scales (x_rows x k/128 floats).
__host__ __device__ inline size_t linear_direct_smem(int x_rows, int k) {
  return sizeof(float) * 9 * 32 * 4 + static_cast<size_t>(x_rows) * (k + 64) +
         sizeof(float) * x_rows * ((k + 127) / 128) + 64;
}

template <int SUBS>
__global__ void __launch_bounds__(320, 2) linear_direct_kernel(const __grid_constant__ LinearDirectParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int RPU = kDirectUnitRuns;
  constexpr int kQ = SUBS == 3 ? 3 : 4;            // warps per row sub-tile
  constexpr int kThreads = SUBS * kQ * 32;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const int tile_ctas = static_cast<int>(gridDim.x) - p.n_tail;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  if (cta >= tile_ctas) {
    PushView pv = p.pv;
#ifdef IQ_TRACE
    pv.trace = p.trace ? p.trace + blockIdx.x * kTraceWords : nullptr;
#endif
    tail_cta(p.tail, pv, p.per_round, cta - tile_ctas, p.n_tail, smem);
    if (tid == 0) { IQ_STAMP(p, 11); IQ_CLOCK(p, 10); }
    return;
  }
  const bool split2 = p.x_kind == IQ_X_BF16_SPLIT2;
  const int k = p.k, m = p.m, n = p.n;
  const int x_rows = split2 ? 2 * m : m;
  float(*red)[32][4] = reinterpret_cast<float(*)[32][4]>(smem);
  uint8_t* xq = smem + sizeof(float) * 9 * 32 * 4;
  float* xs = reinterpret_cast<float*>(xq + static_cast<size_t>(x_rows) * (k + 64));
  StreamShape sh{};                       // (what the staging routines read of it)
  sh.x_pitch = k + 64;
  sh.x_blocks = (k + 127) / 128;
  const int sub = warp / kQ, q = warp - sub * kQ;
  const int row0 = cta * (SUBS * 16) + sub * 16;
  const int g8 = lane >> 2, t = lane & 3;
  const int n_units = k / kDirectUnitBytes;
  const int krow = k >> p.kg_shift;       // weight scale entries per row block

  // ---- ahead of the dependency wait: the first unit's weights into registers, the later
  // units' rows into L2
  auto load_w = [&](DirectW<RPU>& w, int unit) {
    const uint8_t* a = p.w + static_cast<size_t>(row0 + g8) * k + unit * kDirectUnitBytes + t * 16;
    const uint8_t* b = a + static_cast<size_t>(8) * k;
    const float* sc = p.w_scale + static_cast<size_t>(row0 >> p.rg_shift) * krow;
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      w.wa[run] = ldg_nc_u4(a + run * 64);
      w.wb[run] = ldg_nc_u4(b + run * 64);
      w.ws[run] = __ldg(sc + ((unit * kDirectUnitBytes + run * 64) >> p.kg_shift));
    }
  };
  DirectW<RPU> cur, nxt;
  int unit = q;
  if (unit < n_units) load_w(cur, unit);
  for (int u = unit + kQ; u < n_units; u += kQ)
    prefetch_l2(p.w + static_cast<size_t>(row0 + (lane >> 1)) * k + u * kDirectUnitBytes + (lane & 1) * 128);
  after_wait();
  if (tid == 0) IQ_STAMP(p, 1);

  // ---- the activations: staged (and quantised) once per CTA
  if (p.x_kind == IQ_X_BF16_GROUPQ || split2)
    stage_rows_bf16_groupq(xq, xs, sh, static_cast<const __nv_bfloat16*>(p.x), k, m, k, split2,
                           tid, kThreads);
  else
    stage_rows_e4m3(xq, xs, sh, static_cast<const uint8_t*>(p.x), k,
                    p.x_kind == IQ_X_E4M3_GROUP ? p.x_scale : nullptr, m, k, tid, kThreads);
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 2);

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t xq_s = smem_u32(xq), xs_s = smem_u32(xs);
  const bool live_g = g8 < x_rows, live0 = 2 * t < x_rows, live1 = 2 * t + 1 < x_rows;
  while (unit < n_units) {
    if (unit + kQ < n_units) load_w(nxt, unit + kQ);
    const int kb0 = unit * kDirectUnitBytes;
    float part[RPU][4];
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (live_g) xv = lds128(xq_s + g8 * sh.x_pitch + kb0 + run * 64 + t * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) part[run][i] = 0.f;
      mma_e4m3(part[run], cur.wa[run].x, cur.wb[run].x, cur.wa[run].y, cur.wb[run].y, xv.x, xv.y);
      mma_e4m3(part[run], cur.wa[run].z, cur.wb[run].z, cur.wa[run].w, cur.wb[run].w, xv.z, xv.w);
    }
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      const int xblk = (kb0 + run * 64) >> 7;
      const float s0 = live0 ? cur.ws[run] * lds_f32(xs_s + ((2 * t) * sh.x_blocks + xblk) * 4) : 0.f;
      const float s1 = live1 ? cur.ws[run] * lds_f32(xs_s + ((2 * t + 1) * sh.x_blocks + xblk) * 4) : 0.f;
      acc[0] = fmaf(part[run][0], s0, acc[0]);
      acc[1] = fmaf(part[run][1], s1, acc[1]);
      acc[2] = fmaf(part[run][2], s0, acc[2]);
      acc[3] = fmaf(part[run][3], s1, acc[3]);
    }
    unit += kQ;
    cur = nxt;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) red[warp][lane][i] = acc[i];
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 4);

  if (q == 0) {
    int col = lane >> 2;
    const int r0 = (lane & 3) * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + j;
      const int fl = 4 * (r & 7) + (col >> 1), fi = (r >> 3) * 2 + (col & 1);
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kQ; ++w) s += red[sub * kQ + w][fl][fi];
      v[j] = s;
    }
    int row = col;
    bool live = col < m;
    if (split2) {
      // columns 2j and 2j+1 (four lanes apart) are the two terms of row j
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += __shfl_xor_sync(0xffffffffu, v[j], 4);
      row = col >> 1;
      live = (col & 1) == 0 && row < m;
    }
    if (live) {
      const bool push = p.push != 0;
      const uint32_t tag = push ? tag16_of(ld_volatile_u32(p.pv.epoch)) : 0u;
      const int feat = row0 + r0;
      const size_t index = static_cast<size_t>(row) * n + feat;
      if (p.out_f32)
        *reinterpret_cast<float4*>(p.out_f32 + index) = make_float4(v[0], v[1], v[2], v[3]);
      if (p.out) store_row4(p.out, index, v, push, p.pv, tag, row, feat);
    }
    if (lane == 0 && sub == 0) IQ_STAMP(p, 5);
  }
}

}  // namespace iqb
