// The kernels of the block-FP8 tensor-parallel decode path and their C ABI
// (declared in include/iqb200.h), built on the streaming engine of stream_core.cuh:
//
//   iq_linear    row-parallel block-FP8 product (+ fused all-reduce tail)
//   iq_router    bf16 router GEMV + top-k selection in one launch
//   iq_moe_gate  grouped expert Gate/Up + SiLU, each distinct expert streamed once
//   iq_moe_down  grouped expert Down (+ fused all-reduce tail)
//   iq_tail      the all-reduce + residual + RMSNorm epilogue on its own
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <utility>

#include "stream_core.cuh"

namespace iqb {

// ------------------------------------------------------------------------------------
// Scratch layout (bytes): status @0, ticket @64, launch tag @128, tail ticket @132, tile
// counters @256, partials after; behind this basic part the tagged hand-off words of the
// router's logits and the landing zone of a tail that has no peers.
constexpr size_t kScrTicket = 64;
constexpr size_t kScrLaunchTag = 128;    // u32: launches that handed results off as tagged words
constexpr size_t kScrTailTicket = 132;   // u32: tail CTAs of the running launch that are done
constexpr size_t kScrGateDone = 136;     // u32: working CTAs of all Gate launches that have finished (only grows)
constexpr size_t kScrCounters = 256;
constexpr int kMaxTiles = 16384;
constexpr size_t kScrPartials = kScrCounters + sizeof(uint32_t) * kMaxTiles;
constexpr int kMaxGrid = 256;
constexpr size_t kScrBasicBytes = kScrPartials + sizeof(float) * kMaxGrid * 2 * 256 * 8;
constexpr int kMaxRows = 8;
constexpr int kMaxExperts = 512;
constexpr int kZoneMaxH = 8192;
constexpr int kMaxKSlices = 8;          // K slices a router launch may split its rows into
constexpr size_t kScrLogits = kScrBasicBytes;                                    // u64 [8][8][512]
constexpr size_t kScrZone =
    kScrLogits + sizeof(uint64_t) * kMaxKSlices * kMaxRows * kMaxExperts;         // u32 [8][8192]
constexpr size_t kScrBytes = kScrZone + sizeof(uint32_t) * kMaxRows * kZoneMaxH;

__host__ __device__ inline StreamScratch scratch_of(void* base) {
  StreamScratch s;
  uint8_t* b = static_cast<uint8_t*>(base);
  s.status = reinterpret_cast<int*>(b);
  s.ticket = reinterpret_cast<uint32_t*>(b + kScrTicket);
  s.tile_counter = reinterpret_cast<uint32_t*>(b + kScrCounters);
  s.partials = reinterpret_cast<float*>(b + kScrPartials);
  s.trace = nullptr;
  return s;
}

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Per-CTA timelines, compiled in with -DIQ_TRACE only: every launch made while a trace
// buffer is set (iq_trace_set) takes the next slot of it, and each CTA stamps %globaltimer
// at a few points of its life into `trace[cta][point]` (point 15: the SM it ran on).
constexpr int kTraceCtas = 304;
constexpr int kTraceWords = 32;   // 16 %globaltimer stamps, then 16 SM-clock stamps
#ifdef IQ_TRACE
#define IQ_TRACE_FIELD unsigned long long* trace;
#define IQ_TRACE_SCRATCH(scr, p) \
  (scr).trace = (p).trace ? (p).trace + blockIdx.x * kTraceWords : nullptr
#define IQ_STAMP(p, k)                                                                   \
  do {                                                                                   \
    if ((p).trace) (p).trace[blockIdx.x * kTraceWords + (k)] = globaltimer_ns();          \
  } while (0)
#define IQ_CLOCK(p, k)                                                                   \
  do {                                                                                   \
    if ((p).trace)                                                                       \
      (p).trace[blockIdx.x * kTraceWords + 16 + (k)] = static_cast<unsigned long long>(clock64()); \
  } while (0)
__device__ __forceinline__ unsigned long long smid_of() {
  unsigned v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}
#else
#define IQ_TRACE_FIELD
#define IQ_TRACE_SCRATCH(scr, p) do {} while (0)
#define IQ_STAMP(p, k) do {} while (0)
#define IQ_CLOCK(p, k) do {} while (0)
#endif

// Shared-memory carve-up after StreamSmem: activation scales, staged activations, ring.
template <class G>
struct Carve {
  StreamSmem<G>* sm;
  float* sc;      // gathered weight scales [max_items][SCALES_PER_STAGE]
  float* xs;
  uint8_t* xq;
  uint8_t* ring;
};
template <class G>
__host__ __device__ inline size_t smem_fixed_bytes(const StreamShape& sh) {
  size_t off = align_up(sizeof(StreamSmem<G>), 16);
  off += align_up(sizeof(float) * sh.max_items * G::SCALES_PER_STAGE, 16);
  off += align_up(sizeof(float) * sh.x_rows * sh.x_blocks, 16);
  off += static_cast<size_t>(sh.x_rows) * sh.x_pitch;
  return align_up(off, 128);
}
template <class G>
__device__ inline Carve<G> carve(uint8_t* base, const StreamShape& sh) {
  Carve<G> c;
  c.sm = reinterpret_cast<StreamSmem<G>*>(base);
  size_t off = align_up(sizeof(StreamSmem<G>), 16);
  c.sc = reinterpret_cast<float*>(base + off);
  off += align_up(sizeof(float) * sh.max_items * G::SCALES_PER_STAGE, 16);
  c.xs = reinterpret_cast<float*>(base + off);
  off += align_up(sizeof(float) * sh.x_rows * sh.x_blocks, 16);
  c.xq = base + off;
  c.ring = base + smem_fixed_bytes<G>(sh);
  return c;
}

// ------------------------------------------------------------------------------------
// Activation staging (the CTA's `nthr` consumer threads, tid in [0, nthr)).

// Both routines issue a batch of independent 16-byte global loads before touching any of
// them, so a row set costs about one memory latency instead of one per group.  The loads
// bypass L1 (ld.global.cg): in the one-launch layer the rows were written by another CTA
// of the same launch.
constexpr int kStageBatch = 8;

// Two values to e4m3 (saturating) by one conversion: low byte = lo.
__device__ __forceinline__ uint32_t e4m3x2_sat(float lo, float hi) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}
// Vector `i` of a row set with `vec` vectors per row -> (row, vector in the row).  Every
// CTA of a launch stages the same rows, so the staging is bound by instruction issue on
// each SM; a power-of-two row length (the usual case) saves two integer divisions per
// vector.
struct RowVec { int r, v; };
__device__ __forceinline__ RowVec row_vec(int i, int vec, int vec_shift) {
  const int r = vec_shift >= 0 ? i >> vec_shift : i / vec;
  return {r, i - r * vec};
}
__device__ __forceinline__ int shift_of(int vec) {
  return (vec & (vec - 1)) == 0 ? 31 - __clz(vec) : -1;
}

// Raw e4m3 rows (16-byte vectors) + their scales (or 1).
__device__ inline void stage_rows_e4m3(uint8_t* xq, float* xs, const StreamShape& sh,
                                       const uint8_t* src, size_t src_pitch,
                                       const float* src_scale, int rows, int k, int tid,
                                       int nthr) {
  const int vec = k / 16, nvec = rows * vec, vsh = shift_of(vec);
  // the first activation scale of this thread rides along with the first batch of loads
  const int nxs = rows * sh.x_blocks;
  float xs_first = 1.0f;
  if (src_scale && tid < nxs) xs_first = __ldcg(src_scale + tid);
  for (int v0 = 0; v0 < nvec; v0 += nthr * kStageBatch) {
    uint4 raw[kStageBatch];
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * nthr >= nvec) break;   // same for every thread
      const int i = v0 + j * nthr + tid;
      if (i < nvec) {
        const RowVec rv = row_vec(i, vec, vsh);
        raw[j] = __ldcg(reinterpret_cast<const uint4*>(src + rv.r * src_pitch + rv.v * 16));
      }
    }
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * nthr >= nvec) break;
      const int i = v0 + j * nthr + tid;
      if (i < nvec) {
        const RowVec rv = row_vec(i, vec, vsh);
        *reinterpret_cast<uint4*>(xq + rv.r * sh.x_pitch + rv.v * 16) = raw[j];
      }
    }
  }
  if (tid < nxs) xs[tid] = xs_first;
  for (int i = tid + nthr; i < nxs; i += nthr)
    xs[i] = src_scale ? __ldcg(src_scale + i) : 1.0f;
}

// bf16 rows quantised per 1x128 group: scale = amax/448 (1 for an all-zero group), value
// = e4m3(x * (1 / scale)).  A thread holds eight consecutive elements, so a group is sixteen
// consecutive lanes.  With `split2` row r becomes staged rows 2r (the e4m3 value) and
// 2r+1 (the e4m3 of what the first term missed), both under the same scale.
__device__ inline void stage_rows_bf16_groupq(uint8_t* xq, float* xs, const StreamShape& sh,
                                              const __nv_bfloat16* src, size_t src_pitch,
                                              int rows, int k, bool split2, int tid, int nthr) {
  const int vec = k / 8, nvec = rows * vec, vsh = shift_of(vec);
  for (int v0 = 0; v0 < nvec; v0 += nthr * kStageBatch) {
    uint4 raw[kStageBatch];
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * nthr >= nvec) break;   // same for every thread
      const int i = v0 + j * nthr + tid;
      raw[j] = make_uint4(0u, 0u, 0u, 0u);
      if (i < nvec) {
        const RowVec rv = row_vec(i, vec, vsh);
        raw[j] = __ldcg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(rv.r) * src_pitch + rv.v * 8));
      }
    }
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * nthr >= nvec) break;    // whole batch dead: nothing to do
      const int i = v0 + j * nthr + tid;   // uniform trip count: shuffles below
      const bool live = i < nvec;
      const RowVec rv = row_vec(live ? i : 0, vec, vsh);
      const int r = rv.r, v = rv.v;
      // (bf16 -> fp32 is a shift: two logic operations per pair)
      const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
      float f[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        f[2 * q] = __uint_as_float(w[q] << 16);
        f[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
      }
      float amax = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
#pragma unroll
      for (int o = 8; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (!live) continue;               // after the shuffles: dead lanes skip the math
      const float s = amax > 0.f ? amax / 448.0f : 1.0f;
      const float rcp = 1.0f / s;        // one division per vector; values use x * (1/s)
      const int blk = v >> 4;
      if (split2) {
        uint32_t q0[2] = {0u, 0u}, q1[2] = {0u, 0u};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float xn = f[q] * rcp;
          const uint8_t a = f32_to_e4m3_sat(xn);
          q0[q >> 2] |= static_cast<uint32_t>(a) << (8 * (q & 3));
          q1[q >> 2] |= static_cast<uint32_t>(f32_to_e4m3_sat(xn - e4m3_to_f32(a))) << (8 * (q & 3));
        }
        *reinterpret_cast<uint2*>(xq + (2 * r) * sh.x_pitch + v * 8) = make_uint2(q0[0], q0[1]);
        *reinterpret_cast<uint2*>(xq + (2 * r + 1) * sh.x_pitch + v * 8) = make_uint2(q1[0], q1[1]);
        if ((v & 15) == 0) {
          xs[(2 * r) * sh.x_blocks + blk] = s;
          xs[(2 * r + 1) * sh.x_blocks + blk] = s;
        }
      } else {
        // (packed conversions: one instruction per pair of values)
        const uint32_t lo = e4m3x2_sat(f[0] * rcp, f[1] * rcp) | (e4m3x2_sat(f[2] * rcp, f[3] * rcp) << 16);
        const uint32_t hi = e4m3x2_sat(f[4] * rcp, f[5] * rcp) | (e4m3x2_sat(f[6] * rcp, f[7] * rcp) << 16);
        *reinterpret_cast<uint2*>(xq + r * sh.x_pitch + v * 8) = make_uint2(lo, hi);
        if ((v & 15) == 0) xs[r * sh.x_blocks + blk] = s;
      }
    }
  }
}

// Programmatic dependent launch discipline shared by the kernels: a CTA lets its
// dependents be scheduled only AFTER its own wait on its predecessor has returned.  The
// successor kernel therefore starts no earlier than the completion of this kernel's
// predecessor, so before ITS wait it may already read anything written two or more
// launches back (pdl level 2: the Down reads the router's routes, the Gate reads the
// attention tail's activations) as well as weights, and only has to wait for what its
// immediate predecessor writes.
__device__ __forceinline__ void after_wait() {
  pdl_wait();
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------
// The tail: all-reduce of the ranks' bf16 rows, residual add and RMSNorm(s).
//
// Push protocol.  A producing GEMV hands its rows to the tail as 32-bit words, bf16 value
// in the low half and the 16-bit tag of the call in the high half, stored from its epilogue
// into the landing zone `recv[source rank][row][feature]` of EVERY rank (one multimem.st
// per four words; one store per peer without multicast; a local store without peers).  A
// word that shows the call's tag is complete by itself, so the producer needs no fence, no
// counter and no flag, and the tail reads local memory only.
struct PushView {
  uint32_t* recv;             // this rank's landing zone, u32 [world][rows][h]
  uint32_t* recv_mc;          // multicast alias, or null
  uint32_t* const* peer_recv; // device array [world], or null
  uint32_t* epoch;            // local word: completed calls on the zone (the tag's source)
  uint32_t* ticket;           // local word: tail CTAs of the running call that have started
  int world, rank, rows, h;
  unsigned long long* trace;  // trace builds: this CTA's stamps (else null)
};

// Tags run over 1..65535, so a zero-filled zone never looks complete.
__device__ __forceinline__ uint32_t tag16_of(uint32_t epoch) { return epoch % 65535u + 1u; }

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Four consecutive features of `row`, tagged, into every rank's zone.
__device__ __forceinline__ void push_words(const PushView& pv, int row, int feat,
                                           const uint32_t (&w)[4]) {
  const size_t off = (static_cast<size_t>(pv.rank) * pv.rows + row) * pv.h + feat;
  if (pv.recv_mc) {
    multimem_st_u32x4(pv.recv_mc + off, w);
  } else if (pv.world > 1) {
    for (int p = 0; p < pv.world; ++p) st_relaxed_sys_u32x4(pv.peer_recv[p] + off, w);
  } else {
    st_relaxed_gpu_u32x4(pv.recv + off, w);
  }
}

__device__ __forceinline__ uint32_t tagged_bf16(float v, uint32_t tag) {
  return (tag << 16) | static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}

struct TailParams {
  iq_tail_args a;
  PushView pv;
  int push;      // 1: rows arrive through the landing zone
  int n_tail;    // CTAs that share the rows
  int per_round; // sources a tail CTA polls at a time
};

__device__ inline void bf16x8_to_f32(const U4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(p[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ inline U4 f32_to_bf16x8(const float (&f)[8]) {
  U4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) p[j] = __float22bfloat162_rn(make_float2(f[2 * j], f[2 * j + 1]));
  return u;
}
__device__ inline float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// Two values rounded to bf16 by ONE conversion instruction: the packed pair (what a store
// wants) and the two rounded values back in fp32 (two moves).  The tail rounds every element
// up to five times; single conversions were a third of its instructions.
__device__ __forceinline__ uint32_t bf16x2_round(float lo, float hi, float& rlo, float& rhi) {
  const __nv_bfloat162 p = __float22bfloat162_rn(make_float2(lo, hi));
  const uint32_t u = *reinterpret_cast<const uint32_t*>(&p);
  rlo = __uint_as_float(u << 16);
  rhi = __uint_as_float(u & 0xffff0000u);
  return u;
}

// The threads that run a block-wide helper together: the whole CTA (n == 0), or threads
// [0, n) of it meeting on named barrier `id` while the CTA's other warps do something else.
struct BlockBar {
  int id = 0, n = 0;
  __device__ __forceinline__ void sync() const {
    if (n == 0) __syncthreads();
    else named_bar_sync(id, n);
  }
  __device__ __forceinline__ int threads() const { return n == 0 ? static_cast<int>(blockDim.x) : n; }
};

// Block-wide sum with one barrier: every warp drops its sum into `slots`, every thread
// adds the slots up in warp order.  Consecutive calls must alternate `slots` buffers.
__device__ inline float block_sum(float v, float* slots, const BlockBar& bar) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = bar.threads() >> 5;
  v = warp_sum(v);
  if (lane == 0) slots[warp] = v;
  bar.sync();
  float s = 0.f;
  for (int w = 0; w < nwarps; ++w) s += slots[w];
  return s;
}

// The tail runs on 256 threads wherever it runs (a tail CTA of any streaming kernel, the
// last CTA of the pull protocol, the tail kernel), so that its block-wide sums add in one
// order and every form gives the same bits.
constexpr int kTailThreads = 256;
constexpr int kTailVecs = 3;   // 16-byte vectors of a row per thread: h <= 8 * 3 * 256 = 6144

__device__ __forceinline__ void ldg_f32x8(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Row `r` of the landing zone, summed over the source ranks in rank order (fp32, one bf16
// rounding), for this thread's vectors.  The sources are taken `per_round` at a time (as
// many as the CTA's shared memory `zs` holds rows for: [per_round][h] words): every
// (vector, source) chunk of 8 words of a round is copied into shared memory with
// asynchronous 16-byte copies that go to L2, all of them in flight together; a chunk whose
// words do not all show `tag` yet is copied again; a complete round is added up and the
// next one starts.  A thread reads back only what it copied itself.  Returns false when
// the budget ran out.  `warm`: copy each chunk once and take it as it is (see run_tail).
__device__ __forceinline__ bool poll_zone_row(const PushView& pv, uint32_t* zs, int per_round,
                                              int r, uint32_t tag, int tid, int nthr,
                                              int vec_per_row, uint64_t budget_ns, bool warm,
                                              float (&f)[kTailVecs][8]) {
  const size_t src_stride = static_cast<size_t>(pv.rows) * pv.h;
  const uint32_t* row0 = pv.recv + static_cast<size_t>(r) * pv.h;
  const uint32_t zs_s = smem_u32(zs);
  float acc[kTailVecs][8];
#pragma unroll
  for (int i = 0; i < kTailVecs; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  uint64_t t0 = 0;
  bool ok = true;
  for (int p0 = 0; p0 < pv.world && ok; p0 += per_round) {
    const int np = pv.world - p0 < per_round ? pv.world - p0 : per_round;
    uint32_t pend = 0;                                    // bit i*8+p: chunk still incomplete
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i)
      if (tid + i * nthr < vec_per_row) pend |= ((1u << np) - 1u) << (8 * i);
    while (pend) {
#pragma unroll
      for (int i = 0; i < kTailVecs; ++i) {
        const int v = tid + i * nthr;
        for (int p = 0; p < np; ++p) {
          if (!((pend >> (8 * i + p)) & 1u)) continue;
          const uint32_t* src = row0 + (p0 + p) * src_stride + v * 8;
          const uint32_t dst = zs_s + (p * pv.h + v * 8) * 4;
          cp_async16(dst, src);
          cp_async16(dst + 16, src + 4);
        }
      }
      cp_async_wait_all();
#pragma unroll
      for (int i = 0; i < kTailVecs; ++i) {
        const int v = tid + i * nthr;
        for (int p = 0; p < np; ++p) {
          if (!((pend >> (8 * i + p)) & 1u)) continue;
          const uint4 lo = lds128(zs_s + (p * pv.h + v * 8) * 4);
          const uint4 hi = lds128(zs_s + (p * pv.h + v * 8) * 4 + 16);
          const uint32_t all = (lo.x >> 16 == tag) & (lo.y >> 16 == tag) & (lo.z >> 16 == tag) &
                               (lo.w >> 16 == tag) & (hi.x >> 16 == tag) & (hi.y >> 16 == tag) &
                               (hi.z >> 16 == tag) & (hi.w >> 16 == tag);
          if (all) pend &= ~(1u << (8 * i + p));
        }
      }
      if (warm) pend = 0;          // a rehearsal takes whatever the zone holds
      if (pend) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > budget_ns) { ok = false; break; }
      }
    }
    if (!ok) break;
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      for (int p = 0; p < np; ++p) {
        const uint4 lo = lds128(zs_s + (p * pv.h + v * 8) * 4);
        const uint4 hi = lds128(zs_s + (p * pv.h + v * 8) * 4 + 16);
        acc[i][0] += __uint_as_float(lo.x << 16); acc[i][1] += __uint_as_float(lo.y << 16);
        acc[i][2] += __uint_as_float(lo.z << 16); acc[i][3] += __uint_as_float(lo.w << 16);
        acc[i][4] += __uint_as_float(hi.x << 16); acc[i][5] += __uint_as_float(hi.y << 16);
        acc[i][6] += __uint_as_float(hi.z << 16); acc[i][7] += __uint_as_float(hi.w << 16);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kTailVecs; ++i) bf16x8_to_f32(f32_to_bf16x8(acc[i]), f[i]);
  return ok;
}

// Runs on the threads of `bar` (a multiple of 32) for rows r_begin,
// r_begin + r_step, ... of the call.  `red` is shared memory for 4 x 32 floats, `sflag`
// one shared int (push: set to 1 by the caller), `tag` (push) the call's tag, `park` shared
// memory for the residual row (it waits there),
// `zs` (push only) shared memory for per_round x h words.  Without `kPush`,
// rows written by other CTAs of this launch must already be visible (the caller passed
// the ticket) and the pull protocol's signal / wait / switch read applies for world > 1.
// `warm` (push only): a rehearsal -- the same instructions on whatever the buffers hold,
// without waiting and without a single global store.  Code that runs once per launch runs
// at the speed its instructions arrive from L2 (measured here: about 2 us for the 10 KB of
// one row's arithmetic), so a tail CTA, which has nothing to do until its rows arrive,
// goes through the whole path once ahead of time and finds it in the instruction cache
// when it matters.
// Each row is handled entirely in registers and each RMSNorm costs one block barrier.  The
// kernels this runs in keep almost all of the SM's L1 as shared memory, so a spilled
// register would cost an L2 round trip: the loads are ordered to keep few values live
// (the residual stays packed until it is used; each norm weight is fetched just before
// the barrier of the reduction that precedes its use, which hides its latency).
template <bool kPush>
__device__ __forceinline__ void run_tail(const iq_tail_args& a, const PushView& pv, uint32_t tag,
                                         uint8_t* park, uint32_t* zs, int per_round, float* red,
                                         int* sflag, const BlockBar bar = BlockBar{},
                                         int r_begin = 0, int r_step = 1, bool warm = false) {
  const int tid = threadIdx.x, nthr = bar.threads();
  const uint32_t res_s = smem_u32(park);
  const int pstride = a.residual_fp32 ? 32 : 16;      // parked bytes per 8 elements
  const int m = a.m, h = a.h, vec_per_row = h / 8;
  const float inv_h = 1.0f / static_cast<float>(h);
  const bool attn = a.kind == IQ_TAIL_ATTN;

  for (int r = r_begin; r < m; r += r_step) {
    const size_t row_off = static_cast<size_t>(r) * h;
    float* slots0 = red + (r & 1) * 64;        // two reductions per row, alternating rows
    float* slots1 = slots0 + 32;
    // ---- the row's residual: copied asynchronously into this thread's own 32-byte slots
    // of shared memory before the cross-rank wait, so that it costs no registers while the
    // row is awaited (a spilled register would cost an L2 round trip here)
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      const size_t off = row_off + static_cast<size_t>(v) * 8;
      if (a.residual_fp32) {
        const float* rp = static_cast<const float*>(a.residual) + off;
        cp_async16(res_s + v * pstride, rp);
        cp_async16(res_s + v * pstride + 16, rp + 4);
      } else {
        cp_async16(res_s + v * pstride, static_cast<const __nv_bfloat16*>(a.residual) + off);
      }
    }
    cp_async_commit();
    float f[kTailVecs][8];
    float wv[kTailVecs][8];    // w_first (attention tail), then / otherwise w_norm
    // The first norm weight the row meets is loaded now, ahead of the wait for the row: its
    // latency would otherwise sit between the row's arrival and its first use.
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v < vec_per_row) ldg_f32x8((attn ? a.w_first : a.w_norm) + v * 8, wv[i]);
    }
    if (kPush) {
      // ---- the row arrives in the landing zone: poll it, add the ranks
      const uint64_t budget = 1000000ull * (a.timeout_ms ? a.timeout_ms : 2000u);
      if (!poll_zone_row(pv, zs, per_round, r, tag, tid, nthr, vec_per_row, budget, warm, f))
        *sflag = 0;
      bar.sync();
      if (!*sflag) {
        // A source is missing: leave the outputs untouched and let the host read the status.
        if (tid == 0) set_status(a.status, IQ_ERR_PEER_TIMEOUT);
        return;
      }
      if (tid == 0 && pv.trace && !warm) { pv.trace[10] = globaltimer_ns(); pv.trace[16 + 12] = clock64(); }
    } else {
      // ---- cross-rank readiness: signal, then wait while the residual loads are in flight
      if (r == r_begin && a.world > 1) {
        if (tid == 0) {
          const uint32_t target = (*a.epoch + 1u) * static_cast<uint32_t>(a.world);
          if (a.arrive_mc) {
            multimem_red_add_release_u32(a.arrive_mc, 1u);
          } else {
            for (int p = 0; p < a.world; ++p)
              asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(a.peer_arrive[p]), "r"(1u)
                           : "memory");
          }
          const uint64_t budget = 1000000ull * (a.timeout_ms ? a.timeout_ms : 2000u);
          uint64_t t0 = 0;
          int ok = 1;
          for (uint32_t spin = 0;; ++spin) {
            if (static_cast<int32_t>(ld_acquire_sys_u32(a.arrive) - target) >= 0) break;
            if ((spin & 255u) == 255u) {
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > budget) { ok = 0; break; }
            }
          }
          if (!ok) set_status(a.status, IQ_ERR_PEER_TIMEOUT);
          *sflag = ok;
        }
        bar.sync();
        if (!*sflag) {
          // Peers are missing: leave the outputs untouched and let the host read the status.
          if (tid == 0) *a.epoch = *a.epoch + 1u;
          return;
        }
      }
      // ---- the reduced partial
#pragma unroll
      for (int i = 0; i < kTailVecs; ++i) {
        const int v = tid + i * nthr;
        if (v >= vec_per_row) continue;
        const size_t off = row_off + static_cast<size_t>(v) * 8;
        U4 part;
        if (a.world == 1) {
          const uint4 t = __ldcg(reinterpret_cast<const uint4*>(
              static_cast<const __nv_bfloat16*>(a.partial) + off));
          part = U4{t.x, t.y, t.z, t.w};
        } else if (a.partial_mc) {
          part = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(a.partial_mc) + off);
        } else {
          // four peers' vectors in flight at a time, summed in rank order
          float accv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int p0 = 0; p0 < 8; p0 += 4) {
            if (p0 >= a.world) break;
            U4 pvv[4];
#pragma unroll
            for (int p = 0; p < 4; ++p)
              if (p0 + p < a.world)
                pvv[p] = ld_global_u4(static_cast<const __nv_bfloat16*>(a.peer_partials[p0 + p]) + off);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              if (p0 + p >= a.world) continue;
              float t[8];
              bf16x8_to_f32(pvv[p], t);
#pragma unroll
              for (int j = 0; j < 8; ++j) accv[j] += t[j];
            }
          }
          part = f32_to_bf16x8(accv);
        }
        bf16x8_to_f32(part, f[i]);
      }
      cp_async_wait_all();     // the residual (push: the zone's poll has waited for it)
    }

    float inv1 = 0.f;
    if (attn) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kTailVecs; ++i) {
        const int v = tid + i * nthr;
        if (v >= vec_per_row) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[i][j], f[i][j], ss);
      }
      inv1 = rsqrtf(block_sum(ss, slots0, bar) * inv_h + a.eps);
      if (kPush && tid == 0 && pv.trace && !warm) { pv.trace[12] = globaltimer_ns(); pv.trace[16 + 13] = clock64(); }
    }
    // ---- h = residual + (ATTN: bf16(bf16(w1*(ao*inv))*scale) | MLP: bf16(m*scale))
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      const size_t off = row_off + static_cast<size_t>(v) * 8;
      float res[8];
      const uint4 ra = lds128(res_s + v * pstride);
      if (a.residual_fp32) {
        const uint4 rb = lds128(res_s + v * pstride + 16);
        res[0] = __uint_as_float(ra.x); res[1] = __uint_as_float(ra.y);
        res[2] = __uint_as_float(ra.z); res[3] = __uint_as_float(ra.w);
        res[4] = __uint_as_float(rb.x); res[5] = __uint_as_float(rb.y);
        res[6] = __uint_as_float(rb.z); res[7] = __uint_as_float(rb.w);
      } else {
        bf16x8_to_f32(U4{ra.x, ra.y, ra.z, ra.w}, res);
      }
      uint32_t hb[4];
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        float add0, add1;
        if (attn) {
          float n0, n1;
          bf16x2_round(wv[i][j] * (f[i][j] * inv1), wv[i][j + 1] * (f[i][j + 1] * inv1), n0, n1);
          bf16x2_round(n0 * a.scale, n1 * a.scale, add0, add1);
        } else {
          bf16x2_round(f[i][j] * a.scale, f[i][j + 1] * a.scale, add0, add1);
        }
        f[i][j] = res[j] + add0;                 // f now holds h
        f[i][j + 1] = res[j + 1] + add1;
        if (!a.residual_fp32)                    // the norm sees the rounded stream
          hb[j >> 1] = bf16x2_round(f[i][j], f[i][j + 1], f[i][j], f[i][j + 1]);
      }
      if (a.residual_fp32) {
        float* ho = static_cast<float*>(a.h_out) + off;
        if (!warm) {
          *reinterpret_cast<float4*>(ho) = make_float4(f[i][0], f[i][1], f[i][2], f[i][3]);
          *reinterpret_cast<float4*>(ho + 4) = make_float4(f[i][4], f[i][5], f[i][6], f[i][7]);
        }
      } else if (!warm) {
        *reinterpret_cast<U4*>(static_cast<__nv_bfloat16*>(a.h_out) + off) = U4{hb[0], hb[1], hb[2], hb[3]};
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss2 = fmaf(f[i][j], f[i][j], ss2);
      if (attn) ldg_f32x8(a.w_norm + v * 8, wv[i]);   // (the MLP tail holds w_norm already)
    }
    if (kPush && tid == 0 && pv.trace && !warm) { pv.trace[13] = globaltimer_ns(); pv.trace[16 + 14] = clock64(); }
    const float inv2 = rsqrtf(block_sum(ss2, slots1, bar) * inv_h + a.eps);
    if (kPush && tid == 0 && pv.trace && !warm) { pv.trace[14] = globaltimer_ns(); pv.trace[16 + 15] = clock64(); }
    if (a.inv_out && tid == 0 && !warm) a.inv_out[r] = inv2;

    // ---- norm_out = bf16(w_norm * (h * inv)) (+ e4m3 copy, unscaled or per 1x128 group)
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      const bool live = v < vec_per_row;       // uniform over each 16-lane group
      const size_t off = row_off + static_cast<size_t>(live ? v : 0) * 8;
      float o[8];
      uint32_t ob[4];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        ob[j >> 1] = bf16x2_round(live ? wv[i][j] * (f[i][j] * inv2) : 0.f,
                                  live ? wv[i][j + 1] * (f[i][j + 1] * inv2) : 0.f, o[j], o[j + 1]);
        amax = fmaxf(amax, fmaxf(fabsf(o[j]), fabsf(o[j + 1])));
      }
      const bool store = live && !warm;
      if (store)
        *reinterpret_cast<U4*>(static_cast<__nv_bfloat16*>(a.norm_out) + off) = U4{ob[0], ob[1], ob[2], ob[3]};
      if (a.norm_fp8) {
        float sc = 1.0f;
        if (a.norm_fp8_scale) {
          // A 128-element group is sixteen consecutive vectors = sixteen consecutive lanes.
#pragma unroll
          for (int o2 = 8; o2; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
          sc = amax > 0.f ? amax / 448.0f : 1.0f;
          if (store && (v & 15) == 0) a.norm_fp8_scale[static_cast<size_t>(r) * (h / 128) + (v >> 4)] = sc;
        }
        const float rcp = 1.0f / sc;
        const uint32_t q0 = e4m3x2_sat(o[0] * rcp, o[1] * rcp) | (e4m3x2_sat(o[2] * rcp, o[3] * rcp) << 16);
        const uint32_t q1 = e4m3x2_sat(o[4] * rcp, o[5] * rcp) | (e4m3x2_sat(o[6] * rcp, o[7] * rcp) << 16);
        if (store) *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.norm_fp8) + off) = make_uint2(q0, q1);
      }
    }
  }
  if (!kPush && a.world > 1 && tid == 0) *a.epoch = *a.epoch + 1u;
}

// Shared memory for a parked residual row.
__host__ __device__ inline size_t tail_park_bytes(int h, int residual_fp32) {
  return static_cast<size_t>(h) * (residual_fp32 ? 4 : 2);
}

// A tail CTA of the push protocol: CTA `index` of `n_tail` finishes rows index,
// index + n_tail, ...  The last tail CTA to finish closes the call (the zone's epoch moves
// on once every tail CTA has read it).
//
// A tail CTA has nothing to do until its rows arrive, and its code runs once per launch.
// With one row it first makes a REHEARSAL pass ahead of the dependency wait: the same
// instructions on whatever the buffers hold, nothing awaited, not a single global store
// (`warm`, see run_tail), which brings the instructions in.  Measured on the layer of one
// row (hidden 6144, one rank's shard of eight): 45.9 us with the rehearsal, 47.2 us
// without, 47.5 us when the pass was repeated until the dependency resolved (the
// rehearsing CTA takes issue slots from the streaming CTA it shares its SM with), 49.7 us
// when it was made after the wait (it then ends after the rows have arrived).  With
// several rows (several tail CTAs) the rehearsal did not pay (71.0 us without, 72.2 with)
// and is left out.
__device__ __forceinline__ void tail_cta(const iq_tail_args& a, const PushView& pv, int per_round,
                                         int index, int n_tail, uint8_t* smem) {
  float* red = reinterpret_cast<float*>(smem);
  int* sflag = reinterpret_cast<int*>(smem + 512);
  uint32_t* word = reinterpret_cast<uint32_t*>(smem + 516);     // [epoch, closes the call]
  uint8_t* park = smem + 1024;
  uint32_t* zs = reinterpret_cast<uint32_t*>(smem + 1024 + tail_park_bytes(a.h, a.residual_fp32));
  const int tid = threadIdx.x;
  if (tid >= kTailThreads) return;       // (the tail runs on 256 threads: see kTailThreads)
  const BlockBar bar{2, kTailThreads};
  // Both passes go through ONE copy of the tail's code.
#pragma unroll 1
  for (int pass = n_tail == 1 ? 0 : 1; pass < 2; ++pass) {
    const bool warm = pass == 0;
    if (!warm) {
      after_wait();
      if (tid == 0 && pv.trace) { pv.trace[9] = globaltimer_ns(); pv.trace[16 + 11] = clock64(); }
    }
    // The call's tag comes from the zone's epoch.  The epoch may move on once (a) every
    // tail CTA has read it and (b) every producer has: the tail CTA that reads it LAST takes
    // on the job, and does it after its own rows are complete (every producer of the launch
    // contributes to every row, so by then all of them have read the epoch).  That keeps the
    // atomic at the start of the tail, where it waits for data anyway, and off its end.
    if (tid == 0) {
      uint32_t closes = 0, epoch = 0;
      if (!warm) {
        epoch = ld_volatile_u32(pv.epoch);
        closes = 1;
        if (n_tail > 1) {
          closes = atomicAdd(pv.ticket, 1u) == static_cast<uint32_t>(n_tail - 1);
          if (closes) *pv.ticket = 0;
        }
      }
      word[0] = epoch;
      word[1] = closes;
      *sflag = 1;
    }
    bar.sync();
    const uint32_t epoch = word[0];
    run_tail<true>(a, pv, tag16_of(epoch), park, zs, per_round, red, sflag, bar, index, n_tail,
                   warm);
    if (tid == 0 && word[1]) *pv.epoch = epoch + 1u;
    bar.sync();
  }
}

// Sources a tail CTA takes per round when it may use `limit` bytes of shared memory, and
// the shared memory that takes.
__host__ __device__ inline int tail_sources_per_round(int world, int h, int residual_fp32,
                                                      size_t limit) {
  const size_t row = static_cast<size_t>(h) * 4, fixed = 1024 + tail_park_bytes(h, residual_fp32);
  int n = limit > fixed + row ? static_cast<int>((limit - fixed) / row) : 0;
  return n > world ? world : n;
}
// (control words, the parked residual row, the rows of one round)
__host__ __device__ inline size_t tail_cta_smem(int per_round, int h, int residual_fp32) {
  return 1024 + tail_park_bytes(h, residual_fp32) + static_cast<size_t>(per_round) * h * 4;
}

__global__ void __launch_bounds__(kTailThreads) tail_kernel(const TailParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  if (p.push) {
    tail_cta(p.a, p.pv, p.per_round, static_cast<int>(blockIdx.x), p.n_tail, smem);
    return;
  }
  pdl_wait();
  pdl_launch_dependents();   // after the wait: see the note on `after_wait`
  float* red = reinterpret_cast<float*>(smem);
  int* sflag = reinterpret_cast<int*>(smem + 512);
  run_tail<false>(p.a, p.pv, 0u, smem + 1024, nullptr, 0, red, sflag, BlockBar{},
                  static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

// ------------------------------------------------------------------------------------
// iq_linear
enum TailRun : int {
  kTailNone = 0,
  kTailLastCta = 1,   // pull protocol: the last CTA to finish its tiles runs the tail
  kTailCtas = 2,      // push protocol: the launch's last `n_tail` CTAs are tail CTAs
};

struct LinearParams {
  IQ_TRACE_FIELD
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  const void* x;
  const float* x_scale;
  int x_kind, m, k, n;
  const uint8_t* w;
  const float* w_scale;
  __nv_bfloat16* out;
  float* out_f32;           // optional fp32 copy of the result
  void* scratch;
  int tail_run;             // TailRun
  int n_tail;               // tail CTAs at the end of the grid (kTailCtas)
  int push;                 // the epilogue also sends the rows to the landing zone
  int per_round;            // sources a tail CTA polls at a time
  iq_tail_args tail;
  PushView pv;
};

// Four consecutive features of one output row: bf16 into `out`, and (push) tagged into
// the landing zone.
__device__ __forceinline__ void store_row4(__nv_bfloat16* out, size_t index, const float (&v)[4],
                                           bool push, const PushView& pv, uint32_t tag, int row,
                                           int feat) {
  const __nv_bfloat162 lo = __float22bfloat162_rn(make_float2(v[0], v[1]));
  const __nv_bfloat162 hi = __float22bfloat162_rn(make_float2(v[2], v[3]));
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&lo);
  packed.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(out + index) = packed;
  if (push) {
    const uint32_t t = tag << 16;
    const uint32_t w[4] = {t | (packed.x & 0xffffu), t | (packed.x >> 16),
                           t | (packed.y & 0xffffu), t | (packed.y >> 16)};
    push_words(pv, row, feat, w);
  }
}

template <class G>
__global__ void __launch_bounds__(G::BOUND_THREADS, G::CTAS_PER_SM) linear_kernel(const __grid_constant__ LinearParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const StreamShape& sh = p.sh;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int cta = blockIdx.x;
  // CTAs that stream; the rest of the grid (push protocol) finishes the rows.
  const int stream_ctas = static_cast<int>(gridDim.x) - p.n_tail;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  if (cta >= stream_ctas) {
    PushView pv = p.pv;
#ifdef IQ_TRACE
    pv.trace = p.trace ? p.trace + blockIdx.x * kTraceWords : nullptr;
#endif
    tail_cta(p.tail, pv, p.per_round, cta - stream_ctas, p.n_tail, smem);
    if (tid == 0) { IQ_STAMP(p, 11); IQ_CLOCK(p, 10); }
    return;
  }
  const Carve<G> cv = carve<G>(smem, sh);
  StreamScratch scr = scratch_of(p.scratch);
  IQ_TRACE_SCRATCH(scr, p);
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  stream_init<G>(sh, cv.sm);
  if (tid == G::PRODUCER_WARP * 32 && !stream_whole_rows<G>(sh))
    prefetch_tensormap(&p.map0);   // only a map the host filled (K-sliced stages)
  if (tid == 0) {
    GroupDesc& g = cv.sm->groups[0];
    g.w = p.w;
    g.scale = p.w_scale;
    g.row_base = 0;
    g.map_id = 0;
    g.k_base = 0;
    for (int c = 0; c < kMaxCols; ++c) {
      g.col_row[c] = c < sh.x_rows ? c : -1;
      g.col_mul[c] = 1.0f;
      g.col_out[c] = static_cast<int16_t>(c);
    }
  }
  __syncthreads();
  {
    const CtaWork wk = cta_share<G>(sh, stream_ctas, cta, grid);
    if (warp == G::PRODUCER_WARP) {
      // Weights never change: start streaming before the predecessor kernel has finished.
      produce<G>(sh, cv.sm, cv.ring, wk, scr.status, &p.map0, &p.map1);
      if (tid == G::PRODUCER_WARP * 32) IQ_STAMP(p, 3);
      pdl_wait();
    } else if (warp < G::WARPS) {
      float held[kGatherHeld];
      gather_scales_load<G, ElemE4M3>(sh, cv.sm, wk, tid, held);   // weights: before the wait
      // (the walk through the CTA's share: ahead of the wait)
      const ConsumeHead<G> head = consume_head<G>(sh, cv.sm->groups, cv.xq, cv.xs, wk);
      after_wait();
      if (tid == 0) { IQ_STAMP(p, 1); IQ_CLOCK(p, 7); }
      if (p.x_kind == IQ_X_BF16_GROUPQ || p.x_kind == IQ_X_BF16_SPLIT2)
        stage_rows_bf16_groupq(cv.xq, cv.xs, sh, static_cast<const __nv_bfloat16*>(p.x), p.k, p.m,
                               p.k, p.x_kind == IQ_X_BF16_SPLIT2, tid, G::CONSUMER_THREADS);
      else
        stage_rows_e4m3(cv.xq, cv.xs, sh, static_cast<const uint8_t*>(p.x), p.k,
                        p.x_kind == IQ_X_E4M3_GROUP ? p.x_scale : nullptr, p.m, p.k, tid,
                        G::CONSUMER_THREADS);
      if (tid == 0) IQ_CLOCK(p, 8);
      gather_scales_store<G, ElemE4M3>(sh, cv.sm, wk, cv.sc, tid, held);
      named_bar_sync(1, G::CONSUMER_THREADS);
      if (tid == 0) { IQ_STAMP(p, 2); IQ_CLOCK(p, 9); }
      consume<G, ElemE4M3>(sh, cv.sm, cv.ring, cv.xq, cv.xs, cv.sc, wk, scr, &head);
      if (tid == 0) IQ_STAMP(p, 4);
    } else if (warp == G::EPILOGUE_WARP) {
      pdl_wait();
      const bool split2 = p.x_kind == IQ_X_BF16_SPLIT2;
      const int m = p.m, n = p.n;
      __nv_bfloat16* out = p.out;
      const bool push = p.push != 0;
      const uint32_t tag = push ? tag16_of(ld_volatile_u32(p.pv.epoch)) : 0u;
      const PushView& pv = p.pv;
      auto emit = [&](const TileId& id, int r0, int col, const float (&val)[4][G::RT]) {
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub) {
          const int feat = id.tig * G::ROWS + sub * 16 + r0;
          float v[4] = {val[0][sub], val[1][sub], val[2][sub], val[3][sub]};
          int row = col;
          bool live = col < m;
          if (split2) {
            // columns 2j and 2j+1 (four lanes apart) are the two terms of row j: fold them
            // on the even column's lane
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] += __shfl_xor_sync(0xffffffffu, v[j], 4);
            row = col >> 1;
            live = (col & 1) == 0 && row < m;
          }
          if (live) {
            const size_t index = static_cast<size_t>(row) * n + feat;
            if (p.out_f32)
              *reinterpret_cast<float4*>(p.out_f32 + index) = make_float4(v[0], v[1], v[2], v[3]);
            if (out) store_row4(out, index, v, push, pv, tag, row, feat);
          }
        }
      };
      epilogue<G, true>(sh, cv.sm, wk, total, grid, cta, scr, emit);
      if (tid == G::EPILOGUE_WARP * 32) IQ_STAMP(p, 5);
    }
  }
  if (p.tail_run == kTailLastCta && last_cta<G>(cv.sm, scr, gridDim.x)) {
    float* red = reinterpret_cast<float*>(cv.sm->red);
    if (threadIdx.x < kTailThreads)
      run_tail<false>(p.tail, p.pv, 0u, cv.ring, nullptr, 0, red, &cv.sm->is_last_tile,
                      BlockBar{2, kTailThreads});   // (the ring is idle now)
  }
  stream_drain_on_abort<G>(cv.sm);
}

// ------------------------------------------------------------------------------------
// iq_router: bf16 GEMV into fp32 logits, then top-k on the last CTA (one warp per row).
struct RouterParams {
  IQ_TRACE_FIELD
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  const __nv_bfloat16* x;
  const uint8_t* w;
  int m, h, e, top_k, score;
  int k_slices;             // the rows' K range is split over this many groups of tiles
  int* sel;
  float* wt;
  float* logits;
  void* scratch;
};

// Monotone key for finite fp32 with -0 == +0.
__device__ inline uint32_t ordered_key(float v) {
  uint32_t b = __float_as_uint(v);
  if ((b & 0x7fffffffu) == 0) b = 0;
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// One warp selects row `row`: top_k rounds of (largest key, then smallest id), softmax
// or renormalised sigmoid summed in descending-value order, pairs stored by ascending id.
// The rounds are a serial chain on the router's critical path, so each is kept to two
// warp reductions and a few moves: every lane first sorts its own keys (a compile-time
// odd-even merge network, ties to the lower id), then a round compares the lanes' heads and
// the winning lane drops its head.  The winners' probabilities are worked out afterwards,
// one per lane, all at once.
template <int N>
__device__ __forceinline__ void sort_keys_desc(uint32_t (&key)[N], int (&slot)[N]) {
#pragma unroll
  for (int p = 1; p < N; p <<= 1) {
#pragma unroll
    for (int k = p; k >= 1; k >>= 1) {
#pragma unroll
      for (int j = k % p; j + k < N; j += 2 * k) {
#pragma unroll
        for (int i = 0; i < k; ++i) {
          const int a = i + j, b = i + j + k;
          if (b < N && a / (2 * p) == b / (2 * p)) {
            const bool sw = key[b] > key[a] || (key[b] == key[a] && slot[b] < slot[a]);
            const uint32_t ka = key[a], kb = key[b];
            const int sa = slot[a], sb = slot[b];
            key[a] = sw ? kb : ka;
            key[b] = sw ? ka : kb;
            slot[a] = sw ? sb : sa;
            slot[b] = sw ? sa : sb;
          }
        }
      }
    }
  }
}

template <int kMaxPerLane>
__device__ __forceinline__ void select_row_impl(const float* logits, int e, int top_k, int score,
                                                int row, int* sel, float* wt,
                                                bool logits_in_smem, bool store) {
  const int lane = threadIdx.x & 31;
  uint32_t key[kMaxPerLane];
  int slot[kMaxPerLane];
  const int per = (e + 31) / 32;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int id = lane + 32 * j;
    float lv = 0.f;
    if (j < per && id < e)
      lv = logits_in_smem ? logits[static_cast<size_t>(row) * e + id]
                          : __ldcg(logits + static_cast<size_t>(row) * e + id);
    key[j] = (j < per && id < e) ? ordered_key(lv) : 0u;
    slot[j] = j;
  }
  sort_keys_desc<kMaxPerLane>(key, slot);
  int my_id = 0x7fffffff;      // lane t keeps the winner of round t
  uint32_t my_key = 0u;
  int n_sel = 0;
  for (int t = 0; t < top_k; ++t) {
    const uint32_t head = key[0];
    const int head_id = lane + 32 * slot[0];
    const uint32_t wmax = __reduce_max_sync(0xffffffffu, head);
    const int cand = (head == wmax && head != 0u) ? head_id : 0x7fffffff;
    const int win = __reduce_min_sync(0xffffffffu, cand);
    if (win == 0x7fffffff) break;            // fewer than top_k finite logits
    if (lane == t) { my_id = win; my_key = wmax; }
    if (head_id == win && head != 0u) {      // the winning lane drops its head
#pragma unroll
      for (int j = 0; j + 1 < kMaxPerLane; ++j) { key[j] = key[j + 1]; slot[j] = slot[j + 1]; }
      key[kMaxPerLane - 1] = 0u;
    }
    ++n_sel;
  }
  const uint32_t raw = (my_key & 0x80000000u) ? (my_key & 0x7fffffffu) : ~my_key;
  const float val = __uint_as_float(raw);
  const float top_val = __shfl_sync(0xffffffffu, val, 0);
  float my_p = 0.f;
  if (lane < n_sel)
    my_p = score == IQ_ROUTE_SOFTMAX ? expf(__fsub_rn(val, top_val)) : 1.0f / (1.0f + expf(-val));
  // the sum in descending-value order, and the rank of my id among the selected ids
  float sum = 0.f;
  int rank = 0;
  for (int t = 0; t < n_sel; ++t) {
    sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_p, t));
    rank += (__shfl_sync(0xffffffffu, my_id, t) < my_id) ? 1 : 0;
  }
  if (store && lane < n_sel) {
    sel[row * top_k + rank] = my_id;
    wt[row * top_k + rank] = my_p / sum;
  }
}

// The selection runs on one warp at the end of the router's critical path, so its length
// in instructions matters: up to 256 experts take the variant with 8 keys per lane.
__device__ void select_row(const float* logits, int e, int top_k, int score, int row, int* sel,
                           float* wt, bool logits_in_smem = false, bool store = true) {
  if (e <= 256)
    select_row_impl<8>(logits, e, top_k, score, row, sel, wt, logits_in_smem, store);
  else
    select_row_impl<16>(logits, e, top_k, score, row, sel, wt, logits_in_smem, store);   // e <= 512
}

// The router's work is cut into many small pieces: a tile is sixteen experts' rows over ONE
// K slice of `k_slices`, and every CTA takes one tile (the whole matrix is a few megabytes:
// what counts is how little each SM has to pull through, and that the CTAs are small
// enough to sit beside those of the kernels before and after).
// The hand-off inside the launch: a streaming CTA stores each partial logit as a 64-bit
// word (fp32 value, 32-bit tag of the launch) with one relaxed store into
// tagged[slice][row][expert]; the launch's LAST CTA streams nothing and polls those words
// (one warp per row), adds an expert's slices in slice order, writes the plain logits and
// selects.  No fence, ticket or counter on the producers' side.  The tag is the scratch's
// launch counter, which the selecting CTA advances when it is done.
template <class G>
__global__ void __launch_bounds__(G::BOUND_THREADS, G::CTAS_PER_SM) router_kernel(const __grid_constant__ RouterParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const StreamShape& sh = p.sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const int stream_ctas = static_cast<int>(gridDim.x) - 1;
  uint8_t* scratch = static_cast<uint8_t*>(p.scratch);
  uint32_t* launch_tag = reinterpret_cast<uint32_t*>(scratch + kScrLaunchTag);
  uint64_t* tagged = reinterpret_cast<uint64_t*>(scratch + kScrLogits);
  StreamScratch scr = scratch_of(p.scratch);
  IQ_TRACE_SCRATCH(scr, p);
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  if (cta == stream_ctas) {
    // ---- the selecting CTA.  With one row, two passes through one copy of its code: a
    // rehearsal ahead of the dependency wait (words taken as they are, nothing stored) that
    // brings the instructions in, then the launch's own selection (see tail_cta).
    float* lg = reinterpret_cast<float*>(smem);          // [m][e]
    if (tid >= 256) return;                              // (one warp per row, eight at most)
    const BlockBar bar{2, 256};
#pragma unroll 1
    for (int pass = p.m == 1 ? 0 : 1; pass < 2; ++pass) {
      const bool warm = pass == 0;
      if (!warm) {
        after_wait();
        if (tid == 0) { IQ_STAMP(p, 9); IQ_CLOCK(p, 7); }
      }
      const uint32_t tag = warm ? 0u : ld_volatile_u32(launch_tag) + 1u;
      // Polling: the rows' experts are cut into chunks of 32 (one expert per lane) and the
      // chunks dealt over the eight warps, so that a lane has only its expert's K slices in
      // flight and the whole table costs one round trip to L2 per pass when there are no
      // more chunks than warps (one row of 256 experts), not one per group of 32 experts.
      volatile int* failed = reinterpret_cast<volatile int*>(lg + p.m * p.e);
      if (tid == 0) *failed = 0;
      bar.sync();
      {
        const int chunks = (p.e + 31) / 32;
        const int items = p.m * chunks;
        const size_t slice_stride = static_cast<size_t>(kMaxRows) * p.e;
        for (int it = warp; it < items; it += 8) {
          const int row = it / chunks, id = (it - row * chunks) * 32 + lane;
          const uint64_t* src = tagged + static_cast<size_t>(row) * p.e + id;
          uint64_t t0 = 0;
          bool done = id >= p.e;
          float sum = 0.f;
          while (true) {
            if (!done) {
              uint32_t val[kMaxKSlices], seen[kMaxKSlices];
#pragma unroll
              for (int ks = 0; ks < kMaxKSlices; ++ks) {
                val[ks] = 0u;                                   // (+0 beyond k_slices)
                seen[ks] = tag;
                if (ks < p.k_slices) {
                  const uint64_t wv = ld_relaxed_gpu_u64(src + ks * slice_stride);
                  val[ks] = static_cast<uint32_t>(wv);
                  seen[ks] = static_cast<uint32_t>(wv >> 32);
                }
              }
              bool all = true;
              sum = 0.f;
#pragma unroll
              for (int ks = 0; ks < kMaxKSlices; ++ks) {
                all = all && seen[ks] == tag;
                sum += __uint_as_float(val[ks]);
              }
              done = warm || all;
            }
            if (__all_sync(0xffffffffu, done)) break;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kPipeBudgetNs) { *failed = 1; break; }
          }
          if (id < p.e) lg[row * p.e + id] = sum;
        }
      }
      bar.sync();
      if (tid == 0 && !warm) { IQ_STAMP(p, 10); IQ_CLOCK(p, 8); }
      if (warp < p.m) {
        if (*failed == 0) {
          if (tid == 0 && !warm) IQ_CLOCK(p, 9);
          select_row(lg, p.e, p.top_k, p.score, warp, p.sel, p.wt, true, !warm);
          if (tid == 0 && !warm) IQ_CLOCK(p, 10);
          // (the plain logits are for the caller: after the routes, which the next kernel
          // is waiting for)
          if (!warm)
            for (int id = lane; id < p.e; id += 32)
              p.logits[static_cast<size_t>(warp) * p.e + id] = lg[warp * p.e + id];
        } else if (lane == 0) {
          set_status(scr.status, IQ_ERR_PIPE_TIMEOUT);
        }
      }
      bar.sync();
      if (tid == 0 && !warm) *launch_tag = tag;
    }
    if (tid == 0) { IQ_STAMP(p, 11); IQ_CLOCK(p, 11); }
    return;
  }
  const Carve<G> cv = carve<G>(smem, sh);
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  stream_init<G>(sh, cv.sm);
  if (tid == G::PRODUCER_WARP * 32 && !stream_whole_rows<G>(sh))
    prefetch_tensormap(&p.map0);   // only a map the host filled (K-sliced stages)
  if (tid < p.k_slices) {
    GroupDesc& g = cv.sm->groups[tid];
    g.w = p.w;
    g.scale = nullptr;
    g.row_base = 0;
    g.map_id = 0;
    g.k_base = tid * sh.k_bytes;
    for (int c = 0; c < kMaxCols; ++c) {
      g.col_row[c] = c < p.m ? c : -1;
      g.col_mul[c] = 1.0f;
      g.col_out[c] = static_cast<int16_t>(c);
    }
  }
  __syncthreads();
  {
    const CtaWork wk = cta_share<G>(sh, stream_ctas, cta, grid);
    // (the host starts one CTA per tile: a CTA's stages all belong to one K slice, whose
    // part of the activation rows is all it stages)
    const int my_slice = wk.n_items > 0 ? wk.tile0 / wk.tpg : 0;
    if (warp == G::PRODUCER_WARP) {
      produce<G>(sh, cv.sm, cv.ring, wk, scr.status, &p.map0, &p.map1);
      if (tid == G::PRODUCER_WARP * 32) IQ_STAMP(p, 3);
      pdl_wait();
    } else if (warp < G::WARPS) {
      const int vec = sh.k_bytes / 16;   // 16-byte vectors of the slice per bf16 row
      const __nv_bfloat16* x0 = p.x + my_slice * (sh.k_bytes / 2);
      const ConsumeHead<G> head = consume_head<G>(sh, cv.sm->groups, cv.xq, cv.xs, wk);
      after_wait();
      if (tid == 0) IQ_STAMP(p, 1);
      if (wk.n_items > 0) {
        for (int i = tid; i < p.m * vec; i += G::CONSUMER_THREADS) {
          const int r = i / vec, v = i - r * vec;
          *reinterpret_cast<uint4*>(cv.xq + r * sh.x_pitch + v * 16) =
              __ldcg(reinterpret_cast<const uint4*>(x0 + static_cast<size_t>(r) * p.h + v * 8));
        }
      }
      named_bar_sync(1, G::CONSUMER_THREADS);
      if (tid == 0) IQ_STAMP(p, 2);
      consume<G, ElemBF16>(sh, cv.sm, cv.ring, cv.xq, cv.xs, cv.sc, wk, scr, &head);
      if (tid == 0) IQ_STAMP(p, 4);
    } else if (warp == G::EPILOGUE_WARP) {
      pdl_wait();
      const int m = p.m, e = p.e;
      const uint64_t tag = static_cast<uint64_t>(ld_volatile_u32(launch_tag) + 1u) << 32;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[G::RT]) {
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub)
          if (col < m)
            st_relaxed_gpu_u64(tagged + (static_cast<size_t>(id.group) * kMaxRows + col) * e +
                                   id.tig * G::ROWS + sub * 16 + r,
                               tag | __float_as_uint(val[sub]));
      };
      epilogue<G, false>(sh, cv.sm, wk, total, grid, cta, scr, emit);
      if (tid == G::EPILOGUE_WARP * 32) IQ_STAMP(p, 5);
    }
  }
  stream_drain_on_abort<G>(cv.sm);
}

// ------------------------------------------------------------------------------------
// iq_qkv_heads: the attention prologue after the QKV product.  One CTA per (head, row),
// one thread per channel pair's half: thread d owns channel d of the head.
struct HeadsParams {
  iq_heads_args a;
};

__global__ void __launch_bounds__(256) heads_kernel(const HeadsParams p) {
  __shared__ float red[8];
  __shared__ __nv_bfloat16 row[256];
  const iq_heads_args& a = p.a;
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  const int hd = a.head_dim, lane = d & 31, warp = d >> 5, nwarps = (blockDim.x + 31) >> 5;
  const bool is_q = head < a.q_heads, is_k = !is_q && head < a.q_heads + a.kv_heads;
  const int width = (a.q_heads + 2 * a.kv_heads) * hd;
  const bool live = d < hd;
  const float x = live ? a.qkv[static_cast<size_t>(r) * width + head * hd + d] : 0.f;
  long long slot = 0;
  if (!is_q) {
    slot = a.slot[r];
    if (slot < 0 || slot >= a.capacity) {
      if (d == 0) set_status(a.status, IQ_ERR_ROUTE);
      return;
    }
  }
  auto store_kv = [&](void* cache, int kv_head, int ch, __nv_bfloat16 v) {
    const size_t o = (static_cast<size_t>(slot) * a.kv_heads + kv_head) * hd + ch;
    if (a.kv_kind == IQ_ACT_E4M3)
      static_cast<uint8_t*>(cache)[o] = f32_to_e4m3_sat(__bfloat162float(v));
    else
      static_cast<__nv_bfloat16*>(cache)[o] = v;
  };
  if (!is_q && !is_k) {                        // a v head: round and store
    if (live) store_kv(a.v_cache, head - a.q_heads - a.kv_heads, d, __float2bfloat16_rn(x));
    return;
  }
  // RMSNorm over the head in fp32: warp sums in lane order, then the warps in order
  float ss = warp_sum(x * x);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  ss = 0.f;
  for (int w = 0; w < nwarps; ++w) ss += red[w];
  const float inv = rsqrtf(ss / static_cast<float>(hd) + a.eps);
  const float wn = live ? (is_q ? a.w_qn[d] : a.w_kn[d]) : 0.f;
  if (live) row[d] = __float2bfloat16_rn(wn * (x * inv));
  __syncthreads();
  if (!live) return;
  // Partial rotary embedding: channel i pairs with i + half inside the first rotary_dim
  // channels; each product and the sum are rounded to bf16.
  __nv_bfloat16 o = row[d];
  const int rot = a.rotary_dim, half = rot / 2;
  if (d < rot) {
    const __nv_bfloat16* cs = static_cast<const __nv_bfloat16*>(a.cos) + static_cast<size_t>(r) * rot;
    const __nv_bfloat16* sn = static_cast<const __nv_bfloat16*>(a.sin) + static_cast<size_t>(r) * rot;
    const float mine = __bfloat162float(row[d]);
    const float other = d < half ? -__bfloat162float(row[d + half]) : __bfloat162float(row[d - half]);
    const float t0 = bf16_round(mine * __bfloat162float(cs[d]));
    const float t1 = bf16_round(other * __bfloat162float(sn[d]));
    o = __float2bfloat16_rn(t0 + t1);
  }
  if (is_q)
    static_cast<__nv_bfloat16*>(a.q_out)[(static_cast<size_t>(r) * a.q_heads + head) * hd + d] = o;
  else
    store_kv(a.k_cache, head - a.q_heads, d, o);
}

// ------------------------------------------------------------------------------------
// Expert groups of one step: the distinct routed experts in order of first appearance,
// then the shared experts.  Every CTA derives the same table from `sel`.
struct MoeCommon {
  int m, h, i_loc, n_experts, top_k, n_shared;
  const int* sel;
  const float* wt;
  const uint8_t* w;          // expert bank
  const float* w_scale;
  const uint8_t* shared_w;
  const float* shared_scale;
  size_t w_stride, scale_stride;   // bytes / floats between experts
  int rows_per_expert;
};

// Returns the number of groups.  `use_wt`: column multipliers are the routing weights
// (Down) instead of 1 (Gate).  `x_is_pair`: the staged activation row of a column is its
// pair's row (Down) instead of the token's row (Gate).  Called by all threads of `bar`;
// the table is worked out by ONE warp (two pairs per lane, warp-level synchronisation
// only) while the others wait at the single barrier that ends the call: the routes arrive
// right after the dependency wait, so this sits on every CTA's critical path, and a chain
// of block-wide barriers costs far more than the few dozen serial steps it saves.
// With `down_groups` the same pass also fills the Down's table (routing weights as
// multipliers, pair rows as activations) next to the Gate's table in `groups`.
// `shared_first` puts the shared experts at the head of `groups` (not of `down_groups`)
// instead of its tail: their tiles then have indices that do not depend on the routes.
__device__ __noinline__ int build_groups(GroupDesc* groups, const MoeCommon& mc, bool use_wt,
                                         bool x_is_pair, int* status,
                                         int* s_ids /* 64 + kMaxGroups + 1 ints of shared memory */,
                                         const BlockBar bar = BlockBar{},
                                         const int* smem_sel = nullptr,
                                         const float* smem_wt = nullptr,
                                         GroupDesc* down_groups = nullptr,
                                         const MoeCommon* down_mc = nullptr,
                                         bool shared_first = false) {
  const int tid = threadIdx.x;
  const int pairs = mc.m * mc.top_k;            // <= 64
  const int slots = mc.top_k + mc.n_shared;
  const int routed_base = shared_first ? mc.n_shared : 0;
  if (tid < 32) {
    const int lane = tid;
    int e[2] = {-1, -1};
    float wt[2] = {1.0f, 1.0f};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int q = lane + 32 * hf;
      if (q < pairs) {
        // the routes come from global memory, or from the CTA's own copy in shared memory
        e[hf] = smem_sel ? smem_sel[q] : __ldcg(mc.sel + q);
        if (use_wt || down_groups) wt[hf] = smem_wt ? smem_wt[q] : __ldcg(mc.wt + q);
      }
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int q = lane + 32 * hf;
      if (q < pairs) {
        if (e[hf] < 0 || e[hf] >= mc.n_experts) {
          set_status(status, IQ_ERR_ROUTE);
          e[hf] = -1;
        }
        s_ids[q] = e[hf];
      }
    }
    __syncwarp();
    // first pair with my expert, and the group index = number of distinct experts that
    // appear before it
    int first[2] = {lane, lane + 32};
    int gi[2] = {0, 0};
    int n_routed = 0;
    if (pairs <= 32) {
      // one pair per lane: the warp's match / ballot do the search (no loops, no branches)
      const unsigned live = __ballot_sync(0xffffffffu, lane < pairs && e[0] >= 0);
      const unsigned same = __match_any_sync(0xffffffffu, e[0]) & live;
      first[0] = same ? __ffs(same) - 1 : lane;
      const unsigned firsts =
          __ballot_sync(0xffffffffu, lane < pairs && e[0] >= 0 && first[0] == lane);
      gi[0] = __popc(firsts & ((1u << first[0]) - 1u));
      n_routed = __popc(firsts);
    } else {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int q = lane + 32 * hf;
        if (q < pairs) {
          for (int r = 0; r < q; ++r)
            if (s_ids[r] == e[hf]) { first[hf] = r; break; }
          s_ids[64 + q] = (e[hf] >= 0 && first[hf] == q) ? 1 : 0;
        }
      }
      __syncwarp();
      for (int r = 0; r < pairs; ++r) {
        const int f = s_ids[64 + r];
        n_routed += f;
        gi[0] += r < first[0] ? f : 0;
        gi[1] += r < first[1] ? f : 0;
      }
    }
    const int n_groups = n_routed + mc.n_shared;
    if (lane == 0) s_ids[64 + kMaxGroups] = n_groups;
    auto open_group = [](GroupDesc& gd, const MoeCommon& c, int expert) {
      gd.w = c.w + static_cast<size_t>(expert) * c.w_stride;
      gd.scale = c.w_scale + static_cast<size_t>(expert) * c.scale_stride;
      gd.row_base = expert * c.rows_per_expert;
      gd.map_id = 0;
      gd.k_base = 0;
      // all columns unused: multipliers 0, rows -1, outputs 0 (8-byte stores)
      unsigned long long* mul = reinterpret_cast<unsigned long long*>(gd.col_mul);
      unsigned long long* row = reinterpret_cast<unsigned long long*>(gd.col_row);
      unsigned long long* out = reinterpret_cast<unsigned long long*>(gd.col_out);
#pragma unroll
      for (int i = 0; i < 4; ++i) mul[i] = 0ull;
      row[0] = row[1] = ~0ull;
      out[0] = out[1] = 0ull;
    };
    auto shared_group = [&](GroupDesc& gd, const MoeCommon& c, int sidx, bool pair_rows) {
      gd.w = c.shared_w + static_cast<size_t>(sidx) * c.w_stride;
      gd.scale = c.shared_scale + static_cast<size_t>(sidx) * c.scale_stride;
      gd.row_base = sidx * c.rows_per_expert;
      gd.map_id = 1;
      gd.k_base = 0;
      for (int col = 0; col < kMaxCols; ++col) {
        const bool live = col < c.m;
        const int pair_row = col * slots + c.top_k + sidx;
        gd.col_row[col] = static_cast<int16_t>(live ? (pair_rows ? pair_row : col) : -1);
        gd.col_mul[col] = live ? 1.0f : 0.f;
        gd.col_out[col] = static_cast<int16_t>(pair_rows ? col : pair_row);
      }
    };
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int q = lane + 32 * hf;
      if (q < pairs && e[hf] >= 0 && first[hf] == q) {
        open_group(groups[routed_base + gi[hf]], mc, e[hf]);
        if (down_groups) open_group(down_groups[gi[hf]], *down_mc, e[hf]);
      }
    }
    if (lane < mc.n_shared) {
      shared_group(groups[shared_first ? lane : n_groups - mc.n_shared + lane], mc, lane,
                   x_is_pair);
      if (down_groups)
        shared_group(down_groups[n_groups - mc.n_shared + lane], *down_mc, lane, true);
    }
    __syncwarp();
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int q = lane + 32 * hf;
      if (q < pairs && e[hf] >= 0) {
        const int row = q / mc.top_k, slot = q - row * mc.top_k;
        const int pair_row = row * slots + slot;
        GroupDesc& gd = groups[routed_base + gi[hf]];
        gd.col_row[row] = static_cast<int16_t>(x_is_pair ? pair_row : row);
        gd.col_mul[row] = use_wt ? wt[hf] : 1.0f;
        gd.col_out[row] = static_cast<int16_t>(x_is_pair ? row : pair_row);
        if (down_groups) {
          GroupDesc& dd = down_groups[gi[hf]];
          dd.col_row[row] = static_cast<int16_t>(pair_row);
          dd.col_mul[row] = wt[hf];
          dd.col_out[row] = static_cast<int16_t>(row);
        }
      }
    }
  }
  bar.sync();
  return s_ids[64 + kMaxGroups];
}

struct GateParams {
  IQ_TRACE_FIELD
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  MoeCommon mc;
  const uint8_t* x_fp8;
  const float* x_scale;
  const __nv_bfloat16* x_bf16;   // instead of x_fp8: quantised per 1x128 group while staging
  void* act;
  int act_kind;
  void* scratch;
  int pdl_level;
  int early_shared;   // see gate_kernel
};

template <class G>
__device__ __forceinline__ void gate_stage_x(const GateParams& p, const StreamShape& sh,
                                             const Carve<G>& cv, int tid) {
  if (p.x_bf16)
    stage_rows_bf16_groupq(cv.xq, cv.xs, sh, p.x_bf16, p.mc.h, p.mc.m, p.mc.h, false, tid,
                           G::CONSUMER_THREADS);
  else
    stage_rows_e4m3(cv.xq, cv.xs, sh, p.x_fp8, p.mc.h, p.x_scale, p.mc.m, p.mc.h, tid,
                    G::CONSUMER_THREADS);
}

// One stream of the Gate: the tiles of `wk`, every role with its ring / reduction position
// carried in `pos` / `rpos` (the kernel may run two streams back to back).
template <class G>
__device__ __forceinline__ void gate_stream(const GateParams& p, const StreamShape& sh,
                                            const Carve<G>& cv, const StreamScratch& scr,
                                            const CtaWork& wk, long long total, int grid, int cta,
                                            bool stage_x, RingPos& pos, RedPos& rpos) {
  const int tid = threadIdx.x, warp = tid >> 5;
  if (warp == G::PRODUCER_WARP) {
    // (both of the Gate's streams are consumed as they arrive: the first ahead of the
    // dependency wait by design, the second after every role has passed it)
    produce<G>(sh, cv.sm, cv.sm->groups, cv.ring, G::STAGE_BYTES, wk, scr.status, &p.map0, &p.map1,
               pos, false);
  } else if (warp < G::WARPS) {
    float held[kGatherHeld];
    gather_scales_load<G, ElemE4M3>(sh, cv.sm, wk, tid, held);
    if (stage_x) gate_stage_x<G>(p, sh, cv, tid);
    gather_scales_store<G, ElemE4M3>(sh, cv.sm, wk, cv.sc, tid, held);
    named_bar_sync(1, G::CONSUMER_THREADS);
    consume<G, ElemE4M3>(sh, cv.sm, cv.sm->groups, cv.ring, G::STAGE_BYTES, cv.xq, cv.xs, cv.sc, wk,
                         scr, pos, rpos);
  } else if (warp == G::EPILOGUE_WARP) {
    const int i_loc = p.mc.i_loc, m = p.mc.m;
    const int act_kind = p.act_kind;
    void* act = p.act;
    StreamSmem<G>* sm = cv.sm;
    auto emit = [&](const TileId& id, int r, int col, const float (&val)[G::RT]) {
      const GroupDesc& gd = sm->groups[id.group];
      if (col >= m || gd.col_row[col] < 0) return;
      // sub-tiles [0, RT/2) are gate rows, [RT/2, RT) the matching up rows
#pragma unroll
      for (int sub = 0; sub < G::RT / 2; ++sub) {
        const float gte = val[sub], up = val[sub + G::RT / 2];
        const float v = gte / (1.0f + expf(-gte)) * up;
        const size_t o = static_cast<size_t>(gd.col_out[col]) * i_loc +
                         id.tig * (G::ROWS / 2) + sub * 16 + r;
        if (act_kind == IQ_ACT_E4M3)
          static_cast<uint8_t*>(act)[o] = f32_to_e4m3_sat(v);
        else
          static_cast<__nv_bfloat16*>(act)[o] = __float2bfloat16_rn(v);
      }
    };
    epilogue<G, false>(sh, cv.sm, wk, total, grid, cta, scr, rpos, emit);
  }
}

template <class G>
__global__ void __launch_bounds__(G::BOUND_THREADS, G::CTAS_PER_SM) gate_kernel(const __grid_constant__ GateParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  StreamShape sh = p.sh;
  const Carve<G> cv = carve<G>(smem, sh);
  StreamScratch scr = scratch_of(p.scratch);
  IQ_TRACE_SCRATCH(scr, p);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int cta = blockIdx.x, n_cta = static_cast<int>(gridDim.x);
  uint32_t* gate_done = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(p.scratch) + kScrGateDone);
  uint32_t done0 = 0;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
    done0 = ld_volatile_u32(gate_done);
  }
  stream_init<G>(sh, cv.sm);
  if (tid == G::PRODUCER_WARP * 32 && !stream_whole_rows<G>(sh)) {
    prefetch_tensormap(&p.map0);   // only maps the host filled (K-sliced stages)
    if (p.mc.n_shared > 0) prefetch_tensormap(&p.map1);
  }
  RingPos pos;
  RedPos rpos;
  // Level 2: the activations were written two launches back (by the attention tail) and
  // can be staged while the router, the immediate predecessor, is still finishing.
  const bool early_x = p.pdl_level >= 2;
  if (early_x && warp < G::WARPS) gate_stage_x<G>(p, sh, cv, tid);
  // With `early_shared` (host: level 2, shared experts, whole tiles dealt round robin
  // whatever the routes) the shared experts are the first groups, CTA c's first tile is
  // tile c, and if that is a shared expert's tile the CTA streams and finishes it NOW:
  // nothing in it depends on the routes.  A whole tile needs no scratch, and the
  // activation buffer's last reader (the previous layer's Down) finished before the
  // router could start.
  // One row: its routed experts are top_k distinct ids unless the routes are malformed, so
  // everything about the step except WHICH experts is known before the routes are: the
  // number of groups, this CTA's share of the tiles, and the whole group table apart from
  // three fields per routed group.  All of that is worked out here, ahead of the wait
  // (the table from stand-in ids 0..top_k-1).  After the wait every warp reads the routes
  // itself, checks that they are as assumed and fills in those fields -- every warp
  // writes the same values and relies only on its own writes, so no block-wide barrier
  // stands between the routes and the first copy or the scale gather.  (Measured before:
  // 1.8 us for the table and 1 us for the share, in series, after the wait.)
  const bool one_row = p.mc.m == 1 && p.mc.top_k <= 32;
  StreamShape sh_one = sh;
  sh_one.n_groups = p.mc.top_k + p.mc.n_shared;
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  CtaWork wk = cta_work<G>(sh, 0, 0);
  if (one_row) {
    int* stand_in = cv.sm->route_ids + 64 + kMaxGroups + 1;
    if (tid < p.mc.top_k) stand_in[tid] = tid;
    __syncthreads();
    build_groups(cv.sm->groups, p.mc, false, false, nullptr, cv.sm->route_ids, BlockBar{},
                 stand_in, nullptr, nullptr, nullptr, p.early_shared != 0);
    wk = cta_share<G>(sh_one, n_cta, cta, grid);
  }
  int done_tiles = 0;
  if (p.early_shared) {
    const int tpg = stream_tiles_per_group<G>(sh);
    if (tid < p.mc.n_shared) {
      GroupDesc& gd = cv.sm->groups[tid];
      gd.w = p.mc.shared_w + static_cast<size_t>(tid) * p.mc.w_stride;
      gd.scale = p.mc.shared_scale + static_cast<size_t>(tid) * p.mc.scale_stride;
      gd.row_base = tid * p.mc.rows_per_expert;
      gd.map_id = 1;
      gd.k_base = 0;
      for (int c = 0; c < kMaxCols; ++c) {
        const bool live = c < p.mc.m;
        gd.col_row[c] = static_cast<int16_t>(live ? c : -1);
        gd.col_mul[c] = live ? 1.0f : 0.f;
        gd.col_out[c] = static_cast<int16_t>(c * (p.mc.top_k + p.mc.n_shared) + p.mc.top_k + tid);
      }
    }
    __syncthreads();
    if (cta < p.mc.n_shared * tpg) {
      StreamShape sa = sh;
      sa.n_groups = p.mc.n_shared;
      CtaWork wa = cta_work<G>(sa, static_cast<long long>(cta) * stream_stages_per_tile<G>(sa),
                               static_cast<long long>(cta + 1) * stream_stages_per_tile<G>(sa));
      gate_stream<G>(p, sa, cv, scr, wa, 0, n_cta, cta, false, pos, rpos);
      done_tiles = 1;
    }
    __syncthreads();
  }
  after_wait();                     // the routes come from the predecessor
  if (tid == 0) { IQ_STAMP(p, 1); IQ_CLOCK(p, 7); }
  bool as_assumed = false;
  if (one_row) {
    const int lane = tid & 31;
    const int e = lane < p.mc.top_k ? __ldcg(p.mc.sel + lane) : -1 - lane;
    const bool bad = lane < p.mc.top_k && (e < 0 || e >= p.mc.n_experts);
    const bool dup = __popc(__match_any_sync(0xffffffffu, e)) > 1;
    as_assumed = !__any_sync(0xffffffffu, bad || dup);
    if (as_assumed) {
      if (lane < p.mc.top_k) {
        GroupDesc& gd = cv.sm->groups[(p.early_shared ? p.mc.n_shared : 0) + lane];
        gd.w = p.mc.w + static_cast<size_t>(e) * p.mc.w_stride;
        gd.scale = p.mc.w_scale + static_cast<size_t>(e) * p.mc.scale_stride;
        gd.row_base = e * p.mc.rows_per_expert;
      }
      __syncwarp();
      sh.n_groups = sh_one.n_groups;
    } else {
      // Malformed routes (every warp sees that, from the same words): the general path.
      __syncthreads();
    }
  }
  if (!as_assumed) {
    sh.n_groups = build_groups(cv.sm->groups, p.mc, false, false, scr.status, cv.sm->route_ids,
                               BlockBar{}, nullptr, nullptr, nullptr, nullptr, p.early_shared != 0);
  }
  if (tid == 0) IQ_CLOCK(p, 8);
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  if (!as_assumed) wk = cta_share<G>(sh, n_cta, cta, grid);
  if (done_tiles) {                 // the first tile is finished already
    wk.tile0 += wk.tile_step;
    wk.n_items -= wk.spt;
  }
  if (tid == 0) { IQ_STAMP(p, 2); IQ_CLOCK(p, 9); }
  gate_stream<G>(p, sh, cv, scr, wk, total, grid, cta, !early_x, pos, rpos);
  if (tid == 0) IQ_STAMP(p, 4);
  if (tid == G::EPILOGUE_WARP * 32) IQ_STAMP(p, 5);
  // A CTA without work stays on its SM until a working CTA of the launch has finished.
  // The Down's CTAs are placed while this launch runs, next to its CTAs, as many per SM as
  // fit: an SM that an idle CTA left at once would take TWO of them, which then share one
  // SM's shared-memory bandwidth and finish last (measured: 11 us instead of 4.4 us for
  // the Down's consume phase on 4 of 148 SMs).  The counter only grows; its value cannot
  // change between this CTA's start and the launch's first finished CTA.
  if (wk.n_items <= 0 && done_tiles == 0) {
    if (tid == 0) {
      const uint64_t t0 = globaltimer_ns();
      while (ld_volatile_u32(gate_done) == done0 && globaltimer_ns() - t0 < 30000ull) nanosleep_ns(200);
    }
  } else if (tid == G::EPILOGUE_WARP * 32) {
    red_add_relaxed_u32(gate_done, 1u);
  }
  stream_drain_on_abort<G>(cv.sm);
}

struct DownParams {
  IQ_TRACE_FIELD
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  MoeCommon mc;
  const void* act;
  int act_kind;
  __nv_bfloat16* out;
  void* scratch;
  int tail_run;             // TailRun
  int n_tail;
  int push;
  int per_round;
  int pdl_level;
  iq_tail_args tail;
  PushView pv;
};

template <class G>
__global__ void __launch_bounds__(G::BOUND_THREADS, G::CTAS_PER_SM) down_kernel(const __grid_constant__ DownParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  StreamShape sh = p.sh;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int cta = blockIdx.x;
  const int stream_ctas = static_cast<int>(gridDim.x) - p.n_tail;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  if (cta >= stream_ctas) {
    PushView pv = p.pv;
#ifdef IQ_TRACE
    pv.trace = p.trace ? p.trace + blockIdx.x * kTraceWords : nullptr;
#endif
    tail_cta(p.tail, pv, p.per_round, cta - stream_ctas, p.n_tail, smem);
    if (tid == 0) { IQ_STAMP(p, 11); IQ_CLOCK(p, 10); }
    return;
  }
  const Carve<G> cv = carve<G>(smem, sh);
  StreamScratch scr = scratch_of(p.scratch);
  IQ_TRACE_SCRATCH(scr, p);
  stream_init<G>(sh, cv.sm);
  if (tid == G::PRODUCER_WARP * 32 && !stream_whole_rows<G>(sh)) {
    prefetch_tensormap(&p.map0);   // only maps the host filled (K-sliced stages)
    if (p.mc.n_shared > 0) prefetch_tensormap(&p.map1);
  }
  // Level 2: the routes were written two launches back (by the router), so the group
  // table, the weight stream and the scale gather all start while the Gate, the immediate
  // predecessor, is still finishing; only the Gate's activations are waited for.
  const bool early = p.pdl_level >= 2;
  if (!early) after_wait();
  sh.n_groups = build_groups(cv.sm->groups, p.mc, true, true, scr.status, cv.sm->route_ids);
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  {
    const CtaWork wk = cta_share<G>(sh, stream_ctas, cta, grid);
    if (warp == G::PRODUCER_WARP) {
      produce<G>(sh, cv.sm, cv.ring, wk, scr.status, &p.map0, &p.map1);
    } else if (warp < G::WARPS) {
      float held[kGatherHeld];
      gather_scales_load<G, ElemE4M3>(sh, cv.sm, wk, tid, held);
      const int rows = p.mc.m * (p.mc.top_k + p.mc.n_shared);
      // (the walk through the CTA's share: ahead of the wait)
      const ConsumeHead<G> head = consume_head<G>(sh, cv.sm->groups, cv.xq, cv.xs, wk);
      if (early) after_wait();
      if (tid == 0) { IQ_STAMP(p, 1); IQ_CLOCK(p, 7); }
      if (p.act_kind == IQ_ACT_E4M3)
        stage_rows_e4m3(cv.xq, cv.xs, sh, static_cast<const uint8_t*>(p.act), p.mc.i_loc, nullptr,
                        rows, p.mc.i_loc, tid, G::CONSUMER_THREADS);
      else
        stage_rows_bf16_groupq(cv.xq, cv.xs, sh, static_cast<const __nv_bfloat16*>(p.act),
                               p.mc.i_loc, rows, p.mc.i_loc, false, tid, G::CONSUMER_THREADS);
      if (tid == 0) IQ_CLOCK(p, 8);
      gather_scales_store<G, ElemE4M3>(sh, cv.sm, wk, cv.sc, tid, held);
      named_bar_sync(1, G::CONSUMER_THREADS);
      if (tid == 0) { IQ_STAMP(p, 2); IQ_CLOCK(p, 9); }
      consume<G, ElemE4M3>(sh, cv.sm, cv.ring, cv.xq, cv.xs, cv.sc, wk, scr, &head);
      if (tid == 0) IQ_STAMP(p, 4);
    } else if (warp == G::EPILOGUE_WARP) {
      if (early) pdl_wait();
      const int m = p.mc.m, h = p.mc.h;
      __nv_bfloat16* out = p.out;
      const bool push = p.push != 0;
      const uint32_t tag = push ? tag16_of(ld_volatile_u32(p.pv.epoch)) : 0u;
      const PushView& pv = p.pv;
      auto emit = [&](const TileId& id, int r0, int col, const float (&val)[4][G::RT]) {
        if (col >= m) return;
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub) {
          const int feat = id.tile * G::ROWS + sub * 16 + r0;
          const float v[4] = {val[0][sub], val[1][sub], val[2][sub], val[3][sub]};
          store_row4(out, static_cast<size_t>(col) * h + feat, v, push, pv, tag, col, feat);
        }
      };
      epilogue<G, true>(sh, cv.sm, wk, total, grid, cta, scr, emit);
      if (tid == G::EPILOGUE_WARP * 32) IQ_STAMP(p, 5);
    }
  }
  if (p.tail_run == kTailLastCta && last_cta<G>(cv.sm, scr, gridDim.x)) {
    float* red = reinterpret_cast<float*>(cv.sm->red);
    if (threadIdx.x < kTailThreads)
      run_tail<false>(p.tail, p.pv, 0u, cv.ring, nullptr, 0, red, &cv.sm->is_last_tile,
                      BlockBar{2, kTailThreads});   // (the ring is idle now)
  }
  stream_drain_on_abort<G>(cv.sm);
}

}  // namespace iqb

#include "direct.cuh"
#include "direct_gate.cuh"

namespace iqb {

// ------------------------------------------------------------------------------------
// Host side.  The library is entered through a C ABI, possibly from several host threads
// (one per stream): every piece of host state below is guarded by `g_host_mutex`.
static std::mutex g_host_mutex;

static int sm_count() {
  static int per_device[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (per_device[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    per_device[dev] = n;
  }
  return per_device[dev];
}

static int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

// One opt-in to the full shared memory per (kernel, device).
static bool ensure_smem_optin(const void* fn) {
  static std::unordered_set<uint64_t> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  const uint64_t key = (reinterpret_cast<uint64_t>(fn) << 6) ^ static_cast<uint64_t>(dev);
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (done.count(key)) return true;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) !=
      cudaSuccess)
    return false;
  // all of the SM's configurable memory as shared memory: two half-size CTAs must fit
  if (cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared) != cudaSuccess)
    return false;
  done.insert(key);
  return true;
}

// Tensor maps of weight matrices viewed as [total_rows, k_bytes / 4] u32, box = (kc / 4)
// x box_rows, no swizzle.  Encoding costs a driver call, so maps are cached in a hash map
// keyed by address and geometry; a map holds only the address and geometry, never data.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct MapKey {
  const void* ptr;
  long long rows;
  int k_bytes, box_rows, kc;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k_bytes == o.k_bytes && box_rows == o.box_rows &&
           kc == o.kc;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t x = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    x ^= static_cast<uint64_t>(k.rows) * 0xC2B2AE3D27D4EB4Full;
    x ^= (static_cast<uint64_t>(k.k_bytes) << 40) ^ (static_cast<uint64_t>(k.box_rows) << 20) ^
         static_cast<uint64_t>(k.kc);
    return static_cast<size_t>(x ^ (x >> 29));
  }
};
constexpr size_t kMaxCachedMaps = 1 << 16;   // a deep model has a few maps per layer

static int weight_map(CUtensorMap* out, const void* ptr, long long rows, int k_bytes, int box_rows,
                      int kc) {
  static EncodeTiledFn encode = nullptr;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  const MapKey key{ptr, rows, k_bytes, box_rows, kc};
  const auto hit = maps.find(key);
  if (hit != maps.end()) { *out = hit->second; return IQ_OK; }
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return IQ_ERR_CUDA;
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(k_bytes / 4), static_cast<cuuint64_t>(rows)};
  const cuuint64_t gstr[1] = {static_cast<cuuint64_t>(k_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kc / 4), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), gdim,
                            gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "iqb200: cuTensorMapEncodeTiled failed (%d)\n", static_cast<int>(r));
    return IQ_ERR_CUDA;
  }
  if (maps.size() >= kMaxCachedMaps) maps.clear();
  maps.emplace(key, m);
  *out = m;
  return IQ_OK;
}

// Fills map0 (and map1 for the shared experts) when the geometry streams K-slices.
template <class G>
static int fill_maps(CUtensorMap* map0, CUtensorMap* map1, const StreamShape& sh, const void* w,
                     long long rows, const void* shared_w, long long shared_rows) {
  if (stream_whole_rows<G>(sh)) return IQ_OK;      // whole-row stages: untiled copies
  const int box_rows = sh.pair_half > 0 ? G::ROWS / 2 : G::ROWS;
  const int row_bytes = sh.row_bytes ? sh.row_bytes : sh.k_bytes;
  int rc = weight_map(map0, w, rows, row_bytes, box_rows, G::BOXK);
  if (rc != IQ_OK) return rc;
  if (shared_w) rc = weight_map(map1, shared_w, shared_rows, row_bytes, box_rows, G::BOXK);
  return rc;
}

#ifdef IQ_TRACE
static unsigned long long* g_trace_base = nullptr;
static int g_trace_slots = 0, g_trace_next = 0;
template <class Params>
static auto trace_assign(Params& p, int) -> decltype(p.trace, void()) {
  std::lock_guard<std::mutex> lock(g_host_mutex);
  p.trace = nullptr;
  if (g_trace_base && g_trace_next < g_trace_slots)
    p.trace = g_trace_base + static_cast<size_t>(g_trace_next++) * kTraceCtas * kTraceWords;
}
template <class Params>
static void trace_assign(Params&, long) {}
#endif

template <class Kernel, class Params>
static int launch(Kernel kernel, const Params& p_in, int grid, int threads, size_t smem,
                  void* stream, int pdl) {
#ifdef IQ_TRACE
  Params p = p_in;
  trace_assign(p, 0);
#else
  const Params& p = p_in;
#endif
  // One opt-in to the full shared memory per kernel and device.
  if (!ensure_smem_optin(reinterpret_cast<const void*>(kernel))) return IQ_ERR_CUDA;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1] = {};
  int n_attr = 0;
  if (pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, p);
  if (err != cudaSuccess) {
    fprintf(stderr, "iqb200: launch failed: %s\n", cudaGetErrorString(err));
    return IQ_ERR_CUDA;
  }
  return IQ_OK;
}

// Most stages one of `grid` streaming CTAs can own, over every group count the routes can
// produce, under the same rule cta_share applies on the device; 0 when the stream has more
// tiles than the scratch has counters.
template <class G>
static int max_items_any(const StreamShape& sh, int max_groups, int grid) {
  int most = 0;
  for (int n = 1; n <= max_groups; ++n) {
    StreamShape s = sh;
    s.n_groups = n;
    const int n_tiles = stream_num_tiles<G>(s);
    const int spt = stream_stages_per_tile<G>(s);
    if (n_tiles > kMaxTiles) return 0;
    if (spt >= 32768) return 0;        // the gather's multiply-high division needs 16-bit operands
    int items;
    if (tile_aligned_split<G>(n_tiles, spt, grid, s.whole_tiles)) {
      const int g = n_tiles < grid ? n_tiles : grid;
      items = ((n_tiles + g - 1) / g) * spt;
    } else {
      const long long total = static_cast<long long>(n_tiles) * spt;
      items = static_cast<int>((total + grid - 1) / grid);
    }
    if (items >= 32768) return 0;
    if (items > most) most = items;
  }
  return most + 1;
}

// What a CTA of geometry G may take of the SM's shared memory.
template <class G>
constexpr size_t smem_limit() {
  return G::CTAS_PER_SM == 1 ? static_cast<size_t>(kSmemLimit)
                             : static_cast<size_t>(G::SPREAD ? kSmemSpread : kSmemLimitSmall);
}

// Fills the geometry-dependent part of a shape and returns the dynamic shared memory to
// request, or 0 when the ring does not fit.  `grid` is the number of CTAs that stream,
// `max_groups` bounds the group count a kernel may derive from the routes, `other_bytes`
// is what another role of the launch (a tail CTA) needs, `ring_bytes` the ring depth to
// aim for.
template <class G>
static size_t plan_smem(StreamShape& sh, int grid, size_t other_bytes, int max_groups = 1,
                        size_t ring_bytes = 160 * 1024) {
  if (grid < 1) return 0;
  sh.max_items = max_items_any<G>(sh, max_groups, grid);
  if (sh.max_items == 0) return 0;
  const size_t limit = smem_limit<G>();
  const size_t fixed = smem_fixed_bytes<G>(sh);
  if (fixed + 2 * G::STAGE_BYTES > limit || other_bytes > limit) return 0;
  // Ring depth: a bare copy loop saturates HBM with ~96 KB in flight per SM, but the
  // consumers hold a stage or two while they work on it; measured on the layer's kernels
  // with one CTA per SM, 160 KB is where more depth stops paying (96 KB: Gate 46 us,
  // 160 KB: 42 us).  A CTA that shares its SM takes what its half allows.
  int stages = static_cast<int>((limit - fixed) / G::STAGE_BYTES);
  const int want = static_cast<int>((ring_bytes + G::STAGE_BYTES - 1) / G::STAGE_BYTES);
  if (stages > want) stages = want;
  if (stages > kMaxStages) stages = kMaxStages;
  sh.n_stages = stages;
  size_t need = fixed + static_cast<size_t>(stages) * G::STAGE_BYTES;
  if (need < other_bytes) need = other_bytes;
  if (need > limit) return 0;
  return G::SPREAD ? limit : need;      // a spread CTA asks for exactly its class's size
}

// Tuning knobs read once from the environment: IQB200_SHORT_STREAM_MB (streams up to
// this many megabytes per launch run with two CTAs per SM; default 40, 0 = never) and
// IQB200_SHARED_GRID (CTAs such a launch starts per SM: 1 leaves the other half of every
// SM to the next kernel of the chain, 2 takes both halves; default 1; applies to the small
// kind of half-SM CTA only).
static long long env_number(const char* name, long long fallback) {
  const char* v = getenv(name);
  if (!v || !*v) return fallback;
  char* end = nullptr;
  const long long n = strtoll(v, &end, 10);
  return end && *end == 0 && n >= 0 ? n : fallback;
}
static long long short_stream_bytes() {
  static const long long v = env_number("IQB200_SHORT_STREAM_MB", 40) << 20;
  return v;
}
template <class G>
static int grid_for(bool both_halves = false) {
  static const int factor = env_number("IQB200_SHARED_GRID", 1) >= 2 ? 2 : 1;
  return sm_count() * (G::CTAS_PER_SM == 2 && !G::SPREAD ? (both_halves ? 2 : factor) : 1);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_push(const iq_push_args* u, int m, int h) {
  if (u->world < 1 || u->world > 8 || u->rank < 0 || u->rank >= u->world) return IQ_ERR_ARG;
  if (u->rows < m || u->rows > 64 || u->h != h) return IQ_ERR_ARG;
  if (!u->recv || !u->epoch || !u->ticket || !aligned16(u->recv)) return IQ_ERR_ARG;
  if (u->world > 1 && !u->recv_mc && !u->peer_recv) return IQ_ERR_ARG;
  if (u->recv_mc && !aligned16(u->recv_mc)) return IQ_ERR_ARG;
  return IQ_OK;
}

static int check_tail(const iq_tail_args* t) {
  if (!t) return IQ_OK;
  if (t->kind != IQ_TAIL_ATTN && t->kind != IQ_TAIL_MLP) return IQ_ERR_ARG;
  if (t->m < 1 || t->m > 8 || t->h < 128 || t->h % 128 || t->h > 8 * kTailVecs * kTailThreads)
    return IQ_ERR_ARG;
  if (!t->partial || !t->residual || !t->w_norm || !t->h_out || !t->norm_out) return IQ_ERR_ARG;
  if (t->kind == IQ_TAIL_ATTN && !t->w_first) return IQ_ERR_ARG;
  if (t->world < 1 || t->world > 8 || t->rank < 0 || t->rank >= t->world) return IQ_ERR_ARG;
  if (t->push) {
    const int rc = check_push(t->push, t->m, t->h);
    if (rc != IQ_OK) return rc;
    if (t->push->world != t->world || t->push->rank != t->rank) return IQ_ERR_ARG;
  } else if (t->world > 1) {
    if (!t->arrive || !t->epoch) return IQ_ERR_ARG;
    if (!t->arrive_mc && !t->peer_arrive) return IQ_ERR_ARG;
    if (!t->partial_mc && !t->peer_partials) return IQ_ERR_ARG;
  }
  if (!aligned16(t->partial) || !aligned16(t->residual) || !aligned16(t->h_out) ||
      !aligned16(t->norm_out) || !aligned16(t->w_norm))
    return IQ_ERR_ARG;
  return IQ_OK;
}

// The landing zone a launch uses: the caller's, or (no peers) the one inside the scratch.
static int make_push_view(PushView& pv, const iq_push_args* u, void* scratch, size_t scratch_bytes,
                          int h) {
  if (u) {
    pv.recv = u->recv;
    pv.recv_mc = u->recv_mc;
    pv.peer_recv = u->peer_recv;
    pv.epoch = u->epoch;
    pv.ticket = u->ticket;
    pv.world = u->world;
    pv.rank = u->rank;
    pv.rows = u->rows;
    pv.h = u->h;
    return IQ_OK;
  }
  if (!scratch || scratch_bytes < kScrBytes || h > kZoneMaxH) return IQ_ERR_ARG;
  uint8_t* b = static_cast<uint8_t*>(scratch);
  pv.recv = reinterpret_cast<uint32_t*>(b + kScrZone);
  pv.recv_mc = nullptr;
  pv.peer_recv = nullptr;
  pv.epoch = reinterpret_cast<uint32_t*>(b + kScrLaunchTag);
  pv.ticket = reinterpret_cast<uint32_t*>(b + kScrTailTicket);
  pv.world = 1;
  pv.rank = 0;
  pv.rows = kMaxRows;
  pv.h = h;
  return IQ_OK;
}

// How a fused tail runs, and through which zone: push when the tail names a zone or has
// no peers, pull (last CTA) otherwise.
struct TailPlan {
  int tail_run = kTailNone, n_tail = 0, push = 0, per_round = 0;
  size_t smem = 0;      // what a tail CTA needs
  PushView pv{};
};
static int plan_tail(TailPlan& tp, const iq_tail_args* tail, const iq_push_args* push_only,
                     void* scratch, size_t scratch_bytes, int m, int h, size_t smem_limit) {
  if (tail && (tail->push || tail->world == 1)) {
    const int rc = make_push_view(tp.pv, tail->push, scratch, scratch_bytes, h);
    if (rc != IQ_OK) return rc;
    tp.tail_run = kTailCtas;
    tp.n_tail = m;
    tp.push = 1;
    tp.per_round = tail_sources_per_round(tp.pv.world, h, tail->residual_fp32, smem_limit);
    if (tp.per_round < 1) return IQ_ERR_UNSUPPORTED;
    tp.smem = tail_cta_smem(tp.per_round, h, tail->residual_fp32);
  } else if (tail) {
    tp.tail_run = kTailLastCta;
  } else if (push_only) {
    int rc = check_push(push_only, m, h);
    if (rc == IQ_OK) rc = make_push_view(tp.pv, push_only, scratch, scratch_bytes, h);
    if (rc != IQ_OK) return rc;
    tp.push = 1;
  }
  return IQ_OK;
}

template <class G>
static int linear_launch(const iq_linear_args* a, void* stream) {
  LinearParams p{};
  StreamShape& sh = p.sh;
  const bool split2 = a->x_kind == IQ_X_BF16_SPLIT2;
  sh.mode = kRowsPerGroup;
  sh.n_groups = 1;
  sh.rows_per_group = a->n;
  sh.k_bytes = a->k;
  sh.rg_shift = ilog2(a->rg);
  sh.kg_shift = ilog2(a->kg);
  sh.pair_half = 0;
  sh.x_rows = split2 ? 2 * a->m : a->m;
  sh.x_pitch = a->k + 64;
  sh.x_blocks = (a->k + 127) / 128;
  TailPlan tp;
  int rc = plan_tail(tp, a->tail, a->push, a->scratch, a->scratch_bytes, a->m, a->n,
                     smem_limit<G>());
  if (rc != IQ_OK) return rc;
  const int grid = grid_for<G>();
  const size_t smem = plan_smem<G>(sh, grid - tp.n_tail, tp.smem);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  rc = fill_maps<G>(&p.map0, &p.map1, sh, a->w, a->n, nullptr, 0);
  if (rc != IQ_OK) return rc;
  p.x = a->x;
  p.x_scale = a->x_scale;
  p.x_kind = a->x_kind;
  p.m = a->m;
  p.k = a->k;
  p.n = a->n;
  p.w = static_cast<const uint8_t*>(a->w);
  p.w_scale = a->w_scale;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.out_f32 = a->out_f32;
  p.scratch = a->scratch;
  p.tail_run = tp.tail_run;
  p.n_tail = tp.n_tail;
  p.push = tp.push;
  p.per_round = tp.per_round;
  p.pv = tp.pv;
  if (a->tail) {
    p.tail = *a->tail;
    if (!p.tail.status) p.tail.status = scratch_of(a->scratch).status;
  }
  return launch(linear_kernel<G>, p, grid, G::THREADS, smem, stream, a->pdl);
}

// The tail of rows pushed by an earlier launch: one polling CTA per row, taking as many
// sources per round as `smem_limit` bytes of shared memory hold.
static int launch_pushed_tail(const iq_tail_args* a, void* stream, int pdl, size_t smem_limit) {
  TailParams p{};
  p.a = *a;
  if (make_push_view(p.pv, a->push, nullptr, 0, a->h) != IQ_OK) return IQ_ERR_ARG;
  p.push = 1;
  p.n_tail = a->m;
  p.per_round = tail_sources_per_round(p.pv.world, a->h, a->residual_fp32, smem_limit);
  if (p.per_round < 1) return IQ_ERR_UNSUPPORTED;
  return launch(tail_kernel, p, a->m, kTailThreads,
                tail_cta_smem(p.per_round, a->h, a->residual_fp32), stream, pdl);
}

// A tail CTA's shared memory is every CTA's of its launch.  Without peers (or with one) the
// sources of a row fit in 72 KB and several tile CTAs share an SM; with more peers the tail
// takes what a small half-SM CTA may (three sources per round at hidden 6144).
static size_t direct_tail_limit(const iq_tail_args* tail) {
  return tail && tail->world > 2 ? static_cast<size_t>(kSmemLimitSmall) : 72 * 1024;
}

// The direct form (direct.cuh): 32 weight rows per CTA, no ring.
static int linear_direct_launch(const iq_linear_args* a, void* stream) {
  LinearDirectParams p{};
  const bool split2 = a->x_kind == IQ_X_BF16_SPLIT2;
  TailPlan tp;
  // With more than one peer a tail CTA needs about 100 KB for its sources, and a launch's
  // CTAs all get the same shared memory, so only two tile CTAs fit on an SM.  The other
  // form (IQB200_DIRECT_SPLIT_TAIL=1) only pushes the rows here and lets the tail follow
  // as a launch of its own with half an SM's shared memory.  Measured per layer: 62.9 (own
  // launch) against 63.4 us on four GPUs, 64.3 against 57.2 us on eight, so the tail stays
  // in this launch unless the knob says otherwise.
  // The pull protocol's tail (signal, wait, switch read) always follows as its own launch.
  static const bool split_push = env_number("IQB200_DIRECT_SPLIT_TAIL", 0) != 0;
  const bool pull_tail = a->tail && !a->tail->push && a->tail->world > 1;
  const bool split_tail =
      pull_tail || (split_push && a->tail && a->tail->push && a->tail->world > 2);
  int rc = plan_tail(tp, split_tail ? nullptr : a->tail,
                     pull_tail ? nullptr : (split_tail ? a->tail->push : a->push), a->scratch,
                     a->scratch_bytes, a->m, a->n, direct_tail_limit(a->tail));
  if (rc != IQ_OK) return rc;
  size_t smem = linear_direct_smem(split2 ? 2 * a->m : a->m, a->k);
  if (smem > 96 * 1024) return IQ_ERR_UNSUPPORTED;
  if (tp.smem > smem) smem = tp.smem;
  p.x = a->x;
  p.x_scale = a->x_scale;
  p.x_kind = a->x_kind;
  p.m = a->m;
  p.k = a->k;
  p.n = a->n;
  p.rg_shift = ilog2(a->rg);
  p.kg_shift = ilog2(a->kg);
  p.w = static_cast<const uint8_t*>(a->w);
  p.w_scale = a->w_scale;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.out_f32 = a->out_f32;
  p.scratch = a->scratch;
  p.n_tail = tp.n_tail;
  p.push = tp.push;
  p.per_round = tp.per_round;
  p.pv = tp.pv;
  if (a->tail && !split_tail) {
    p.tail = *a->tail;
    if (!p.tail.status) p.tail.status = scratch_of(a->scratch).status;
  }
  // (32 rows per CTA measured faster than 48 for the o_proj: 9.3 against 10.1 us)
  static const bool rows48 = env_number("IQB200_LINEAR_DIRECT_ROWS48", 0) != 0;
  if (rows48 && a->n % 48 == 0)
    rc = launch(linear_direct_kernel<3>, p, a->n / 48 + tp.n_tail, 288, smem, stream, a->pdl);
  else
    rc = launch(linear_direct_kernel<2>, p, a->n / 32 + tp.n_tail, 256, smem, stream, a->pdl);
  if (rc != IQ_OK || !split_tail) return rc;
  iq_tail_args t = *a->tail;
  if (!t.status) t.status = scratch_of(a->scratch).status;
  if (pull_tail) return iq_tail(&t, stream, a->pdl);
  return launch_pushed_tail(&t, stream, a->pdl, kSmemSpread);
}

}  // namespace iqb

using namespace iqb;

extern "C" size_t iq_scratch_bytes(void) { return kScrBytes; }

extern "C" int iq_sm_count(void) { return sm_count(); }

extern "C" int iq_status_read(void* scratch, int* code, int clear, void* stream) {
  if (!scratch || !code) return IQ_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(code, scratch, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return IQ_ERR_CUDA;
  if (clear && cudaMemsetAsync(scratch, 0, sizeof(int), s) != cudaSuccess) return IQ_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return IQ_ERR_CUDA;
  return IQ_OK;
}

extern "C" int iq_tail(const iq_tail_args* a, void* stream, int pdl) {
  if (!a) return IQ_ERR_ARG;
  const int rc = check_tail(a);
  if (rc != IQ_OK) return rc;
  if (sm_count() == 0) return IQ_ERR_CUDA;
  TailParams p{};
  p.a = *a;
  if (a->push) {
    // a small CTA that can sit beside a streaming kernel's: half an SM's shared memory
    return launch_pushed_tail(a, stream, pdl, kSmemLimitSmall);
  }
  // rows in `partial`: one CTA per row without peers, one CTA (one signal / wait) with
  return launch(tail_kernel, p, a->world == 1 ? a->m : 1, kTailThreads,
                tail_cta_smem(0, a->h, a->residual_fp32), stream, pdl);
}

extern "C" int iq_linear(const iq_linear_args* a, void* stream) {
  if (!a || !a->x || !a->w || !a->w_scale || !a->scratch) return IQ_ERR_ARG;
  if (!a->out && (!a->out_f32 || a->tail || a->push)) return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBasicBytes) return IQ_ERR_ARG;
  if (a->x_kind < IQ_X_BF16_GROUPQ || a->x_kind > IQ_X_E4M3_UNSCALED) return IQ_ERR_ARG;
  if (a->x_kind == IQ_X_E4M3_GROUP && !a->x_scale) return IQ_ERR_ARG;
  const int max_m = a->x_kind == IQ_X_BF16_SPLIT2 ? 4 : 8;
  if (a->m < 1 || a->m > max_m) return IQ_ERR_ARG;
  if (a->k < 64 || a->k % 64 || a->n < 16 || a->n % 16) return IQ_ERR_ARG;
  if (a->x_kind != IQ_X_E4M3_UNSCALED && a->k % 128) return IQ_ERR_ARG;   // 1x128 groups
  if ((a->rg != 64 && a->rg != 128) || (a->kg != 64 && a->kg != 128)) return IQ_ERR_ARG;
  if (!aligned16(a->x) || !aligned16(a->w) || !aligned16(a->out) || !aligned16(a->out_f32))
    return IQ_ERR_ARG;
  if (a->tail) {
    const int rc = check_tail(a->tail);
    if (rc != IQ_OK) return rc;
    if (a->tail->partial != a->out || a->tail->m != a->m || a->tail->h != a->n) return IQ_ERR_ARG;
  }
  if (sm_count() == 0) return IQ_ERR_CUDA;
  const int k = a->k, n = a->n;
  // A short stream takes CTAs of eight (six) consumer warps on half an SM each, one per SM
  // (the spread kind), so that a neighbour in the launch chain can set up and prefetch
  // beside it (see Geo); a long stream takes the whole SM.
  if (static_cast<long long>(n) * k <= short_stream_bytes()) {
    // (falls through to a whole-SM geometry when half an SM cannot hold the rows and a ring)
    int rc = IQ_ERR_UNSUPPORTED;
    // The direct form (direct.cuh) for streams of up to IQB200_LINEAR_DIRECT_MB megabytes
    // (default 16; 0 turns it off) of many short rows -- the row-parallel o_proj of a shard:
    // K a multiple of 256 and at most 2048, at least 2048 rows (32 per CTA).  (The
    // column-parallel QKV of a shard, 1280 rows of 6144, would be 40 CTAs with long rows:
    // measured 14.8 against the engine's 9.5 us.)
    static const long long direct_bytes = env_number("IQB200_LINEAR_DIRECT_MB", 16) << 20;
    if (static_cast<long long>(n) * k <= direct_bytes && k % 256 == 0 && k <= 2048 && n >= 2048 &&
        n % kDirectRows == 0 && a->kg >= 64)
      rc = linear_direct_launch(a, stream);
    if (rc != IQ_ERR_UNSUPPORTED) return rc;
    // One 48-row tile per CTA (its k-stages worked on in batches) where that leaves no CTA
    // with more rows than 16-row tiles would: a CTA pays the hand-over of a finished tile
    // to its epilogue warp once instead of three times (IQB200_LINEAR_TILE48=0 turns it off).
    static const bool tile48 = env_number("IQB200_LINEAR_TILE48", 1) != 0;
    if (tile48 && k % 256 == 0 && n % 48 == 0) {
      const int ctas = std::max(1, sm_count() - (a->tail || a->push ? a->m : 0));
      const int most16 = (n / 16 + ctas - 1) / ctas * 16;
      const int most48 = (n / 48 + ctas - 1) / ctas * 48;
      static const bool runs4 = env_number("IQB200_LINEAR_RUNS4", 0) != 0;
      if (most48 <= most16 && runs4 && k % 512 == 0) rc = linear_launch<Geo<3, 2, 4, 3>>(a, stream);
      if (most48 <= most16 && rc == IQ_ERR_UNSUPPORTED) rc = linear_launch<Geo<3, 2, 2, 3>>(a, stream);
    }
    if (rc != IQ_ERR_UNSUPPORTED) return rc;
    if (k % 1024 == 0 && n % 16 == 0) rc = linear_launch<Geo<1, 8, 2, 3>>(a, stream);
    else if (k % 768 == 0 && n % 32 == 0) rc = linear_launch<Geo<2, 4, 3, 3>>(a, stream);
    else if (k % 512 == 0 && n % 32 == 0) rc = linear_launch<Geo<2, 4, 2, 3>>(a, stream);
    else if (k % 256 == 0 && n % 64 == 0) rc = linear_launch<Geo<4, 2, 2, 3>>(a, stream);
    else if (k % 192 == 0 && n % 32 == 0) rc = linear_launch<Geo<2, 3, 1, 3>>(a, stream);
    if (rc != IQ_ERR_UNSUPPORTED) return rc;
  }
  // k a multiple of 2048: 16 rows x 2 KB stages on sixteen consumer warps.  The other form
  // (IQB200_K2048_ROWS32=1: 32 rows x 1 KB on eight warps, as for k = 1024) measured 18.3
  // against 15.0 us for a 50 MB o_proj and 31.1 against 29.6 us for a 113 MB expert Down.
  static const bool rows32 = env_number("IQB200_K2048_ROWS32", 0) != 0;
  if (k % 2048 == 0 && n % 16 == 0 && !(rows32 && n % 32 == 0))
    return linear_launch<Geo<1, 16, 2>>(a, stream);
  // k = 1024: 32-row stages (half as many tile hand-offs) measured 0.25 us faster
  if (k % 1024 == 0 && n % 32 == 0) return linear_launch<Geo<2, 8, 2>>(a, stream);
  if (k % 1024 == 0 && n % 16 == 0) return linear_launch<Geo<1, 16, 1>>(a, stream);
  if (k % 768 == 0 && n % 64 == 0) return linear_launch<Geo<4, 4, 3>>(a, stream);
  if (k % 512 == 0 && n % 32 == 0) return linear_launch<Geo<2, 8, 1>>(a, stream);
  if (k % 256 == 0 && n % 64 == 0) return linear_launch<Geo<4, 4, 1>>(a, stream);
  if (k % 192 == 0 && n % 256 == 0) return linear_launch<Geo<16, 1, 3>>(a, stream);
  if (k % 128 == 0 && n % 128 == 0) return linear_launch<Geo<8, 2, 1>>(a, stream);
  if (k % 64 == 0 && n % 256 == 0) return linear_launch<Geo<16, 1, 1>>(a, stream);
  return IQ_ERR_UNSUPPORTED;
}

extern "C" int iq_qkv_heads(const iq_heads_args* a, void* stream) {
  if (!a || !a->qkv || !a->w_qn || !a->w_kn || !a->cos || !a->sin || !a->slot || !a->q_out ||
      !a->k_cache || !a->v_cache)
    return IQ_ERR_ARG;
  if (a->m < 1 || a->m > 64 || a->q_heads < 1 || a->kv_heads < 1 || a->capacity < 1)
    return IQ_ERR_ARG;
  if (a->head_dim < 2 || a->head_dim > 256 || a->head_dim % 2) return IQ_ERR_ARG;
  if (a->rotary_dim < 0 || a->rotary_dim > a->head_dim || a->rotary_dim % 2) return IQ_ERR_ARG;
  if (a->kv_kind != IQ_ACT_BF16 && a->kv_kind != IQ_ACT_E4M3) return IQ_ERR_ARG;
  HeadsParams p{};
  p.a = *a;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(a->q_heads + 2 * a->kv_heads),
                     static_cast<unsigned>(a->m), 1);
  cfg.blockDim = dim3(static_cast<unsigned>((a->head_dim + 31) / 32 * 32), 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1] = {};
  if (a->pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  const cudaError_t err = cudaLaunchKernelEx(&cfg, heads_kernel, p);
  if (err != cudaSuccess) {
    fprintf(stderr, "iqb200: launch failed: %s\n", cudaGetErrorString(err));
    return IQ_ERR_CUDA;
  }
  return IQ_OK;
}

template <class G>
static int router_launch(const iq_router_args* a, void* stream) {
  RouterParams p{};
  StreamShape& sh = p.sh;
  // One CTA per tile, K cut into as many slices as gives every SM at most one CTA (and a
  // slice a whole number of stages).
  const int row_tiles = (a->e + G::ROWS - 1) / G::ROWS;
  const int row_stages = a->h * 2 / G::KC;
  static const int max_slices = static_cast<int>(env_number("IQB200_ROUTER_SLICES", kMaxKSlices));
  int k_slices = 1;
  for (int ks = 2; ks <= kMaxKSlices && ks <= max_slices; ++ks)
    if (row_stages % ks == 0 && row_tiles * ks + 1 <= sm_count()) k_slices = ks;
  if (row_tiles + 1 > sm_count()) return IQ_ERR_UNSUPPORTED;
  sh.whole_tiles = 2;
  sh.mode = kRowsPerGroup;
  sh.n_groups = k_slices;
  sh.rows_per_group = a->e;
  sh.k_bytes = a->h * 2 / k_slices;
  sh.row_bytes = a->h * 2;
  sh.rg_shift = 7;
  sh.kg_shift = 7;
  sh.pair_half = 0;
  sh.x_rows = a->m;
  sh.x_pitch = sh.k_bytes + 64;
  sh.x_blocks = 1;
  const int grid = row_tiles * k_slices + 1;
  // the launch's last CTA selects; it keeps the rows' logits in shared memory
  // (the ring holds a CTA's whole tile: it is in shared memory before the dependency wait
  // returns)
  const size_t tile_bytes = static_cast<size_t>(G::ROWS) * sh.k_bytes;
  const size_t smem =
      plan_smem<G>(sh, grid - 1, sizeof(float) * a->m * a->e + 16, k_slices, tile_bytes);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  p.k_slices = k_slices;
  const int mrc = fill_maps<G>(&p.map0, &p.map1, sh, a->w, a->e, nullptr, 0);
  if (mrc != IQ_OK) return mrc;
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.w = static_cast<const uint8_t*>(a->w);
  p.m = a->m;
  p.h = a->h;
  p.e = a->e;
  p.top_k = a->top_k;
  p.score = a->score;
  p.sel = a->sel;
  p.wt = a->wt;
  p.logits = a->logits;
  p.scratch = a->scratch;
  return launch(router_kernel<G>, p, grid, G::THREADS, smem, stream, a->pdl);
}

extern "C" int iq_router(const iq_router_args* a, void* stream) {
  if (!a || !a->x || !a->w || !a->sel || !a->wt || !a->logits || !a->scratch) return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBytes) return IQ_ERR_ARG;
  if (a->m < 1 || a->m > 8 || a->h < 512 || a->h % 512) return IQ_ERR_ARG;
  if (a->e < 16 || a->e % 16 || a->e > kMaxExperts || a->top_k < 1 || a->top_k > 32 ||
      a->top_k > a->e)
    return IQ_ERR_ARG;
  if (a->score != IQ_ROUTE_SOFTMAX && a->score != IQ_ROUTE_SIGMOID) return IQ_ERR_ARG;
  if (!aligned16(a->x) || !aligned16(a->w)) return IQ_ERR_ARG;
  if (sm_count() < 2) return IQ_ERR_CUDA;
  // (h % 512 == 0: a row is a whole number of 1 KiB stages)
  return router_launch<Geo<1, 8, 2, 2>>(a, stream);
}

static int fill_moe(MoeCommon& mc, int m, int h, int i_loc, int n_experts, int top_k, int n_shared,
                    const int* sel, const float* wt) {
  if (m < 1 || m > 8 || top_k < 1 || m * top_k > 64 || n_shared < 0 || n_shared > 4)
    return IQ_ERR_ARG;
  if (m * top_k + n_shared > kMaxGroups) return IQ_ERR_ARG;
  if (n_experts < 1 || !sel) return IQ_ERR_ARG;
  mc.m = m;
  mc.h = h;
  mc.i_loc = i_loc;
  mc.n_experts = n_experts;
  mc.top_k = top_k;
  mc.n_shared = n_shared;
  mc.sel = sel;
  mc.wt = wt;
  return IQ_OK;
}

template <class G>
static int gate_launch(const iq_moe_gate_args* a, void* stream) {
  GateParams p{};
  int rc = fill_moe(p.mc, a->m, a->h, a->i_loc, a->n_experts, a->top_k, a->n_shared, a->sel,
                    nullptr);
  if (rc != IQ_OK) return rc;
  p.mc.w = static_cast<const uint8_t*>(a->fc);
  p.mc.w_scale = a->fc_scale;
  p.mc.shared_w = static_cast<const uint8_t*>(a->shared_fc);
  p.mc.shared_scale = a->shared_fc_scale;
  p.mc.w_stride = static_cast<size_t>(2) * a->i_loc * a->h;
  p.mc.scale_stride = static_cast<size_t>(2 * a->i_loc / 64) * (a->h / 128);
  p.mc.rows_per_expert = 2 * a->i_loc;
  StreamShape& sh = p.sh;
  sh.mode = kRowsPerGroup;
  sh.n_groups = 1;                 // set in the kernel from the routes
  sh.rows_per_group = 2 * a->i_loc;
  sh.k_bytes = a->h;
  sh.rg_shift = 6;
  sh.kg_shift = 7;
  sh.pair_half = a->i_loc;
  sh.x_rows = a->m;
  sh.x_pitch = a->h + 64;
  sh.x_blocks = a->h / 128;
  // Early start on the shared experts (pdl level 2 only): needs whole tiles for every group
  // count valid routes can produce, so that a CTA's first tile is known before the routes.
  const int grid = grid_for<G>();
  bool early = a->pdl >= 2 && a->n_shared > 0;
  if (early) {
    // Only where a CTA has several tiles: with one tile per CTA the early CTAs gain nothing
    // for the launch (they have no second tile to move on to), but they reach their
    // dependency wait -- and release the NEXT kernel's CTAs -- microseconds late (measured:
    // 8 us at one tile of 196 KB per CTA).
    StreamShape t = sh;
    t.n_groups = a->n_shared + a->top_k;
    if (stream_num_tiles<G>(t) <= grid) early = false;
  }
  if (early) {
    for (int n = a->n_shared + a->top_k; n <= a->n_shared + a->m * a->top_k && early; ++n) {
      StreamShape t = sh;
      t.n_groups = n;
      early = tile_aligned_split<G>(stream_num_tiles<G>(t), stream_stages_per_tile<G>(t), grid, 0);
    }
  }
  if (early) {
    sh.whole_tiles = 2;
    sh.round_robin = 1;
  }
  p.early_shared = early ? 1 : 0;
  const size_t smem = plan_smem<G>(sh, grid, 0, a->m * a->top_k + a->n_shared);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  const int mrc = fill_maps<G>(&p.map0, &p.map1, sh, a->fc,
                               static_cast<long long>(a->n_experts) * 2 * a->i_loc, a->shared_fc,
                               static_cast<long long>(a->n_shared) * 2 * a->i_loc);
  if (mrc != IQ_OK) return mrc;
  p.x_fp8 = static_cast<const uint8_t*>(a->x_fp8);
  p.x_scale = a->x_scale;
  p.x_bf16 = static_cast<const __nv_bfloat16*>(a->x_bf16);
  p.act = a->act;
  p.act_kind = a->act_kind;
  p.scratch = a->scratch;
  p.pdl_level = a->pdl;
  return launch(gate_kernel<G>, p, grid, G::THREADS, smem, stream, a->pdl);
}

// Bytes the expert kernels stream for `m` rows: every routed pair a distinct expert (the
// most there can be), plus the shared experts.
static long long expert_stream_bytes(int m, int top_k, int n_experts, int n_shared,
                                     long long bytes_per_expert) {
  const int routed = m * top_k < n_experts ? m * top_k : n_experts;
  return (routed + n_shared) * bytes_per_expert;
}

// The direct form for one row (direct_gate.cuh): sixteen features of one group per CTA.
static int gate_direct_launch(const iq_moe_gate_args* a, void* stream, bool eight) {
  GateDirectParams p{};
  int rc = fill_moe(p.mc, a->m, a->h, a->i_loc, a->n_experts, a->top_k, a->n_shared, a->sel, nullptr);
  if (rc != IQ_OK) return rc;
  p.mc.w = static_cast<const uint8_t*>(a->fc);
  p.mc.w_scale = a->fc_scale;
  p.mc.shared_w = static_cast<const uint8_t*>(a->shared_fc);
  p.mc.shared_scale = a->shared_fc_scale;
  p.mc.w_stride = static_cast<size_t>(2) * a->i_loc * a->h;
  p.mc.scale_stride = static_cast<size_t>(2 * a->i_loc / 64) * (a->h / 128);
  p.mc.rows_per_expert = 2 * a->i_loc;
  p.x_fp8 = static_cast<const uint8_t*>(a->x_fp8);
  p.x_scale = a->x_scale;
  p.x_bf16 = static_cast<const __nv_bfloat16*>(a->x_bf16);
  p.act = a->act;
  p.act_kind = a->act_kind;
  p.scratch = a->scratch;
  p.pdl_level = a->pdl;
  if (eight) {
    const int grid = (a->top_k + a->n_shared) * (a->i_loc / 8);
    return launch(gate_direct8_kernel, p, grid, 256, gate_direct_smem(a->h), stream, a->pdl);
  }
  const int grid = (a->top_k + a->n_shared) * (a->i_loc / 16);
  return launch(gate_direct_kernel, p, grid, 256, gate_direct_smem(a->h), stream, a->pdl);
}

extern "C" int iq_moe_gate(const iq_moe_gate_args* a, void* stream) {
  if (!a || (!a->x_fp8 && !a->x_bf16) || !a->fc || !a->fc_scale || !a->act || !a->scratch)
    return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBasicBytes) return IQ_ERR_ARG;
  if (a->n_shared > 0 && (!a->shared_fc || !a->shared_fc_scale)) return IQ_ERR_ARG;
  if (a->act_kind != IQ_ACT_E4M3 && a->act_kind != IQ_ACT_BF16) return IQ_ERR_ARG;
  if (a->h < 1024 || a->h % 1024 || a->i_loc < 64 || a->i_loc % 64) return IQ_ERR_ARG;
  if (!aligned16(a->x_fp8) || !aligned16(a->x_bf16) || !aligned16(a->fc)) return IQ_ERR_ARG;
  if (sm_count() == 0) return IQ_ERR_CUDA;
  const long long bytes = expert_stream_bytes(a->m, a->top_k, a->n_experts, a->n_shared,
                                              2ll * a->i_loc * a->h);
  if (bytes <= short_stream_bytes()) {
    // One row and a stream of up to IQB200_GATE_DIRECT_MB megabytes (default 12; 0 turns it
    // off): the direct form.  Measured, one row: 6.3 against 8.1 us at 9.4 MB (hidden 3072,
    // expert width 192), but 15.5 against 12.2 us at 28 MB (hidden 6144, width 256), where a
    // warp's three units in flight are too few to keep HBM busy.
    static const long long direct_bytes = env_number("IQB200_GATE_DIRECT_MB", 12) << 20;
    if (bytes <= direct_bytes && a->m == 1 && a->h % 512 == 0 && a->i_loc % 64 == 0 &&
        a->top_k <= 32)
      return gate_direct_launch(a, stream, false);
    // Longer one-row streams: eight features per CTA (IQB200_GATE_DIRECT8=0 turns it off).
    static const bool direct8 = env_number("IQB200_GATE_DIRECT8", 0) != 0;
    if (direct8 && a->m == 1 && a->h % 1024 == 0 && a->i_loc % 64 == 0 && a->top_k <= 32)
      return gate_direct_launch(a, stream, true);
    static const bool runs3 = env_number("IQB200_GATE_RUNS3", 0) != 0;
    int rc = IQ_ERR_UNSUPPORTED;
    if (runs3 && a->h % 768 == 0) rc = gate_launch<Geo<2, 4, 3, 3>>(a, stream);
    if (rc == IQ_ERR_UNSUPPORTED) rc = gate_launch<Geo<2, 4, 2, 3>>(a, stream);
    if (rc != IQ_ERR_UNSUPPORTED) return rc;
  }
  return gate_launch<Geo<2, 8, 2>>(a, stream);
}

template <class G>
static int down_launch(const iq_moe_down_args* a, void* stream) {
  DownParams p{};
  int rc = fill_moe(p.mc, a->m, a->h, a->i_loc, a->n_experts, a->top_k, a->n_shared, a->sel, a->wt);
  if (rc != IQ_OK) return rc;
  p.mc.w = static_cast<const uint8_t*>(a->proj);
  p.mc.w_scale = a->proj_scale;
  p.mc.shared_w = static_cast<const uint8_t*>(a->shared_proj);
  p.mc.shared_scale = a->shared_proj_scale;
  p.mc.w_stride = static_cast<size_t>(a->h) * a->i_loc;
  p.mc.scale_stride = static_cast<size_t>(a->h / 128) * (a->i_loc / 64);
  p.mc.rows_per_expert = a->h;
  StreamShape& sh = p.sh;
  sh.mode = kConcatK;
  sh.n_groups = 1;
  sh.rows_per_group = a->h;
  sh.k_bytes = a->i_loc;
  sh.rg_shift = 7;
  sh.kg_shift = 6;
  sh.pair_half = 0;
  sh.x_rows = a->m * (a->top_k + a->n_shared);
  sh.x_pitch = a->i_loc + 64;
  sh.x_blocks = (a->i_loc + 127) / 128;
  TailPlan tp;
  rc = plan_tail(tp, a->tail, a->push, a->scratch, a->scratch_bytes, a->m, a->h, smem_limit<G>());
  if (rc != IQ_OK) return rc;
  // (a short Down runs as small half-SM CTAs beside the spread CTAs of the Gate before it
  // and of the o_proj after it: one per SM, because every SM has exactly one half free)
  const int grid = grid_for<G>();
  const size_t smem = plan_smem<G>(sh, grid - tp.n_tail, tp.smem, a->m * a->top_k + a->n_shared);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  const int mrc = fill_maps<G>(&p.map0, &p.map1, sh, a->proj,
                               static_cast<long long>(a->n_experts) * a->h, a->shared_proj,
                               static_cast<long long>(a->n_shared) * a->h);
  if (mrc != IQ_OK) return mrc;
  p.act = a->act;
  p.act_kind = a->act_kind;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.scratch = a->scratch;
  p.tail_run = tp.tail_run;
  p.n_tail = tp.n_tail;
  p.push = tp.push;
  p.per_round = tp.per_round;
  p.pv = tp.pv;
  p.pdl_level = a->pdl;
  if (a->tail) {
    p.tail = *a->tail;
    if (!p.tail.status) p.tail.status = scratch_of(a->scratch).status;
  }
  return launch(down_kernel<G>, p, grid, G::THREADS, smem, stream, a->pdl);
}

// The direct form (direct.cuh): 32 weight rows per CTA, no ring.
template <int RT, int RPU>
static int down_direct_launch(const iq_moe_down_args* a, void* stream) {
  DownDirectParams p{};
  int rc = fill_moe(p.mc, a->m, a->h, a->i_loc, a->n_experts, a->top_k, a->n_shared, a->sel, a->wt);
  if (rc != IQ_OK) return rc;
  p.mc.w = static_cast<const uint8_t*>(a->proj);
  p.mc.w_scale = a->proj_scale;
  p.mc.shared_w = static_cast<const uint8_t*>(a->shared_proj);
  p.mc.shared_scale = a->shared_proj_scale;
  p.mc.w_stride = static_cast<size_t>(a->h) * a->i_loc;
  p.mc.scale_stride = static_cast<size_t>(a->h / 128) * (a->i_loc / 64);
  p.mc.rows_per_expert = a->h;
  TailPlan tp;
  // (see linear_direct_launch)
  static const bool split_push = env_number("IQB200_DIRECT_SPLIT_TAIL", 0) != 0;
  const bool pull_tail = a->tail && !a->tail->push && a->tail->world > 1;
  const bool split_tail =
      pull_tail || (split_push && a->tail && a->tail->push && a->tail->world > 2);
  rc = plan_tail(tp, split_tail ? nullptr : a->tail,
                 pull_tail ? nullptr : (split_tail ? a->tail->push : a->push), a->scratch,
                 a->scratch_bytes, a->m, a->h, direct_tail_limit(a->tail));
  if (rc != IQ_OK) return rc;
  size_t smem = down_direct_smem(a->m * (a->top_k + a->n_shared), a->i_loc);
  if (tp.smem > smem) smem = tp.smem;
  p.act = a->act;
  p.act_kind = a->act_kind;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.scratch = a->scratch;
  p.n_tail = tp.n_tail;
  p.push = tp.push;
  p.per_round = tp.per_round;
  p.pv = tp.pv;
  p.pdl_level = a->pdl;
  if (a->tail && !split_tail) {
    p.tail = *a->tail;
    if (!p.tail.status) p.tail.status = scratch_of(a->scratch).status;
  }
  // (48 rows per CTA -- one CTA per SM beside the Gate's, all resident at once -- made the
  // Down itself faster, 11.1 against 12.4 us, but the layer slower, 40.4 against 39.5 us:
  // 32 rows is the default, IQB200_DOWN_DIRECT_ROWS48=1 selects 48 for one or two rows)
  static const bool rows48 = env_number("IQB200_DOWN_DIRECT_ROWS48", 0) != 0;
  if (rows48 && a->h % 48 == 0 && a->m <= 2)
    rc = launch(down_direct_kernel<RT, RPU, 3>, p, a->h / 48 + tp.n_tail, 288, smem, stream,
                a->pdl);
  else
    rc = launch(down_direct_kernel<RT, RPU, 2>, p, a->h / 32 + tp.n_tail, 256, smem, stream,
                a->pdl);
  if (rc != IQ_OK || !split_tail) return rc;
  iq_tail_args t = *a->tail;
  if (!t.status) t.status = scratch_of(a->scratch).status;
  if (pull_tail) return iq_tail(&t, stream, a->pdl);
  return launch_pushed_tail(&t, stream, a->pdl, kSmemSpread);
}

extern "C" int iq_moe_down(const iq_moe_down_args* a, void* stream) {
  if (!a || !a->act || !a->proj || !a->proj_scale || !a->out || !a->wt || !a->scratch)
    return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBasicBytes) return IQ_ERR_ARG;
  if (a->n_shared > 0 && (!a->shared_proj || !a->shared_proj_scale)) return IQ_ERR_ARG;
  if (a->act_kind != IQ_ACT_E4M3 && a->act_kind != IQ_ACT_BF16) return IQ_ERR_ARG;
  if (a->h < 128 || a->h % 128 || a->i_loc < 64 || a->i_loc % 64) return IQ_ERR_ARG;
  if (a->act_kind == IQ_ACT_BF16 && a->i_loc % 128) return IQ_ERR_ARG;
  if (!aligned16(a->act) || !aligned16(a->proj) || !aligned16(a->out)) return IQ_ERR_ARG;
  if (a->tail) {
    const int rc = check_tail(a->tail);
    if (rc != IQ_OK) return rc;
    if (a->tail->partial != a->out || a->tail->m != a->m || a->tail->h != a->h) return IQ_ERR_ARG;
  }
  if (sm_count() == 0) return IQ_ERR_CUDA;
  const int k = a->i_loc;
  const long long bytes = expert_stream_bytes(a->m, a->top_k, a->n_experts, a->n_shared,
                                              static_cast<long long>(a->h) * a->i_loc);
  if (bytes <= short_stream_bytes()) {
    // A stream this short runs in the direct form where that exists (an expert width of at
    // most 512): see direct.cuh.  IQB200_DOWN_DIRECT=0 turns it off.
    static const bool direct = env_number("IQB200_DOWN_DIRECT", 1) != 0;
    if (direct && a->h % kDirectRows == 0 && a->m * (a->top_k + a->n_shared) <= kDirectMaxRows) {
      int rc = IQ_ERR_UNSUPPORTED;
      if (k == 512) rc = down_direct_launch<8, 2>(a, stream);
      else if (k == 256) rc = down_direct_launch<4, 2>(a, stream);
      else if (k == 192) rc = down_direct_launch<3, 1>(a, stream);
      else if (k == 128) rc = down_direct_launch<2, 2>(a, stream);
      else if (k == 64) rc = down_direct_launch<1, 1>(a, stream);
      if (rc != IQ_ERR_UNSUPPORTED) return rc;
    }
    // two CTAs per SM (see Geo); fall through when the staged activations leave no room
    int rc = IQ_ERR_UNSUPPORTED;
    if (k % 1024 == 0) rc = down_launch<Geo<1, 8, 2>>(a, stream);
    else if (k % 512 == 0 && a->h % 32 == 0) rc = down_launch<Geo<2, 4, 2>>(a, stream);
    else if (k % 256 == 0 && a->h % 32 == 0) {
      // Whole tiles per CTA: the launch takes as long as the CTA with the most rows.  With
      // 32-row tiles 6144 rows are 192 tiles, two for every third of 147 CTAs (64 rows);
      // 48-row tiles give 128 CTAs one tile each.
      const int ctas = std::max(1, sm_count() - a->m);
      const int most32 = (a->h / 32 + ctas - 1) / ctas * 32;
      const int most48 = a->h % 48 == 0 ? (a->h / 48 + ctas - 1) / ctas * 48 : 1 << 30;
      if (most48 < most32) rc = down_launch<Geo<3, 2, 2, 2>>(a, stream);
      if (rc == IQ_ERR_UNSUPPORTED) rc = down_launch<Geo<2, 4, 1>>(a, stream);
    }
    else if (k % 192 == 0 && a->h % 32 == 0) rc = down_launch<Geo<2, 3, 1>>(a, stream);
    if (rc != IQ_ERR_UNSUPPORTED) return rc;
  }
  // k = 1024: 32 rows x 1 KB stages (two 64-byte runs per warp) measured 5 % faster than
  // 16 rows x 1 KB; at k = 512 the wider tile (64 rows) measured slower and is not used.
  static const bool rows32 = env_number("IQB200_K2048_ROWS32", 0) != 0;   // (see iq_linear)
  if (k % 2048 == 0 && !(rows32 && a->h % 32 == 0)) return down_launch<Geo<1, 16, 2>>(a, stream);
  if (k % 1024 == 0 && a->h % 32 == 0) return down_launch<Geo<2, 8, 2>>(a, stream);
  if (k % 1024 == 0) return down_launch<Geo<1, 16, 1>>(a, stream);
  if (k % 512 == 0 && a->h % 32 == 0) return down_launch<Geo<2, 8, 1>>(a, stream);
  if (k % 256 == 0 && a->h % 64 == 0) return down_launch<Geo<4, 4, 1>>(a, stream);
  if (k % 192 == 0 && a->h % 256 == 0) return down_launch<Geo<16, 1, 3>>(a, stream);
  if (k % 128 == 0 && a->h % 128 == 0) return down_launch<Geo<8, 2, 1>>(a, stream);
  return IQ_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------
// iq_linear_static: iq_linear for callers that cannot obtain device memory.
//
// Some callers of this library cannot allocate on the device at the point where they
// call it: a plugin running inside a host application's stream capture (cudaMalloc is
// illegal there), a serving loop whose memory budget was handed out in full at start-up,
// or a host that is only given raw pointers to inputs and outputs.  For them the work
// area of the streaming GEMV (split-tile partial sums, tile counters, the CTA ticket and
// the status word) lives in this file-scope device array instead of a caller buffer.
// Every GPU that loads the library holds the array (kScrBasicBytes, about 4.3 MB) until exit.
//
// `g_static_scratch` below is a host-side stand-in when named in host code, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device with that device current.
constexpr int kStaticMaxN = 65536;   // largest output width served from the static area
constexpr int kStaticMaxK = 65536;   // largest contraction length
static __device__ __align__(256) uint8_t g_static_scratch[kScrBasicBytes];
static void* g_static_ptr[64] = {};   // per device, guarded by g_host_mutex

// The array's device address on the current device; looked up on the first call.
static int static_scratch_ptr(void** out, bool resolve) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return IQ_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (!g_static_ptr[dev] && resolve) {
    // First call on this device: resolve the array's device address.  Do this before any
    // stream capture begins.
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || !ptr) {
      fprintf(stderr, "iqb200: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(err));
      return IQ_ERR_CUDA;
    }
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return IQ_OK;
}

extern "C" int iq_linear_static(const iq_linear_args* a, void* stream) {
  if (!a) return IQ_ERR_ARG;
  if (a->tail) {
    fprintf(stderr, "iqb200: iq_linear_static does not run a fused tail\n");
    return IQ_ERR_UNSUPPORTED;
  }
  if (a->n > kStaticMaxN || a->k > kStaticMaxK) {
    fprintf(stderr,
            "iqb200: iq_linear_static serves n <= %d and k <= %d from its built-in work area; "
            "got n=%d k=%d (use iq_linear with a caller scratch buffer)\n",
            kStaticMaxN, kStaticMaxK, a->n, a->k);
    return IQ_ERR_UNSUPPORTED;
  }
  void* base = nullptr;
  const int prc = static_scratch_ptr(&base, true);
  if (prc != IQ_OK) return prc;
  // The array keeps whatever the last call left.  The kernel expects the status word,
  // the ticket and the tile counters at zero; the partial-sum area is written before it
  // is read and needs no clearing.
  if (cudaMemsetAsync(base, 0, kScrPartials, static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return IQ_ERR_CUDA;
  iq_linear_args b = *a;
  b.scratch = base;
  b.scratch_bytes = kScrBasicBytes;
  b.push = nullptr;
  return iq_linear(&b, stream);
}

extern "C" int iq_linear_static_status(int* code, void* stream) {
  if (!code) return IQ_ERR_ARG;
  void* base = nullptr;
  const int prc = static_scratch_ptr(&base, false);
  if (prc != IQ_OK) return prc;
  *code = 0;
  if (!base) return IQ_OK;              // no call has been made on this device yet
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(code, base, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return IQ_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return IQ_ERR_CUDA;
  return IQ_OK;
}

#ifdef IQ_TRACE
// Trace builds only: `base` receives slots x 304 x 16 u64 stamps, one slot per launch in
// launch order from now on (NULL stops tracing).
extern "C" void iq_trace_set(void* base, int slots) {
  std::lock_guard<std::mutex> lock(iqb::g_host_mutex);
  iqb::g_trace_base = static_cast<unsigned long long*>(base);
  iqb::g_trace_slots = slots;
  iqb::g_trace_next = 0;
}
#endif
