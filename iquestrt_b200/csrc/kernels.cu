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

#include <mutex>
#include <utility>
#include <vector>

#include "stream_core.cuh"

namespace iqb {

// ------------------------------------------------------------------------------------
// Scratch layout (bytes): status @0, ticket @64, tile counters @256, partials after.
constexpr size_t kScrTicket = 64;
constexpr size_t kScrCounters = 256;
constexpr int kMaxTiles = 16384;
constexpr size_t kScrPartials = kScrCounters + sizeof(uint32_t) * kMaxTiles;
constexpr int kMaxGrid = 256;
constexpr size_t kScrBasicBytes = kScrPartials + sizeof(float) * kMaxGrid * 2 * 256 * 8;
// The one-launch layer keeps its tagged hand-off words in an area of their own behind the
// basic scratch: the other kernels never write there, so a word can only carry a tag that
// a one-launch layer gave it.
constexpr size_t kScrLayerBytes = 3 * 1024 * 1024 + 256 * 1024;
constexpr size_t kScrBytes = kScrBasicBytes + kScrLayerBytes;

__host__ __device__ inline StreamScratch scratch_of(void* base) {
  StreamScratch s;
  uint8_t* b = static_cast<uint8_t*>(base);
  s.status = reinterpret_cast<int*>(b);
  s.ticket = reinterpret_cast<uint32_t*>(b + kScrTicket);
  s.tile_counter = reinterpret_cast<uint32_t*>(b + kScrCounters);
  s.partials = reinterpret_cast<float*>(b + kScrPartials);
  return s;
}

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

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
// Activation staging (consumer threads only, tid in [0, 256)).

// Both routines issue a batch of independent 16-byte global loads before touching any of
// them, so a row set costs about one memory latency instead of one per group.  The loads
// bypass L1 (ld.global.cg): in the one-launch layer the rows were written by another CTA
// of the same launch.
constexpr int kStageBatch = 8;

// Raw e4m3 rows (16-byte vectors) + their scales (or 1).
__device__ inline void stage_rows_e4m3(uint8_t* xq, float* xs, const StreamShape& sh,
                                       const uint8_t* src, size_t src_pitch,
                                       const float* src_scale, int rows, int k, int tid) {
  const int vec = k / 16, nvec = rows * vec;
  // the first activation scale of this thread rides along with the first batch of loads
  const int nxs = rows * sh.x_blocks;
  float xs_first = 1.0f;
  if (src_scale && tid < nxs) xs_first = __ldcg(src_scale + tid);
  for (int v0 = 0; v0 < nvec; v0 += kConsumerThreads * kStageBatch) {
    uint4 raw[kStageBatch];
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * kConsumerThreads >= nvec) break;   // same for every thread
      const int i = v0 + j * kConsumerThreads + tid;
      if (i < nvec) {
        const int r = i / vec, v = i - r * vec;
        raw[j] = __ldcg(reinterpret_cast<const uint4*>(src + r * src_pitch + v * 16));
      }
    }
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * kConsumerThreads >= nvec) break;
      const int i = v0 + j * kConsumerThreads + tid;
      if (i < nvec) {
        const int r = i / vec, v = i - r * vec;
        *reinterpret_cast<uint4*>(xq + r * sh.x_pitch + v * 16) = raw[j];
      }
    }
  }
  if (tid < nxs) xs[tid] = xs_first;
  for (int i = tid + kConsumerThreads; i < nxs; i += kConsumerThreads)
    xs[i] = src_scale ? __ldcg(src_scale + i) : 1.0f;
}

// bf16 rows quantised per 1x128 group: scale = amax/448 (1 for an all-zero group), value
// = e4m3(x * (1 / scale)).  A thread holds eight consecutive elements, so a group is sixteen
// consecutive lanes.  With `split2` row r becomes staged rows 2r (the e4m3 value) and
// 2r+1 (the e4m3 of what the first term missed), both under the same scale.
__device__ inline void stage_rows_bf16_groupq(uint8_t* xq, float* xs, const StreamShape& sh,
                                              const __nv_bfloat16* src, size_t src_pitch,
                                              int rows, int k, bool split2, int tid) {
  const int vec = k / 8, nvec = rows * vec;
  for (int v0 = 0; v0 < nvec; v0 += kConsumerThreads * kStageBatch) {
    uint4 raw[kStageBatch];
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * kConsumerThreads >= nvec) break;   // same for every thread
      const int i = v0 + j * kConsumerThreads + tid;
      raw[j] = make_uint4(0u, 0u, 0u, 0u);
      if (i < nvec) {
        const int r = i / vec, v = i - r * vec;
        raw[j] = __ldcg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * src_pitch + v * 8));
      }
    }
#pragma unroll
    for (int j = 0; j < kStageBatch; ++j) {
      if (v0 + j * kConsumerThreads >= nvec) break;    // whole batch dead: nothing to do
      const int i = v0 + j * kConsumerThreads + tid;   // uniform trip count: shuffles below
      const bool live = i < nvec;
      const int ii = live ? i : 0;
      const int r = ii / vec, v = ii - r * vec;
      float f[8];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 t = __bfloat1622float2(p[q]);
        f[2 * q] = t.x;
        f[2 * q + 1] = t.y;
      }
      float amax = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
#pragma unroll
      for (int o = 8; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (!live) continue;               // after the shuffles: dead lanes skip the math
      const float s = amax > 0.f ? amax / 448.0f : 1.0f;
      const float rcp = 1.0f / s;        // one division per vector; values use x * (1/s)
      uint32_t q0[2] = {0u, 0u}, q1[2] = {0u, 0u};
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float xn = f[q] * rcp;
        const uint8_t a = f32_to_e4m3_sat(xn);
        q0[q >> 2] |= static_cast<uint32_t>(a) << (8 * (q & 3));
        if (split2)
          q1[q >> 2] |= static_cast<uint32_t>(f32_to_e4m3_sat(xn - e4m3_to_f32(a))) << (8 * (q & 3));
      }
      const int blk = v >> 4;
      if (split2) {
        *reinterpret_cast<uint2*>(xq + (2 * r) * sh.x_pitch + v * 8) = make_uint2(q0[0], q0[1]);
        *reinterpret_cast<uint2*>(xq + (2 * r + 1) * sh.x_pitch + v * 8) = make_uint2(q1[0], q1[1]);
        if ((v & 15) == 0) {
          xs[(2 * r) * sh.x_blocks + blk] = s;
          xs[(2 * r + 1) * sh.x_blocks + blk] = s;
        }
      } else {
        *reinterpret_cast<uint2*>(xq + r * sh.x_pitch + v * 8) = make_uint2(q0[0], q0[1]);
        if ((v & 15) == 0) xs[r * sh.x_blocks + blk] = s;
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// The tail: all-reduce of the ranks' bf16 rows, residual add and RMSNorm(s).
struct TailParams {
  iq_tail_args a;
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

constexpr int kTailVecs = 2;   // 16-byte vectors of a row per thread: h <= 8 * 2 * threads

__device__ __forceinline__ void ldg_f32x8(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Runs on the threads of `bar` (a multiple of 32; h <= 16 * threads).  `red` is shared
// memory for 4 x 32 floats, `sflag` one shared int.  Rows written by other CTAs of this
// launch must already be visible (the caller passed the ticket).  Rows are handled one
// after the other, each entirely in registers, and each RMSNorm costs one block barrier.
// The kernels this runs in keep almost all of the SM's L1 as shared memory, so a spilled
// register would cost an L2 round trip: the loads are ordered to keep few values live
// (the residual stays packed until it is used; each norm weight is fetched just before
// the barrier of the reduction that precedes its use, which hides its latency).
__device__ __forceinline__ void run_tail(const iq_tail_args& a, __nv_bfloat16* /*rows_s*/,
                                         float* red, int* sflag, const BlockBar bar = BlockBar{}) {
  const int tid = threadIdx.x, nthr = bar.threads();
  const int m = a.m, h = a.h, vec_per_row = h / 8;
  const float inv_h = 1.0f / static_cast<float>(h);
  const bool attn = a.kind == IQ_TAIL_ATTN;

  for (int r = 0; r < m; ++r) {
    const size_t row_off = static_cast<size_t>(r) * h;
    float* slots0 = red + (r & 1) * 64;        // two reductions per row, alternating rows
    float* slots1 = slots0 + 32;
    // ---- the row's residual, issued before the cross-rank wait and kept packed
    uint4 res_raw[kTailVecs][2];
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      const size_t off = row_off + static_cast<size_t>(v) * 8;
      if (a.residual_fp32) {
        const float* rp = static_cast<const float*>(a.residual) + off;
        res_raw[i][0] = __ldcg(reinterpret_cast<const uint4*>(rp));
        res_raw[i][1] = __ldcg(reinterpret_cast<const uint4*>(rp + 4));
      } else {
        res_raw[i][0] = __ldcg(
            reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.residual) + off));
      }
    }
    // ---- cross-rank readiness: signal, then wait while the residual loads are in flight
    if (r == 0 && a.world > 1) {
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
    float f[kTailVecs][8];
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
          U4 pv[4];
#pragma unroll
          for (int p = 0; p < 4; ++p)
            if (p0 + p < a.world)
              pv[p] = ld_global_u4(static_cast<const __nv_bfloat16*>(a.peer_partials[p0 + p]) + off);
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            if (p0 + p >= a.world) continue;
            float t[8];
            bf16x8_to_f32(pv[p], t);
#pragma unroll
            for (int j = 0; j < 8; ++j) accv[j] += t[j];
          }
        }
        part = f32_to_bf16x8(accv);
      }
      bf16x8_to_f32(part, f[i]);
    }

    float wv[kTailVecs][8];    // w_first, later w_norm
    float inv1 = 0.f;
    if (attn) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kTailVecs; ++i) {
        const int v = tid + i * nthr;
        if (v >= vec_per_row) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[i][j], f[i][j], ss);
        ldg_f32x8(a.w_first + v * 8, wv[i]);      // lands while the reduction's barrier is waited
      }
      inv1 = rsqrtf(block_sum(ss, slots0, bar) * inv_h + a.eps);
    }
    // ---- h = residual + (ATTN: bf16(bf16(w1*(ao*inv))*scale) | MLP: bf16(m*scale))
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      const size_t off = row_off + static_cast<size_t>(v) * 8;
      float res[8];
      if (a.residual_fp32) {
        const float* r0 = reinterpret_cast<const float*>(&res_raw[i][0]);
        const float* r1 = reinterpret_cast<const float*>(&res_raw[i][1]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { res[j] = r0[j]; res[4 + j] = r1[j]; }
      } else {
        bf16x8_to_f32(U4{res_raw[i][0].x, res_raw[i][0].y, res_raw[i][0].z, res_raw[i][0].w}, res);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float add;
        if (attn) {
          const float nrm = bf16_round(wv[i][j] * (f[i][j] * inv1));
          add = bf16_round(nrm * a.scale);
        } else {
          add = bf16_round(f[i][j] * a.scale);
        }
        f[i][j] = res[j] + add;                 // f now holds h
      }
      if (a.residual_fp32) {
        float* ho = static_cast<float*>(a.h_out) + off;
        *reinterpret_cast<float4*>(ho) = make_float4(f[i][0], f[i][1], f[i][2], f[i][3]);
        *reinterpret_cast<float4*>(ho + 4) = make_float4(f[i][4], f[i][5], f[i][6], f[i][7]);
      } else {
        const U4 hb = f32_to_bf16x8(f[i]);
        *reinterpret_cast<U4*>(static_cast<__nv_bfloat16*>(a.h_out) + off) = hb;
        bf16x8_to_f32(hb, f[i]);            // the norm sees the rounded stream
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss2 = fmaf(f[i][j], f[i][j], ss2);
      ldg_f32x8(a.w_norm + v * 8, wv[i]);
    }
    const float inv2 = rsqrtf(block_sum(ss2, slots1, bar) * inv_h + a.eps);
    if (a.inv_out && tid == 0) a.inv_out[r] = inv2;

    // ---- norm_out = bf16(w_norm * (h * inv)) (+ e4m3 copy, unscaled or per 1x128 group)
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      const bool live = v < vec_per_row;       // uniform over each 16-lane group
      const size_t off = row_off + static_cast<size_t>(live ? v : 0) * 8;
      float o[8];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = live ? bf16_round(wv[i][j] * (f[i][j] * inv2)) : 0.f;
        amax = fmaxf(amax, fabsf(o[j]));
      }
      if (live)
        *reinterpret_cast<U4*>(static_cast<__nv_bfloat16*>(a.norm_out) + off) = f32_to_bf16x8(o);
      if (a.norm_fp8) {
        float sc = 1.0f;
        if (a.norm_fp8_scale) {
          // A 128-element group is sixteen consecutive vectors = sixteen consecutive lanes.
#pragma unroll
          for (int o2 = 8; o2; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
          sc = amax > 0.f ? amax / 448.0f : 1.0f;
          if (live && (v & 15) == 0) a.norm_fp8_scale[static_cast<size_t>(r) * (h / 128) + (v >> 4)] = sc;
        }
        const float rcp = 1.0f / sc;
        uint32_t q0 = 0, q1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q0 |= static_cast<uint32_t>(f32_to_e4m3_sat(o[j] * rcp)) << (8 * j);
          q1 |= static_cast<uint32_t>(f32_to_e4m3_sat(o[j + 4] * rcp)) << (8 * j);
        }
        if (live) *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.norm_fp8) + off) = make_uint2(q0, q1);
      }
    }
  }
  if (a.world > 1 && tid == 0) *a.epoch = *a.epoch + 1u;
}

__global__ void __launch_bounds__(kThreads, 1) tail_kernel(const TailParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_wait();
  pdl_launch_dependents();   // after the wait: see the note on `after_wait` below
  float* red = reinterpret_cast<float*>(smem);
  int* sflag = reinterpret_cast<int*>(smem + 512);
  // Sixteen warps everywhere the tail runs, so that its block-wide sums add in one order.
  if (threadIdx.x < kConsumerThreads)
    run_tail(p.a, reinterpret_cast<__nv_bfloat16*>(smem + 1024), red, sflag,
             BlockBar{2, kConsumerThreads});
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
// iq_linear
struct LinearParams {
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  const void* x;
  const float* x_scale;
  int x_kind, m, k, n;
  const uint8_t* w;
  const float* w_scale;
  __nv_bfloat16* out;
  void* scratch;
  int has_tail;
  iq_tail_args tail;
};

template <class G>
__global__ void __launch_bounds__(kThreads, 1) linear_kernel(const __grid_constant__ LinearParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const StreamShape& sh = p.sh;
  const Carve<G> cv = carve<G>(smem, sh);
  const StreamScratch scr = scratch_of(p.scratch);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  const int cta = blockIdx.x;
  stream_init<G>(sh, cv.sm);
  if (tid == kProducerWarp * 32 && !(sh.k_bytes == G::KC && G::NBOX == 1))
    prefetch_tensormap(&p.map0);   // only a map the host filled (K-sliced stages)
  if (tid == 0) {
    GroupDesc& g = cv.sm->groups[0];
    g.w = p.w;
    g.scale = p.w_scale;
    g.row_base = 0;
    g.map_id = 0;
    for (int c = 0; c < kMaxCols; ++c) {
      g.col_row[c] = c < sh.x_rows ? c : -1;
      g.col_mul[c] = 1.0f;
      g.col_out[c] = static_cast<int16_t>(c);
    }
  }
  __syncthreads();
  {
    const CtaWork wk = cta_share<G>(sh, static_cast<int>(gridDim.x), cta, grid);
    if (warp == kProducerWarp) {
      // Weights never change: start streaming before the predecessor kernel has finished.
      produce<G>(sh, cv.sm, cv.ring, wk, scr.status, &p.map0, &p.map1);
      pdl_wait();
    } else if (warp < kConsumerWarps) {
      float held[kGatherHeld];
      gather_scales_load<G, ElemE4M3>(sh, cv.sm, wk, tid, held);   // weights: before the wait
      after_wait();
      if (p.x_kind == IQ_X_BF16_GROUPQ || p.x_kind == IQ_X_BF16_SPLIT2)
        stage_rows_bf16_groupq(cv.xq, cv.xs, sh, static_cast<const __nv_bfloat16*>(p.x), p.k, p.m,
                               p.k, p.x_kind == IQ_X_BF16_SPLIT2, tid);
      else
        stage_rows_e4m3(cv.xq, cv.xs, sh, static_cast<const uint8_t*>(p.x), p.k,
                        p.x_kind == IQ_X_E4M3_GROUP ? p.x_scale : nullptr, p.m, p.k, tid);
      gather_scales_store<G, ElemE4M3>(sh, cv.sm, wk, cv.sc, tid, held);
      named_bar_sync(1, kConsumerThreads);
      consume<G, ElemE4M3>(sh, cv.sm, cv.ring, cv.xq, cv.xs, cv.sc, wk, scr);
    } else {
      pdl_wait();
      const bool split2 = p.x_kind == IQ_X_BF16_SPLIT2;
      const int m = p.m, n = p.n;
      __nv_bfloat16* out = p.out;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[G::RT]) {
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub) {
          const int row = id.tig * G::ROWS + sub * 16 + r;
          if (split2) {
            // columns 2j and 2j+1 are the two terms of row j: fold them on the even lane
            const float other = __shfl_xor_sync(0xffffffffu, val[sub], 1);
            if ((col & 1) == 0 && (col >> 1) < m)
              out[static_cast<size_t>(col >> 1) * n + row] = __float2bfloat16_rn(val[sub] + other);
          } else if (col < m) {
            out[static_cast<size_t>(col) * n + row] = __float2bfloat16_rn(val[sub]);
          }
        }
      };
      epilogue<G>(sh, cv.sm, wk, total, grid, cta, scr, emit);
    }
  }
  if (!p.has_tail) {
    stream_drain_on_abort<G>(cv.sm);
    return;
  }
  if (last_cta<G>(cv.sm, scr, gridDim.x)) {
    // The ring is idle now: its first bytes hold the reduced rows.
    float* red = reinterpret_cast<float*>(cv.sm->red);
    if (threadIdx.x < kConsumerThreads)
      run_tail(p.tail, reinterpret_cast<__nv_bfloat16*>(cv.ring), red, &cv.sm->is_last_tile,
               BlockBar{2, kConsumerThreads});
  }
  stream_drain_on_abort<G>(cv.sm);
}

// ------------------------------------------------------------------------------------
// iq_router: bf16 GEMV into fp32 logits, then top-k on the last CTA (one warp per row).
struct RouterParams {
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  const __nv_bfloat16* x;
  const uint8_t* w;
  int m, h, e, top_k, score;
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
template <int kMaxPerLane>
__device__ __forceinline__ void select_row_impl(const float* logits, int e, int top_k, int score,
                                                int row, int* sel, float* wt,
                                                bool logits_in_smem) {
  const int lane = threadIdx.x & 31;
  uint32_t key[kMaxPerLane];
  const int per = (e + 31) / 32;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int id = lane + 32 * j;
    float lv = 0.f;
    if (j < per && id < e)
      lv = logits_in_smem ? logits[static_cast<size_t>(row) * e + id]
                          : __ldcg(logits + static_cast<size_t>(row) * e + id);
    key[j] = (j < per && id < e) ? ordered_key(lv) : 0u;
  }
  int my_id = 0x7fffffff;
  float top_val = 0.f, sum = 0.f, my_p = 0.f;
  for (int t = 0; t < top_k; ++t) {
    uint32_t best = 0;
    int best_id = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int id = lane + 32 * j;
      if (key[j] > best) { best = key[j]; best_id = id; }   // ascending id: first max wins
    }
    const uint32_t wmax = __reduce_max_sync(0xffffffffu, best);
    const int cand = (best == wmax && best != 0u) ? best_id : 0x7fffffff;
    const int win = __reduce_min_sync(0xffffffffu, cand);
    if (win == 0x7fffffff) break;            // fewer than top_k finite logits
    const uint32_t kbits = wmax;
    const uint32_t raw = (kbits & 0x80000000u) ? (kbits & 0x7fffffffu) : ~kbits;
    const float val = __uint_as_float(raw);
    if (t == 0) top_val = val;
    const float p = score == IQ_ROUTE_SOFTMAX ? expf(__fsub_rn(val, top_val))
                                              : 1.0f / (1.0f + expf(-val));
    sum = __fadd_rn(sum, p);
    if (lane == t) { my_id = win; my_p = p; }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if ((win & 31) == lane && (win >> 5) == j) key[j] = 0u;
  }
  // rank of my id among the selected ids
  int rank = 0;
  for (int t = 0; t < top_k; ++t) {
    const int other = __shfl_sync(0xffffffffu, my_id, t);
    rank += (other < my_id) ? 1 : 0;
  }
  if (lane < top_k && my_id != 0x7fffffff) {
    sel[row * top_k + rank] = my_id;
    wt[row * top_k + rank] = my_p / sum;
  }
}

// The selection runs on one warp at the end of the router's critical path, so its length
// in instructions matters: up to 256 experts take the variant with 8 keys per lane.
__device__ void select_row(const float* logits, int e, int top_k, int score, int row, int* sel,
                           float* wt, bool logits_in_smem = false) {
  if (e <= 256)
    select_row_impl<8>(logits, e, top_k, score, row, sel, wt, logits_in_smem);
  else
    select_row_impl<16>(logits, e, top_k, score, row, sel, wt, logits_in_smem);   // e <= 512
}

template <class G>
__global__ void __launch_bounds__(kThreads, 1) router_kernel(const __grid_constant__ RouterParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const StreamShape& sh = p.sh;
  const Carve<G> cv = carve<G>(smem, sh);
  const StreamScratch scr = scratch_of(p.scratch);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  const int cta = blockIdx.x;
  stream_init<G>(sh, cv.sm);
  if (tid == kProducerWarp * 32 && !(sh.k_bytes == G::KC && G::NBOX == 1))
    prefetch_tensormap(&p.map0);   // only a map the host filled (K-sliced stages)
  if (tid == 0) {
    GroupDesc& g = cv.sm->groups[0];
    g.w = p.w;
    g.scale = nullptr;
    g.row_base = 0;
    g.map_id = 0;
    for (int c = 0; c < kMaxCols; ++c) {
      g.col_row[c] = c < p.m ? c : -1;
      g.col_mul[c] = 1.0f;
      g.col_out[c] = static_cast<int16_t>(c);
    }
  }
  __syncthreads();
  {
    const CtaWork wk = cta_share<G>(sh, static_cast<int>(gridDim.x), cta, grid);
    if (warp == kProducerWarp) {
      produce<G>(sh, cv.sm, cv.ring, wk, scr.status, &p.map0, &p.map1);
      pdl_wait();
    } else if (warp < kConsumerWarps) {
      after_wait();
      const int vec = p.h / 8;   // 16-byte vectors per bf16 row
      for (int i = tid; i < p.m * vec; i += kConsumerThreads) {
        const int r = i / vec, v = i - r * vec;
        *reinterpret_cast<uint4*>(cv.xq + r * sh.x_pitch + v * 16) =
            *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(r) * p.h + v * 8);
      }
      named_bar_sync(1, kConsumerThreads);
      consume<G, ElemBF16>(sh, cv.sm, cv.ring, cv.xq, cv.xs, cv.sc, wk, scr);
    } else {
      pdl_wait();
      const int m = p.m, e = p.e;
      float* logits = p.logits;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[G::RT]) {
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub)
          if (col < m)
            logits[static_cast<size_t>(col) * e + id.tig * G::ROWS + sub * 16 + r] = val[sub];
      };
      epilogue<G>(sh, cv.sm, wk, total, grid, cta, scr, emit);
    }
  }
  if (last_cta<G>(cv.sm, scr, gridDim.x)) {
    if (warp < p.m) select_row(p.logits, p.e, p.top_k, p.score, warp, p.sel, p.wt);
  }
  stream_drain_on_abort<G>(cv.sm);
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
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  MoeCommon mc;
  const uint8_t* x_fp8;
  const float* x_scale;
  void* act;
  int act_kind;
  void* scratch;
  int pdl_level;
  int early_shared;   // see gate_kernel
};

// One stream of the Gate: the tiles of `wk`, every role with its ring / reduction position
// carried in `pos` / `rpos` (the kernel may run two streams back to back).
template <class G>
__device__ __forceinline__ void gate_stream(const GateParams& p, const StreamShape& sh,
                                            const Carve<G>& cv, const StreamScratch& scr,
                                            const CtaWork& wk, long long total, int grid, int cta,
                                            bool stage_x, RingPos& pos, RedPos& rpos) {
  const int tid = threadIdx.x, warp = tid >> 5;
  if (warp == kProducerWarp) {
    produce<G>(sh, cv.sm, cv.sm->groups, cv.ring, G::STAGE_BYTES, wk, scr.status, &p.map0, &p.map1,
               pos);
  } else if (warp < kConsumerWarps) {
    float held[kGatherHeld];
    gather_scales_load<G, ElemE4M3>(sh, cv.sm, wk, tid, held);
    if (stage_x)
      stage_rows_e4m3(cv.xq, cv.xs, sh, p.x_fp8, p.mc.h, p.x_scale, p.mc.m, p.mc.h, tid);
    gather_scales_store<G, ElemE4M3>(sh, cv.sm, wk, cv.sc, tid, held);
    named_bar_sync(1, kConsumerThreads);
    consume<G, ElemE4M3>(sh, cv.sm, cv.sm->groups, cv.ring, G::STAGE_BYTES, cv.xq, cv.xs, cv.sc, wk,
                         scr, pos, rpos);
  } else {
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
    epilogue<G>(sh, cv.sm, wk, total, grid, cta, scr, rpos, emit);
  }
}

template <class G>
__global__ void __launch_bounds__(kThreads, 1) gate_kernel(const __grid_constant__ GateParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  StreamShape sh = p.sh;
  const Carve<G> cv = carve<G>(smem, sh);
  const StreamScratch scr = scratch_of(p.scratch);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int cta = blockIdx.x, n_cta = static_cast<int>(gridDim.x);
  stream_init<G>(sh, cv.sm);
  if (tid == kProducerWarp * 32 && !(sh.k_bytes == G::KC && G::NBOX == 1)) {
    prefetch_tensormap(&p.map0);   // only maps the host filled (K-sliced stages)
    if (p.mc.n_shared > 0) prefetch_tensormap(&p.map1);
  }
  RingPos pos;
  RedPos rpos;
  // Level 2: the activations were written two launches back (by the attention tail) and
  // can be staged while the router, the immediate predecessor, is still finishing.
  const bool early_x = p.pdl_level >= 2;
  if (early_x && warp < kConsumerWarps)
    stage_rows_e4m3(cv.xq, cv.xs, sh, p.x_fp8, p.mc.h, p.x_scale, p.mc.m, p.mc.h, tid);
  // With `early_shared` (host: level 2, shared experts, whole tiles dealt round robin
  // whatever the routes) the shared experts are the first groups, CTA c's first tile is
  // tile c, and if that is a shared expert's tile the CTA streams and finishes it NOW:
  // nothing in it depends on the routes.  A whole tile needs no scratch, and the
  // activation buffer's last reader (the previous layer's Down) finished before the
  // router could start.
  int done_tiles = 0;
  if (p.early_shared) {
    const int tpg = stream_tiles_per_group<G>(sh);
    if (tid < p.mc.n_shared) {
      GroupDesc& gd = cv.sm->groups[tid];
      gd.w = p.mc.shared_w + static_cast<size_t>(tid) * p.mc.w_stride;
      gd.scale = p.mc.shared_scale + static_cast<size_t>(tid) * p.mc.scale_stride;
      gd.row_base = tid * p.mc.rows_per_expert;
      gd.map_id = 1;
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
  sh.n_groups = build_groups(cv.sm->groups, p.mc, false, false, scr.status, cv.sm->route_ids,
                             BlockBar{}, nullptr, nullptr, nullptr, nullptr, p.early_shared != 0);
  const long long total =
      static_cast<long long>(stream_num_tiles<G>(sh)) * stream_stages_per_tile<G>(sh);
  int grid = 0;   // CTAs that take part in the stream (set by cta_share)
  CtaWork wk = cta_share<G>(sh, n_cta, cta, grid);
  if (done_tiles) {                 // the first tile is finished already
    wk.tile0 += wk.tile_step;
    wk.n_items -= wk.spt;
  }
  gate_stream<G>(p, sh, cv, scr, wk, total, grid, cta, !early_x, pos, rpos);
  stream_drain_on_abort<G>(cv.sm);
}

struct DownParams {
  CUtensorMap map0, map1;   // weight tensor maps (unused for whole-row stages)
  StreamShape sh;
  MoeCommon mc;
  const void* act;
  int act_kind;
  __nv_bfloat16* out;
  void* scratch;
  int has_tail;
  int pdl_level;
  iq_tail_args tail;
};

template <class G>
__global__ void __launch_bounds__(kThreads, 1) down_kernel(const __grid_constant__ DownParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  StreamShape sh = p.sh;
  const Carve<G> cv = carve<G>(smem, sh);
  const StreamScratch scr = scratch_of(p.scratch);
  const int tid = threadIdx.x, warp = tid >> 5;
  stream_init<G>(sh, cv.sm);
  if (tid == kProducerWarp * 32 && !(sh.k_bytes == G::KC && G::NBOX == 1)) {
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
  const int cta = blockIdx.x;
  {
    const CtaWork wk = cta_share<G>(sh, static_cast<int>(gridDim.x), cta, grid);
    if (warp == kProducerWarp) {
      produce<G>(sh, cv.sm, cv.ring, wk, scr.status, &p.map0, &p.map1);
    } else if (warp < kConsumerWarps) {
      float held[kGatherHeld];
      gather_scales_load<G, ElemE4M3>(sh, cv.sm, wk, tid, held);
      if (early) after_wait();
      const int rows = p.mc.m * (p.mc.top_k + p.mc.n_shared);
      if (p.act_kind == IQ_ACT_E4M3)
        stage_rows_e4m3(cv.xq, cv.xs, sh, static_cast<const uint8_t*>(p.act), p.mc.i_loc, nullptr,
                        rows, p.mc.i_loc, tid);
      else
        stage_rows_bf16_groupq(cv.xq, cv.xs, sh, static_cast<const __nv_bfloat16*>(p.act),
                               p.mc.i_loc, rows, p.mc.i_loc, false, tid);
      gather_scales_store<G, ElemE4M3>(sh, cv.sm, wk, cv.sc, tid, held);
      named_bar_sync(1, kConsumerThreads);
      consume<G, ElemE4M3>(sh, cv.sm, cv.ring, cv.xq, cv.xs, cv.sc, wk, scr);
    } else {
      if (early) pdl_wait();
      const int m = p.mc.m, h = p.mc.h;
      __nv_bfloat16* out = p.out;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[G::RT]) {
        if (col >= m) return;
#pragma unroll
        for (int sub = 0; sub < G::RT; ++sub)
          out[static_cast<size_t>(col) * h + id.tile * G::ROWS + sub * 16 + r] =
              __float2bfloat16_rn(val[sub]);
      };
      epilogue<G>(sh, cv.sm, wk, total, grid, cta, scr, emit);
    }
  }
  if (!p.has_tail) {
    stream_drain_on_abort<G>(cv.sm);
    return;
  }
  if (last_cta<G>(cv.sm, scr, gridDim.x)) {
    float* red = reinterpret_cast<float*>(cv.sm->red);
    if (threadIdx.x < kConsumerThreads)
      run_tail(p.tail, reinterpret_cast<__nv_bfloat16*>(cv.ring), red, &cv.sm->is_last_tile,
               BlockBar{2, kConsumerThreads});
  }
  stream_drain_on_abort<G>(cv.sm);
}

}  // namespace iqb

#include "layer_fused.cuh"

namespace iqb {

// ------------------------------------------------------------------------------------
// Host side
static int g_sm_count = 0;
static int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_sm_count = n;
  }
  return g_sm_count;
}

static int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

// One opt-in to the full shared memory per (kernel, device).  Callers are serialised per
// process by the GIL or by their own stream discipline; the table is append-only.
static bool ensure_smem_optin(const void* fn) {
  struct Entry { const void* fn; int dev; };
  static Entry done[256];
  static int n_done = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  for (int i = 0; i < n_done; ++i)
    if (done[i].fn == fn && done[i].dev == dev) return true;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) !=
      cudaSuccess)
    return false;
  if (n_done < 256) done[n_done++] = Entry{fn, dev};
  return true;
}

// Tensor maps of weight matrices viewed as [total_rows, k_bytes / 4] u32, box = (kc / 4)
// x box_rows, no swizzle.  Encoding costs a driver call, so maps are cached by key; a map
// holds only the address and geometry, never data.
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
static std::mutex g_map_mutex;
static std::vector<std::pair<MapKey, CUtensorMap>> g_maps;

static int weight_map(CUtensorMap* out, const void* ptr, long long rows, int k_bytes, int box_rows,
                      int kc) {
  static EncodeTiledFn encode = nullptr;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{ptr, rows, k_bytes, box_rows, kc};
  for (const auto& kv : g_maps)
    if (kv.first == key) { *out = kv.second; return IQ_OK; }
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
  if (g_maps.size() >= 4096) g_maps.clear();
  g_maps.emplace_back(key, m);
  *out = m;
  return IQ_OK;
}

// Fills map0 (and map1 for the shared experts) when the geometry streams K-slices.
template <class G>
static int fill_maps(CUtensorMap* map0, CUtensorMap* map1, const StreamShape& sh, const void* w,
                     long long rows, const void* shared_w, long long shared_rows) {
  if (sh.k_bytes == G::KC && G::NBOX == 1) return IQ_OK;      // whole-row stages: untiled copies
  const int box_rows = sh.pair_half > 0 ? G::ROWS / 2 : G::ROWS;
  int rc = weight_map(map0, w, rows, sh.k_bytes, box_rows, G::BOXK);
  if (rc != IQ_OK) return rc;
  if (shared_w) rc = weight_map(map1, shared_w, shared_rows, sh.k_bytes, box_rows, G::BOXK);
  return rc;
}

template <class Kernel, class Params>
static int launch(Kernel kernel, const Params& p, int grid, size_t smem, void* stream, int pdl,
                  bool cooperative = false) {
  // One opt-in to the full shared memory per kernel and device (this function is
  // instantiated per kernel, so the flags are per kernel).
  if (!ensure_smem_optin(reinterpret_cast<const void*>(kernel))) return IQ_ERR_CUDA;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2] = {};
  int n_attr = 0;
  if (cooperative) {
    attr[n_attr].id = cudaLaunchAttributeCooperative;
    attr[n_attr].val.cooperative = 1;
    ++n_attr;
  }
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

// Most stages one CTA can own, over every group count the routes can produce, under the
// same rule cta_share applies on the device; 0 when the stream has more tiles than the
// scratch has counters.
template <class G>
static int max_items_any(const StreamShape& sh, int max_groups) {
  const int grid = sm_count() > 0 ? sm_count() : 1;
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

// Fills the geometry-dependent part of a shape and returns the dynamic shared memory to
// request, or 0 when the ring does not fit.
// `max_groups` bounds the group count a kernel may derive from the routes.
template <class G>
static size_t plan_smem(StreamShape& sh, size_t tail_bytes, int max_groups = 1) {
  sh.max_items = max_items_any<G>(sh, max_groups);
  if (sh.max_items == 0) return 0;
  const size_t fixed = smem_fixed_bytes<G>(sh);
  if (fixed + 2 * G::STAGE_BYTES > static_cast<size_t>(kSmemLimit)) return 0;
  // Ring depth: a bare copy loop saturates HBM with ~96 KB in flight per SM, but the
  // consumers hold a stage or two while they work on it; measured on the layer's kernels,
  // 160 KB is where more depth stops paying (96 KB: Gate 46 us, 160 KB: 42 us).
  int stages = static_cast<int>((kSmemLimit - fixed) / G::STAGE_BYTES);
  const int want = (160 * 1024 + G::STAGE_BYTES - 1) / G::STAGE_BYTES;
  if (stages > want) stages = want;
  if (stages > kMaxStages) stages = kMaxStages;
  sh.n_stages = stages;
  size_t need = fixed + static_cast<size_t>(stages) * G::STAGE_BYTES;
  if (need < fixed + tail_bytes) need = fixed + tail_bytes;
  return need <= static_cast<size_t>(kSmemLimit) ? need : 0;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_tail(const iq_tail_args* t) {
  if (!t) return IQ_OK;
  if (t->kind != IQ_TAIL_ATTN && t->kind != IQ_TAIL_MLP) return IQ_ERR_ARG;
  if (t->m < 1 || t->m > 8 || t->h < 128 || t->h % 128 || t->h > 8 * kTailVecs * kConsumerThreads)
    return IQ_ERR_ARG;
  if (!t->partial || !t->residual || !t->w_norm || !t->h_out || !t->norm_out) return IQ_ERR_ARG;
  if (t->kind == IQ_TAIL_ATTN && !t->w_first) return IQ_ERR_ARG;
  if (t->world < 1 || t->world > 8 || t->rank < 0 || t->rank >= t->world) return IQ_ERR_ARG;
  if (t->world > 1) {
    if (!t->arrive || !t->epoch) return IQ_ERR_ARG;
    if (!t->arrive_mc && !t->peer_arrive) return IQ_ERR_ARG;
    if (!t->partial_mc && !t->peer_partials) return IQ_ERR_ARG;
  }
  if (!aligned16(t->partial) || !aligned16(t->residual) || !aligned16(t->h_out) ||
      !aligned16(t->norm_out) || !aligned16(t->w_norm))
    return IQ_ERR_ARG;
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
  const size_t tail_bytes = a->tail ? static_cast<size_t>(a->tail->m) * a->tail->h * 2 : 0;
  const size_t smem = plan_smem<G>(sh, tail_bytes);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  const int mrc = fill_maps<G>(&p.map0, &p.map1, sh, a->w, a->n, nullptr, 0);
  if (mrc != IQ_OK) return mrc;
  p.x = a->x;
  p.x_scale = a->x_scale;
  p.x_kind = a->x_kind;
  p.m = a->m;
  p.k = a->k;
  p.n = a->n;
  p.w = static_cast<const uint8_t*>(a->w);
  p.w_scale = a->w_scale;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.scratch = a->scratch;
  p.has_tail = a->tail != nullptr;
  if (a->tail) {
    p.tail = *a->tail;
    if (!p.tail.status) p.tail.status = scratch_of(a->scratch).status;
  }
  return launch(linear_kernel<G>, p, sm_count(), smem, stream, a->pdl);
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
  const size_t smem = 1024 + static_cast<size_t>(a->m) * a->h * 2;
  if (smem > static_cast<size_t>(kSmemLimit)) return IQ_ERR_UNSUPPORTED;
  return launch(tail_kernel, p, 1, smem, stream, pdl);
}

extern "C" int iq_linear(const iq_linear_args* a, void* stream) {
  if (!a || !a->x || !a->w || !a->w_scale || !a->out || !a->scratch) return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBasicBytes) return IQ_ERR_ARG;
  if (a->x_kind < IQ_X_BF16_GROUPQ || a->x_kind > IQ_X_E4M3_UNSCALED) return IQ_ERR_ARG;
  if (a->x_kind == IQ_X_E4M3_GROUP && !a->x_scale) return IQ_ERR_ARG;
  const int max_m = a->x_kind == IQ_X_BF16_SPLIT2 ? 4 : 8;
  if (a->m < 1 || a->m > max_m) return IQ_ERR_ARG;
  if (a->k < 64 || a->k % 64 || a->n < 16 || a->n % 16) return IQ_ERR_ARG;
  if (a->x_kind != IQ_X_E4M3_UNSCALED && a->k % 128) return IQ_ERR_ARG;   // 1x128 groups
  if ((a->rg != 64 && a->rg != 128) || (a->kg != 64 && a->kg != 128)) return IQ_ERR_ARG;
  if (!aligned16(a->x) || !aligned16(a->w) || !aligned16(a->out)) return IQ_ERR_ARG;
  if (a->tail) {
    const int rc = check_tail(a->tail);
    if (rc != IQ_OK) return rc;
    if (a->tail->partial != a->out || a->tail->m != a->m || a->tail->h != a->n) return IQ_ERR_ARG;
  }
  if (sm_count() == 0) return IQ_ERR_CUDA;
  const int k = a->k, n = a->n;
  if (k % 2048 == 0 && n % 16 == 0) return linear_launch<Geo<1, 16, 2>>(a, stream);
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

template <class G>
static int router_launch(const iq_router_args* a, void* stream) {
  RouterParams p{};
  StreamShape& sh = p.sh;
  sh.whole_tiles = 1;
  sh.mode = kRowsPerGroup;
  sh.n_groups = 1;
  sh.rows_per_group = a->e;
  sh.k_bytes = a->h * 2;
  sh.rg_shift = 7;
  sh.kg_shift = 7;
  sh.pair_half = 0;
  sh.x_rows = a->m;
  sh.x_pitch = a->h * 2 + 64;
  sh.x_blocks = 1;
  const size_t smem = plan_smem<G>(sh, 0);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
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
  return launch(router_kernel<G>, p, sm_count(), smem, stream, a->pdl);
}

extern "C" int iq_router(const iq_router_args* a, void* stream) {
  if (!a || !a->x || !a->w || !a->sel || !a->wt || !a->logits || !a->scratch) return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBasicBytes) return IQ_ERR_ARG;
  if (a->m < 1 || a->m > 8 || a->h < 512 || a->h % 512) return IQ_ERR_ARG;
  if (a->e < 16 || a->e % 16 || a->e > 512 || a->top_k < 1 || a->top_k > 32 || a->top_k > a->e)
    return IQ_ERR_ARG;
  if (a->score != IQ_ROUTE_SOFTMAX && a->score != IQ_ROUTE_SIGMOID) return IQ_ERR_ARG;
  if (!aligned16(a->x) || !aligned16(a->w)) return IQ_ERR_ARG;
  if (sm_count() == 0) return IQ_ERR_CUDA;
  if ((a->h * 2) % 2048 == 0) return router_launch<Geo<1, 16, 2>>(a, stream);
  return router_launch<Geo<1, 16, 1>>(a, stream);
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

extern "C" int iq_moe_gate(const iq_moe_gate_args* a, void* stream) {
  if (!a || !a->x_fp8 || !a->fc || !a->fc_scale || !a->act || !a->scratch) return IQ_ERR_ARG;
  if (a->scratch_bytes < kScrBasicBytes) return IQ_ERR_ARG;
  if (a->n_shared > 0 && (!a->shared_fc || !a->shared_fc_scale)) return IQ_ERR_ARG;
  if (a->act_kind != IQ_ACT_E4M3 && a->act_kind != IQ_ACT_BF16) return IQ_ERR_ARG;
  if (a->h < 1024 || a->h % 1024 || a->i_loc < 64 || a->i_loc % 64) return IQ_ERR_ARG;
  if (!aligned16(a->x_fp8) || !aligned16(a->fc)) return IQ_ERR_ARG;
  using G = Geo<2, 8, 2>;
  GateParams p{};
  int rc = fill_moe(p.mc, a->m, a->h, a->i_loc, a->n_experts, a->top_k, a->n_shared, a->sel,
                    nullptr);
  if (rc != IQ_OK) return rc;
  if (sm_count() == 0) return IQ_ERR_CUDA;
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
  bool early = a->pdl >= 2 && a->n_shared > 0;
  if (early) {
    const int grid = sm_count();
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
  const size_t smem = plan_smem<G>(sh, 0, a->m * a->top_k + a->n_shared);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  const int mrc = fill_maps<G>(&p.map0, &p.map1, sh, a->fc,
                               static_cast<long long>(a->n_experts) * 2 * a->i_loc, a->shared_fc,
                               static_cast<long long>(a->n_shared) * 2 * a->i_loc);
  if (mrc != IQ_OK) return mrc;
  p.x_fp8 = static_cast<const uint8_t*>(a->x_fp8);
  p.x_scale = a->x_scale;
  p.act = a->act;
  p.act_kind = a->act_kind;
  p.scratch = a->scratch;
  p.pdl_level = a->pdl;
  return launch(gate_kernel<G>, p, sm_count(), smem, stream, a->pdl);
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
  const size_t tail_bytes = a->tail ? static_cast<size_t>(a->tail->m) * a->tail->h * 2 : 0;
  const size_t smem = plan_smem<G>(sh, tail_bytes, a->m * a->top_k + a->n_shared);
  if (smem == 0) return IQ_ERR_UNSUPPORTED;
  const int mrc = fill_maps<G>(&p.map0, &p.map1, sh, a->proj,
                               static_cast<long long>(a->n_experts) * a->h, a->shared_proj,
                               static_cast<long long>(a->n_shared) * a->h);
  if (mrc != IQ_OK) return mrc;
  p.act = a->act;
  p.act_kind = a->act_kind;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.scratch = a->scratch;
  p.has_tail = a->tail != nullptr;
  p.pdl_level = a->pdl;
  if (a->tail) {
    p.tail = *a->tail;
    if (!p.tail.status) p.tail.status = scratch_of(a->scratch).status;
  }
  return launch(down_kernel<G>, p, sm_count(), smem, stream, a->pdl);
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
  // k = 1024: 32 rows x 1 KB stages (two 64-byte runs per warp) measured 5 % faster than
  // 16 rows x 1 KB; at k = 512 the wider tile (64 rows) measured slower and is not used.
  if (k % 2048 == 0) return down_launch<Geo<1, 16, 2>>(a, stream);
  if (k % 1024 == 0 && a->h % 32 == 0) return down_launch<Geo<2, 8, 2>>(a, stream);
  if (k % 1024 == 0) return down_launch<Geo<1, 16, 1>>(a, stream);
  if (k % 512 == 0 && a->h % 32 == 0) return down_launch<Geo<2, 8, 1>>(a, stream);
  if (k % 256 == 0 && a->h % 64 == 0) return down_launch<Geo<4, 4, 1>>(a, stream);
  if (k % 192 == 0 && a->h % 256 == 0) return down_launch<Geo<16, 1, 3>>(a, stream);
  if (k % 128 == 0 && a->h % 128 == 0) return down_launch<Geo<8, 2, 1>>(a, stream);
  return IQ_ERR_UNSUPPORTED;
}

namespace iqb {

// ------------------------------------------------------------------------------------
// iq_decode_layer: the four streams in one cooperative launch.
static void shape_linear(StreamShape& sh, const iq_linear_args* a) {
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
}
static void shape_router(StreamShape& sh, const iq_router_args* a) {
  sh.whole_tiles = 1;
  sh.mode = kRowsPerGroup;
  sh.n_groups = 1;
  sh.rows_per_group = a->e;
  sh.k_bytes = a->h * 2;
  sh.rg_shift = 7;
  sh.kg_shift = 7;
  sh.pair_half = 0;
  sh.x_rows = a->m;
  sh.x_pitch = a->h * 2 + 64;
  sh.x_blocks = 1;
}
static void shape_gate(StreamShape& sh, const iq_moe_gate_args* a) {
  sh.mode = kRowsPerGroup;
  sh.n_groups = 1;
  sh.rows_per_group = 2 * a->i_loc;
  sh.k_bytes = a->h;
  sh.rg_shift = 6;
  sh.kg_shift = 7;
  sh.pair_half = a->i_loc;
  sh.x_rows = a->m;
  sh.x_pitch = a->h + 64;
  sh.x_blocks = a->h / 128;
}
static void shape_down(StreamShape& sh, const iq_moe_down_args* a) {
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
}

template <class G>
static int max_items_of(const StreamShape& sh, int max_groups) {
  return max_items_any<G>(sh, max_groups);
}

static void fill_moe_gate(MoeCommon& mc, const iq_moe_gate_args* a) {
  mc.w = static_cast<const uint8_t*>(a->fc);
  mc.w_scale = a->fc_scale;
  mc.shared_w = static_cast<const uint8_t*>(a->shared_fc);
  mc.shared_scale = a->shared_fc_scale;
  mc.w_stride = static_cast<size_t>(2) * a->i_loc * a->h;
  mc.scale_stride = static_cast<size_t>(2 * a->i_loc / 64) * (a->h / 128);
  mc.rows_per_expert = 2 * a->i_loc;
}
static void fill_moe_down(MoeCommon& mc, const iq_moe_down_args* a) {
  mc.w = static_cast<const uint8_t*>(a->proj);
  mc.w_scale = a->proj_scale;
  mc.shared_w = static_cast<const uint8_t*>(a->shared_proj);
  mc.shared_scale = a->shared_proj_scale;
  mc.w_stride = static_cast<size_t>(a->h) * a->i_loc;
  mc.scale_stride = static_cast<size_t>(a->h / 128) * (a->i_loc / 64);
  mc.rows_per_expert = a->h;
}

template <class GO, class GD>
static int layer_launch(const iq_decode_layer_args* a, void* stream, int pdl) {
  using GR = Geo<1, 16, 2>;
  using GG = Geo<2, 8, 2>;
  const iq_linear_args& o = a->oproj;
  const iq_router_args& r = a->router;
  const iq_moe_gate_args& g = a->gate;
  const iq_moe_down_args& d = a->down;
  LayerParams p{};
  shape_linear(p.sh_o, &o);
  shape_router(p.sh_r, &r);
  shape_gate(p.sh_g, &g);
  shape_down(p.sh_d, &d);
  const int max_groups = g.m * g.top_k + g.n_shared;
  p.sh_o.max_items = max_items_of<GO>(p.sh_o, 1);
  p.sh_r.max_items = max_items_of<GR>(p.sh_r, 1);
  p.sh_g.max_items = max_items_of<GG>(p.sh_g, max_groups);
  p.sh_d.max_items = max_items_of<GD>(p.sh_d, max_groups);
  if (!p.sh_o.max_items || !p.sh_r.max_items || !p.sh_g.max_items || !p.sh_d.max_items)
    return IQ_ERR_UNSUPPORTED;
  // Shared memory: the fixed structures, then one scale table, one activation-scale table
  // and one activation area, each sized for the stream that needs most, then the ring.
  auto maxz = [](size_t x, size_t y) { return x > y ? x : y; };
  size_t sc = static_cast<size_t>(p.sh_o.max_items) * GO::SCALES_PER_STAGE;
  sc = maxz(sc, static_cast<size_t>(p.sh_g.max_items) * GG::SCALES_PER_STAGE);
  sc = maxz(sc, static_cast<size_t>(p.sh_d.max_items) * GD::SCALES_PER_STAGE);
  // Activation rows: o_proj's, then the router's with the Gate's beside them (both are
  // written by the attention tail), then the Down's; each set overlays the one before.
  const size_t xq_router = align_up(static_cast<size_t>(p.sh_r.x_rows) * p.sh_r.x_pitch, 16);
  size_t xs = 0, xq = xq_router + static_cast<size_t>(p.sh_g.x_rows) * p.sh_g.x_pitch;
  for (const StreamShape* sh : {&p.sh_o, &p.sh_g, &p.sh_d}) {
    xs = maxz(xs, static_cast<size_t>(sh->x_rows) * sh->x_blocks);
    xq = maxz(xq, static_cast<size_t>(sh->x_rows) * sh->x_pitch);
  }
  size_t off = align_up(sizeof(StreamSmem<GO>), 16);
  p.off_extra = static_cast<uint32_t>(off);
  off += align_up(sizeof(LayerSmemExtra), 16);
  p.off_sc = static_cast<uint32_t>(off);
  off += align_up(sizeof(float) * sc, 16);
  p.off_xs = static_cast<uint32_t>(off);
  off += align_up(sizeof(float) * xs, 16);
  p.off_xq = static_cast<uint32_t>(off);
  p.off_xq_gate = static_cast<uint32_t>(off + xq_router);
  off += align_up(xq, 16);
  off = align_up(off, 128);
  p.off_ring = static_cast<uint32_t>(off);
  int slot_bytes = GO::STAGE_BYTES;
  for (int b : {GR::STAGE_BYTES, GG::STAGE_BYTES, GD::STAGE_BYTES})
    if (b > slot_bytes) slot_bytes = b;
  p.slot_bytes = slot_bytes;
  int slots = static_cast<int>((static_cast<size_t>(kSmemLimit) - off) / slot_bytes);
  if (off + 2 * static_cast<size_t>(slot_bytes) > static_cast<size_t>(kSmemLimit)) return IQ_ERR_UNSUPPORTED;
  const int want = (160 * 1024 + slot_bytes - 1) / slot_bytes;
  if (slots > want) slots = want;
  if (slots > kMaxStages) slots = kMaxStages;
  p.sh_o.n_stages = p.sh_r.n_stages = p.sh_g.n_stages = p.sh_d.n_stages = slots;
  const size_t smem = off + static_cast<size_t>(slots) * slot_bytes;

  CUtensorMap unused;
  int rc = fill_maps<GO>(&p.map_o, &unused, p.sh_o, o.w, o.n, nullptr, 0);
  if (rc == IQ_OK) rc = fill_maps<GR>(&p.map_r, &unused, p.sh_r, r.w, r.e, nullptr, 0);
  if (rc == IQ_OK)
    rc = fill_maps<GG>(&p.map_g0, &p.map_g1, p.sh_g, g.fc,
                       static_cast<long long>(g.n_experts) * 2 * g.i_loc, g.shared_fc,
                       static_cast<long long>(g.n_shared) * 2 * g.i_loc);
  if (rc == IQ_OK)
    rc = fill_maps<GD>(&p.map_d0, &p.map_d1, p.sh_d, d.proj,
                       static_cast<long long>(d.n_experts) * d.h, d.shared_proj,
                       static_cast<long long>(d.n_shared) * d.h);
  if (rc != IQ_OK) return rc;

  p.x = o.x;
  p.x_scale = o.x_scale;
  p.x_kind = o.x_kind;
  p.m = o.m;
  p.k_o = o.k;
  p.h = o.n;
  p.w_o = static_cast<const uint8_t*>(o.w);
  p.w_o_scale = o.w_scale;
  p.out_o = static_cast<__nv_bfloat16*>(o.out);
  p.tail_a = *o.tail;
  p.w_r = static_cast<const uint8_t*>(r.w);
  p.e = r.e;
  p.top_k = r.top_k;
  p.score = r.score;
  p.sel = r.sel;
  p.wt = r.wt;
  p.logits = r.logits;
  rc = fill_moe(p.mc_g, g.m, g.h, g.i_loc, g.n_experts, g.top_k, g.n_shared, g.sel, nullptr);
  if (rc == IQ_OK)
    rc = fill_moe(p.mc_d, d.m, d.h, d.i_loc, d.n_experts, d.top_k, d.n_shared, d.sel, d.wt);
  if (rc != IQ_OK) return rc;
  fill_moe_gate(p.mc_g, &g);
  fill_moe_down(p.mc_d, &d);
  p.act = g.act;
  p.act_kind = g.act_kind;
  p.out_d = static_cast<__nv_bfloat16*>(d.out);
  p.tail_m = *d.tail;
  p.scratch = o.scratch;
  int* status = scratch_of(o.scratch).status;
  if (!p.tail_a.status) p.tail_a.status = status;
  if (!p.tail_m.status) p.tail_m.status = status;
  unsigned peer_ms = p.tail_a.timeout_ms ? p.tail_a.timeout_ms : 2000u;
  const unsigned peer_ms_m = p.tail_m.timeout_ms ? p.tail_m.timeout_ms : 2000u;
  if (peer_ms_m > peer_ms) peer_ms = peer_ms_m;
  p.wait_ms = peer_ms + 500u;

  auto kernel = layer_kernel<GO, GD>;
  if (!ensure_smem_optin(reinterpret_cast<const void*>(kernel))) return IQ_ERR_CUDA;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem) != cudaSuccess ||
      per_sm < 1) {
    fprintf(stderr, "iqb200: iq_decode_layer needs one resident CTA per SM (%zu B shared)\n", smem);
    return IQ_ERR_UNSUPPORTED;
  }
  return launch(kernel, p, sm_count(), smem, stream, pdl, true);
}

}  // namespace iqb

using namespace iqb;

extern "C" int iq_decode_layer(const iq_decode_layer_args* a, void* stream, int pdl) {
  if (!a) return IQ_ERR_ARG;
  const iq_linear_args& o = a->oproj;
  const iq_router_args& r = a->router;
  const iq_moe_gate_args& g = a->gate;
  const iq_moe_down_args& d = a->down;
  // ---- each part as its own entry point would check it
  if (!o.x || !o.w || !o.w_scale || !o.out || !o.scratch || !o.tail || !d.tail) return IQ_ERR_ARG;
  if (o.scratch_bytes < kScrBytes) return IQ_ERR_ARG;
  if (r.scratch != o.scratch || g.scratch != o.scratch || d.scratch != o.scratch) return IQ_ERR_ARG;
  if (o.x_kind < IQ_X_BF16_GROUPQ || o.x_kind > IQ_X_E4M3_UNSCALED) return IQ_ERR_ARG;
  if (o.x_kind == IQ_X_E4M3_GROUP && !o.x_scale) return IQ_ERR_ARG;
  const int max_m = o.x_kind == IQ_X_BF16_SPLIT2 ? 4 : 8;
  if (o.m < 1 || o.m > max_m) return IQ_ERR_ARG;
  if ((o.rg != 64 && o.rg != 128) || (o.kg != 64 && o.kg != 128)) return IQ_ERR_ARG;
  if (o.k < 1024 || o.k % 1024 || o.n < 1024 || o.n % 1024) return IQ_ERR_UNSUPPORTED;
  if (!aligned16(o.x) || !aligned16(o.w) || !aligned16(o.out)) return IQ_ERR_ARG;
  if (!r.x || !r.w || !r.sel || !r.wt || !r.logits) return IQ_ERR_ARG;
  if (r.e < 16 || r.e % 16 || r.e > 512 || r.top_k < 1 || r.top_k > 32 || r.top_k > r.e)
    return IQ_ERR_ARG;
  if (r.score != IQ_ROUTE_SOFTMAX && r.score != IQ_ROUTE_SIGMOID) return IQ_ERR_ARG;
  if (!aligned16(r.x) || !aligned16(r.w)) return IQ_ERR_ARG;
  if (!g.x_fp8 || !g.fc || !g.fc_scale || !g.act || !g.sel) return IQ_ERR_ARG;
  if (g.n_shared > 0 && (!g.shared_fc || !g.shared_fc_scale)) return IQ_ERR_ARG;
  if (g.act_kind != IQ_ACT_E4M3 && g.act_kind != IQ_ACT_BF16) return IQ_ERR_ARG;
  if (!aligned16(g.x_fp8) || !aligned16(g.fc)) return IQ_ERR_ARG;
  if (!d.act || !d.proj || !d.proj_scale || !d.out || !d.wt || !d.sel) return IQ_ERR_ARG;
  if (d.n_shared > 0 && (!d.shared_proj || !d.shared_proj_scale)) return IQ_ERR_ARG;
  if (!aligned16(d.act) || !aligned16(d.proj) || !aligned16(d.out)) return IQ_ERR_ARG;
  // ---- the four parts describe one layer
  const int m = o.m, h = o.n;
  if (r.m != m || g.m != m || d.m != m) return IQ_ERR_ARG;
  if (r.h != h || g.h != h || d.h != h) return IQ_ERR_ARG;
  if (g.i_loc != d.i_loc || g.top_k != d.top_k || g.n_shared != d.n_shared ||
      g.n_experts != d.n_experts || g.act_kind != d.act_kind)
    return IQ_ERR_ARG;
  if (r.top_k != g.top_k || r.e != g.n_experts) return IQ_ERR_ARG;
  // ---- what one part writes is what the next one reads
  if (r.x != o.tail->norm_out || g.x_fp8 != o.tail->norm_fp8 || g.x_scale != o.tail->norm_fp8_scale)
    return IQ_ERR_ARG;
  if (g.sel != r.sel || d.sel != r.sel || d.wt != r.wt || d.act != g.act) return IQ_ERR_ARG;
  if (g.i_loc < 256 || g.i_loc % 256) return IQ_ERR_UNSUPPORTED;
  int rc = check_tail(o.tail);
  if (rc == IQ_OK) rc = check_tail(d.tail);
  if (rc != IQ_OK) return rc;
  if (o.tail->kind != IQ_TAIL_ATTN || d.tail->kind != IQ_TAIL_MLP) return IQ_ERR_ARG;
  if (o.tail->partial != o.out || o.tail->m != m || o.tail->h != h) return IQ_ERR_ARG;
  if (d.tail->partial != d.out || d.tail->m != m || d.tail->h != h) return IQ_ERR_ARG;
  if (h > kLayerMaxH) return IQ_ERR_UNSUPPORTED;
  if (o.tail->timeout_ms > 3000u || d.tail->timeout_ms > 3000u) return IQ_ERR_ARG;
  if (sm_count() == 0) return IQ_ERR_CUDA;
  const bool o2 = o.k % 2048 == 0;
  const int i = g.i_loc;
  using Geo2048 = Geo<1, 16, 2>;
  using Geo1024 = Geo<1, 16, 1>;
  using Geo512 = Geo<2, 8, 1>;
  using Geo256 = Geo<4, 4, 1>;
#define IQ_LAYER_DISPATCH(GD)                                                   \
  return o2 ? layer_launch<Geo<1, 16, 2>, GD>(a, stream, pdl)                   \
            : layer_launch<Geo<1, 16, 1>, GD>(a, stream, pdl)
  if (i % 2048 == 0) { IQ_LAYER_DISPATCH(Geo2048); }
  if (i % 1024 == 0) { IQ_LAYER_DISPATCH(Geo1024); }
  if (i % 512 == 0) { IQ_LAYER_DISPATCH(Geo512); }
  IQ_LAYER_DISPATCH(Geo256);
#undef IQ_LAYER_DISPATCH
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
static void* g_static_ptr[64] = {};

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
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return IQ_ERR_CUDA;
  if (!g_static_ptr[dev]) {
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
  // The array keeps whatever the last call left.  The kernel expects the status word,
  // the ticket and the tile counters at zero; the partial-sum area is written before it
  // is read and needs no clearing.
  if (cudaMemsetAsync(g_static_ptr[dev], 0, kScrPartials, static_cast<cudaStream_t>(stream)) !=
      cudaSuccess)
    return IQ_ERR_CUDA;
  iq_linear_args b = *a;
  b.scratch = g_static_ptr[dev];
  b.scratch_bytes = kScrBasicBytes;
  return iq_linear(&b, stream);
}
