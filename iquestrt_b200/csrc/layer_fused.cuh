// The whole decode layer of the path in ONE launch (included by kernels.cu).
//
//   o_proj stream -> attention all-reduce tail -> router stream -> top-k
//   -> expert Gate/Up stream -> expert Down stream -> MLP all-reduce tail
//
// Four weight streams run back to back through one shared-memory ring.  The producer warp
// never waits for the steps between them: while the attention tail is computed, every
// CTA's ring is already filling with router weights; while the Gate's last tiles are
// reduced, the Down's first stages are landing.
//
// What separates two streams is a grid-wide hand-off, and its cost is the number of
// dependent global-memory round trips in it (each is about a microsecond on this part),
// not arithmetic.  So:
//
//   * Results that other CTAs consume inside the launch travel as self-validating words:
//     the value and the tag of this launch in one aligned scalar store.  The writer needs
//     no fence, no counter and no flag; a reader simply re-reads a word until it carries
//     this launch's tag.  The o_proj and Down rows (bf16 + 16-bit tag), the router logits
//     and the fp32 partials of tiles split between CTAs (32 bits + 32-bit tag) go this
//     way.  The Gate's activations are larger (every CTA reads all of them), so they keep
//     a counter: one fence and one release-add per CTA, one poll per reader.
//   * The steps between the streams are not given to one CTA whose result the others
//     then wait for and fetch: EVERY CTA reads the complete rows from L2 and computes the
//     step itself (residual add and RMSNorms of the tails, top-k of the router).  The
//     arithmetic is a few thousand elements, and the results land directly in the CTA's
//     shared memory as the next stream's activations.  Each CTA writes only its 1/148
//     share of the results that must also exist in global memory.
//
// With tensor parallelism the rows must first be summed over the ranks, and that cannot be
// done 148 times (every copy would cross NVLink): CTA 0 collects the local rows, stores
// them into the symmetric buffer, runs the cross-rank hand-shake and the multimem (or
// peer-load) reduction, and publishes the reduced rows as tagged words in local memory,
// which is what the other CTAs' tails read.
//
// CTAs of this launch wait on one another, so the launch is cooperative (all CTAs are
// resident together, one per SM).  Every wait is bounded: a wait that runs out records
// IQ_ERR_PIPE_TIMEOUT (or IQ_ERR_PEER_TIMEOUT), raises the CTA's abort flag, and every role
// then skips its remaining work but still walks through all the CTA-level barriers, so
// the CTA always exits.
//
// The numerics are those of the four separate kernels: the same item split, the same
// accumulation order, the same rounding points in the tails, so the outputs are
// bit-identical to the four-launch layer.
#pragma once

namespace iqb {

// Hand-off words of the one-launch layer inside the scratch.
constexpr size_t kScrEpoch = 96;     // completed one-launch layers on this scratch (never reset)
constexpr size_t kScrExit = 104;     // CTAs that have finished; the last one closes the launch
constexpr size_t kScrCntG = 192;     // CTAs whose Gate tiles are all emitted
// Tagged words, in the layer's own area behind the basic scratch.
constexpr size_t kScrLayer = kScrBasicBytes;
constexpr size_t kScrParts = kScrLayer;                        // u64 [256][2][512] split-tile partials
constexpr size_t kScrRowsO = kScrLayer + 2 * 1024 * 1024;      // u32 [8][8192] o_proj rows
constexpr size_t kScrRowsD = kScrRowsO + 256 * 1024;           // u32 [8][8192] Down rows
constexpr size_t kScrRowsA = kScrRowsD + 256 * 1024;           // u32: attention rows summed over ranks
constexpr size_t kScrRowsM = kScrRowsA + 256 * 1024;           // u32: MLP rows summed over ranks
constexpr size_t kScrLogits = kScrRowsM + 256 * 1024;          // u64 [8][512] router logits
static_assert(kScrLogits + 8 * 512 * 8 <= kScrBytes - 65536, "layer area fits below the trace area");
constexpr int kLayerMaxH = 8192;
constexpr int kLayerMaxTileRows = 64;   // rows of the largest tile geometry the layer uses

__device__ __forceinline__ uint32_t tag16_of(uint32_t epoch) { return epoch % 65535u + 1u; }
// The split-tile partials of the four streams share one area, so their tag also names the
// stream (0..3): a word left by an earlier stream of the same launch is not valid for a
// later one.
__device__ __forceinline__ uint32_t tag32_of(uint32_t epoch, uint32_t stream) {
  return epoch * 4u + stream + 1u;
}

constexpr int kBarConsumers = 1;      // the 16 consumer warps
constexpr int kBarHelpers = 2;        // the same warps inside tail / table helpers
constexpr int kBarTables = 4;         // all warps: the Gate/Down group tables are ready

struct LayerSmemExtra {
  GroupDesc g_oproj;
  GroupDesc g_router;
  GroupDesc g_down[kMaxGroups];
  int n_groups;
  int flag;            // broadcast word of the consumer warps
  int pad[2];
  int sel[64];         // this CTA's copy of the routes
  float wt[64];
};

struct LayerParams {
  CUtensorMap map_o, map_r, map_g0, map_g1, map_d0, map_d1;
  StreamShape sh_o, sh_r, sh_g, sh_d;
  // o_proj + attention tail
  const void* x;
  const float* x_scale;
  int x_kind, m, k_o, h;
  const uint8_t* w_o;
  const float* w_o_scale;
  __nv_bfloat16* out_o;
  iq_tail_args tail_a;
  // router
  const uint8_t* w_r;
  int e, top_k, score;
  int* sel;
  float* wt;
  float* logits;
  // experts
  MoeCommon mc_g, mc_d;
  void* act;
  int act_kind;
  __nv_bfloat16* out_d;
  iq_tail_args tail_m;
  void* scratch;
  int slot_bytes;          // ring slot pitch (the largest stage of the four streams)
  uint32_t off_extra, off_sc, off_xs, off_xq, off_xq_gate, off_ring;   // shared-memory layout
  uint32_t wait_ms;        // budget of the grid-wide hand-offs
};

// One thread: spins until *word >= target.  False when the budget runs out or the CTA
// has aborted.
__device__ inline bool poll_word(const uint32_t* word, uint32_t target, uint32_t budget_ms,
                                 const volatile int* abort) {
  if (*abort) return false;
  const uint64_t budget = 1000000ull * budget_ms;
  uint64_t t0 = 0;
#pragma unroll 1
  for (uint32_t spin = 0;; ++spin) {
    if (ld_acquire_gpu_u32(word) >= target) return true;
    if ((spin & 127u) == 127u) {
      if (*abort) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget) return false;
    }
  }
}

// Epilogue warp, after its last tile of a stream: counts the CTA in.
__device__ __forceinline__ void count_in(uint32_t* counter) {
  __threadfence();
  __syncwarp();
  if ((threadIdx.x & 31) == 0)
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(counter), "r"(1u) : "memory");
}

// Consumer warps: wait until `*word >= target`; ends with the consumer warps in step and
// everything written before the word was raised visible to L2-level loads.
template <class S>
__device__ __forceinline__ void wait_word(S* sm, const uint32_t* word, uint32_t target,
                                          uint32_t budget_ms, int* status) {
  if (threadIdx.x == 0 && !poll_word(word, target, budget_ms, &sm->abort_flag)) {
    if (!sm->abort_flag) set_status(status, IQ_ERR_PIPE_TIMEOUT);
    sm->abort_flag = 1;
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

// Eight consecutive tagged row words (bf16 value | tag << 16) -> eight floats.  Re-reads
// until all eight carry `tag`; false (with the CTA's abort flag raised) when that does not
// happen within `budget_ms`.
template <class S>
__device__ __forceinline__ bool poll_row_vec(S* sm, const uint32_t* src, uint32_t tag,
                                             uint32_t budget_ms, int* status, uint32_t (&w)[8]) {
  uint64_t t0 = 0;
#pragma unroll 1
  for (uint32_t spin = 0;; ++spin) {
    uint32_t a[4], b[4];
    ld_relaxed_gpu_u32x4(src, a);
    ld_relaxed_gpu_u32x4(src + 4, b);
    bool ok = true;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ok = ok && (a[j] >> 16) == tag && (b[j] >> 16) == tag;
      w[j] = a[j];
      w[4 + j] = b[j];
    }
    if (ok) return true;
    if ((spin & 63u) == 63u) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (sm->abort_flag || now - t0 > 1000000ull * budget_ms) {
        if (!sm->abort_flag) set_status(status, IQ_ERR_PIPE_TIMEOUT);
        sm->abort_flag = 1;
        return false;
      }
    }
  }
}

// CTA 0, consumer warps, TP > 1.  Collects this rank's rows from their tagged words
// (`local`), stores them as plain bf16 into the symmetric buffer the peers read, runs the
// cross-rank hand-shake of `a` (see run_tail), sums the rows over the ranks and publishes
// the sums as tagged words in `reduced` (local memory).  When the peers do not arrive the
// status is IQ_ERR_PEER_TIMEOUT and nothing is published.
template <class S>
__device__ __forceinline__ void reduce_rows_over_ranks(S* sm, LayerSmemExtra* ex,
                                                       const iq_tail_args& a, const uint32_t* local,
                                                       uint32_t* reduced, uint32_t tag,
                                                       uint32_t budget_ms) {
  const int tid = threadIdx.x;
  const int nvec = a.m * (a.h / 8);
  __nv_bfloat16* mine = const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(a.partial));
  for (int v = tid; v < nvec; v += kConsumerThreads) {
    uint32_t w[8];
    if (!poll_row_vec(sm, local + static_cast<size_t>(v) * 8, tag, budget_ms, a.status, w)) break;
    uint4 packed;
    packed.x = (w[0] & 0xffffu) | (w[1] << 16);
    packed.y = (w[2] & 0xffffu) | (w[3] << 16);
    packed.z = (w[4] & 0xffffu) | (w[5] << 16);
    packed.w = (w[6] & 0xffffu) | (w[7] << 16);
    *reinterpret_cast<uint4*>(mine + static_cast<size_t>(v) * 8) = packed;
  }
  __threadfence_system();
  named_bar_sync(kBarConsumers, kConsumerThreads);
  if (tid == 0) {
    int ok = sm->abort_flag ? 0 : 1;
    if (ok) {
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
      for (uint32_t spin = 0;; ++spin) {
        if (static_cast<int32_t>(ld_acquire_sys_u32(a.arrive) - target) >= 0) break;
        if ((spin & 255u) == 255u) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > budget) { ok = 0; break; }
        }
      }
      if (!ok) {
        set_status(a.status, IQ_ERR_PEER_TIMEOUT);
        sm->abort_flag = 1;
      }
      *a.epoch = *a.epoch + 1u;
    }
    ex->flag = ok;
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
  if (!ex->flag) return;
  for (int v = tid; v < nvec; v += kConsumerThreads) {
    const size_t off = static_cast<size_t>(v) * 8;
    U4 part;
    if (a.partial_mc) {
      part = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(a.partial_mc) + off);
    } else {
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
    const uint32_t hi = tag << 16;
    const uint32_t pk[4] = {part.x, part.y, part.z, part.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      st_relaxed_gpu_u32(reduced + off + 2 * j, hi | (pk[j] & 0xffffu));
      st_relaxed_gpu_u32(reduced + off + 2 * j + 1, hi | (pk[j] >> 16));
    }
  }
}

// Where a tail's results go besides global memory: the next streams' activation rows in
// this CTA's shared memory (null = none).
struct TailSinks {
  uint8_t* x_bf16 = nullptr;   // normalised rows as bf16, row pitch `pitch_bf16` bytes
  int pitch_bf16 = 0;
  uint8_t* x_fp8 = nullptr;    // the same rows as e4m3, row pitch `pitch_fp8` bytes
  int pitch_fp8 = 0;
  float* x_fp8_scale = nullptr;   // their 1x128 scales (or 1), `blocks` entries per row
  int blocks = 0;
};

// The tail of `a` on rows that are already summed over the ranks (`rows`, bf16 [m,h] in
// global memory), run by the sixteen consumer warps of EVERY CTA.  Same arithmetic and
// rounding points as run_tail.  Each CTA stores to global memory only the 16-byte vectors
// v with v % n_cta == cta; all of the normalised row goes to `sinks`.
// What a tail needs besides the rows themselves, for one row.  All of it is requested in
// one go together with the row, so the whole tail pays ONE global round trip (a dependent
// global load costs about a microsecond here) instead of one per operand.
struct TailOperands {
  uint4 res_raw[kTailVecs][2];   // residual, still packed
  float w1[kTailVecs][8];        // w_first (attention tail only)
  float w2[kTailVecs][8];        // w_norm
};

__device__ __forceinline__ void tail_fetch_operands(const iq_tail_args& a, int r, TailOperands& op) {
  const int tid = threadIdx.x, vec_per_row = a.h / 8;
#pragma unroll
  for (int i = 0; i < kTailVecs; ++i) {
    const int v = tid + i * kConsumerThreads;
    if (v >= vec_per_row) continue;
    const size_t off = static_cast<size_t>(r) * a.h + static_cast<size_t>(v) * 8;
    if (a.residual_fp32) {
      const float* rp = static_cast<const float*>(a.residual) + off;
      op.res_raw[i][0] = __ldcg(reinterpret_cast<const uint4*>(rp));
      op.res_raw[i][1] = __ldcg(reinterpret_cast<const uint4*>(rp + 4));
    } else {
      op.res_raw[i][0] = __ldcg(
          reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.residual) + off));
    }
    if (a.kind == IQ_TAIL_ATTN) ldg_f32x8(a.w_first + v * 8, op.w1[i]);
    ldg_f32x8(a.w_norm + v * 8, op.w2[i]);
  }
}

// The tail of `a` on rows that are already summed over the ranks (`rows`, tagged words
// [m][h]), run by the sixteen consumer warps of EVERY CTA.  Same arithmetic and rounding
// points as run_tail.  Each CTA stores to global memory only the 16-byte vectors v with
// v % n_cta == cta; all of the normalised row goes to `sinks`.
template <class S>
__device__ __forceinline__ void tail_everywhere(S* sm, const iq_tail_args& a, const uint32_t* rows,
                                                uint32_t tag, uint32_t budget_ms, float* red,
                                                const TailSinks& sinks, int cta, int n_cta) {
  TailOperands op;
  const BlockBar bar{kBarHelpers, kConsumerThreads};
  const int tid = threadIdx.x, nthr = kConsumerThreads;
  const int m = a.m, h = a.h, vec_per_row = h / 8;
  const float inv_h = 1.0f / static_cast<float>(h);
  const bool attn = a.kind == IQ_TAIL_ATTN;

  for (int r = 0; r < m; ++r) {
    const size_t row_off = static_cast<size_t>(r) * h;
    float* slots0 = red + (r & 1) * 64;
    float* slots1 = slots0 + 32;
    // the operands are requested first and land while the row's words are awaited
    tail_fetch_operands(a, r, op);
    float f[kTailVecs][8];
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      uint32_t w[8];
      poll_row_vec(sm, rows + row_off + static_cast<size_t>(v) * 8, tag, budget_ms, a.status, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[i][j] = __uint_as_float(w[j] << 16);
    }
    float inv1 = 0.f;
    if (attn) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kTailVecs; ++i) {
        if (tid + i * nthr >= vec_per_row) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[i][j], f[i][j], ss);
      }
      inv1 = rsqrtf(block_sum(ss, slots0, bar) * inv_h + a.eps);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      if (v >= vec_per_row) continue;
      const size_t off = row_off + static_cast<size_t>(v) * 8;
      const bool mine = (v % n_cta) == cta;
      float res[8];
      if (a.residual_fp32) {
        const float* r0 = reinterpret_cast<const float*>(&op.res_raw[i][0]);
        const float* r1 = reinterpret_cast<const float*>(&op.res_raw[i][1]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { res[j] = r0[j]; res[4 + j] = r1[j]; }
      } else {
        bf16x8_to_f32(U4{op.res_raw[i][0].x, op.res_raw[i][0].y, op.res_raw[i][0].z,
                         op.res_raw[i][0].w}, res);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float add;
        if (attn) {
          const float nrm = bf16_round(op.w1[i][j] * (f[i][j] * inv1));
          add = bf16_round(nrm * a.scale);
        } else {
          add = bf16_round(f[i][j] * a.scale);
        }
        f[i][j] = res[j] + add;                 // f now holds h
      }
      if (a.residual_fp32) {
        if (mine) {
          float* ho = static_cast<float*>(a.h_out) + off;
          *reinterpret_cast<float4*>(ho) = make_float4(f[i][0], f[i][1], f[i][2], f[i][3]);
          *reinterpret_cast<float4*>(ho + 4) = make_float4(f[i][4], f[i][5], f[i][6], f[i][7]);
        }
      } else {
        const U4 hb = f32_to_bf16x8(f[i]);
        if (mine) *reinterpret_cast<U4*>(static_cast<__nv_bfloat16*>(a.h_out) + off) = hb;
        bf16x8_to_f32(hb, f[i]);            // the norm sees the rounded stream
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss2 = fmaf(f[i][j], f[i][j], ss2);
    }
    const float inv2 = rsqrtf(block_sum(ss2, slots1, bar) * inv_h + a.eps);
    if (a.inv_out && tid == 0 && cta == 0) a.inv_out[r] = inv2;

#pragma unroll
    for (int i = 0; i < kTailVecs; ++i) {
      const int v = tid + i * nthr;
      const bool live = v < vec_per_row;       // uniform over each 16-lane group
      const int vv = live ? v : 0;
      const size_t off = row_off + static_cast<size_t>(vv) * 8;
      const bool mine = live && (vv % n_cta) == cta;
      float o[8];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = live ? bf16_round(op.w2[i][j] * (f[i][j] * inv2)) : 0.f;
        amax = fmaxf(amax, fabsf(o[j]));
      }
      const U4 ob = f32_to_bf16x8(o);
      if (mine) *reinterpret_cast<U4*>(static_cast<__nv_bfloat16*>(a.norm_out) + off) = ob;
      if (live && sinks.x_bf16)
        *reinterpret_cast<U4*>(sinks.x_bf16 + r * sinks.pitch_bf16 + vv * 16) = ob;
      if (a.norm_fp8) {
        float sc = 1.0f;
        if (a.norm_fp8_scale) {
#pragma unroll
          for (int o2 = 8; o2; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
          sc = amax > 0.f ? amax / 448.0f : 1.0f;
          // one CTA writes a whole group's scale: the one that owns the group's first vector
          if (mine && (vv & 15) == 0)
            a.norm_fp8_scale[static_cast<size_t>(r) * (h / 128) + (vv >> 4)] = sc;
        }
        if (live && sinks.x_fp8_scale && (vv & 15) == 0)
          sinks.x_fp8_scale[r * sinks.blocks + (vv >> 4)] = sc;
        const float rcp = 1.0f / sc;
        uint32_t q0 = 0, q1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q0 |= static_cast<uint32_t>(f32_to_e4m3_sat(o[j] * rcp)) << (8 * j);
          q1 |= static_cast<uint32_t>(f32_to_e4m3_sat(o[j + 4] * rcp)) << (8 * j);
        }
        if (mine) *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.norm_fp8) + off) = make_uint2(q0, q1);
        if (live && sinks.x_fp8)
          *reinterpret_cast<uint2*>(sinks.x_fp8 + r * sinks.pitch_fp8 + vv * 8) = make_uint2(q0, q1);
      }
    }
  }
}

#ifdef IQB_TRACE
// Development builds only: thread 0 of every CTA stamps %globaltimer into the top 64 KB
// of the scratch at the points of interest.
#define IQB_STAMP(i) do { if (tid == 0) trace[i] = globaltimer_ns(); } while (0)
#else
#define IQB_STAMP(i) do { } while (0)
#endif

template <class GO, class GD>
__global__ void __launch_bounds__(kThreads, 1) layer_kernel(const __grid_constant__ LayerParams p) {
  using GR = Geo<1, 16, 2>;   // router rows are bf16: 2 KB per 1024 elements
  using GG = Geo<2, 8, 2>;
  using Smem = StreamSmem<GO>;
  extern __shared__ __align__(128) uint8_t smem[];
  Smem* sm = reinterpret_cast<Smem*>(smem);
  LayerSmemExtra* ex = reinterpret_cast<LayerSmemExtra*>(smem + p.off_extra);
  float* sc = reinterpret_cast<float*>(smem + p.off_sc);
  float* xs = reinterpret_cast<float*>(smem + p.off_xs);
  uint8_t* xq = smem + p.off_xq;
  uint8_t* xq_gate = smem + p.off_xq_gate;   // the Gate's rows live beside the router's
  uint8_t* ring = smem + p.off_ring;
  const StreamScratch scr = scratch_of(p.scratch);
  uint8_t* scr_bytes = static_cast<uint8_t*>(p.scratch);
  uint32_t* cnt_g = reinterpret_cast<uint32_t*>(scr_bytes + kScrCntG);
  const uint32_t* epoch_word = reinterpret_cast<const uint32_t*>(scr_bytes + kScrEpoch);
  uint64_t* parts = reinterpret_cast<uint64_t*>(scr_bytes + kScrParts);
  uint32_t* rows_o = reinterpret_cast<uint32_t*>(scr_bytes + kScrRowsO);
  uint32_t* rows_d = reinterpret_cast<uint32_t*>(scr_bytes + kScrRowsD);
  uint64_t* logits_t = reinterpret_cast<uint64_t*>(scr_bytes + kScrLogits);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int cta = blockIdx.x, n_cta = static_cast<int>(gridDim.x);
  const int slot_bytes = p.slot_bytes;
#ifdef IQB_TRACE
  unsigned long long* trace =
      reinterpret_cast<unsigned long long*>(scr_bytes + kScrBytes - 65536) + cta * 32;
#endif
  IQB_STAMP(0);

  stream_init<GO>(p.sh_o, sm);
  if (tid == 0) {
    GroupDesc& g = ex->g_oproj;
    g.w = p.w_o;
    g.scale = p.w_o_scale;
    g.row_base = 0;
    g.map_id = 0;
    for (int c = 0; c < kMaxCols; ++c) {
      g.col_row[c] = c < p.sh_o.x_rows ? c : -1;
      g.col_mul[c] = 1.0f;
      g.col_out[c] = static_cast<int16_t>(c);
    }
  } else if (tid == 32) {
    GroupDesc& g = ex->g_router;
    g.w = p.w_r;
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

  int grid_o = 0, grid_r = 0, grid_g = 0, grid_d = 0;
  const CtaWork wk_o = cta_share<GO>(p.sh_o, n_cta, cta, grid_o);
  const CtaWork wk_r = cta_share<GR>(p.sh_r, n_cta, cta, grid_r);

  if (warp == kProducerWarp) {
    // ================================================================ producer
    RingPos pos;
    produce<GO>(p.sh_o, sm, &ex->g_oproj, ring, slot_bytes, wk_o, scr.status, &p.map_o, &p.map_o,
                pos);
    if (!sm->abort_flag)
      produce<GR>(p.sh_r, sm, &ex->g_router, ring, slot_bytes, wk_r, scr.status, &p.map_r,
                  &p.map_r, pos);
    named_bar_sync(kBarTables, kThreads);
    StreamShape sh_g = p.sh_g, sh_d = p.sh_d;
    sh_g.n_groups = sh_d.n_groups = ex->n_groups;
    const CtaWork wk_g = cta_share<GG>(sh_g, n_cta, cta, grid_g);
    const CtaWork wk_d = cta_share<GD>(sh_d, n_cta, cta, grid_d);
    if (!sm->abort_flag)
      produce<GG>(sh_g, sm, sm->groups, ring, slot_bytes, wk_g, scr.status, &p.map_g0, &p.map_g1,
                  pos);
    if (!sm->abort_flag)
      produce<GD>(sh_d, sm, ex->g_down, ring, slot_bytes, wk_d, scr.status, &p.map_d0, &p.map_d1,
                  pos);
    pdl_wait();
  } else if (warp < kConsumerWarps) {
    // ================================================================ consumers
    RingPos pos;
    RedPos rpos;
    const BlockBar helpers{kBarHelpers, kConsumerThreads};
    float* red = reinterpret_cast<float*>(ex->g_down);   // 128 floats; the Down's table is idle
    float held[kGatherHeld];

    // ---- o_proj
    gather_scales_load<GO, ElemE4M3>(p.sh_o, &ex->g_oproj, wk_o, tid, held);
    after_wait();
    IQB_STAMP(1);
    if (p.x_kind == IQ_X_BF16_GROUPQ || p.x_kind == IQ_X_BF16_SPLIT2)
      stage_rows_bf16_groupq(xq, xs, p.sh_o, static_cast<const __nv_bfloat16*>(p.x), p.k_o, p.m,
                             p.k_o, p.x_kind == IQ_X_BF16_SPLIT2, tid);
    else
      stage_rows_e4m3(xq, xs, p.sh_o, static_cast<const uint8_t*>(p.x), p.k_o,
                      p.x_kind == IQ_X_E4M3_GROUP ? p.x_scale : nullptr, p.m, p.k_o, tid);
    IQB_STAMP(14);
    gather_scales_store<GO, ElemE4M3>(p.sh_o, &ex->g_oproj, wk_o, sc, tid, held);
    named_bar_sync(kBarConsumers, kConsumerThreads);
    IQB_STAMP(15);
    if (!sm->abort_flag)
      consume<GO, ElemE4M3>(p.sh_o, sm, &ex->g_oproj, ring, slot_bytes, xq, xs, sc, wk_o, scr, pos,
                            rpos);
    IQB_STAMP(2);

    // ---- attention tail, in every CTA, straight into the router's and the Gate's rows
    const uint32_t epoch = __ldcg(epoch_word);    // stable: the last CTA out advances it
    const uint32_t tag16 = tag16_of(epoch), tag32 = tag32_of(epoch, 1);   // 1: the router's
    {
      const uint32_t* rows = rows_o;
      if (p.tail_a.world > 1) {
        uint32_t* reduced = reinterpret_cast<uint32_t*>(scr_bytes + kScrRowsA);
        rows = reduced;
        if (cta == 0 && !sm->abort_flag)
          reduce_rows_over_ranks(sm, ex, p.tail_a, rows_o, reduced, tag16, p.wait_ms);
      }
      TailSinks sinks;
      sinks.x_bf16 = xq;
      sinks.pitch_bf16 = p.sh_r.x_pitch;
      sinks.x_fp8 = xq_gate;
      sinks.pitch_fp8 = p.sh_g.x_pitch;
      sinks.x_fp8_scale = xs;
      sinks.blocks = p.sh_g.x_blocks;
      // every consumer warp of this CTA is past its last o_proj stage before the rows of
      // the next streams overwrite the o_proj activations
      named_bar_sync(kBarConsumers, kConsumerThreads);
      IQB_STAMP(3);
      if (!sm->abort_flag)
        tail_everywhere(sm, p.tail_a, rows, tag16, p.wait_ms, red, sinks, cta, n_cta);
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    IQB_STAMP(4);

    // ---- router
    if (!sm->abort_flag)
      consume<GR, ElemBF16>(p.sh_r, sm, &ex->g_router, ring, slot_bytes, xq, xs, sc, wk_r, scr, pos,
                            rpos);
    IQB_STAMP(5);
    named_bar_sync(kBarConsumers, kConsumerThreads);   // the router's rows are no longer read
    {
      // the logits, as soon as their words carry this launch's tag, into shared memory
      float* s_logits = reinterpret_cast<float*>(xq);
      const int n_logits = p.m * p.e;
      for (int i = tid; i < n_logits && !sm->abort_flag; i += kConsumerThreads) {
        uint64_t t0 = 0;
        for (uint32_t spin = 0;; ++spin) {
          const uint64_t w = ld_relaxed_gpu_u64(logits_t + i);
          if (static_cast<uint32_t>(w >> 32) == tag32) {
            s_logits[i] = __uint_as_float(static_cast<uint32_t>(w));
            break;
          }
          if ((spin & 63u) == 63u) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (sm->abort_flag || now - t0 > 1000000ull * p.wait_ms) {
              if (!sm->abort_flag) set_status(scr.status, IQ_ERR_PIPE_TIMEOUT);
              sm->abort_flag = 1;
              break;
            }
          }
        }
      }
      named_bar_sync(kBarConsumers, kConsumerThreads);
      IQB_STAMP(6);
      // top-k in every CTA (one warp per row) into the CTA's own copy of the routes
      if (!sm->abort_flag && warp < p.m)
        select_row(s_logits, p.e, p.top_k, p.score, warp, ex->sel, ex->wt, true);
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    if (cta == 0 && tid < p.m * p.top_k) {
      p.sel[tid] = ex->sel[tid];
      p.wt[tid] = ex->wt[tid];
    }
    IQB_STAMP(7);

    // ---- the group tables of both expert streams, then the Gate
    const int n_groups = build_groups(sm->groups, p.mc_g, false, false, scr.status, sm->route_ids,
                                      helpers, ex->sel, ex->wt, ex->g_down, &p.mc_d);
    if (tid == 0) ex->n_groups = n_groups;
    named_bar_sync(kBarTables, kThreads);
    IQB_STAMP(8);
    StreamShape sh_g = p.sh_g, sh_d = p.sh_d;
    sh_g.n_groups = sh_d.n_groups = n_groups;
    const CtaWork wk_g = cta_share<GG>(sh_g, n_cta, cta, grid_g);
    const CtaWork wk_d = cta_share<GD>(sh_d, n_cta, cta, grid_d);
    gather_scales_load<GG, ElemE4M3>(sh_g, sm->groups, wk_g, tid, held);
    gather_scales_store<GG, ElemE4M3>(sh_g, sm->groups, wk_g, sc, tid, held);
    named_bar_sync(kBarConsumers, kConsumerThreads);
    if (!sm->abort_flag)
      consume<GG, ElemE4M3>(sh_g, sm, sm->groups, ring, slot_bytes, xq_gate, xs, sc, wk_g, scr, pos,
                            rpos);
    IQB_STAMP(9);

    // ---- Down: its scales are fetched while the other CTAs finish their Gate tiles
    gather_scales_load<GD, ElemE4M3>(sh_d, ex->g_down, wk_d, tid, held);
    wait_word(sm, cnt_g, static_cast<uint32_t>(n_cta), p.wait_ms, scr.status);
    IQB_STAMP(10);
    {
      const int rows = p.mc_d.m * (p.mc_d.top_k + p.mc_d.n_shared);
      if (p.act_kind == IQ_ACT_E4M3)
        stage_rows_e4m3(xq, xs, sh_d, static_cast<const uint8_t*>(p.act), p.mc_d.i_loc, nullptr,
                        rows, p.mc_d.i_loc, tid);
      else
        stage_rows_bf16_groupq(xq, xs, sh_d, static_cast<const __nv_bfloat16*>(p.act),
                               p.mc_d.i_loc, rows, p.mc_d.i_loc, false, tid);
    }
    gather_scales_store<GD, ElemE4M3>(sh_d, ex->g_down, wk_d, sc, tid, held);
    named_bar_sync(kBarConsumers, kConsumerThreads);
    if (!sm->abort_flag)
      consume<GD, ElemE4M3>(sh_d, sm, ex->g_down, ring, slot_bytes, xq, xs, sc, wk_d, scr, pos,
                            rpos);
    IQB_STAMP(11);

    // ---- MLP tail, in every CTA, each writing its share of the layer's outputs
    {
      const uint32_t* rows = rows_d;
      if (p.tail_m.world > 1) {
        uint32_t* reduced = reinterpret_cast<uint32_t*>(scr_bytes + kScrRowsM);
        rows = reduced;
        if (cta == 0 && !sm->abort_flag)
          reduce_rows_over_ranks(sm, ex, p.tail_m, rows_d, reduced, tag16, p.wait_ms);
      }
      // The Down's table doubles as the reduction slots again: every consumer warp of this
      // CTA must be past its last Down stage.
      named_bar_sync(kBarConsumers, kConsumerThreads);
      IQB_STAMP(12);
      if (!sm->abort_flag)
        tail_everywhere(sm, p.tail_m, rows, tag16, p.wait_ms, red, TailSinks{}, cta, n_cta);
    }
    // ---- the last CTA to get here closes the launch: the next one gets a new tag
    if (tid == 0 && !sm->abort_flag) {
      uint32_t* exit_cnt = reinterpret_cast<uint32_t*>(scr_bytes + kScrExit);
      if (atomicAdd(exit_cnt, 1u) == static_cast<uint32_t>(n_cta - 1)) {
        *cnt_g = 0u;
        *exit_cnt = 0u;
        *reinterpret_cast<uint32_t*>(scr_bytes + kScrEpoch) = epoch + 1u;
      }
    }
  } else {
    // ================================================================ epilogue warp
    RedPos rpos;
    pdl_wait();
    const uint32_t epoch = __ldcg(epoch_word);
    const uint32_t tag16 = tag16_of(epoch);
    {
      const long long total =
          static_cast<long long>(stream_num_tiles<GO>(p.sh_o)) * stream_stages_per_tile<GO>(p.sh_o);
      const bool split2 = p.x_kind == IQ_X_BF16_SPLIT2;
      const bool plain = p.tail_a.world == 1;   // with peers, CTA 0 fills the symmetric buffer
      const int m = p.m, n = p.h;
      __nv_bfloat16* out = p.out_o;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[GO::RT]) {
#pragma unroll
        for (int sub = 0; sub < GO::RT; ++sub) {
          const int row = id.tig * GO::ROWS + sub * 16 + r;
          float v = val[sub];
          int orow = col;
          bool live = col < m;
          if (split2) {
            // columns 2j and 2j+1 are the two terms of row j: fold them on the even lane
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            orow = col >> 1;
            live = (col & 1) == 0 && orow < m;
          }
          const __nv_bfloat16 b = __float2bfloat16_rn(v);
          if (live && plain) out[static_cast<size_t>(orow) * n + row] = b;
          // every row's words are rewritten by every launch, live or not
          if (!split2 || (col & 1) == 0)
            st_relaxed_gpu_u32(rows_o + static_cast<size_t>(orow) * n + row,
                               (tag16 << 16) | __bfloat16_as_ushort(b));
        }
      };
      if (!sm->abort_flag)
        epilogue_resident<GO>(p.sh_o, sm, wk_o, total, grid_o, cta, scr, parts, tag32_of(epoch, 0), rpos,
                              emit);
    }
    {
      const long long total =
          static_cast<long long>(stream_num_tiles<GR>(p.sh_r)) * stream_stages_per_tile<GR>(p.sh_r);
      const int m = p.m, e = p.e;
      const uint32_t tag32 = tag32_of(epoch, 1);
      float* logits = p.logits;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[GR::RT]) {
#pragma unroll
        for (int sub = 0; sub < GR::RT; ++sub)
          if (col < m) {
            const size_t o = static_cast<size_t>(col) * e + id.tig * GR::ROWS + sub * 16 + r;
            logits[o] = val[sub];
            st_relaxed_gpu_u64(logits_t + o,
                               (static_cast<uint64_t>(tag32) << 32) | __float_as_uint(val[sub]));
          }
      };
      if (!sm->abort_flag)
        epilogue_resident<GR>(p.sh_r, sm, wk_r, total, grid_r, cta, scr, parts, tag32, rpos, emit);
    }
    named_bar_sync(kBarTables, kThreads);
    StreamShape sh_g = p.sh_g, sh_d = p.sh_d;
    sh_g.n_groups = sh_d.n_groups = ex->n_groups;
    const CtaWork wk_g = cta_share<GG>(sh_g, n_cta, cta, grid_g);
    const CtaWork wk_d = cta_share<GD>(sh_d, n_cta, cta, grid_d);
    {
      const long long total =
          static_cast<long long>(stream_num_tiles<GG>(sh_g)) * stream_stages_per_tile<GG>(sh_g);
      const int i_loc = p.mc_g.i_loc, m = p.mc_g.m;
      const int act_kind = p.act_kind;
      void* act = p.act;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[GG::RT]) {
        const GroupDesc& gd = sm->groups[id.group];
        if (col >= m || gd.col_row[col] < 0) return;
#pragma unroll
        for (int sub = 0; sub < GG::RT / 2; ++sub) {
          const float gte = val[sub], up = val[sub + GG::RT / 2];
          const float v = gte / (1.0f + expf(-gte)) * up;
          const size_t o = static_cast<size_t>(gd.col_out[col]) * i_loc +
                           id.tig * (GG::ROWS / 2) + sub * 16 + r;
          if (act_kind == IQ_ACT_E4M3)
            static_cast<uint8_t*>(act)[o] = f32_to_e4m3_sat(v);
          else
            static_cast<__nv_bfloat16*>(act)[o] = __float2bfloat16_rn(v);
        }
      };
      if (!sm->abort_flag)
        epilogue_resident<GG>(sh_g, sm, wk_g, total, grid_g, cta, scr, parts, tag32_of(epoch, 2), rpos,
                              emit);
    }
    count_in(cnt_g);
    {
      const long long total =
          static_cast<long long>(stream_num_tiles<GD>(sh_d)) * stream_stages_per_tile<GD>(sh_d);
      const bool plain = p.tail_m.world == 1;
      const int m = p.mc_d.m, h = p.mc_d.h;
      __nv_bfloat16* out = p.out_d;
      auto emit = [&](const TileId& id, int r, int col, const float (&val)[GD::RT]) {
#pragma unroll
        for (int sub = 0; sub < GD::RT; ++sub) {
          const size_t o = static_cast<size_t>(col) * h + id.tile * GD::ROWS + sub * 16 + r;
          const __nv_bfloat16 b = __float2bfloat16_rn(val[sub]);
          if (col < m && plain) out[o] = b;
          st_relaxed_gpu_u32(rows_d + o, (tag16 << 16) | __bfloat16_as_ushort(b));
        }
      };
      if (!sm->abort_flag)
        epilogue_resident<GD>(sh_d, sm, wk_d, total, grid_d, cta, scr, parts, tag32_of(epoch, 3), rpos,
                              emit);
    }
  }
  __syncthreads();
  IQB_STAMP(13);
  stream_drain_on_abort<GO>(sm);
}

}  // namespace iqb
