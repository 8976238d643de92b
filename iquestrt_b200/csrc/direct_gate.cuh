// The direct form of the expert Gate/Up + SiLU for ONE row (see direct.cuh for the idea).
//
// A CTA owns sixteen features of one group (a routed pair of the row, or a shared expert):
// the sixteen gate rows and the sixteen matching up rows of that expert.  Warp (half, q) of
// its eight owns the gate (half 0) or up (half 1) rows and quarter q of K, which it walks in
// units of 128 bytes with three units of 16-byte loads in flight; the activation row is
// staged in shared memory ahead of the dependency wait (it was written two launches back).
// After the wait every warp reads its pair's expert id itself -- no table, no barrier -- and
// starts loading.  The eight fragments meet in shared memory; eight lanes of one warp form
// SiLU(gate) * up and store the sixteen activations.  Shared experts do not depend on the
// routes: their CTAs load before the wait.
#pragma once

namespace iqb {

struct GateDirectParams {
  IQ_TRACE_FIELD
  MoeCommon mc;
  const uint8_t* x_fp8;
  const float* x_scale;
  const __nv_bfloat16* x_bf16;
  void* act;
  int act_kind;
  void* scratch;
  int pdl_level;
};

constexpr int kGateUnitRuns = 2;                 // 64-byte runs per unit
constexpr int kGateUnitBytes = kGateUnitRuns * 64;

__host__ __device__ inline size_t gate_direct_smem(int h) {
  return sizeof(float) * 8 * 32 * 4 + static_cast<size_t>(h + 64) + sizeof(float) * (h / 128) + 64;
}

__global__ void __launch_bounds__(320, 2) gate_direct_kernel(const __grid_constant__ GateDirectParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int RPU = kGateUnitRuns;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = p.mc.h, i_loc = p.mc.i_loc, top_k = p.mc.top_k;
  const int tpg = i_loc >> 4;                    // feature tiles per group
  const int group = static_cast<int>(blockIdx.x) / tpg, ft = static_cast<int>(blockIdx.x) - group * tpg;
  const bool routed = group < top_k;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  float(*red)[32][4] = reinterpret_cast<float(*)[32][4]>(smem);
  uint8_t* xq = smem + sizeof(float) * 8 * 32 * 4;
  float* xs = reinterpret_cast<float*>(xq + h + 64);
  const bool early_x = p.pdl_level >= 2;
  StreamShape sh{};                              // (what the staging routines read of it)
  sh.x_pitch = h + 64;
  sh.x_blocks = h / 128;
  auto stage_x = [&]() {
    if (p.x_bf16)
      stage_rows_bf16_groupq(xq, xs, sh, p.x_bf16, h, 1, h, false, tid, 256);
    else
      stage_rows_e4m3(xq, xs, sh, p.x_fp8, h, p.x_scale, 1, h, tid, 256);
  };
  if (early_x) stage_x();

  const int half = warp >> 2, q = warp & 3;
  const int g8 = lane >> 2, t = lane & 3;
  const int row0 = half * i_loc + ft * 16;       // first of the warp's 16 rows in its expert
  const int k0 = q * (h >> 2);                   // the warp's quarter of K
  const int n_units = (h >> 2) / kGateUnitBytes;
  const int krow = h >> 7;                       // weight scale entries per 64-row block
  const uint8_t* wbase = nullptr;
  const float* sbase = nullptr;
  auto set_expert = [&](const uint8_t* w, const float* sc) {
    wbase = w + static_cast<size_t>(row0 + g8) * h + k0 + t * 16;
    sbase = sc + static_cast<size_t>(row0 >> 6) * krow + (k0 >> 7);
  };
  auto load_w = [&](DirectW<RPU>& w, int unit) {
    const uint8_t* a = wbase + unit * kGateUnitBytes;
    const uint8_t* b = a + static_cast<size_t>(8) * h;
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      w.wa[run] = ldg_nc_u4(a + run * 64);
      w.wb[run] = ldg_nc_u4(b + run * 64);
    }
    w.ws[0] = __ldg(sbase + unit);               // (one 128-byte unit lies in one scale block)
  };
  DirectW<RPU> b0, b1, b2;
  bool live = true;
  if (!routed) {
    const int s = group - top_k;
    set_expert(p.mc.shared_w + static_cast<size_t>(s) * p.mc.w_stride,
               p.mc.shared_scale + static_cast<size_t>(s) * p.mc.scale_stride);
    load_w(b0, 0);
    if (n_units > 1) load_w(b1, 1);
    if (n_units > 2) load_w(b2, 2);
  }
  after_wait();
  if (tid == 0) IQ_STAMP(p, 1);
  if (routed) {
    const int e = __ldcg(p.mc.sel + group);
    live = e >= 0 && e < p.mc.n_experts;
    if (live) {
      set_expert(p.mc.w + static_cast<size_t>(e) * p.mc.w_stride,
                 p.mc.w_scale + static_cast<size_t>(e) * p.mc.scale_stride);
      load_w(b0, 0);
      if (n_units > 1) load_w(b1, 1);
      if (n_units > 2) load_w(b2, 2);
    } else if (tid == 0) {
      set_status(scratch_of(p.scratch).status, IQ_ERR_ROUTE);
    }
  }
  if (!early_x) stage_x();
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 2);
  if (!live) return;                              // (a malformed route: nothing is written)

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t xq_s = smem_u32(xq) + k0 + t * 16, xs_s = smem_u32(xs) + (k0 >> 7) * 4;
  auto fold = [&](const DirectW<RPU>& w, int unit) {
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (g8 == 0) xv = lds128(xq_s + unit * kGateUnitBytes + run * 64);   // column 0 = the row
      mma_e4m3(part, w.wa[run].x, w.wb[run].x, w.wa[run].y, w.wb[run].y, xv.x, xv.y);
      mma_e4m3(part, w.wa[run].z, w.wb[run].z, w.wa[run].w, w.wb[run].w, xv.z, xv.w);
    }
    const float s = w.ws[0] * lds_f32(xs_s + unit * 4);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(part[i], s, acc[i]);
  };
  for (int unit = 0; unit < n_units; unit += 3) {
    fold(b0, unit);
    if (unit + 3 < n_units) load_w(b0, unit + 3);
    if (unit + 1 < n_units) {
      fold(b1, unit + 1);
      if (unit + 4 < n_units) load_w(b1, unit + 4);
    }
    if (unit + 2 < n_units) {
      fold(b2, unit + 2);
      if (unit + 5 < n_units) load_w(b2, unit + 5);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) red[warp][lane][i] = acc[i];
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 4);

  // ---- lanes 0, 4, ..., 28 of warp 0 hold column 0 of rows r and r+8 of the fragments
  if (warp == 0 && t == 0) {
    float gate_lo = 0.f, gate_hi = 0.f, up_lo = 0.f, up_hi = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      gate_lo += red[w][lane][0];
      gate_hi += red[w][lane][2];
      up_lo += red[4 + w][lane][0];
      up_hi += red[4 + w][lane][2];
    }
    const float v_lo = gate_lo / (1.0f + expf(-gate_lo)) * up_lo;
    const float v_hi = gate_hi / (1.0f + expf(-gate_hi)) * up_hi;
    const size_t o = static_cast<size_t>(group) * i_loc + ft * 16 + g8;   // pair row = group
    if (p.act_kind == IQ_ACT_E4M3) {
      static_cast<uint8_t*>(p.act)[o] = f32_to_e4m3_sat(v_lo);
      static_cast<uint8_t*>(p.act)[o + 8] = f32_to_e4m3_sat(v_hi);
    } else {
      static_cast<__nv_bfloat16*>(p.act)[o] = __float2bfloat16_rn(v_lo);
      static_cast<__nv_bfloat16*>(p.act)[o + 8] = __float2bfloat16_rn(v_hi);
    }
    if (lane == 0) IQ_STAMP(p, 5);
  }
}


// ------------------------------------------------------------------------------------
// The same for longer streams: EIGHT features per CTA.  An MMA tile's sixteen rows are the
// eight gate rows and the eight matching up rows, so a lane that holds gate row r in its
// fragment holds up row r as well and SiLU(gate) * up needs no exchange; the CTA's eight
// warps each take an eighth of K.  Twice as many CTAs as with sixteen features (two per SM at
// hidden 6144, expert width 256): twice as many loads in flight, which is what a stream
// that is not in L2 needs.
__global__ void __launch_bounds__(320, 2) gate_direct8_kernel(const __grid_constant__ GateDirectParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int RPU = kGateUnitRuns;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = p.mc.h, i_loc = p.mc.i_loc, top_k = p.mc.top_k;
  const int tpg = i_loc >> 3;                    // feature tiles (of eight) per group
  const int group = static_cast<int>(blockIdx.x) / tpg, ft = static_cast<int>(blockIdx.x) - group * tpg;
  const bool routed = group < top_k;
  if (tid == 0) {
    IQ_STAMP(p, 0);
#ifdef IQ_TRACE
    if (p.trace) p.trace[blockIdx.x * kTraceWords + 15] = smid_of();
#endif
  }
  float(*red)[32][4] = reinterpret_cast<float(*)[32][4]>(smem);
  uint8_t* xq = smem + sizeof(float) * 8 * 32 * 4;
  float* xs = reinterpret_cast<float*>(xq + h + 64);
  const bool early_x = p.pdl_level >= 2;
  StreamShape sh{};                              // (what the staging routines read of it)
  sh.x_pitch = h + 64;
  sh.x_blocks = h / 128;
  auto stage_x = [&]() {
    if (p.x_bf16)
      stage_rows_bf16_groupq(xq, xs, sh, p.x_bf16, h, 1, h, false, tid, 256);
    else
      stage_rows_e4m3(xq, xs, sh, p.x_fp8, h, p.x_scale, 1, h, tid, 256);
  };
  if (early_x) stage_x();

  const int g8 = lane >> 2, t = lane & 3;
  const int gate_row = ft * 8, up_row = i_loc + ft * 8;   // first rows of the two halves
  const int k0 = warp * (h >> 3);                // the warp's eighth of K
  const int n_units = (h >> 3) / kGateUnitBytes;
  const int krow = h >> 7;                       // weight scale entries per 64-row block
  const uint8_t *ga = nullptr, *ua = nullptr;
  const float *gs = nullptr, *us = nullptr;
  auto set_expert = [&](const uint8_t* w, const float* sc) {
    ga = w + static_cast<size_t>(gate_row + g8) * h + k0 + t * 16;
    ua = w + static_cast<size_t>(up_row + g8) * h + k0 + t * 16;
    gs = sc + static_cast<size_t>(gate_row >> 6) * krow + (k0 >> 7);
    us = sc + static_cast<size_t>(up_row >> 6) * krow + (k0 >> 7);
  };
  auto load_w = [&](DirectW<RPU>& w, int unit) {
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      w.wa[run] = ldg_nc_u4(ga + unit * kGateUnitBytes + run * 64);
      w.wb[run] = ldg_nc_u4(ua + unit * kGateUnitBytes + run * 64);
    }
    w.ws[0] = __ldg(gs + unit);                  // (one 128-byte unit lies in one scale block)
    w.ws[1] = __ldg(us + unit);
  };
  DirectW<RPU> b0, b1, b2;
  bool live = true;
  if (!routed) {
    const int s = group - top_k;
    set_expert(p.mc.shared_w + static_cast<size_t>(s) * p.mc.w_stride,
               p.mc.shared_scale + static_cast<size_t>(s) * p.mc.scale_stride);
    load_w(b0, 0);
    if (n_units > 1) load_w(b1, 1);
    if (n_units > 2) load_w(b2, 2);
  }
  after_wait();
  if (tid == 0) IQ_STAMP(p, 1);
  if (routed) {
    const int e = __ldcg(p.mc.sel + group);
    live = e >= 0 && e < p.mc.n_experts;
    if (live) {
      set_expert(p.mc.w + static_cast<size_t>(e) * p.mc.w_stride,
                 p.mc.w_scale + static_cast<size_t>(e) * p.mc.scale_stride);
      load_w(b0, 0);
      if (n_units > 1) load_w(b1, 1);
      if (n_units > 2) load_w(b2, 2);
    } else if (tid == 0) {
      set_status(scratch_of(p.scratch).status, IQ_ERR_ROUTE);
    }
  }
  if (!early_x) stage_x();
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 2);
  if (!live) return;                              // (a malformed route: nothing is written)

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t xq_s = smem_u32(xq) + k0 + t * 16, xs_s = smem_u32(xs) + (k0 >> 7) * 4;
  auto fold = [&](const DirectW<RPU>& w, int unit) {
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int run = 0; run < RPU; ++run) {
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (g8 == 0) xv = lds128(xq_s + unit * kGateUnitBytes + run * 64);   // column 0 = the row
      mma_e4m3(part, w.wa[run].x, w.wb[run].x, w.wa[run].y, w.wb[run].y, xv.x, xv.y);
      mma_e4m3(part, w.wa[run].z, w.wb[run].z, w.wa[run].w, w.wb[run].w, xv.z, xv.w);
    }
    const float xsc = lds_f32(xs_s + unit * 4);
    const float sg = w.ws[0] * xsc, su = w.ws[1] * xsc;
    acc[0] = fmaf(part[0], sg, acc[0]);           // fragment rows 0..7: gate
    acc[1] = fmaf(part[1], sg, acc[1]);
    acc[2] = fmaf(part[2], su, acc[2]);           // fragment rows 8..15: up
    acc[3] = fmaf(part[3], su, acc[3]);
  };
  for (int unit = 0; unit < n_units; unit += 3) {
    fold(b0, unit);
    if (unit + 3 < n_units) load_w(b0, unit + 3);
    if (unit + 1 < n_units) {
      fold(b1, unit + 1);
      if (unit + 4 < n_units) load_w(b1, unit + 4);
    }
    if (unit + 2 < n_units) {
      fold(b2, unit + 2);
      if (unit + 5 < n_units) load_w(b2, unit + 5);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) red[warp][lane][i] = acc[i];
  __syncthreads();
  if (tid == 0) IQ_STAMP(p, 4);

  // ---- lanes 0, 4, ..., 28 of warp 0: column 0 of gate row r (c0) and up row r (c2)
  if (warp == 0 && t == 0) {
    float gate = 0.f, up = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      gate += red[w][lane][0];
      up += red[w][lane][2];
    }
    const float v = gate / (1.0f + expf(-gate)) * up;
    const size_t o = static_cast<size_t>(group) * i_loc + ft * 8 + g8;   // pair row = group
    if (p.act_kind == IQ_ACT_E4M3)
      static_cast<uint8_t*>(p.act)[o] = f32_to_e4m3_sat(v);
    else
      static_cast<__nv_bfloat16*>(p.act)[o] = __float2bfloat16_rn(v);
    if (lane == 0) IQ_STAMP(p, 5);
  }
}

}  // namespace iqb
