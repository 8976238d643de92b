/* C ABI of libiqb200: the block-FP8 tensor-parallel decode path on B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*),
 * launches asynchronously on that stream, allocates nothing and is CUDA-graph
 * capturable.  The return value is an IQ_* code for errors found on the host (bad
 * arguments, launch failure).  Errors found on the device (a pipeline or peer wait that
 * ran out of time, an expert id out of range) are written to the status word at the
 * start of the caller's scratch buffer; read it with iq_status_read.  No kernel traps
 * and no device-side wait is unbounded.
 *
 * The citations name the reference interface (IQuestRT, path inside that project) each
 * entry point stands in for; the reference binds its kernels as pybind functions taking
 * int64 raw device pointers (iquestrt/kernels/sm100_moe_fp8.py:192-193,345-346,
 * iquestrt/kernels/router.py:218-219, iquestrt/kernels/ar_tail.py:20-48).
 */
#ifndef IQB200_H_
#define IQB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  IQ_OK = 0,
  IQ_ERR_ARG = 1,
  IQ_ERR_CUDA = 2,
  IQ_ERR_PIPE_TIMEOUT = 3,
  IQ_ERR_PEER_TIMEOUT = 4,
  IQ_ERR_ROUTE = 5,
  IQ_ERR_UNSUPPORTED = 6
};

/* Activation formats of iq_linear. */
enum {
  IQ_X_BF16_GROUPQ = 0,   /* bf16 in; quantised in the kernel per 1x128 group (e4m3, fp32 amax/448) */
  IQ_X_BF16_SPLIT2 = 1,   /* bf16 in; two e4m3 terms per value (W8A16-faithful), m <= 4 */
  IQ_X_E4M3_GROUP = 2,    /* e4m3 in with fp32 [m, k/128] group scales */
  IQ_X_E4M3_UNSCALED = 3  /* e4m3 in, no scales (the reference's MoE activation format) */
};

enum { IQ_TAIL_NONE = 0, IQ_TAIL_ATTN = 1, IQ_TAIL_MLP = 2 };
enum { IQ_ROUTE_SOFTMAX = 0, IQ_ROUTE_SIGMOID = 1 };
enum { IQ_ACT_E4M3 = 0, IQ_ACT_BF16 = 1 };

/* The `pdl` field of the argument structs: 0 = plain launch; 1 = launch with the
 * programmatic-stream-serialization attribute (the kernel streams its weights before
 * waiting for its predecessor, and lets its own successor start once that wait has
 * returned); 2 = as 1, and the caller also guarantees that iq_moe_gate's x_fp8/x_scale,
 * resp. iq_moe_down's sel/wt, were written at least TWO launches earlier on the stream,
 * so they too are read before the wait (as in the layer: attention tail -> router ->
 * Gate -> Down, every launch made with pdl >= 1).  At level 2 iq_moe_gate with shared
 * experts also WRITES the shared experts' rows of `act` before its wait, so the launch
 * immediately before it must not read `act` (in the layer that launch is the router). */

/* Bytes of scratch every streaming entry point needs.  The caller zero-fills it once;
 * each launch leaves its counters zeroed again (the status word and the launch counter
 * that tags hand-off words persist).  Launches that share a scratch buffer must be
 * ordered on one stream. */
size_t iq_scratch_bytes(void);

/* Copies the device status word at the start of `scratch` to *code after synchronising
 * `stream`, and clears it when `clear` is non-zero. */
int iq_status_read(void* scratch, int* code, int clear, void* stream);

/* Number of SMs the library sizes its persistent grids for on the current device. */
int iq_sm_count(void);

/* The all-reduce + residual + RMSNorm epilogue ("tail").  Standalone it replaces
 * MultimemARTail.__call__ / .h_inv_xpad_fp8_pdl_overlap_local
 * (iquestrt/kernels/ar_tail.py:1407-1550, kernels L185-592) for kind IQ_TAIL_ATTN and
 * MultimemMLPTail.__call__ (iquestrt/kernels/ar_tail.py:1574-1622, kernel L597-707) for
 * kind IQ_TAIL_MLP; fused it runs inside iq_linear / iq_moe_down after the last tile.
 *
 *   ATTN: ao = AR(partial); h = bf16(residual + bf16(bf16(w_first*(ao*inv))*scale));
 *         norm_out = bf16(w_norm*(h*inv2))
 *   MLP:  m = AR(partial);  h = bf16(residual + bf16(m*scale));
 *         norm_out = bf16(w_norm*(h*inv))
 *
 * Two all-reduce protocols exist for world > 1.
 *
 * Pull (`push` == NULL): every rank adds one to every rank's `arrive` counter (one
 * multimem.red through `arrive_mc`, else one store per peer through `peer_arrive`), waits
 * (bounded by timeout_ms) until its own counter shows all ranks of this call, then reads
 * the switch-reduced rows with multimem.ld_reduce through `partial_mc` (else sums the
 * peers' rows through `peer_partials` in rank order).
 *
 * Push (`push` != NULL): the producing GEMV stores every finished tile of its rows, as
 * 32-bit words that carry the bf16 value and a 16-bit tag of the call, straight from its
 * epilogue into a per-source landing zone on EVERY rank (one multimem.st per 16 bytes
 * through `recv_mc`, else one store per peer through `peer_recv`).  The tail polls its
 * own rank's landing zone (local memory only) until every word of a row carries the
 * call's tag (bounded by timeout_ms), adds the sources in rank order in fp32 and rounds
 * once to bf16.  There is no flag, counter or fence on the producer's side, and no load
 * crosses NVLink.  world == 1 uses the same hand-off through a zone inside the scratch.
 * Rows are independent: each row of a call is finished by its own CTA. */
typedef struct iq_push_args {
  int world, rank;
  int rows;                      /* rows the zone is laid out for (>= m) */
  int h;
  uint32_t* recv;                /* this rank's zone: u32 [world][rows][h] */
  uint32_t* recv_mc;             /* multicast alias of `recv`, or NULL */
  uint32_t* const* peer_recv;    /* device array [world] of the ranks' zones, or NULL */
  uint32_t* epoch;               /* local device word: completed calls on this zone */
  uint32_t* ticket;              /* local device word, zero between calls */
} iq_push_args;

typedef struct iq_tail_args {
  int kind;
  int world, rank;
  int m, h;
  const void* partial;               /* bf16 [m,h], this rank's rows in its symmetric buffer */
  const void* partial_mc;            /* multicast alias of `partial`, or NULL */
  const void* const* peer_partials;  /* device array [world], or NULL */
  uint32_t* arrive;                  /* this rank's arrival counter in the symmetric buffer */
  uint32_t* arrive_mc;               /* multicast alias of `arrive`, or NULL */
  uint32_t* const* peer_arrive;      /* device array [world], or NULL */
  uint32_t* epoch;                   /* local device word: completed calls on this buffer */
  const void* residual;              /* bf16 [m,h], or fp32 when residual_fp32 */
  int residual_fp32;
  const float* w_first;              /* ATTN: [h] fp32 */
  const float* w_norm;               /* [h] fp32 */
  float scale, eps;
  void* h_out;                       /* bf16 [m,h] (fp32 when residual_fp32) */
  void* norm_out;                    /* bf16 [m,h] */
  void* norm_fp8;                    /* optional e4m3 [m,h] */
  float* norm_fp8_scale;             /* optional fp32 [m,h/128]: NULL = unscaled cast */
  float* inv_out;                    /* optional fp32 [m]: rsqrt of the last norm */
  int* status;                       /* device status word (normally the scratch's) */
  unsigned timeout_ms;               /* peer wait budget; 0 = 2000 */
  const iq_push_args* push;          /* push protocol (see above), or NULL */
} iq_tail_args;

/* The tail on its own, one CTA per row (the pull protocol with world > 1: one CTA).  With
 * `push`, the rows must have been produced by iq_linear / iq_moe_down calls given the
 * same `push`. */
int iq_tail(const iq_tail_args* a, void* stream, int pdl);

/* out[m,n] bf16 = x[m,k] . dequant(w[n,k] e4m3, w_scale)^T, optionally followed in the
 * same kernel by the tail.  Replaces reference.linear
 * (iquestrt/model/reference.py:23-27) and OProjGemv.__call__ / build_gemv_block
 * (iquestrt/kernels/oproj.py:83-171).  w_scale is [n/rg, k/kg] fp32 (rg, kg in
 * {64,128}); when `tail` is given, `out` must be tail->partial.
 *
 * With a tail that uses the push protocol (or world == 1) the last m CTAs of the launch
 * take no part in the GEMV: CTA i of them finishes row i (polls the landing zone, adds
 * the ranks, residual, RMSNorms) while the others are still streaming.  With the pull
 * protocol the last CTA to finish its tiles runs the tail for all rows.  `push` without
 * `tail` only sends the rows (for a later iq_tail with the same `push`). */
typedef struct iq_linear_args {
  const void* x;
  const float* x_scale;
  int x_kind;
  int m, k, n;
  const void* w;
  const float* w_scale;
  int rg, kg;
  void* out;
  void* scratch;
  size_t scratch_bytes;
  const iq_tail_args* tail;
  int pdl;
  const iq_push_args* push;
  float* out_f32;           /* optional fp32 [m,n]: the result before its bf16 rounding;
                               with it `out` may be NULL (then no tail and no push) */
} iq_linear_args;

int iq_linear(const iq_linear_args* a, void* stream);

/* iq_linear without a caller scratch buffer.  It has no counterpart in the reference: it
 * exists for callers that cannot allocate device memory where they call the library (a
 * plugin invoked while the host application captures a stream, a server whose memory
 * was handed out in full at start-up, a host that only ever receives input and output
 * pointers).  The work area lives in a device array built into the library, about
 * 4.3 MB on every GPU that loads it.  a->scratch and a->scratch_bytes are ignored;
 * a->tail must be NULL; n and k must each be at most 65536, larger shapes are refused
 * with IQ_ERR_UNSUPPORTED and a message on stderr.  The call allocates and frees no
 * device memory.  The first call on a device looks the array's address up and should
 * come before any stream capture.  All calls on a device share the one array: it keeps
 * the previous call's contents (the part that must start at zero is cleared on the
 * stream before each launch), and calls that overlap on the GPU race -- order them on
 * one stream.  A device-side error (a pipeline wait that ran out) is recorded in the
 * array's status word until the next iq_linear_static call on the device clears it: read
 * it with iq_linear_static_status before making that next call. */
int iq_linear_static(const iq_linear_args* a, void* stream);

/* Copies the status word of iq_linear_static's built-in work area on the current device
 * to *code after synchronising `stream` (0 when no call has been made yet).  Allocates
 * nothing.  It has no counterpart in the reference either. */
int iq_linear_static_status(int* code, void* stream);

/* The attention prologue after the column-parallel QKV product (iq_linear with out_f32):
 * per (head, row) the fp32 product is normalised (q and k heads: RMSNorm over the head
 * with w_qn / w_kn, bf16 result), q and k get the partial rotary embedding over their
 * first rotary_dim channels (neox halves; products and sum each rounded to bf16), q goes
 * to q_out and k, v into row slot[row] of the caches (bf16, or e4m3 saturating when
 * kv_kind is IQ_ACT_E4M3).  Replaces the heads kernel of the reference's prologue
 * (iquestrt/kernels/prologue.py:147-238 `build_heads`; algebra
 * iquestrt/model/reference.py:101-112).  head_dim <= 256 and even, rotary_dim even. */
typedef struct iq_heads_args {
  const float* qkv;         /* fp32 [m, (q_heads + 2*kv_heads) * head_dim] */
  int m, q_heads, kv_heads, head_dim, rotary_dim;
  const float* w_qn;        /* [head_dim] fp32 */
  const float* w_kn;
  const void* cos;          /* bf16 [m, rotary_dim] */
  const void* sin;
  float eps;
  const int64_t* slot;      /* [m] cache rows */
  void* q_out;              /* bf16 [m, q_heads, head_dim] */
  void* k_cache;            /* [capacity, kv_heads, head_dim] */
  void* v_cache;
  int capacity;
  int kv_kind;              /* IQ_ACT_BF16 or IQ_ACT_E4M3 */
  int* status;              /* optional device status word: IQ_ERR_ROUTE on a slot out of range */
  int pdl;
} iq_heads_args;

int iq_qkv_heads(const iq_heads_args* a, void* stream);

/* Router: logits = x[m,h] bf16 . w[e,h]^T bf16 (fp32 accumulate), top_k with ties to the
 * lower expert id, weights = softmax over the selected logits (reference) or their
 * sigmoids renormalised, pairs stored in ascending expert id per row.  Replaces
 * RouterSelect.__call__ / router_q8_fused_kernel (iquestrt/kernels/router.py:416-563,
 * 658-699; select_row L43-115). */
typedef struct iq_router_args {
  const void* x;
  const void* w;
  int m, h, e, top_k;
  int score;
  int* sel;        /* [m*top_k] int32 */
  float* wt;       /* [m*top_k] fp32 */
  float* logits;   /* [m,e] fp32, written */
  void* scratch;
  size_t scratch_bytes;
  int pdl;
} iq_router_args;

int iq_router(const iq_router_args* a, void* stream);

/* Expert Gate/Up + SiLU for the routed pairs of m rows (each distinct expert streamed
 * once) plus n_shared shared experts: act[row*(top_k+n_shared)+slot][i_loc] =
 * silu(gate) * up.  Replaces moe_gate (iquestrt/kernels/sm100_moe_fp8.py:110-188) and
 * the Gate half of DenseMlp (iquestrt/kernels/oproj.py:174-197).  fc is
 * [E, 2*i_loc, h] e4m3 ([gate; up]) with scales [E, 2*i_loc/64, h/128]; the shared
 * expert uses the same shapes without the leading E.  The activations come as e4m3
 * (x_fp8, with x_scale or unscaled) or, when x_bf16 is given, as bf16 rows that the kernel
 * quantises per 1x128 group itself (x_fp8 / x_scale are then ignored). */
typedef struct iq_moe_gate_args {
  const void* x_fp8;        /* [m,h] e4m3 */
  const float* x_scale;     /* [m,h/128] or NULL (unscaled) */
  int m, h, i_loc, n_experts, top_k, n_shared;
  const int* sel;
  const void* fc;
  const float* fc_scale;
  const void* shared_fc;
  const float* shared_fc_scale;
  void* act;
  int act_kind;             /* IQ_ACT_E4M3 (unscaled, saturating) or IQ_ACT_BF16 */
  void* scratch;
  size_t scratch_bytes;
  int pdl;
  const void* x_bf16;       /* optional [m,h] bf16 (see above) */
} iq_moe_gate_args;

int iq_moe_gate(const iq_moe_gate_args* a, void* stream);

/* Expert Down: out[row] bf16 = sum_slot wt * dequant(proj[e_slot]) . act[row,slot]
 * (+ shared experts with weight 1), optionally followed in the same kernel by the
 * tail.  Replaces moe_down (iquestrt/kernels/sm100_moe_fp8.py:265-341),
 * MoeDecodeKernels.__call__ (iquestrt/kernels/moe_gemv.py:47-61) and the Down half of
 * DenseMlp.  proj is [E, h, i_loc] e4m3 with scales [E, h/128, i_loc/64].  A bf16 `act`
 * is quantised in the kernel per 1x128 group; an e4m3 `act` is used as is. */
typedef struct iq_moe_down_args {
  const void* act;
  int act_kind;
  int m, h, i_loc, n_experts, top_k, n_shared;
  const int* sel;
  const float* wt;
  const void* proj;
  const float* proj_scale;
  const void* shared_proj;
  const float* shared_proj_scale;
  void* out;                /* bf16 [m,h] */
  void* scratch;
  size_t scratch_bytes;
  const iq_tail_args* tail;
  int pdl;
  const iq_push_args* push; /* as in iq_linear_args */
} iq_moe_down_args;

int iq_moe_down(const iq_moe_down_args* a, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* IQB200_H_ */
