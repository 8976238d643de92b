"""Tensor-level wrappers of the C ABI: shape/dtype checks, pointer marshalling, stream.

These are the calls the reference-shaped holders in `iquestrt_b200.kernels` make.  Every
function launches on torch's current CUDA stream, allocates nothing when its outputs
are passed in, and raises on any non-zero return code.  PyTorch is used for device
memory and streams only."""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import (ACT_BF16, ACT_E4M3, ROUTE_SIGMOID, ROUTE_SOFTMAX, TAIL_ATTN, TAIL_MLP,
                   X_BF16_GROUPQ, X_BF16_SPLIT2, X_E4M3_GROUP, X_E4M3_UNSCALED)

E4M3 = torch.float8_e4m3fn

__all__ = ["Scratch", "TailSpec", "linear", "linear_static", "linear_static_status", "qkv_heads",
           "router",
           "moe_gate", "moe_down", "tail",
           "X_BF16_GROUPQ", "X_BF16_SPLIT2", "X_E4M3_GROUP", "X_E4M3_UNSCALED",
           "TAIL_ATTN", "TAIL_MLP", "ROUTE_SOFTMAX", "ROUTE_SIGMOID", "ACT_E4M3", "ACT_BF16"]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _need(name, t, dtype, shape=None, device=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor, got {t.device}")
    if device is not None and t.device != device:
        raise ValueError(f"{name} must be on {device}, got {t.device}")
    if t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


class Scratch:
    """The zero-filled work area the streaming kernels share (split-tile partials, tile
    counters, the CTA ticket and the device status word).  One per stream of calls."""

    def __init__(self, device="cuda"):
        lib = _lib.load()
        self.bytes = int(lib.iq_scratch_bytes())
        self.buf = torch.zeros(self.bytes, dtype=torch.uint8, device=device)
        self.ptr = self.buf.data_ptr()

    def status(self, clear: bool = True) -> int:
        """Synchronises the current stream and returns the device status code.  After an
        error the whole work area is zeroed (with `clear`): a launch that gave up may have
        left counters and hand-off words behind."""
        code = C.c_int(0)
        _lib.check("iq_status_read",
                   _lib.load().iq_status_read(self.ptr, C.byref(code), int(clear), _stream()))
        if code.value and clear:
            self.buf.zero_()
        return code.value

    def raise_on_error(self, where: str = "device status") -> None:
        code = self.status()
        if code:
            raise _lib.IqError(where, code)


@dataclass
class TailSpec:
    """Arguments of the all-reduce + residual + RMSNorm epilogue (see `iq_tail_args`).

    `partial` is this rank's bf16 [m,h] rows; for world > 1 it must live in a symmetric
    buffer and `comm` (a `parallel.SymmSlot`) supplies the multicast / peer addresses."""

    kind: int
    partial: torch.Tensor
    residual: torch.Tensor
    w_norm: torch.Tensor
    h_out: torch.Tensor
    norm_out: torch.Tensor
    scale: float = 1.0
    eps: float = 1e-6
    w_first: torch.Tensor | None = None
    norm_fp8: torch.Tensor | None = None
    norm_fp8_scale: torch.Tensor | None = None
    inv_out: torch.Tensor | None = None
    comm: object | None = None
    timeout_ms: int = 2000
    _keep: list = field(default_factory=list, repr=False)

    def to_c(self, status_ptr: int) -> _lib.TailArgs:
        m, h = self.partial.shape
        dev = self.partial.device
        _need("partial", self.partial, torch.bfloat16)
        fp32 = self.residual.dtype == torch.float32
        _need("residual", self.residual, torch.float32 if fp32 else torch.bfloat16, (m, h), dev)
        _need("w_norm", self.w_norm, torch.float32, (h,), dev)
        _need("h_out", self.h_out, torch.float32 if fp32 else torch.bfloat16, (m, h), dev)
        _need("norm_out", self.norm_out, torch.bfloat16, (m, h), dev)
        if self.kind == TAIL_ATTN:
            _need("w_first", self.w_first, torch.float32, (h,), dev)
        if self.norm_fp8 is not None:
            _need("norm_fp8", self.norm_fp8, E4M3, (m, h), dev)
        if self.norm_fp8_scale is not None:
            _need("norm_fp8_scale", self.norm_fp8_scale, torch.float32, (m, h // 128), dev)
        if self.inv_out is not None:
            _need("inv_out", self.inv_out, torch.float32, (m,), dev)
        a = _lib.TailArgs()
        a.kind = self.kind
        a.m, a.h = m, h
        a.partial = self.partial.data_ptr()
        if self.comm is None:
            a.world, a.rank = 1, 0
        else:
            self.comm.fill(a, self.partial)
        a.residual = self.residual.data_ptr()
        a.residual_fp32 = int(fp32)
        a.w_first = _ptr(self.w_first)
        a.w_norm = self.w_norm.data_ptr()
        a.scale, a.eps = float(self.scale), float(self.eps)
        a.h_out = self.h_out.data_ptr()
        a.norm_out = self.norm_out.data_ptr()
        a.norm_fp8 = _ptr(self.norm_fp8)
        a.norm_fp8_scale = _ptr(self.norm_fp8_scale)
        a.inv_out = _ptr(self.inv_out)
        a.status = status_ptr
        a.timeout_ms = int(self.timeout_ms)
        return a


_SCRATCH: dict[int, Scratch] = {}


def default_scratch(device=None) -> Scratch:
    """The per-device scratch the reference-shaped holders share (their calls are ordered
    on one stream, as one captured decode step is)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _SCRATCH:
        _SCRATCH[index] = Scratch(torch.device("cuda", index))
    return _SCRATCH[index]


def tail(spec: TailSpec, scratch: Scratch, *, pdl: bool = False) -> None:
    """The epilogue on its own: one CTA (`iq_tail`)."""
    a = spec.to_c(scratch.ptr)
    _lib.check("iq_tail", _lib.load().iq_tail(C.byref(a), _stream(), int(pdl)))


def _linear_args(x, w, w_scale, out, x_kind, x_scale, block):
    """Checks the operands of the block-FP8 GEMV and fills the part of `iq_linear_args`
    that `linear` and `linear_static` share."""
    m, k = x.shape
    n = w.shape[0]
    dev = x.device
    _need("w", w, E4M3, (n, k), dev)
    rg, kg = block
    _need("w_scale", w_scale, torch.float32, (n // rg, k // kg), dev)
    if x_kind is None:
        if x.dtype == torch.bfloat16:
            x_kind = X_BF16_GROUPQ
        else:
            x_kind = X_E4M3_GROUP if x_scale is not None else X_E4M3_UNSCALED
    _need("x", x, torch.bfloat16 if x_kind in (X_BF16_GROUPQ, X_BF16_SPLIT2) else E4M3, None, dev)
    if x_kind == X_E4M3_GROUP:
        _need("x_scale", x_scale, torch.float32, (m, k // 128), dev)
    if out is not None:
        _need("out", out, torch.bfloat16, (m, n), dev)
    a = _lib.LinearArgs()
    a.x, a.x_scale, a.x_kind = x.data_ptr(), _ptr(x_scale), x_kind
    a.m, a.k, a.n = m, k, n
    a.w, a.w_scale, a.rg, a.kg = w.data_ptr(), w_scale.data_ptr(), rg, kg
    a.out = _ptr(out)
    return a


def linear(x, w, w_scale, *, scratch: Scratch, out=None, x_kind=None, x_scale=None,
           block=(128, 128), tail: TailSpec | None = None, push=None, out_f32=None,
           pdl: bool = False):
    """`out[m,n] bf16 = x[m,k] @ dequant(w[n,k], w_scale).T` on the streaming GEMV kernel,
    optionally followed in the same launch by `tail` (whose `partial` must be `out`).

    `x` is bf16 (quantised in the kernel per 1x128 group, or split in two e4m3 terms with
    `x_kind=X_BF16_SPLIT2`) or e4m3 (with `x_scale [m,k/128]`, or unscaled).  `push` (a
    `parallel.SymmSlot`) sends the rows to that slot's landing zone on every rank without
    running a tail, for a later `tail(...)` on the same slot.  `out_f32 [m,n]` receives the
    result before its bf16 rounding; with it and no `out` only the fp32 result is written
    (and returned)."""
    only_f32 = out is None and out_f32 is not None and tail is None and push is None
    if out is None and not only_f32:
        out = torch.empty(x.shape[0], w.shape[0], dtype=torch.bfloat16, device=x.device)
    if out_f32 is not None:
        _need("out_f32", out_f32, torch.float32, (x.shape[0], w.shape[0]), x.device)
    a = _linear_args(x, w, w_scale, out, x_kind, x_scale, block)
    a.out_f32 = _ptr(out_f32)
    a.scratch, a.scratch_bytes = scratch.ptr, scratch.bytes
    t = None
    if tail is not None:
        t = tail.to_c(scratch.ptr)
        a.tail = C.pointer(t)
    elif push is not None and push.world > 1 and push.protocol == "push":
        a.push = C.pointer(push.push_args())
    a.pdl = int(pdl)
    _lib.check("iq_linear", _lib.load().iq_linear(C.byref(a), _stream()))
    return out_f32 if only_f32 else out


def qkv_heads(qkv, w_qn, w_kn, cos, sin, slot, q_out, k_cache, v_cache, *, q_heads: int,
              kv_heads: int, rotary_dim: int, eps: float, scratch: Scratch | None = None,
              pdl: bool = False):
    """The attention prologue after the QKV product (`iq_qkv_heads`): `qkv [m, (q_heads +
    2 kv_heads) * D]` fp32 -> `q_out [m, q_heads, D]` bf16 (normalised, roped), k and v
    into rows `slot [m]` (int64) of `k_cache` / `v_cache [capacity, kv_heads, D]` (bf16 or
    e4m3)."""
    m = qkv.shape[0]
    dev = qkv.device
    d = q_out.shape[-1]
    _need("qkv", qkv, torch.float32, (m, (q_heads + 2 * kv_heads) * d), dev)
    _need("w_qn", w_qn, torch.float32, (d,), dev)
    _need("w_kn", w_kn, torch.float32, (d,), dev)
    _need("cos", cos, torch.bfloat16, (m, rotary_dim), dev)
    _need("sin", sin, torch.bfloat16, (m, rotary_dim), dev)
    _need("slot", slot, torch.int64, (m,), dev)
    _need("q_out", q_out, torch.bfloat16, (m, q_heads, d), dev)
    if k_cache.dtype not in (torch.bfloat16, E4M3) or v_cache.dtype != k_cache.dtype:
        raise ValueError("the KV caches must both be bf16 or both e4m3")
    cap = k_cache.shape[0]
    _need("k_cache", k_cache, k_cache.dtype, (cap, kv_heads, d), dev)
    _need("v_cache", v_cache, k_cache.dtype, (cap, kv_heads, d), dev)
    a = _lib.HeadsArgs()
    a.qkv = qkv.data_ptr()
    a.m, a.q_heads, a.kv_heads, a.head_dim, a.rotary_dim = m, q_heads, kv_heads, d, rotary_dim
    a.w_qn, a.w_kn, a.cos, a.sin = w_qn.data_ptr(), w_kn.data_ptr(), cos.data_ptr(), sin.data_ptr()
    a.eps, a.slot, a.q_out = float(eps), slot.data_ptr(), q_out.data_ptr()
    a.k_cache, a.v_cache, a.capacity = k_cache.data_ptr(), v_cache.data_ptr(), cap
    a.kv_kind = ACT_E4M3 if k_cache.dtype == E4M3 else ACT_BF16
    a.status = None if scratch is None else scratch.ptr
    a.pdl = int(pdl)
    _lib.check("iq_qkv_heads", _lib.load().iq_qkv_heads(C.byref(a), _stream()))
    return q_out


def router(x, weight, *, top_k: int, scratch: Scratch, score: int = ROUTE_SOFTMAX, sel=None,
           wt=None, logits=None, pdl: bool = False):
    """Router GEMV + top-k in one launch: returns `(sel int32 [m*top_k], wt fp32 [m*top_k],
    logits fp32 [m,e])`, pairs in ascending expert id per row."""
    m, h = x.shape
    e = weight.shape[0]
    dev = x.device
    _need("x", x, torch.bfloat16, None, dev)
    _need("weight", weight, torch.bfloat16, (e, h), dev)
    if sel is None:
        sel = torch.empty(m * top_k, dtype=torch.int32, device=dev)
    if wt is None:
        wt = torch.empty(m * top_k, dtype=torch.float32, device=dev)
    if logits is None:
        logits = torch.empty(m, e, dtype=torch.float32, device=dev)
    _need("sel", sel, torch.int32, None, dev)
    _need("wt", wt, torch.float32, None, dev)
    _need("logits", logits, torch.float32, (m, e), dev)
    if sel.numel() < m * top_k or wt.numel() < m * top_k:
        raise ValueError("sel/wt must hold m*top_k entries")
    a = _lib.RouterArgs()
    a.x, a.w = x.data_ptr(), weight.data_ptr()
    a.m, a.h, a.e, a.top_k, a.score = m, h, e, top_k, score
    a.sel, a.wt, a.logits = sel.data_ptr(), wt.data_ptr(), logits.data_ptr()
    a.scratch, a.scratch_bytes, a.pdl = scratch.ptr, scratch.bytes, int(pdl)
    _lib.check("iq_router", _lib.load().iq_router(C.byref(a), _stream()))
    return sel, wt, logits


def moe_gate(x_fp8, sel, fc, fc_scale, act, *, m: int, top_k: int, scratch: Scratch,
             x_scale=None, shared_fc=None, shared_fc_scale=None, pdl: bool = False):
    """Gate/Up + SiLU of the routed pairs of the first `m` rows (+ shared experts) into
    `act [m*(top_k+n_shared), i_loc]` (e4m3 unscaled, or bf16).  `x_fp8` is e4m3 (with
    `x_scale`, or unscaled) or bf16 (quantised per 1x128 group inside the kernel)."""
    e, two_i, h = fc.shape
    i_loc = two_i // 2
    dev = fc.device
    _need("fc", fc, E4M3, None, dev)
    _need("fc_scale", fc_scale, torch.float32, (e, two_i // 64, h // 128), dev)
    x_is_bf16 = x_fp8.dtype == torch.bfloat16
    _need("x", x_fp8, torch.bfloat16 if x_is_bf16 else E4M3, None, dev)
    if x_fp8.shape[-1] != h or x_fp8.shape[0] < m:
        raise ValueError(f"x must be [>= {m}, {h}], got {tuple(x_fp8.shape)}")
    _need("sel", sel, torch.int32, None, dev)
    n_shared = 0
    if shared_fc is not None:
        n_shared = 1 if shared_fc.dim() == 2 else shared_fc.shape[0]
        _need("shared_fc", shared_fc, E4M3, None, dev)
        _need("shared_fc_scale", shared_fc_scale, torch.float32, None, dev)
        if shared_fc.numel() != n_shared * two_i * h:
            raise ValueError("shared_fc must have the experts' [2*i_loc, h] shape")
    slots = top_k + n_shared
    if act.dtype not in (E4M3, torch.bfloat16):
        raise ValueError("act must be e4m3 or bf16")
    _need("act", act, act.dtype, None, dev)
    if act.numel() < m * slots * i_loc:
        raise ValueError("act too small")
    if x_scale is not None:
        _need("x_scale", x_scale, torch.float32, None, dev)
    a = _lib.MoeGateArgs()
    if x_is_bf16:
        a.x_bf16 = x_fp8.data_ptr()
    else:
        a.x_fp8, a.x_scale = x_fp8.data_ptr(), _ptr(x_scale)
    a.m, a.h, a.i_loc, a.n_experts, a.top_k, a.n_shared = m, h, i_loc, e, top_k, n_shared
    a.sel, a.fc, a.fc_scale = sel.data_ptr(), fc.data_ptr(), fc_scale.data_ptr()
    a.shared_fc, a.shared_fc_scale = _ptr(shared_fc), _ptr(shared_fc_scale)
    a.act, a.act_kind = act.data_ptr(), ACT_E4M3 if act.dtype == E4M3 else ACT_BF16
    a.scratch, a.scratch_bytes, a.pdl = scratch.ptr, scratch.bytes, int(pdl)
    _lib.check("iq_moe_gate", _lib.load().iq_moe_gate(C.byref(a), _stream()))
    return act


def moe_down(act, sel, wt, proj, proj_scale, out, *, m: int, top_k: int, scratch: Scratch,
             shared_proj=None, shared_proj_scale=None, tail: TailSpec | None = None,
             push=None, pdl: bool = False):
    """Down of the routed pairs (+ shared experts) into `out[:m]` bf16 `[m,h]`, optionally
    followed in the same launch by `tail`; `push` as in `linear`."""
    e, h, i_loc = proj.shape
    dev = proj.device
    _need("proj", proj, E4M3, None, dev)
    _need("proj_scale", proj_scale, torch.float32, (e, h // 128, i_loc // 64), dev)
    _need("sel", sel, torch.int32, None, dev)
    _need("wt", wt, torch.float32, None, dev)
    _need("out", out, torch.bfloat16, None, dev)
    if out.shape[-1] != h or out.shape[0] < m:
        raise ValueError(f"out must be [>= {m}, {h}]")
    n_shared = 0
    if shared_proj is not None:
        n_shared = 1 if shared_proj.dim() == 2 else shared_proj.shape[0]
        _need("shared_proj", shared_proj, E4M3, None, dev)
        _need("shared_proj_scale", shared_proj_scale, torch.float32, None, dev)
    if act.dtype not in (E4M3, torch.bfloat16):
        raise ValueError("act must be e4m3 or bf16")
    _need("act", act, act.dtype, None, dev)
    a = _lib.MoeDownArgs()
    a.act, a.act_kind = act.data_ptr(), ACT_E4M3 if act.dtype == E4M3 else ACT_BF16
    a.m, a.h, a.i_loc, a.n_experts, a.top_k, a.n_shared = m, h, i_loc, e, top_k, n_shared
    a.sel, a.wt = sel.data_ptr(), wt.data_ptr()
    a.proj, a.proj_scale = proj.data_ptr(), proj_scale.data_ptr()
    a.shared_proj, a.shared_proj_scale = _ptr(shared_proj), _ptr(shared_proj_scale)
    a.out = out.data_ptr()
    a.scratch, a.scratch_bytes = scratch.ptr, scratch.bytes
    t = None
    if tail is not None:
        t = tail.to_c(scratch.ptr)
        a.tail = C.pointer(t)
    elif push is not None and push.world > 1 and push.protocol == "push":
        a.push = C.pointer(push.push_args())
    a.pdl = int(pdl)
    _lib.check("iq_moe_down", _lib.load().iq_moe_down(C.byref(a), _stream()))
    return out[:m]


def linear_static(x, w, w_scale, out, *, x_kind=None, x_scale=None, block=(128, 128),
                  pdl: bool = False):
    """`linear` for callers that cannot allocate device memory where they call it (inside a
    host application's stream capture, or with a memory budget spent in full at start-up):
    the kernel's work area is a device array built into the library, so no scratch buffer
    is passed and `out` must be given.  Limits: n, k <= 65536, no fused tail.  All calls on
    a device share that array, so order them on one stream; the first call on a device
    should come before any stream capture.  A device-side error of the call stays readable
    through `linear_static_status` until the next `linear_static` on the device."""
    a = _linear_args(x, w, w_scale, out, x_kind, x_scale, block)
    a.pdl = int(pdl)
    _lib.check("iq_linear_static", _lib.load().iq_linear_static(C.byref(a), _stream()))
    return out


def linear_static_status() -> int:
    """Synchronises the current stream and returns the device status code the last
    `linear_static` call on this device left (0 = none)."""
    code = C.c_int(0)
    _lib.check("iq_linear_static_status",
               _lib.load().iq_linear_static_status(C.byref(code), _stream()))
    return code.value
