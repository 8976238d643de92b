"""ctypes binding of `libiqb200.so` (the C ABI declared in `include/iqb200.h`).

There is no fallback: if the library is missing or a call returns a non-zero code the
operators raise."""

from __future__ import annotations

import ctypes as C
import os

from . import _build

IQ_OK, IQ_ERR_ARG, IQ_ERR_CUDA, IQ_ERR_PIPE_TIMEOUT, IQ_ERR_PEER_TIMEOUT, IQ_ERR_ROUTE, \
    IQ_ERR_UNSUPPORTED = range(7)
ERR_NAMES = {
    IQ_OK: "ok", IQ_ERR_ARG: "bad argument", IQ_ERR_CUDA: "CUDA call failed",
    IQ_ERR_PIPE_TIMEOUT: "shared-memory pipeline wait timed out",
    IQ_ERR_PEER_TIMEOUT: "a peer rank did not arrive in time",
    IQ_ERR_ROUTE: "expert id out of range", IQ_ERR_UNSUPPORTED: "unsupported shape",
}

X_BF16_GROUPQ, X_BF16_SPLIT2, X_E4M3_GROUP, X_E4M3_UNSCALED = range(4)
TAIL_NONE, TAIL_ATTN, TAIL_MLP = range(3)
ROUTE_SOFTMAX, ROUTE_SIGMOID = range(2)
ACT_E4M3, ACT_BF16 = range(2)

EXPORTS = ("iq_scratch_bytes", "iq_status_read", "iq_sm_count", "iq_tail", "iq_linear",
           "iq_linear_static", "iq_linear_static_status", "iq_qkv_heads", "iq_router",
           "iq_moe_gate", "iq_moe_down")


class IqError(RuntimeError):
    def __init__(self, where: str, code: int):
        super().__init__(f"{where}: {ERR_NAMES.get(code, 'error')} (code {code})")
        self.code = code


class PushArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("rank", C.c_int), ("rows", C.c_int), ("h", C.c_int),
        ("recv", C.c_void_p), ("recv_mc", C.c_void_p), ("peer_recv", C.c_void_p),
        ("epoch", C.c_void_p), ("ticket", C.c_void_p),
    ]


class TailArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int), ("world", C.c_int), ("rank", C.c_int), ("m", C.c_int), ("h", C.c_int),
        ("partial", C.c_void_p), ("partial_mc", C.c_void_p), ("peer_partials", C.c_void_p),
        ("arrive", C.c_void_p), ("arrive_mc", C.c_void_p), ("peer_arrive", C.c_void_p),
        ("epoch", C.c_void_p), ("residual", C.c_void_p), ("residual_fp32", C.c_int),
        ("w_first", C.c_void_p), ("w_norm", C.c_void_p), ("scale", C.c_float), ("eps", C.c_float),
        ("h_out", C.c_void_p), ("norm_out", C.c_void_p), ("norm_fp8", C.c_void_p),
        ("norm_fp8_scale", C.c_void_p), ("inv_out", C.c_void_p), ("status", C.c_void_p),
        ("timeout_ms", C.c_uint), ("push", C.POINTER(PushArgs)),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_scale", C.c_void_p), ("x_kind", C.c_int),
        ("m", C.c_int), ("k", C.c_int), ("n", C.c_int),
        ("w", C.c_void_p), ("w_scale", C.c_void_p), ("rg", C.c_int), ("kg", C.c_int),
        ("out", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
        ("tail", C.POINTER(TailArgs)), ("pdl", C.c_int), ("push", C.POINTER(PushArgs)),
        ("out_f32", C.c_void_p),
    ]


class HeadsArgs(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p),
        ("m", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int),
        ("rotary_dim", C.c_int),
        ("w_qn", C.c_void_p), ("w_kn", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("eps", C.c_float), ("slot", C.c_void_p), ("q_out", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("capacity", C.c_int),
        ("kv_kind", C.c_int), ("status", C.c_void_p), ("pdl", C.c_int),
    ]


class RouterArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p),
        ("m", C.c_int), ("h", C.c_int), ("e", C.c_int), ("top_k", C.c_int), ("score", C.c_int),
        ("sel", C.c_void_p), ("wt", C.c_void_p), ("logits", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("pdl", C.c_int),
    ]


class MoeGateArgs(C.Structure):
    _fields_ = [
        ("x_fp8", C.c_void_p), ("x_scale", C.c_void_p),
        ("m", C.c_int), ("h", C.c_int), ("i_loc", C.c_int), ("n_experts", C.c_int),
        ("top_k", C.c_int), ("n_shared", C.c_int),
        ("sel", C.c_void_p), ("fc", C.c_void_p), ("fc_scale", C.c_void_p),
        ("shared_fc", C.c_void_p), ("shared_fc_scale", C.c_void_p),
        ("act", C.c_void_p), ("act_kind", C.c_int),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("pdl", C.c_int),
        ("x_bf16", C.c_void_p),
    ]


class MoeDownArgs(C.Structure):
    _fields_ = [
        ("act", C.c_void_p), ("act_kind", C.c_int),
        ("m", C.c_int), ("h", C.c_int), ("i_loc", C.c_int), ("n_experts", C.c_int),
        ("top_k", C.c_int), ("n_shared", C.c_int),
        ("sel", C.c_void_p), ("wt", C.c_void_p), ("proj", C.c_void_p), ("proj_scale", C.c_void_p),
        ("shared_proj", C.c_void_p), ("shared_proj_scale", C.c_void_p),
        ("out", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
        ("tail", C.POINTER(TailArgs)), ("pdl", C.c_int), ("push", C.POINTER(PushArgs)),
    ]


_LIB = None


def lib_path() -> str:
    """The library to load: `IQB200_LIB` (a prebuilt `libiqb200.so` elsewhere) or the in-tree
    build."""
    return os.environ.get("IQB200_LIB") or _build.LIB


def load() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (`iquestrt_b200._build.build`)."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m iquestrt_b200._build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
        lib = C.CDLL(path)
        lib.iq_scratch_bytes.restype = C.c_size_t
        lib.iq_scratch_bytes.argtypes = []
        lib.iq_sm_count.restype = C.c_int
        lib.iq_sm_count.argtypes = []
        lib.iq_status_read.restype = C.c_int
        lib.iq_status_read.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_void_p]
        lib.iq_tail.restype = C.c_int
        lib.iq_tail.argtypes = [C.POINTER(TailArgs), C.c_void_p, C.c_int]
        for name, struct in (("iq_linear", LinearArgs), ("iq_linear_static", LinearArgs),
                             ("iq_qkv_heads", HeadsArgs), ("iq_router", RouterArgs),
                             ("iq_moe_gate", MoeGateArgs), ("iq_moe_down", MoeDownArgs)):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(struct), C.c_void_p]
        lib.iq_linear_static_status.restype = C.c_int
        lib.iq_linear_static_status.argtypes = [C.POINTER(C.c_int), C.c_void_p]
        _LIB = lib
    return _LIB


def check(where: str, code: int) -> None:
    if code != IQ_OK:
        raise IqError(where, code)
