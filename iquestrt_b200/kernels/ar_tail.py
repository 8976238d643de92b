"""All-reduce fused with the residual add and RMSNorm(s) (mirrors MultimemARTail /
MultimemMLPTail, iquestrt/kernels/ar_tail.py:1260-1622).

Each holder can run its epilogue as its own launch (`__call__`, the reference's form) or
hand a `spec(...)` to the producing GEMV (`OProjGemv.__call__(..., tail=spec)`,
`MoeDecodeKernels.__call__(..., tail=spec)`), which then performs the all-reduce from
inside its own epilogue."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from .. import ops, parallel
from .tail import TailKernels


def _check(name, t, dtype, device, numel=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.device != device:
        raise ValueError(f"{name} must be on {device}, got {t.device}")
    if t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if numel is not None and t.numel() != numel:
        raise ValueError(f"{name} must contain {numel} elements, got {t.numel()}")


class MultimemARTail:
    """All-reduce + residual + two RMSNorms (the attention tail)."""

    def __init__(self, ao_buffers: Sequence[torch.Tensor], *, group=None, tail: TailKernels,
                 scratch=None, timeout_ms: int = 2000):
        if not isinstance(tail, TailKernels):
            raise TypeError("tail must be a TailKernels instance")
        buffers = tuple(ao_buffers)
        if len(buffers) != 2:
            raise ValueError("the all-reduce needs exactly two alternating buffers, got "
                             f"{len(buffers)}")
        self.tail = tail
        self.q_len, self.hidden = tail.q_len, tail.hidden
        self.device = buffers[0].device
        self._slots = {}
        for i, buf in enumerate(buffers):
            _check(f"buffer {i}", buf, torch.bfloat16, self.device)
            slot = parallel.slot_of(buf)
            if slot is None:
                raise ValueError(f"buffer {i} is not a symmetric workspace slot")
            if buf.shape[-1] != self.hidden or buf.shape[0] < self.q_len:
                raise ValueError(f"buffer {i} must be [>= {self.q_len}, {self.hidden}]")
            self._slots[buf.data_ptr()] = slot
        if buffers[0].data_ptr() == buffers[1].data_ptr():
            raise ValueError("the two buffers alias")
        self.world, self.rank = next(iter(self._slots.values())).world, \
            next(iter(self._slots.values())).rank
        self.group = group
        self.ao_buffers = buffers
        self.timeout_ms = timeout_ms
        self.inv = torch.empty(self.q_len, dtype=torch.float32, device=self.device)
        self._scratch = scratch

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.device)
        return self._scratch

    def _slot(self, buf, name):
        try:
            return self._slots[buf.data_ptr()]
        except KeyError as exc:
            raise ValueError(f"{name} must be the [:Q] base view of one of the two "
                             "registered symmetric buffers") from exc

    def spec(self, ao, residual, w_ao, w_ffn, a_scale, f_scale, *, rows=None, h_out=None,
             norm_out=None, norm_fp8=None, norm_fp8_scale=None, inv_out=None) -> ops.TailSpec:
        """The attention tail's arguments for `ao` (a view of a registered buffer)."""
        q = self.q_len if rows is None else rows
        slot = self._slot(ao, "ao")
        fp32 = residual.dtype == torch.float32
        _check("residual", residual, torch.float32 if fp32 else torch.bfloat16, self.device)
        _check("w_ao", w_ao, torch.float32, self.device, self.hidden)
        _check("w_ffn", w_ffn, torch.float32, self.device, self.hidden)
        self.tail._prep(a_scale, f_scale)
        if h_out is None:
            h_out = self.tail.h32 if fp32 else self.tail.h
        if norm_out is None:
            norm_out = self.tail.hn
        return ops.TailSpec(
            kind=ops.TAIL_ATTN, partial=ao[:q], residual=residual[:q], w_first=w_ao,
            w_norm=w_ffn, h_out=h_out[:q], norm_out=norm_out[:q], scale=float(a_scale),
            eps=self.tail.eps, norm_fp8=None if norm_fp8 is None else norm_fp8[:q],
            norm_fp8_scale=None if norm_fp8_scale is None else norm_fp8_scale[:q],
            inv_out=None if inv_out is None else inv_out[:q], comm=slot,
            timeout_ms=self.timeout_ms)

    def __call__(self, ao, residual, w_ao, w_ffn, a_scale, f_scale, *, pdl=False):
        """Reduce `ao` and write/return `(tail.h, tail.hn)`; an fp32 `residual` keeps the
        sum fp32: `(tail.h32, tail.hn)`."""
        spec = self.spec(ao, residual, w_ao, w_ffn, a_scale, f_scale)
        ops.tail(spec, self.scratch, pdl=pdl)
        return spec.h_out, spec.norm_out

    def h_inv_xpad_fp8_pdl_overlap_local(self, ao, residual, w_ao, w_ffn, inv_out, x_pad,
                                         x_pad_fp8, a_scale, f_scale, *, fp32_residual=False,
                                         x_pad_scale=None, pdl=False):
        """The MoE layer's attention tail: `h`, the second norm's inverse RMS, and the
        router / MoE inputs `x_pad` (bf16) and `x_pad_fp8` (e4m3; with 1x128 group scales
        into `x_pad_scale` when given)."""
        if fp32_residual != (residual.dtype == torch.float32):
            raise ValueError("fp32_residual does not match the residual's dtype")
        spec = self.spec(ao, residual, w_ao, w_ffn, a_scale, f_scale, norm_out=x_pad,
                         norm_fp8=x_pad_fp8, norm_fp8_scale=x_pad_scale, inv_out=inv_out)
        ops.tail(spec, self.scratch, pdl=pdl)
        return spec.h_out


class MultimemMLPTail(MultimemARTail):
    """MoE all-reduce + `out = residual + mlp * f_scale` + the next attention norm."""

    def __init__(self, mlp_buffers: Sequence[torch.Tensor], *, group=None, tail: TailKernels,
                 norm_out: torch.Tensor, scratch=None, timeout_ms: int = 2000):
        super().__init__(mlp_buffers, group=group, tail=tail, scratch=scratch,
                         timeout_ms=timeout_ms)
        _check("norm_out", norm_out, torch.bfloat16, self.device, self.q_len * self.hidden)
        self.norm_out = norm_out

    def spec(self, mlp_out, residual, f_scale, w_norm, *, rows=None, out=None,
             norm_fp8=None, norm_fp8_scale=None) -> ops.TailSpec:
        q = self.q_len if rows is None else rows
        slot = self._slot(mlp_out, "mlp_out")
        _check("residual", residual, torch.bfloat16, self.device)
        _check("w_norm", w_norm, torch.float32, self.device, self.hidden)
        a_scale = self.tail._scales[0]
        self.tail._prep(1.0 if a_scale is None else a_scale, f_scale)
        out = self.tail.out if out is None else out
        return ops.TailSpec(
            kind=ops.TAIL_MLP, partial=mlp_out[:q], residual=residual[:q], w_norm=w_norm,
            h_out=out[:q], norm_out=self.norm_out.view(self.q_len, self.hidden)[:q],
            scale=float(f_scale), eps=self.tail.eps,
            norm_fp8=None if norm_fp8 is None else norm_fp8[:q],
            norm_fp8_scale=None if norm_fp8_scale is None else norm_fp8_scale[:q],
            comm=slot, timeout_ms=self.timeout_ms)

    def __call__(self, mlp_out, residual, f_scale, w_norm, *, pdl=False):
        spec = self.spec(mlp_out, residual, f_scale, w_norm)
        ops.tail(spec, self.scratch, pdl=pdl)
        return spec.h_out, spec.norm_out
