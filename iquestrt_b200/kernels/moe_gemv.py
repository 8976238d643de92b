"""The decode MoE holder: grouped block-FP8 Gate+SiLU then Down (mirrors
MoeDecodeKernels, iquestrt/kernels/moe_gemv.py:8-61)."""

import torch

from .. import ops, parallel

ROW_BM = 16


class MoeDecodeKernels:
    """Block-FP8 Gate+SiLU, then block-FP8 Down into a rotating symmetric output.

    Each distinct routed expert of the live rows is streamed once and applied to every
    row routed to it.  `act_format="e4m3"` keeps the reference's unscaled e4m3
    activations; `"bf16"` carries the Gate's output in bf16 and quantises it per 1x128
    group inside the Down (the benchmark configuration's format).  `n_shared` shared
    experts (same shapes as a routed expert) join both kernels as extra groups."""

    def __init__(self, experts: int, topk: int, hidden: int, i_loc: int, *, ws, q_len: int,
                 live_rows=(), n_shared: int = 0, act_format: str = "e4m3", scratch=None):
        if not 1 <= q_len <= 8 or q_len * topk > 64:
            raise ValueError(f"the MoE covers 1..8 rows and at most 64 routed pairs, got "
                             f"Q={q_len}, top_k={topk}")
        if hidden % 1024 or i_loc % 64:
            raise ValueError(f"unsupported MoE shape H={hidden}, I_loc={i_loc}")
        if act_format not in ("e4m3", "bf16"):
            raise ValueError(f"act_format must be 'e4m3' or 'bf16', got {act_format!r}")
        if act_format == "bf16" and i_loc % 128:
            raise ValueError("1x128 activation groups need I_loc % 128 == 0")
        live_rows = tuple(live_rows)
        if not all(1 <= r <= q_len for r in live_rows):
            raise ValueError(f"live_rows must be in 1..{q_len}, got {live_rows}")
        self.experts, self.topk, self.hidden, self.i_loc = experts, topk, hidden, i_loc
        self.q_len, self.n_shared = q_len, n_shared
        slots = topk + n_shared
        self.x_pad = ws.slot(("moe", "x_pad"), (ROW_BM, hidden), torch.bfloat16)
        self.x_pad_fp8 = ws.slot(("moe", "x_pad_fp8"), (ROW_BM, hidden), torch.float8_e4m3fn)
        self.x_pad_scale = ws.slot(("moe", "x_pad_scale"), (ROW_BM, hidden // 128),
                                   torch.float32)
        act_dtype = torch.float8_e4m3fn if act_format == "e4m3" else torch.bfloat16
        self.act = ws.slot(("moe", "act"), (q_len * slots, i_loc), act_dtype)
        self.act_fp8 = self.act if act_format == "e4m3" else None
        self.outputs = tuple(
            ws.slot(("moe", "out", index), (ROW_BM, hidden), torch.bfloat16, symm=True)
            for index in range(2))
        self._out_index = 0
        self._scratch = scratch

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.act.device)
        return self._scratch

    def next_out(self) -> torch.Tensor:
        """The next of the two output slots (see `OProjGemv`)."""
        out = self.outputs[self._out_index]
        self._out_index ^= 1
        return out

    def __call__(self, sel, wt, fc, fc_scale, proj, proj_scale, *, rows=None, x_scale=None,
                 shared=None, tail=None, push=None, out=None, pdl=False):
        """Routed pairs `sel`/`wt` [Q*topk] -> [rows, H] bf16, unreduced across ranks.

        `x_pad_fp8` (and `x_scale`, when the activations carry 1x128 group scales) were
        written by the attention tail; `sel` is int32, ascending by expert id within each
        row.  `shared = (fc, fc_scale, proj, proj_scale)` of the shared experts.  `tail`
        runs the MLP all-reduce epilogue inside the Down launch; `push` (the output's
        symmetric slot) only sends the rows, for a tail launched separately."""
        rows = self.q_len if rows is None else rows
        if not 1 <= rows <= self.q_len:
            raise ValueError(f"rows must be in 1..{self.q_len}, got {rows}")
        if (shared is None) != (self.n_shared == 0):
            raise ValueError("shared expert weights do not match n_shared")
        if out is None:
            out = self.next_out()
        if tail is None and push is None:
            push = parallel.slot_of(out)        # the slot's only reader is its all-reduce tail
        sfc = sfs = spj = sps = None
        if shared is not None:
            sfc, sfs, spj, sps = shared
        ops.moe_gate(self.x_pad_fp8, sel, fc, fc_scale, self.act, m=rows, top_k=self.topk,
                     scratch=self.scratch, x_scale=x_scale, shared_fc=sfc,
                     shared_fc_scale=sfs, pdl=pdl)
        return ops.moe_down(self.act, sel, wt, proj, proj_scale, out, m=rows, top_k=self.topk,
                            scratch=self.scratch, shared_proj=spj, shared_proj_scale=sps,
                            tail=tail, push=push, pdl=pdl)
