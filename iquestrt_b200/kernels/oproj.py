"""Row-parallel block-FP8 GEMV holders (mirror iquestrt/kernels/oproj.py:147-197)."""

import torch

from .. import ops

BM = 16   # rows of the symmetric output slots (the reference pads its MMA M to 16)


class OProjGemv:
    """`ao [Q, q_dim] @ dequant(w_o).T` into one of two alternating symmetric output slots.

    The slots alternate because the all-reduce has no output barrier: a rank that has
    finished call n may already write call n+1's partial while a peer still reads call
    n's.  Pass `tail=` (an `ops.TailSpec` from `MultimemARTail.spec(...)`) to run the
    all-reduce epilogue inside the same launch.

    `activation` picks how the bf16 `ao` meets the e4m3 weight: "group" quantises it per
    1x128 group in the kernel (the benchmark configuration's format); "w8a16" keeps bf16
    precision with two e4m3 terms per value (the reference's W8A16 product), Q <= 4."""

    def __init__(self, q_dim: int, hidden: int, *, ws, q_len: int, activation="group",
                 scratch=None):
        if not 1 <= q_len <= 8:
            raise ValueError(f"the OProj covers 1..8 rows, got {q_len}")
        if activation not in ("group", "w8a16"):
            raise ValueError(f"activation must be 'group' or 'w8a16', got {activation!r}")
        if activation == "w8a16" and q_len > 4:
            raise ValueError("the two-term W8A16 product covers at most 4 rows")
        self.q_dim, self.hidden, self.q_len = q_dim, hidden, q_len
        self.x_kind = ops.X_BF16_GROUPQ if activation == "group" else ops.X_BF16_SPLIT2
        self.outputs = tuple(
            ws.slot(("oproj", key), (BM, hidden), torch.bfloat16, symm=True)
            for key in ("out", "out_alt"))
        self._next_output = 0
        self._scratch = scratch

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.outputs[0].device)
        return self._scratch

    def next_out(self) -> torch.Tensor:
        out = self.outputs[self._next_output]
        self._next_output = (self._next_output + 1) % len(self.outputs)
        return out

    def __call__(self, ao, w_o, w_scale, *, out=None, tail=None, pdl=False):
        """ao [Q, q_dim] bf16 contiguous, w_o [hidden, q_dim] e4m3 with its rank-local
        [hidden/128, q_dim/128] scales -> [Q, hidden] bf16 (unreduced across ranks)."""
        if out is None:
            out = self.next_out()
        view = out[:self.q_len]
        ops.linear(ao.reshape(self.q_len, self.q_dim), w_o, w_scale, scratch=self.scratch,
                   out=view, x_kind=self.x_kind, tail=tail, pdl=pdl)
        return view


class DenseMlp:
    """Dense SwiGLU MLP: block-FP8 Gate/Up + SiLU, block-FP8 Down into `out` (the
    reference's layer-0 MLP; the benchmark configuration's shared expert has the same
    form).  Runs on the grouped-expert kernels with the dense weights as one group."""

    def __init__(self, hidden: int, inter: int, *, ws, q_len: int, scratch=None):
        if not 1 <= q_len <= 8:
            raise ValueError(f"the dense MLP covers 1..8 rows, got {q_len}")
        self.q_len, self.inter, self.hidden = q_len, inter, hidden
        self.x_fp8 = ws.slot(("dense", "x_fp8"), (q_len, hidden), torch.float8_e4m3fn)
        self.x_scale = ws.slot(("dense", "x_scale"), (q_len, hidden // 128), torch.float32)
        self.act = ws.slot(("dense", "act"), (q_len, inter), torch.bfloat16)
        self.sel = ws.slot(("dense", "sel"), (q_len,), torch.int32)
        self.wt = ws.slot(("dense", "wt"), (q_len,), torch.float32)
        self.wt.fill_(1.0)
        self._scratch = scratch

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.act.device)
        return self._scratch

    def __call__(self, x_fp8, x_scale, w_gate_up, gate_up_scale, w_down, down_scale, out, *,
                 tail=None, pdl=False):
        """`x_fp8 [Q, hidden]` e4m3 with `x_scale [Q, hidden/128]` (or None) -> out[:Q]
        bf16, the rank's partial Down output.  Scale tables at grain (64, 128) for
        gate/up and (128, 64) for down, like the expert banks."""
        q = self.q_len
        ops.moe_gate(x_fp8, self.sel, w_gate_up.unsqueeze(0), gate_up_scale.unsqueeze(0),
                     self.act, m=q, top_k=1, scratch=self.scratch, x_scale=x_scale, pdl=pdl)
        return ops.moe_down(self.act, self.sel, self.wt, w_down.unsqueeze(0),
                            down_scale.unsqueeze(0), out, m=q, top_k=1,
                            scratch=self.scratch, tail=tail, pdl=pdl)
