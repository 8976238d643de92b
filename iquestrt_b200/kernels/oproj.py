"""Row-parallel block-FP8 GEMV holders (mirror iquestrt/kernels/oproj.py:147-197)."""

import torch

from .. import ops, parallel

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

    def __call__(self, ao, w_o, w_scale, *, out=None, tail=None, push=None, pdl=False):
        """ao [Q, q_dim] bf16 contiguous, w_o [hidden, q_dim] e4m3 with its rank-local
        [hidden/128, q_dim/128] scales -> [Q, hidden] bf16 (unreduced across ranks).
        `push` (the output's symmetric slot) also sends the rows to every rank's landing
        zone, for an all-reduce tail launched separately."""
        if out is None:
            out = self.next_out()
        if tail is None and push is None:
            push = parallel.slot_of(out)        # the slot's only reader is its all-reduce tail
        view = out[:self.q_len]
        ops.linear(ao.reshape(self.q_len, self.q_dim), w_o, w_scale, scratch=self.scratch,
                   out=view, x_kind=self.x_kind, tail=tail, push=push, pdl=pdl)
        return view


class DenseMlp:
    """Dense SwiGLU MLP: block-FP8 Gate/Up + SiLU, block-FP8 Down into `out` (the
    reference's layer-0 MLP, iquestrt/kernels/oproj.py:174-197; the benchmark
    configuration's shared expert has the same form).  Runs on the grouped-expert kernels
    with the dense weights as one group."""

    def __init__(self, hidden: int, inter: int, *, ws, q_len: int, scratch=None):
        if not 1 <= q_len <= 8:
            raise ValueError(f"the dense MLP covers 1..8 rows, got {q_len}")
        if hidden % 1024 or inter % 128:
            raise ValueError(f"unsupported dense MLP shape H={hidden}, I={inter}")
        self.q_len, self.inter, self.hidden = q_len, inter, hidden
        self.act = ws.slot(("dense", "act"), (q_len, inter), torch.bfloat16)
        self.sel = ws.slot(("dense", "sel"), (q_len,), torch.int32)
        self.wt = ws.slot(("dense", "wt"), (q_len,), torch.float32)
        self.wt.fill_(1.0)
        self._scratch = scratch
        self._tables: dict[tuple[int, int], torch.Tensor] = {}

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.act.device)
        return self._scratch

    def _grain64(self, table: torch.Tensor, dim: int, blocks: int) -> torch.Tensor:
        """The kernels read expert-style tables (one entry per 64 rows of gate/up, per 64
        columns of down).  A checkpoint-grain table (one entry per 128) is widened once per
        weight and kept, so that calls inside a captured graph allocate nothing."""
        if table.shape[dim] == 2 * blocks:
            return table
        if table.shape[dim] != blocks:
            raise ValueError(f"scale table {tuple(table.shape)} does not tile the dense weight")
        key = (table.data_ptr(), dim)
        if key not in self._tables:
            self._tables[key] = table.repeat_interleave(2, dim).contiguous()
        return self._tables[key]

    def __call__(self, hn, w_gate_up, gate_up_scale, w_down, down_scale, out, *, x_scale=None,
                 tail=None, pdl=False):
        """`hn [Q, hidden]` bf16 (quantised per 1x128 group inside the Gate kernel) -> out[:Q]
        bf16, the rank's partial Down output.  `w_gate_up [2I, hidden]` and `w_down
        [hidden, I]` are e4m3 with fp32 scale tables at the checkpoint's 128 grain or at
        the expert kernels' 64 grain.  An `hn` that is already e4m3 is used as is, with
        `x_scale [Q, hidden/128]` (or unscaled when that is None)."""
        q = self.q_len
        gu_scale = self._grain64(gate_up_scale, 0, 2 * self.inter // 128)
        dn_scale = self._grain64(down_scale, 1, self.inter // 128)
        ops.moe_gate(hn, self.sel, w_gate_up.unsqueeze(0), gu_scale.unsqueeze(0), self.act, m=q,
                     top_k=1, scratch=self.scratch, x_scale=x_scale, pdl=pdl)
        return ops.moe_down(self.act, self.sel, self.wt, w_down.unsqueeze(0),
                            dn_scale.unsqueeze(0), out, m=q, top_k=1, scratch=self.scratch,
                            tail=tail, pdl=pdl)
