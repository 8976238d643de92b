"""The MoE router of one decode step in one launch (mirrors RouterSelect,
iquestrt/kernels/router.py:658-699)."""

import torch

from .. import ops


class RouterSelect:
    """x_pad[:Q] -> (sel [Q*k] int32, ascending within each row; wt [Q*k] fp32).

    `score="softmax"` is the reference's rule (softmax over the selected logits);
    `score="sigmoid"` renormalises the selected logits' sigmoids (the benchmark
    configuration).  Calls share the per-device scratch, so they must be serialised on one
    stream, which one captured step is."""

    def __init__(self, n_experts: int, top_k: int, hidden: int, *, device, ws, q_len: int,
                 score: str = "softmax", scratch=None):
        if score not in ("softmax", "sigmoid"):
            raise ValueError(f"score must be 'softmax' or 'sigmoid', got {score!r}")
        if not 1 <= q_len <= 8:
            raise ValueError(f"the router covers 1..8 rows, got {q_len}")
        if hidden % 512 or n_experts % 16 or n_experts > 512 or not 1 <= top_k <= n_experts:
            raise ValueError(f"unsupported router shape H={hidden}, E={n_experts}, k={top_k}")
        target = torch.device(device)
        index = torch.cuda.current_device() if target.index is None else target.index
        self.device = torch.device("cuda", index)
        self.n_experts, self.top_k, self.hidden, self.q_len = n_experts, top_k, hidden, q_len
        self.score = ops.ROUTE_SOFTMAX if score == "softmax" else ops.ROUTE_SIGMOID
        self.sel = ws.slot(("router", "sel"), (q_len * top_k,), torch.int32)
        self.wt = ws.slot(("router", "wt"), (q_len * top_k,), torch.float32)
        self.logits = ws.slot(("router", "logits"), (q_len, n_experts), torch.float32)
        self._scratch = scratch

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.device)
        return self._scratch

    def __call__(self, x_pad: torch.Tensor, weight: torch.Tensor, *, rows=None, pdl=False):
        rows = self.q_len if rows is None else rows
        if not 1 <= rows <= self.q_len:
            raise ValueError(f"rows must be in 1..{self.q_len}, got {rows}")
        for tensor, shape, name in ((x_pad, (None, self.hidden), "x_pad"),
                                    (weight, (self.n_experts, self.hidden), "weight")):
            if (tensor.device != self.device or tensor.dtype != torch.bfloat16
                    or tensor.dim() != 2 or tensor.shape[1] != shape[1]
                    or (shape[0] is not None and tensor.shape[0] != shape[0])
                    or not tensor.is_contiguous()):
                raise ValueError(f"router {name} expected contiguous bf16 [*, {shape[1]}] on "
                                 f"{self.device}, got {tensor.dtype} {tuple(tensor.shape)} on "
                                 f"{tensor.device}")
        if x_pad.shape[0] < rows:
            raise ValueError(f"x_pad holds {x_pad.shape[0]} rows, need {rows}")
        ops.router(x_pad[:rows], weight, top_k=self.top_k, scratch=self.scratch,
                   score=self.score, sel=self.sel, wt=self.wt, logits=self.logits[:rows],
                   pdl=pdl)
        return self.sel, self.wt
