"""Layer-tail arena state (mirrors iquestrt/kernels/tail.py:6-39)."""

import torch


class TailKernels:
    """The arena slots the all-reduce tails write.  `eps` and the two residual scales are
    passed to the kernels by value (a captured graph bakes them in either way), so they
    are plain floats here rather than one-element device tensors."""

    def __init__(self, hidden: int, eps: float, *, ws, q_len: int):
        self.hidden = hidden
        self.q_len = q_len
        self.eps = float(eps)

        def slot(key, shape, dtype):
            return ws.slot(("tail", key), shape, dtype)

        self.h = slot("h", (q_len, hidden), torch.bfloat16)
        self.hn = slot("hn", (q_len, hidden), torch.bfloat16)
        self.out = slot("out", (q_len, hidden), torch.bfloat16)
        # The recursive draft's fp32 residual stream.
        self.h32 = slot("h32", (q_len, hidden), torch.float32)
        self.out32 = slot("out32", (q_len, hidden), torch.float32)
        self._scales = (None, None)

    def _prep(self, a_scale, f_scale):
        self._scales = (a_scale, f_scale)
