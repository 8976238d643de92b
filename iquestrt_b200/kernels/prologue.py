"""The attention prologue of one decode layer: column-parallel block-FP8 QKV product, then
per-head q/k RMSNorm, partial rotary embedding and the KV-cache write (mirrors
`PrologueKernels`, iquestrt/kernels/prologue.py:240-296).

The QKV product has no all-reduce (its OUTPUT dim is sharded): it is the streaming GEMV of
`ops.linear` with the fp32 result kept (the reference's heads kernel also normalises the
un-rounded fp32 product).  The heads step is one small launch, `ops.qkv_heads`."""

import torch

from .. import ops


class PrologueKernels:
    """QKV + heads over arena slots for `q_len` rows of a rank's head shard."""

    def __init__(self, hidden: int, q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                 eps: float, *, ws, q_len: int, activation: str | None = None, scratch=None):
        if not 1 <= q_len <= 8:
            raise ValueError(f"the prologue covers 1..8 rows, got {q_len}")
        if activation is None:
            # the reference's QKV product is W8A16: keep bf16 precision (two e4m3 terms per
            # activation) where the rows fit the MMA's eight columns
            activation = "w8a16" if q_len <= 4 else "group"
        if activation not in ("group", "w8a16") or (activation == "w8a16" and q_len > 4):
            raise ValueError(f"unsupported activation {activation!r} for {q_len} rows")
        self.x_kind = ops.X_BF16_SPLIT2 if activation == "w8a16" else ops.X_BF16_GROUPQ
        if head_dim % 2 or head_dim > 256 or rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"unsupported head shape D={head_dim}, rotary={rotary_dim}")
        self.hidden, self.q_len, self.eps = hidden, q_len, float(eps)
        self.q_heads, self.kv_heads, self.head_dim = q_heads, kv_heads, head_dim
        self.rotary_dim = rotary_dim
        self.n_qkv = (q_heads + 2 * kv_heads) * head_dim

        def slot(key, shape, dtype):
            return ws.slot(("prologue", key), shape, dtype)

        self.qkv = slot("qkv", (q_len, self.n_qkv), torch.float32)
        self.q = slot("q", (q_len, q_heads, head_dim), torch.bfloat16)
        self._scratch = scratch

    @property
    def scratch(self):
        if self._scratch is None:
            self._scratch = ops.default_scratch(self.qkv.device)
        return self._scratch

    def call_prenorm(self, xn, w_qkv, w_scale, w_qn, w_kn, cos, sin, slot, k_cache, v_cache, *,
                     pdl=False):
        """QKV + heads when `xn [Q, hidden]` (bf16) was emitted by the MLP all-reduce tail:
        returns `(xn, q [Q, q_heads, D])`; k and v go straight into rows `slot` of the
        caches.  `w_qkv [n_qkv, hidden]` is e4m3 with its rank-local `[n_qkv/128,
        hidden/128]` scale table."""
        xn = xn.reshape(self.q_len, self.hidden)
        ops.linear(xn, w_qkv, w_scale, scratch=self.scratch, x_kind=self.x_kind,
                   out_f32=self.qkv, pdl=pdl)
        return xn, self.heads(w_qn, w_kn, cos, sin, slot, k_cache, v_cache, pdl=pdl)

    def heads(self, w_qn, w_kn, cos, sin, slot, k_cache, v_cache, *, pdl=False):
        """The heads step over `self.qkv` -> q [Q, q_heads, D]."""
        q = self.q_len
        return ops.qkv_heads(self.qkv, w_qn, w_kn,
                             cos.reshape(q, -1)[:, :self.rotary_dim].contiguous(),
                             sin.reshape(q, -1)[:, :self.rotary_dim].contiguous(),
                             slot.reshape(q), self.q, k_cache, v_cache, q_heads=self.q_heads,
                             kv_heads=self.kv_heads, rotary_dim=self.rotary_dim, eps=self.eps,
                             scratch=self.scratch, pdl=pdl)
