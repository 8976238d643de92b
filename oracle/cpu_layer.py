"""The decode layer on host cores with the reference's torch algebra (bf16 activations,
fp32 dequantise-and-matmul).  TEST INFRASTRUCTURE / CPU BASELINE ONLY.

Composes `oracle.ref_path` in the order of the reference's `layer_forward`
(iquestrt/model/reference.py:124-143) with its MoE (iquestrt/kernels/prefill.py:142-185)
restricted to the routed experts, plus the benchmark configuration's shared expert as a
dense SwiGLU MLP (iquestrt/model/reference.py:70-74)."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ref_path as R


def shared_expert(hn, lw, s):
    gu = R.linear(hn, lw["shared_fc"][s], lw["shared_fc_scale"][s], (64, 128))
    half = gu.shape[-1] // 2
    act = F.silu(gu[:, :half]) * gu[:, half:]
    return R.linear(act, lw["shared_proj"][s], lw["shared_proj_scale"][s], (128, 64))


def layer_cpu(lw_ranks, ao_ranks, residual, *, top_k, n_shared, eps, a_scale=1.0, f_scale=1.0,
              score="softmax", routes=None):
    """One layer over `len(lw_ranks)` simulated TP ranks: per-rank partial products, a
    Python sum for each all-reduce.  `routes = (sel, wt)` replaces the layer's own top-k
    (to compare two implementations on identical routes when a top-k margin is too small
    for them to agree).  Returns (out, norm_out, sel, wt)."""
    parts = [R.linear(ao, lw["o_proj"], lw["o_scale"]) for lw, ao in zip(lw_ranks, ao_ranks)]
    lw0 = lw_ranks[0]
    h, hn = R.layer_residual_algebra(parts, residual, lw0["attn_out_norm"],
                                     lw0["feed_forward_norm"], a_scale, eps)
    logits = R.router_logits(hn, lw0["router"])
    sel, wt, _ = R.select_topk(logits, top_k, score)
    if routes is not None:
        sel, wt = routes
    mlp = None
    for lw in lw_ranks:
        part = R.moe_prefill(hn, sel, wt, lw["fc"], lw["fc_scale"], lw["proj"], lw["proj_scale"])
        for s in range(n_shared):
            part = part + shared_expert(hn, lw, s)
        mlp = part if mlp is None else mlp + part
    out = h + mlp * f_scale
    return out, R.rms_norm(out, lw0["next_attention_norm"], eps), sel, wt
