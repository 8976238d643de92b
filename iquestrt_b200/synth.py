"""Seeded synthetic weights and activations of the decode layer, at any TP degree.

There is no checkpoint, so every weight is random-init with the distributions of the
benchmark configurations: e4m3 weights from N(0,1) clamped to +-448, fp32 scales
log-uniform in [2^-12, 2^-6] per 128x128 block of the GLOBAL matrix, then sharded the
way the reference shards its checkpoint (row-parallel o_proj and expert proj on the
contraction dim, expert fc on its rows, router replicated; rank-local expert scale tables
at grain 64 -- iquestrt/weights.py:358-439, iquestrt/blockfp8.py:24-36).  Every rank of
a TP group derives its shard from the same global tensors, so TP=1/2/4/8 see the same
problem."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .blockfp8 import shard_scale

E4M3 = torch.float8_e4m3fn
BLOCK = 128
EXPERT_GRAIN = 64


@dataclass(frozen=True)
class LayerShape:
    hidden: int = 6144
    q_dim: int = 8192          # o_proj contraction (q heads x head_dim), sharded over TP
    n_experts: int = 256
    top_k: int = 8
    inter: int = 2048          # expert intermediate, sharded over TP
    n_shared: int = 1
    eps: float = 1e-6

    def local(self, tp: int):
        if self.q_dim % (tp * BLOCK) or self.inter % (tp * EXPERT_GRAIN):
            raise ValueError(f"TP={tp} does not tile q_dim={self.q_dim} / inter={self.inter}")
        return self.q_dim // tp, self.inter // tp


BASELINE = LayerShape()
# The reference model's own dimensions (iquestrt/engine.py:291-295,
# iquestrt/kernels/sm100_moe_fp8.py:11): no shared expert.
REFERENCE_Q1 = LayerShape(hidden=3072, q_dim=6144, n_experts=256, top_k=8, inter=1536,
                          n_shared=0)


def _gen(device, *seed):
    g = torch.Generator(device=device)
    s = 0x9E3779B97F4A7C15
    for v in seed:
        s = (s * 6364136223846793005 + int(v) + 1442695040888963407) % (1 << 63)
    g.manual_seed(s)
    return g


def fp8_weight(rows, cols, gen, device):
    """e4m3 [rows, cols] from N(0,1) clamped to +-448."""
    w = torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float32)
    return w.clamp_(-448.0, 448.0).to(E4M3)


def block_scales(rows, cols, gen, device):
    """fp32 [rows/128, cols/128], log-uniform in [2^-12, 2^-6]."""
    u = torch.rand(rows // BLOCK, cols // BLOCK, generator=gen, device=device,
                   dtype=torch.float32)
    return torch.exp2(-12.0 + 6.0 * u)


def _expert_shard(shape: LayerShape, tp, rank, device, *seed):
    """One expert's rank-local ([gate;up] fc, fc_scale, proj, proj_scale)."""
    h, i = shape.hidden, shape.inter
    il = i // tp
    g = _gen(device, *seed)
    gate_up = fp8_weight(2 * i, h, g, device)
    gu_scale = block_scales(2 * i, h, g, device)
    down = fp8_weight(h, i, g, device)
    d_scale = block_scales(h, i, g, device)
    r0 = rank * il
    fc = torch.cat([gate_up[r0:r0 + il], gate_up[i + r0:i + r0 + il]], 0).contiguous()
    fc_scale = torch.cat([shard_scale(gu_scale, 0, r0, il, EXPERT_GRAIN),
                          shard_scale(gu_scale, 0, i + r0, il, EXPERT_GRAIN)], 0).contiguous()
    proj = down[:, r0:r0 + il].contiguous()
    proj_scale = shard_scale(d_scale, 1, r0, il, EXPERT_GRAIN).contiguous()
    return fc, fc_scale, proj, proj_scale


def make_layer(shape: LayerShape, *, tp=1, rank=0, device="cuda", seed=0, layer=0):
    """Rank-local weights of one decode layer as a dict of tensors on `device`."""
    if not 0 <= rank < tp:
        raise ValueError(f"rank {rank} outside a tensor-parallel group of {tp}")
    h = shape.hidden
    ql, il = shape.local(tp)
    out = {}
    g = _gen(device, seed, layer, 1)
    o_full = fp8_weight(h, shape.q_dim, g, device)
    o_scale = block_scales(h, shape.q_dim, g, device)
    out["o_proj"] = o_full[:, rank * ql:(rank + 1) * ql].contiguous()
    out["o_scale"] = shard_scale(o_scale, 1, rank * ql, ql, BLOCK).contiguous()
    del o_full
    for name in ("attn_out_norm", "feed_forward_norm", "next_attention_norm"):
        out[name] = 0.5 + torch.rand(h, generator=g, device=device, dtype=torch.float32)
    router = torch.randn(shape.n_experts, h, generator=g, device=device,
                         dtype=torch.float32) * 0.02
    out["router"] = router.to(torch.bfloat16)
    e = shape.n_experts
    fc = torch.empty(e, 2 * il, h, dtype=E4M3, device=device)
    fc_scale = torch.empty(e, 2 * il // EXPERT_GRAIN, h // BLOCK, dtype=torch.float32,
                           device=device)
    proj = torch.empty(e, h, il, dtype=E4M3, device=device)
    proj_scale = torch.empty(e, h // BLOCK, il // EXPERT_GRAIN, dtype=torch.float32,
                             device=device)
    for x in range(e):
        fc[x], fc_scale[x], proj[x], proj_scale[x] = _expert_shard(
            shape, tp, rank, device, seed, layer, 2, x)
    out.update(fc=fc, fc_scale=fc_scale, proj=proj, proj_scale=proj_scale)
    if shape.n_shared:
        parts = [_expert_shard(shape, tp, rank, device, seed, layer, 3, s)
                 for s in range(shape.n_shared)]
        out["shared_fc"] = torch.stack([p[0] for p in parts]).contiguous()
        out["shared_fc_scale"] = torch.stack([p[1] for p in parts]).contiguous()
        out["shared_proj"] = torch.stack([p[2] for p in parts]).contiguous()
        out["shared_proj_scale"] = torch.stack([p[3] for p in parts]).contiguous()
    return out


@dataclass(frozen=True)
class HeadShape:
    """Attention heads of the benchmark's decoder slice: 64 query and 8 key/value heads of
    128 channels, rotary embedding on the first 32."""
    q_heads: int = 64
    kv_heads: int = 8
    head_dim: int = 128
    rotary_dim: int = 32
    theta: float = 10000.0

    def local(self, tp: int):
        if self.q_heads % tp or self.kv_heads % tp:
            raise ValueError(f"TP={tp} does not divide {self.q_heads} / {self.kv_heads} heads")
        return self.q_heads // tp, self.kv_heads // tp


HEADS = HeadShape()


def make_prologue(shape: LayerShape, heads: HeadShape = HEADS, *, tp=1, rank=0, device="cuda",
                  seed=0, layer=0):
    """Rank-local weights of one layer's attention prologue: the column-parallel QKV weight
    (this rank's query heads, then its key heads, then its value heads: rows of the global
    [q | k | v] matrix) with its block scales, and the q / k norm weights."""
    qh, kh = heads.local(tp)
    d, h = heads.head_dim, shape.hidden
    g = _gen(device, seed, layer, 7)
    parts, scales = [], []
    # (one global tensor per projection, generated whole so that every TP degree sees the
    # same problem; a rank keeps its heads' rows)
    for n_heads, mine in ((heads.q_heads, qh), (heads.kv_heads, kh), (heads.kv_heads, kh)):
        w = fp8_weight(n_heads * d, h, g, device)
        sc = block_scales(n_heads * d, h, g, device)
        r0, n = rank * mine * d, mine * d
        parts.append(w[r0:r0 + n])
        scales.append(shard_scale(sc, 0, r0, n, BLOCK))
    return {"w_qkv": torch.cat(parts, 0).contiguous(),
            "w_qkv_scale": torch.cat(scales, 0).contiguous(),
            "w_qn": 0.5 + torch.rand(d, generator=g, device=device, dtype=torch.float32),
            "w_kn": 0.5 + torch.rand(d, generator=g, device=device, dtype=torch.float32)}


def rope_tables(positions, heads: HeadShape = HEADS, *, device="cuda"):
    """bf16 (cos, sin) `[len(positions), rotary_dim]` of the partial rotary embedding (the
    two halves of the rotated channels share their angles)."""
    rot = heads.rotary_dim
    pos = torch.as_tensor(positions, dtype=torch.float32)
    inv = heads.theta ** (-torch.arange(0, rot, 2, dtype=torch.float32) / rot)
    ang = torch.cat([pos[:, None] * inv[None, :]] * 2, dim=-1)
    return ang.cos().bfloat16().to(device), ang.sin().bfloat16().to(device)


def make_step_inputs(shape: LayerShape, m, *, tp=1, rank=0, device="cuda", seed=0, step=0):
    """Activations of one decode step: the attention output `ao [m, q_dim/tp]` (this rank's
    head slice of a global N(0,1) tensor) and the residual `[m, hidden]`, both bf16."""
    ql, _ = shape.local(tp)
    g = _gen(device, seed, 1000 + step)
    ao = torch.randn(m, shape.q_dim, generator=g, device=device, dtype=torch.float32)
    res = torch.randn(m, shape.hidden, generator=g, device=device, dtype=torch.float32)
    return (ao[:, rank * ql:(rank + 1) * ql].to(torch.bfloat16).contiguous(),
            res.to(torch.bfloat16))


def make_linear_case(n, k, m, *, device="cuda", seed=0):
    """Benchmark configuration 0: bf16 activation ~N(0,1) `[m,k]`, e4m3 weight `[n,k]`,
    fp32 128x128 block scales."""
    g = _gen(device, seed, 7)
    x = torch.randn(m, k, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    w = fp8_weight(n, k, g, device)
    s = block_scales(n, k, g, device)
    return x, w, s
