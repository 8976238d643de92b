"""Generates `tests/golden/*.pt` by running the REFERENCE's own Python code on CPU.

Run where the reference is checked out, giving the checkout's root:

    python tests/golden/make_golden.py <reference_root>          # both fixture files
    python tests/golden/make_golden.py <reference_root> heads    # reference_heads.pt only

The reference has no golden vectors for this path, so these fixtures are outputs of the
reference itself on small seeded inputs: `iquestrt.blockfp8.dequant / shard_scale`,
`iquestrt.model.reference.linear / rms_norm / dense_mlp / layer_forward` (with a stub
attention and an injected all-reduce over simulated ranks), and
`iquestrt.kernels.prefill.moe` with only its Triton `_combine` launch replaced by the
same arithmetic in torch (separately rounded multiply and add, routes in ascending
expert order).  The fixtures pin `oracle/ref_path.py`; nothing at test time reads the
reference."""

from __future__ import annotations

import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
E4M3 = torch.float8_e4m3fn


def fp8(rows, cols, g):
    return torch.randn(rows, cols, generator=g).clamp_(-448, 448).to(E4M3)


def scales(r, c, g):
    return torch.exp2(-12 + 6 * torch.rand(r, c, generator=g))


class _Combine:
    """CPU stand-in for the Triton launch `_combine[grid](down, weights, inverse, out, H,
    top_k, B)` with the kernel's arithmetic (iquestrt/kernels/prefill.py:117-139)."""

    def __getitem__(self, grid):
        def run(down, weights, inverse, out, h, top_k, b, **_):
            rows = out.shape[0]
            for row in range(rows):
                acc = torch.zeros(h, dtype=torch.float32)
                for slot in range(top_k):
                    route = int(inverse[row * top_k + slot])
                    value = down[route].to(torch.bfloat16).to(torch.float32)
                    product = value * weights[row, slot]
                    acc = acc + product
                out[row] = acc.to(out.dtype)
        return run


def main(ref_root):
    sys.path.insert(0, ref_root)
    from iquestrt import blockfp8
    from iquestrt.kernels import prefill
    from iquestrt.model import reference

    g = torch.Generator().manual_seed(1234)
    out = {}

    # ---- blockfp8.dequant / shard_scale
    q = fp8(256, 384, g)
    s = scales(2, 3, g)
    out["dequant"] = dict(q=q, s=s, f64=blockfp8.dequant(q, s),
                          f32=blockfp8.dequant(q, s, dtype=torch.float32))
    q64 = fp8(128, 256, g)
    s64 = scales(2, 2, g)
    out["dequant_64x128"] = dict(q=q64, s=s64, block=(64, 128),
                                 f32=blockfp8.dequant(q64, s64, (64, 128), torch.float32))
    table = scales(4, 6, g)
    out["shard_scale"] = [
        dict(table=table, dim=d, start=st, length=ln, grain=gr,
             out=blockfp8.shard_scale(table, d, st, ln, gr))
        for d, st, ln, gr in [(0, 128, 256, 128), (1, 192, 192, 64), (0, 64, 64, 64),
                              (1, 0, 768, 128)]]

    # ---- reference.linear / rms_norm (configuration-0 shapes, reduced)
    x = torch.randn(3, 384, generator=g).bfloat16()
    out["linear"] = dict(x=x, q=q, s=s, y=reference.linear(x, q, s))
    w = 0.5 + torch.rand(384, generator=g)
    out["rms_norm"] = dict(x=x, w=w, eps=1e-6, y=reference.rms_norm(x, w, 1e-6),
                           y32=reference.rms_norm(x.float(), w, 1e-6))

    # ---- prefill.moe with the Triton combine replaced (E=8, top-4, H=256, I=128)
    e, top_k, h, inter = 8, 4, 256, 128
    lw = types.SimpleNamespace(
        router=torch.randn(e, h, generator=g) * 0.02,
        experts_fc=torch.stack([fp8(2 * inter, h, g) for _ in range(e)]),
        fc_scale=torch.stack([scales(2 * inter // 64, h // 128, g) for _ in range(e)]),
        experts_proj=torch.stack([fp8(h, inter, g) for _ in range(e)]),
        proj_scale=torch.stack([scales(h // 128, inter // 64, g) for _ in range(e)]))
    cfg = types.SimpleNamespace(top_k=top_k)
    xm = torch.randn(5, h, generator=g).bfloat16()
    prefill._combine = _Combine()
    prefill.triton = types.SimpleNamespace(cdiv=lambda a, b: -(-a // b))
    y = prefill.moe(xm, lw, cfg)
    logits = torch.nn.functional.linear(xm.to(lw.router.dtype), lw.router)
    wts, ids = torch.topk(logits, top_k, dim=-1)
    wts = torch.softmax(wts, dim=-1, dtype=torch.float32)
    ids, order = ids.sort(dim=-1)
    out["moe"] = dict(x=xm, router=lw.router, fc=lw.experts_fc, fc_scale=lw.fc_scale,
                      proj=lw.experts_proj, proj_scale=lw.proj_scale, top_k=top_k,
                      logits=logits, ids=ids, weights=wts.gather(1, order), y=y)

    # ---- dense_mlp (the shared-expert analogue) and the layer's residual algebra
    dl = types.SimpleNamespace(
        dense_gate_up=fp8(2 * 256, h, g), gate_up_scale=scales(4, 2, g),
        dense_down=fp8(h, 256, g), down_scale=scales(2, 2, g))
    out["dense_mlp"] = dict(x=xm, gate_up=dl.dense_gate_up, gate_up_scale=dl.gate_up_scale,
                            down=dl.dense_down, down_scale=dl.down_scale,
                            y=reference.dense_mlp(xm, dl))

    # layer_forward with 2 simulated ranks: run it once per rank with an all_reduce that
    # adds the other rank's partial (computed first with an identity all-reduce).
    heads, hd, q_dim = 2, 128, 256          # per rank
    world = 2
    o_full = fp8(h, q_dim * world, g)
    o_scale_full = scales(h // 128, q_dim * world // 128, g)
    norms = {k: 0.5 + torch.rand(h, generator=g)
             for k in ("attention_norm", "attn_out_norm", "feed_forward_norm")}
    hidden = torch.randn(4, h, generator=g).bfloat16()
    attn_out = [torch.randn(4, heads, hd, generator=g).bfloat16() for _ in range(world)]
    a_scale, f_scale = 0.8, 1.1

    def run_rank(r, all_reduce):
        lwr = types.SimpleNamespace(
            attention_norm=norms["attention_norm"], attn_out_norm=norms["attn_out_norm"],
            feed_forward_norm=norms["feed_forward_norm"], ffn_out_norm=None,
            qkv=fp8(384, h, torch.Generator().manual_seed(5)),
            qkv_scale=scales(3, 2, torch.Generator().manual_seed(6)),
            q_norm=torch.ones(hd), k_norm=torch.ones(hd), sink_k=None,
            o_proj=o_full[:, r * q_dim:(r + 1) * q_dim].contiguous(),
            o_scale=blockfp8.shard_scale(o_scale_full, 1, r * q_dim, q_dim, 128))
        shard = types.SimpleNamespace(q_dim=q_dim, kv_dim=64, num_q_heads=heads, num_kv_heads=1)
        # qkv split must total 384 = 256 + 64 + 64 with head_dim 128 -> kv heads of 64 do
        # not divide; give k/v one head of 64 via head_dim-independent stub below.
        cfgr = types.SimpleNamespace(rms_norm_eps=1e-6, head_dim=64, rotary_dim=64,
                                     softmax_scale=1.0, top_k=top_k)
        shard = types.SimpleNamespace(q_dim=q_dim, kv_dim=64, num_q_heads=4, num_kv_heads=1)
        lwr.q_norm, lwr.k_norm = torch.ones(64), torch.ones(64)
        mw = types.SimpleNamespace(cfg=cfgr, folded=False, shard=shard)
        spec = types.SimpleNamespace(attn_out_scale=a_scale, ffn_out_scale=f_scale,
                                     use_sandwich_norm=False, is_dense_mlp=False,
                                     sliding_window=None, idx=0)
        cos = torch.ones(4, 64, dtype=torch.bfloat16)
        sin = torch.zeros(4, 64, dtype=torch.bfloat16)
        captured = {}

        def attention_fn(q_, k_, v_, **kw):
            return attn_out[r].reshape(4, 4, 64)

        def moe_fn(hn, lw_, cfg_):
            captured["hn"] = hn.clone()
            return torch.zeros_like(hn)

        y = reference.layer_forward(hidden, torch.arange(4), spec, lwr, mw, rope=(cos, sin),
                                    all_reduce=all_reduce, attention_fn=attention_fn,
                                    moe_fn=moe_fn)
        partial = reference.linear(attn_out[r].reshape(4, q_dim), lwr.o_proj, lwr.o_scale)
        return y, captured["hn"], partial

    partials = [run_rank(r, None)[2] for r in range(world)]

    def make_all_reduce(r):
        calls = {"n": 0}

        def all_reduce(t):
            if calls["n"] == 0:                 # the o_proj reduce; the MoE one adds zeros
                t.copy_(partials[0] + partials[1])
            calls["n"] += 1
        return all_reduce

    y0, hn0, _ = run_rank(0, make_all_reduce(0))
    xn = reference.rms_norm(hidden, norms["attention_norm"], 1e-6)
    out["layer_residual"] = dict(partials=partials, base=xn, w_ao=norms["attn_out_norm"],
                                 w_ffn=norms["feed_forward_norm"], a_scale=a_scale, eps=1e-6,
                                 h=y0, hn=hn0)

    path = os.path.join(HERE, "reference_outputs.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def heads(ref_root):
    """`tests/golden/reference_heads.pt`: the attention prologue after the QKV product
    (iquestrt/model/reference.py:101-112: per-head q/k RMSNorm, then `apply_partial_rope`
    with `rope_tables`), for a partial and a full rotary width."""
    sys.path.insert(0, ref_root)
    from iquestrt.model import reference
    g = torch.Generator().manual_seed(4321)
    cases = []
    for q_heads, kv_heads, hd, rotary in ((8, 1, 128, 32), (6, 1, 128, 128), (4, 2, 64, 16)):
        rows = 4
        qkv = (torch.randn(rows, (q_heads + 2 * kv_heads) * hd, generator=g) * 2).bfloat16()
        w_qn = 0.5 + torch.rand(hd, generator=g)
        w_kn = 0.5 + torch.rand(hd, generator=g)
        positions = torch.tensor([5, 100, 4095, 77])
        cos, sin = reference.rope_tables(positions, rotary, 10000.0, "cpu", torch.bfloat16)
        q, k, v = qkv.split([q_heads * hd, kv_heads * hd, kv_heads * hd], dim=-1)
        q = reference.rms_norm(q.view(-1, q_heads, hd), w_qn, 1e-6)
        k = reference.rms_norm(k.view(-1, kv_heads, hd), w_kn, 1e-6)
        q = reference.apply_partial_rope(q, cos, sin, rotary)
        k = reference.apply_partial_rope(k, cos, sin, rotary)
        cases.append(dict(qkv=qkv, q_heads=q_heads, kv_heads=kv_heads, head_dim=hd,
                          rotary_dim=rotary, w_qn=w_qn, w_kn=w_kn, positions=positions,
                          theta=10000.0, cos=cos, sin=sin, eps=1e-6, q=q, k=k,
                          v=v.view(-1, kv_heads, hd)))
    path = os.path.join(HERE, "reference_heads.pt")
    torch.save(cases, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: python tests/golden/make_golden.py <reference_root> [heads]")
    if len(sys.argv) == 3 and sys.argv[2] == "heads":
        heads(sys.argv[1])
    else:
        main(sys.argv[1])
        heads(sys.argv[1])
