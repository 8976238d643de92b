"""The decode layer (o_proj + attention tail, router, Gate, Down + MLP tail: four launches)
against the CPU oracle, through the reference-shaped holders, on one GPU.

Two bars: (1) the decode numerics restated in the oracle, stage by stage, to bf16
rounding; (2) the reference's own layer algebra with bf16 activations
(iquestrt/model/reference.py:124-143 + iquestrt/kernels/prefill.py:142-185), within the
path's 2e-2 relative Frobenius tolerance on the layer outputs."""

import pytest
import torch

from oracle import ref_path as R

pytestmark = pytest.mark.gpu

PATH_TOL = 2e-2


def _layer_case(shape, tp, rank, m, seed):
    from iquestrt_b200 import synth
    lw = synth.make_layer(shape, tp=tp, rank=rank, device="cuda", seed=seed)
    ao, res = synth.make_step_inputs(shape, m, tp=tp, rank=rank, device="cuda", seed=seed)
    return lw, ao, res


def _cpu(d):
    return {k: v.cpu() for k, v in d.items()}


def _oracle_layer(shape, lw, ao, res, m, formats, a_scale, f_scale):
    """The layer on CPU with the decode numerics of `formats`; returns every stage."""
    eps = shape.eps
    bench = formats == "benchmark"
    if bench:
        aq, a_s = R.quant_act_group(ao)
        part = R.linear_a8(aq, a_s, lw["o_proj"], lw["o_scale"])
    else:
        part = R.linear(ao, lw["o_proj"], lw["o_scale"])
    h, hn, hn8, _ = R.attention_tail([part], res, lw["attn_out_norm"], lw["feed_forward_norm"],
                                     a_scale, eps)
    logits = R.router_logits(hn, lw["router"])
    sel, wt, margin = R.select_topk(logits, shape.top_k, "sigmoid" if bench else "softmax")
    return dict(part=part, h=h, hn=hn, logits=logits, sel=sel, wt=wt, margin=margin)


def _oracle_moe(shape, lw, hn, sel, wt, formats):
    bench = formats == "benchmark"
    m = hn.shape[0]
    e = shape.n_experts
    il = lw["proj"].shape[2]
    if bench:
        xq, xs = R.quant_act_group(hn)
    else:
        xq, xs = R.to_e4m3_sat(hn), None
    act = R.gate_decode(xq, sel, lw["fc"], lw["fc_scale"], xs)
    proj, pjs, sel_all, wt_all = lw["proj"], lw["proj_scale"], sel, wt
    if shape.n_shared:
        sh = R.gate_decode(xq, torch.zeros(m, 1, dtype=torch.int32), lw["shared_fc"],
                           lw["shared_fc_scale"], xs)
        act = torch.cat([act, sh], 1)
        proj = torch.cat([proj, lw["shared_proj"]], 0)
        pjs = torch.cat([pjs, lw["shared_proj_scale"]], 0)
        sel_all = torch.cat([sel, torch.full((m, 1), e, dtype=torch.int32)], 1)
        wt_all = torch.cat([wt, torch.ones(m, 1)], 1)
    slots = act.shape[1]
    if bench:
        ab = act.bfloat16()
        aq, a_s = R.quant_act_group(ab.reshape(m * slots, il))
        aq, a_s = aq.view(m, slots, il), a_s.view(m, slots, il // 128)
    else:
        aq, a_s = R.to_e4m3_sat(act), None
    return R.down_decode(aq, sel_all, wt_all, proj, pjs, a_s)


def _dense_shared(hn, lw, s):
    gu = R.linear(hn, lw["shared_fc"][s], lw["shared_fc_scale"][s], (64, 128))
    half = gu.shape[-1] // 2
    act = torch.nn.functional.silu(gu[:, :half]) * gu[:, half:]
    return R.linear(act, lw["shared_proj"][s], lw["shared_proj_scale"][s], (128, 64))


@pytest.mark.parametrize("m,tp,formats,fused", [
    (1, 8, "benchmark", True),     # configuration 2's rank shard, M=1
    (4, 8, "benchmark", True),     # M=4 (MTP verify)
    (4, 8, "benchmark", False),    # the two tails as their own launches
    (2, 8, "reference", True),     # the reference model's numerics at its own shapes
    (1, 1, "benchmark", True),     # the benchmark's TP=1 layer at full width (what bench.py times)
    (4, 1, "benchmark", True),
    (3, 2, "benchmark", True),     # TP=2 shard widths (Down K = 1024)
])
def test_decode_layer_against_oracle(m, tp, formats, fused):
    from iquestrt_b200 import synth
    if formats == "benchmark":
        shape = synth.LayerShape(n_experts=32)
    else:
        shape = synth.LayerShape(hidden=3072, q_dim=6144, n_experts=32, top_k=8, inter=1536,
                                 n_shared=0)
    a_scale, f_scale = 0.9, 1.1
    lw, ao, res = _layer_case(shape, tp, min(1, tp - 1), m, seed=5 + m)
    layer = _single_rank_layer(shape, m, tp, formats, a_scale, f_scale)
    out, norm_out = layer.step(ao, res, lw, fused=fused)
    layer.check()
    out, norm_out = out.cpu(), norm_out.cpu()
    c = _cpu(lw)
    o = _oracle_layer(shape, c, ao.cpu(), res.cpu(), m, formats, a_scale, f_scale)
    q = m
    # stage by stage
    assert R.rel_fro(layer.tail.h[:q].cpu(), o["h"]) <= 4e-3
    assert R.rel_fro(layer.moe.x_pad[:q].cpu(), o["hn"]) <= 4e-3
    sel = layer.router.sel.cpu().view(q, shape.top_k)
    wt = layer.router.wt.cpu().view(q, shape.top_k)
    for r in range(q):
        if o["margin"][r] > 1e-3:
            assert torch.equal(sel[r], o["sel"][r])
    # MoE + MLP tail from the kernel's own routes and normalised rows
    hn_k = layer.moe.x_pad[:q].cpu()
    mlp = _oracle_moe(shape, c, hn_k, sel, wt, formats)
    want_out, want_norm = R.mlp_tail([mlp], layer.tail.h[:q].cpu(), f_scale,
                                     c["next_attention_norm"], shape.eps)
    assert R.rel_fro(out, want_out) <= 4e-3
    assert R.rel_fro(norm_out, want_norm) <= 4e-3
    # the reference's bf16-activation algebra on the same routes
    part = R.linear(ao.cpu(), c["o_proj"], c["o_scale"])
    h_ref, hn_ref = R.layer_residual_algebra([part], res.cpu(), c["attn_out_norm"],
                                             c["feed_forward_norm"], a_scale, shape.eps)
    mlp_ref = R.moe_prefill(hn_ref, sel, wt, c["fc"], c["fc_scale"], c["proj"], c["proj_scale"])
    for s in range(shape.n_shared):
        mlp_ref = mlp_ref + _dense_shared(hn_ref, c, s)
    out_ref = h_ref + mlp_ref * f_scale
    norm_ref = R.rms_norm(out_ref, c["next_attention_norm"], shape.eps)
    assert R.rel_fro(out, out_ref) <= PATH_TOL
    assert R.rel_fro(norm_out, norm_ref) <= PATH_TOL


def _single_rank_layer(shape, m, tp, formats, a_scale, f_scale, **kw):
    """A TP rank's shard run alone: the layer object is built for the shard's local
    widths with world size 1 (no all-reduce peers)."""
    from iquestrt_b200 import synth
    from iquestrt_b200.layer import DecodeLayer
    q_loc, i_loc = shape.local(tp)
    local = synth.LayerShape(hidden=shape.hidden, q_dim=q_loc, n_experts=shape.n_experts,
                             top_k=shape.top_k, inter=i_loc, n_shared=shape.n_shared,
                             eps=shape.eps)
    return DecodeLayer(local, q_len=m, tp=1, formats=formats, a_scale=a_scale,
                       f_scale=f_scale, **kw)


def test_captured_layer_steps_replay_identically():
    from iquestrt_b200 import synth
    from iquestrt_b200.layer import CapturedSteps
    shape = synth.LayerShape(n_experts=16)
    m, tp = 1, 8
    lw, ao, res = _layer_case(shape, tp, 0, m, seed=3)
    layer = _single_rank_layer(shape, m, tp, "benchmark", 1.0, 1.0)
    eager_out, eager_norm = layer.step(ao, res, lw)
    layer.check()
    eager_out, eager_norm = eager_out.clone(), eager_norm.clone()
    cap = CapturedSteps(layer, [(ao, res, lw), (ao, res, lw)])
    for _ in range(3):
        cap.replay()
    torch.cuda.synchronize()
    layer.check()
    out, norm = cap.results[-1]
    assert torch.equal(out.view(torch.int16), eager_out.view(torch.int16))
    assert torch.equal(norm.view(torch.int16), eager_norm.view(torch.int16))


def _path_error(layer, shape, lw, ao, res, a_scale, f_scale):
    """Relative Frobenius error of one layer step against the reference's bf16-activation
    algebra evaluated on the kernel's own routes."""
    out, norm_out = layer.step(ao, res, lw)
    layer.check()
    c = _cpu(lw)
    q = ao.shape[0]
    sel = layer.router.sel.cpu().view(q, shape.top_k)
    wt = layer.router.wt.cpu().view(q, shape.top_k)
    part = R.linear(ao.cpu(), c["o_proj"], c["o_scale"])
    h_ref, hn_ref = R.layer_residual_algebra([part], res.cpu(), c["attn_out_norm"],
                                             c["feed_forward_norm"], a_scale, shape.eps)
    mlp_ref = R.moe_prefill(hn_ref, sel, wt, c["fc"], c["fc_scale"], c["proj"], c["proj_scale"])
    for s in range(shape.n_shared):
        mlp_ref = mlp_ref + _dense_shared(hn_ref, c, s)
    out_ref = h_ref + mlp_ref * f_scale
    norm_ref = R.rms_norm(out_ref, c["next_attention_norm"], shape.eps)
    return R.rel_fro(out.cpu(), out_ref), R.rel_fro(norm_out.cpu(), norm_ref)


@pytest.mark.parametrize("m", [1, 4])
def test_path_tolerance_over_seeds(m):
    """The 2e-2 bar over eight seeds, not one draw.  With the W8A16-faithful o_proj (two
    e4m3 terms per activation) every seed must pass.  With single-term 1x128-group e4m3
    activations everywhere (the benchmark format) the quantisation of the activations
    alone sits close to the bar: the maximum over the seeds is printed and must stay
    within 2.5e-2."""
    from iquestrt_b200 import synth
    shape = synth.LayerShape(n_experts=16)
    tp = 8
    worst = {}
    for act in ("w8a16", "group"):
        layer = _single_rank_layer(shape, m, tp, "benchmark", 1.0, 1.0, oproj_activation=act)
        errs = []
        for seed in range(8):
            lw, ao, res = _layer_case(shape, tp, seed % tp, m, seed=100 + seed)
            errs.append(max(_path_error(layer, shape, lw, ao, res, 1.0, 1.0)))
        worst[act] = max(errs)
        print(f"m={m} o_proj activation {act}: rel. Frobenius over 8 seeds "
              f"min {min(errs):.3e} max {max(errs):.3e}")
    assert worst["w8a16"] <= PATH_TOL
    assert worst["group"] <= 2.5e-2


def test_host_step_matches_device_step():
    """`HostStep` (host buffers in, one graph launch with the copies inside, host buffer
    out) returns what `DecodeLayer.step` returns on the same inputs, call after call."""
    from iquestrt_b200 import synth
    from iquestrt_b200.layer import HostStep
    shape = synth.LayerShape(n_experts=16)
    layer = _single_rank_layer(shape, 1, 8, "benchmark", 1.0, 1.0)
    lw, _, _ = _layer_case(shape, 8, 0, 1, seed=3)
    hs = HostStep(layer, lw)
    for call in range(3):
        ao, res = synth.make_step_inputs(shape, 1, tp=8, rank=0, device="cuda", seed=40 + call)
        want, _ = layer.step(ao, res, lw)
        want = want.cpu()
        got = hs(ao.cpu(), res.cpu())
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    layer.check()
    assert hs.h2d_bytes == 2 * (ao.numel() + res.numel()) and hs.d2h_bytes == 2 * want.numel()


def test_decode_slice_chain_against_oracle():
    """Four chained layers with their attention prologues (`DecodeSlice`, the attention core
    a stand-in): every layer's out / norm / q within the path tolerance of the reference's
    algebra on that layer's inputs, routes equal under the margin rule (the check the bench's
    `--workload slice4` prints), and a CUDA-graph replay of the step bit-identical to the
    eager step."""
    import types
    import bench
    from iquestrt_b200 import synth
    from iquestrt_b200.layer import DecodeSlice
    args = types.SimpleNamespace(no_multicast=False, protocol="push")
    report = bench.slice_parity(args, 1, 0, torch.device("cuda", 0), None, rows_list=(2,))
    assert report["ok"], report
    assert report["rel_fro_out"] <= PATH_TOL and report["rel_fro_q"] <= PATH_TOL

    shape = synth.LayerShape(n_experts=16)
    ql, il = shape.local(8)
    shard = synth.LayerShape(hidden=shape.hidden, q_dim=ql, n_experts=16, inter=il)
    heads = synth.HeadShape(q_heads=8, kv_heads=1)
    layers = [(synth.make_layer(shard, device="cuda", seed=5, layer=i),
               synth.make_prologue(shard, heads, device="cuda", seed=5, layer=i))
              for i in range(4)]
    sl = DecodeSlice(shard, layers, heads=heads, q_len=1)
    aos, res0, xn0 = bench.slice_inputs(synth, shard, 1, 1, 0, "cuda", 4)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(2):
            out, norm = sl.step(res0, xn0, aos)
        stream.synchronize()
        want = (out.clone(), norm.clone(), sl.k_cache[3][sl.slot].clone())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(4):
                out_g, norm_g = sl.step(res0, xn0, aos)
        for _ in range(3):
            g.replay()
        stream.synchronize()
    sl.check()
    assert torch.equal(out_g.view(torch.int16), want[0].view(torch.int16))
    assert torch.equal(norm_g.view(torch.int16), want[1].view(torch.int16))
    assert torch.equal(sl.k_cache[3][sl.slot].view(torch.uint8), want[2].view(torch.uint8))
