"""Pins the CPU oracle (`oracle/ref_path.py`) against outputs of the reference's own
Python code (`tests/golden/reference_outputs.pt`, made by `tests/golden/make_golden.py`),
plus closed-form cases.  CPU only."""

import os

import pytest
import torch

from oracle import ref_path as R

GOLD = os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.pt")


@pytest.fixture(scope="module")
def gold():
    return torch.load(GOLD, weights_only=False)


def _bits(t):
    return t.contiguous().view(torch.int16) if t.dtype == torch.bfloat16 else t


def test_dequant_matches_reference_bitwise(gold):
    d = gold["dequant"]
    assert torch.equal(R.dequant(d["q"], d["s"]), d["f64"])
    assert torch.equal(R.dequant(d["q"], d["s"], dtype=torch.float32), d["f32"])
    d = gold["dequant_64x128"]
    assert torch.equal(R.dequant(d["q"], d["s"], d["block"], torch.float32), d["f32"])


def test_dequant_rejects_mistiled_scale():
    q = torch.zeros(256, 256).to(R.E4M3)
    with pytest.raises(ValueError):
        R.dequant(q, torch.ones(2, 3))


def test_shard_scale_matches_reference(gold):
    for c in gold["shard_scale"]:
        got = R.shard_scale(c["table"], c["dim"], c["start"], c["length"], c["grain"])
        assert torch.equal(got, c["out"])
    with pytest.raises(ValueError):
        R.shard_scale(gold["shard_scale"][0]["table"], 0, 32, 64, 64)


def test_shard_scale_of_synthetic_generator_is_the_reference_rule(gold):
    from iquestrt_b200 import synth
    for c in gold["shard_scale"]:
        got = synth.shard_scale(c["table"], c["dim"], c["start"], c["length"], c["grain"])
        assert torch.equal(got, c["out"])


def test_linear_and_rms_norm_match_reference_bitwise(gold):
    d = gold["linear"]
    assert torch.equal(_bits(R.linear(d["x"], d["q"], d["s"])), _bits(d["y"]))
    d = gold["rms_norm"]
    assert torch.equal(_bits(R.rms_norm(d["x"], d["w"], d["eps"])), _bits(d["y"]))
    assert torch.equal(R.rms_norm(d["x"].float(), d["w"], d["eps"]), d["y32"])


def test_router_selection_matches_reference(gold):
    d = gold["moe"]
    logits = R.router_logits(d["x"], d["router"])
    assert torch.equal(logits, d["logits"])
    sel, wt, margin = R.select_topk(logits, d["top_k"], "softmax")
    assert torch.equal(sel.long(), d["ids"])
    assert torch.allclose(wt, d["weights"], rtol=1e-6, atol=1e-8)
    assert (margin >= 0).all()


def test_moe_prefill_matches_reference(gold):
    d = gold["moe"]
    got = R.moe_prefill(d["x"], d["ids"], d["weights"], d["fc"], d["fc_scale"], d["proj"],
                        d["proj_scale"])
    # The reference multiplies all rows routed to an expert in one fp32 GEMM, the oracle one
    # row at a time: the fp32 sums may differ in the last bit, i.e. at most a bf16 ulp in
    # a few outputs.
    assert R.rel_fro(got, d["y"]) <= 2e-3
    diff = (got.float() - d["y"].float()).abs()
    assert (diff <= d["y"].float().abs() * 2.0 ** -7 + 1e-12).all()


def test_dense_mlp_matches_reference_bitwise(gold):
    d = gold["dense_mlp"]
    got = R.dense_mlp(d["x"], d["gate_up"], d["gate_up_scale"], d["down"], d["down_scale"])
    assert torch.equal(_bits(got), _bits(d["y"]))


def test_layer_residual_algebra_matches_reference_bitwise(gold):
    d = gold["layer_residual"]
    h, hn = R.layer_residual_algebra(d["partials"], d["base"], d["w_ao"], d["w_ffn"],
                                     d["a_scale"], d["eps"])
    assert torch.equal(_bits(h), _bits(d["h"]))
    assert torch.equal(_bits(hn), _bits(d["hn"]))


def test_decode_tail_numerics_agree_with_reference_algebra(gold):
    """The decode kernels' rounding points (oracle `attention_tail`) against the
    reference's layer algebra: inside the path tolerance with a wide margin."""
    d = gold["layer_residual"]
    h, hn, hn8, inv2 = R.attention_tail(d["partials"], d["base"], d["w_ao"], d["w_ffn"],
                                        d["a_scale"], d["eps"])
    assert R.rel_fro(h, d["h"]) <= 5e-3
    assert R.rel_fro(hn, d["hn"]) <= 5e-3
    assert R.rel_fro(hn8.float(), d["hn"]) <= 6e-2       # e4m3 keeps three mantissa bits
    assert inv2.shape == (d["h"].shape[0],)


def test_decode_moe_numerics_agree_with_reference_algebra(gold):
    """Decode Gate/Down with e4m3 activations against the reference's bf16-activation MoE:
    the difference is the activation quantisation itself (about 2^-4 relative per
    element, averaging to a few percent of the routed output)."""
    d = gold["moe"]
    sel = d["ids"].to(torch.int32)
    m, k = sel.shape
    il = d["proj"].shape[2]
    # 1x128 group scales keep these synthetic magnitudes (weights ~2^-9, so SiLU*Up ~1e-4)
    # inside e4m3's range; an unscaled cast would flush them to zero.
    xq, xs = R.quant_act_group(d["x"])
    act = R.gate_decode(xq, sel, d["fc"], d["fc_scale"], xs)
    aq, a_s = R.quant_act_group(act.bfloat16().reshape(m * k, il))
    out = R.down_decode(aq.view(m, k, il), sel, d["weights"], d["proj"], d["proj_scale"],
                        a_s.view(m, k, il // 128))
    assert R.rel_fro(out, d["y"]) <= 1e-1
    # the Gate alone, on the same dequantised input as the reference algebra: tight
    x_deq = R.dequant_act_group(xq, xs)
    for r in range(m):
        e = int(sel[r, 0])
        w = R.dequant(d["fc"][e], d["fc_scale"][e], (64, 128), dtype=torch.float32)
        gu = torch.mv(w, x_deq[r])
        ref_act = torch.nn.functional.silu(gu[:il]) * gu[il:]
        assert R.rel_fro(act[r, 0], ref_act) <= 1e-4


# ------------------------------------------------------------------ closed-form cases

def test_quant_act_group_roundtrip_and_zero_group():
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    x[0, :128] = torch.linspace(-3, 3, 128).bfloat16()
    q, s = R.quant_act_group(x)
    assert s[0, 1] == 1.0 and s[1, 0] == 1.0             # all-zero groups
    assert torch.isclose(s[0, 0], torch.tensor(3.0 / 448))
    back = R.dequant_act_group(q, s)
    assert (back[0, :128] - x[0, :128].float()).abs().max() <= 3.0 * 2.0 ** -4
    assert q.float().abs().max() <= 448


def test_to_e4m3_sat_saturates():
    v = torch.tensor([1e6, -1e6, 448.0, 500.0, float("inf")])
    assert R.to_e4m3_sat(v).float().tolist() == [448.0, -448.0, 448.0, 448.0, 448.0]


def test_select_topk_ties_and_modes():
    lg = torch.zeros(1, 16)
    lg[0, 9] = 1.0
    lg[0, 3] = -0.0
    sel, wt, margin = R.select_topk(lg, 4, "softmax")
    assert sel[0].tolist() == [0, 1, 2, 9]               # tie -> lower id, -0 == +0
    assert margin[0] == 0
    e = torch.exp(torch.tensor(-1.0))
    assert torch.allclose(wt[0], torch.tensor([e, e, e, 1.0]) / (1 + 3 * e))
    sel2, wt2, _ = R.select_topk(lg, 4, "sigmoid")
    assert torch.equal(sel, sel2)
    sg = torch.sigmoid(torch.tensor([0.0, 0.0, 0.0, 1.0]))
    assert torch.allclose(wt2[0], sg / sg.sum())


def test_all_reduce_rounds_once():
    a = torch.tensor([[1.0, 2.0 ** -9]]).bfloat16()
    parts = [a, a, a, a]
    got = R.all_reduce_bf16(parts)
    assert got.dtype == torch.bfloat16
    assert got[0, 0] == 4.0 and got[0, 1] == 2.0 ** -7


def test_mlp_tail_identity_cases():
    h = 256
    m = torch.randn(2, h).bfloat16()
    zero = torch.zeros(2, h, dtype=torch.bfloat16)
    out, nrm = R.mlp_tail([m], zero, 1.0, torch.ones(h), 0.0)
    assert torch.equal(out, m)
    assert torch.allclose(nrm.float().pow(2).mean(-1), torch.ones(2), atol=2e-2)


def test_attention_prologue_matches_reference_bitwise():
    """`rope_tables`, `apply_partial_rope` and the per-head q/k norm of the oracle against
    outputs of the reference's own torch functions (`tests/golden/reference_heads.pt`);
    the decode form (fp32 product into the norm) stays within bf16 rounding of it."""
    cases = torch.load(os.path.join(os.path.dirname(__file__), "golden", "reference_heads.pt"),
                       weights_only=False)
    assert len(cases) == 3
    for c in cases:
        cos, sin = R.rope_tables(c["positions"], c["rotary_dim"], c["theta"])
        assert torch.equal(_bits(cos), _bits(c["cos"])) and torch.equal(_bits(sin), _bits(c["sin"]))
        q, k, v = R.heads_prefill(c["qkv"], c["q_heads"], c["kv_heads"], c["head_dim"], c["w_qn"],
                                  c["w_kn"], cos, sin, c["rotary_dim"], c["eps"])
        assert torch.equal(_bits(q), _bits(c["q"]))
        assert torch.equal(_bits(k), _bits(c["k"]))
        assert torch.equal(_bits(v), _bits(c["v"]))
        # unrotated channels pass through the rope bit-exact
        plain = R.rms_norm(c["qkv"][:, :c["q_heads"] * c["head_dim"]]
                           .reshape(-1, c["q_heads"], c["head_dim"]), c["w_qn"], c["eps"])
        assert torch.equal(_bits(q[..., c["rotary_dim"]:]), _bits(plain[..., c["rotary_dim"]:]))
        qd, kd, vd = R.heads_decode(c["qkv"].float(), c["q_heads"], c["kv_heads"], c["head_dim"],
                                    c["w_qn"], c["w_kn"], cos, sin, c["rotary_dim"], c["eps"])
        assert torch.equal(_bits(vd), _bits(c["v"]))
        assert R.rel_fro(qd, c["q"]) <= 4e-3 and R.rel_fro(kd, c["k"]) <= 4e-3
