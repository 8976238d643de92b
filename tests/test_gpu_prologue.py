"""The attention prologue on the GPU: column-parallel block-FP8 QKV product (fp32 result),
then the heads step (per-head q/k RMSNorm, partial rotary embedding, KV-cache write),
through the C ABI against the CPU oracle and against outputs of the reference's own
torch functions (`tests/golden/reference_heads.pt`)."""

import os

import pytest
import torch

from oracle import ref_path as R

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
GOLD = os.path.join(os.path.dirname(__file__), "golden", "reference_heads.pt")


def _bits(t):
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("kv_dtype", [torch.bfloat16, E4M3])
def test_heads_against_reference_outputs(scratch, kv_dtype):
    """Fed the reference fixture's bf16 QKV rows (as fp32), the heads kernel reproduces the
    reference's q, k and v bit for bit: the fp32 normalisation of a bf16-valued product
    rounds to the same bf16."""
    from iquestrt_b200 import ops
    for c in torch.load(GOLD, weights_only=False):
        rows, qh, kh, d, rot = c["qkv"].shape[0], c["q_heads"], c["kv_heads"], c["head_dim"], \
            c["rotary_dim"]
        cap = 32
        q = torch.zeros(rows, qh, d, dtype=torch.bfloat16, device="cuda")
        kc = torch.zeros(cap, kh, d, dtype=kv_dtype, device="cuda")
        vc = torch.zeros(cap, kh, d, dtype=kv_dtype, device="cuda")
        slot = torch.tensor([3, 0, 31, 17], dtype=torch.int64, device="cuda")
        ops.qkv_heads(c["qkv"].float().cuda(), c["w_qn"].cuda(), c["w_kn"].cuda(), c["cos"].cuda(),
                      c["sin"].cuda(), slot, q, kc, vc, q_heads=qh, kv_heads=kh, rotary_dim=rot,
                      eps=c["eps"], scratch=scratch)
        assert scratch.status() == 0
        want_q, want_k, want_v = R.heads_decode(c["qkv"].float(), qh, kh, d, c["w_qn"], c["w_kn"],
                                                c["cos"], c["sin"], rot, c["eps"])
        assert torch.equal(_bits(q.cpu()), _bits(want_q))
        got_k, got_v = kc[slot].cpu(), vc[slot].cpu()
        if kv_dtype == torch.bfloat16:
            assert torch.equal(_bits(got_k), _bits(want_k))
            assert torch.equal(_bits(got_v), _bits(want_v))
            # and the reference's torch functions themselves, to bf16 rounding of the norm
            assert R.rel_fro(q.cpu(), c["q"]) <= 4e-3 and R.rel_fro(got_k, c["k"]) <= 4e-3
            assert torch.equal(_bits(got_v), _bits(c["v"]))
        else:
            assert torch.equal(got_k.view(torch.uint8), R.to_e4m3_sat(want_k).view(torch.uint8))
            assert torch.equal(got_v.view(torch.uint8), R.to_e4m3_sat(want_v).view(torch.uint8))
        untouched = torch.ones(cap, dtype=torch.bool)
        untouched[slot.cpu()] = False
        assert int(kc[untouched.cuda()].float().abs().sum()) == 0


def test_heads_slot_out_of_range_sets_status(scratch):
    from iquestrt_b200 import ops
    c = torch.load(GOLD, weights_only=False)[0]
    qh, kh, d, rot = c["q_heads"], c["kv_heads"], c["head_dim"], c["rotary_dim"]
    q = torch.zeros(4, qh, d, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(8, kh, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    slot = torch.tensor([0, 1, 8, 2], dtype=torch.int64, device="cuda")     # 8 == capacity
    ops.qkv_heads(c["qkv"].float().cuda(), c["w_qn"].cuda(), c["w_kn"].cuda(), c["cos"].cuda(),
                  c["sin"].cuda(), slot, q, kc, vc, q_heads=qh, kv_heads=kh, rotary_dim=rot,
                  eps=c["eps"], scratch=scratch)
    assert scratch.status() == 5                                            # IQ_ERR_ROUTE
    assert scratch.status() == 0


@pytest.mark.parametrize("m,tp", [(1, 8), (4, 8), (2, 1)])
def test_prologue_holder_qkv_then_heads(m, tp):
    """`PrologueKernels.call_prenorm`: xn [m, 6144] -> QKV product over a rank's heads
    (64 q / 8 kv heads of 128 channels, sharded over `tp`) -> q, and k / v in the cache."""
    from iquestrt_b200 import ops, synth
    from iquestrt_b200.kernels import PrologueKernels
    from iquestrt_b200.workspace import Workspace
    hidden, d, rot = 6144, 128, 32
    qh, kh = 64 // tp, 8 // tp
    n_qkv = (qh + 2 * kh) * d
    ws = Workspace(device="cuda")
    scr = ops.Scratch("cuda")
    pro = PrologueKernels(hidden, qh, kh, d, rot, 1e-6, ws=ws, q_len=m, scratch=scr)
    ws.freeze()
    g = synth._gen("cuda", 5, m, tp)
    w = synth.fp8_weight(n_qkv, hidden, g, "cuda")
    ws_ = synth.block_scales(n_qkv, hidden, g, "cuda")
    xn = torch.randn(m, hidden, generator=g, device="cuda").bfloat16()
    w_qn = 0.5 + torch.rand(d, generator=g, device="cuda")
    w_kn = 0.5 + torch.rand(d, generator=g, device="cuda")
    pos = torch.tensor([7, 4000, 31999, 123][:m])
    cos, sin = R.rope_tables(pos, rot, 10000.0)
    cap = 64
    kc = torch.zeros(cap, kh, d, dtype=E4M3, device="cuda")
    vc = torch.zeros_like(kc)
    slot = torch.arange(10, 10 + m, dtype=torch.int64, device="cuda")
    for _ in range(2):
        _, q = pro.call_prenorm(xn, w, ws_, w_qn, w_kn, cos.cuda(), sin.cuda(), slot, kc, vc)
    assert scr.status() == 0
    # the fp32 product against the reference's W8A16 product before its rounding (bf16
    # activations; the kernel carries them as two e4m3 terms)
    want = torch.nn.functional.linear(xn.cpu().float(),
                                      R.dequant(w.cpu(), ws_.cpu(), dtype=torch.float32))
    got = pro.qkv.cpu()
    assert R.rel_fro(got, want) <= 4e-3
    # heads on the kernel's own product: bit-exact against the oracle's decode form
    wq, wk, wv = R.heads_decode(got, qh, kh, d, w_qn.cpu(), w_kn.cpu(), cos, sin, rot, 1e-6)
    assert torch.equal(_bits(q.cpu()), _bits(wq))
    assert torch.equal(kc[slot].cpu().view(torch.uint8), R.to_e4m3_sat(wk).view(torch.uint8))
    assert torch.equal(vc[slot].cpu().view(torch.uint8), R.to_e4m3_sat(wv).view(torch.uint8))
    # and the reference's algebra (bf16 activations into the product) within path tolerance
    ref_qkv = R.linear(xn.cpu(), w.cpu(), ws_.cpu())
    rq, rk, rv = R.heads_prefill(ref_qkv, qh, kh, d, w_qn.cpu(), w_kn.cpu(), cos, sin, rot, 1e-6)
    assert R.rel_fro(q.cpu(), rq) <= 2e-2
    # single-term 1x128-group activations (the benchmark format) stay within e4m3 precision
    pro_g = PrologueKernels(hidden, qh, kh, d, rot, 1e-6, ws=Workspace(device="cuda"), q_len=m,
                            activation="group", scratch=scr)
    _, qg = pro_g.call_prenorm(xn, w, ws_, w_qn, w_kn, cos.cuda(), sin.cuda(), slot, kc, vc)
    assert scr.status() == 0
    xq, xs = R.quant_act_group(xn.cpu())
    want_g = R.linear_a8(xq, xs, w.cpu(), ws_.cpu(), out_dtype=torch.float32)
    assert R.rel_fro(pro_g.qkv.cpu(), want_g) <= 1e-4
    assert R.rel_fro(qg.cpu(), rq) <= 4e-2
