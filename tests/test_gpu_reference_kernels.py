"""This build's expert Gate, expert Down and router beside the REFERENCE'S OWN kernels on
the same GPU, same seeded inputs, at the reference's shapes (hidden 3072, 256 experts
top-8, expert width 192 per rank, up to 8 rows).

The reference's kernels are its unmodified `load_inline` sources (iquestrt/kernels/
sm100_moe_fp8.py:110-188 `moe_gate`, :265-341 `moe_down`; iquestrt/kernels/router.py:416-563
`router_q8_fused_kernel`), compiled by `oracle/build_ref.py` into `oracle/_ref/`.  The
tests skip when those modules have not been built.  They also pin the oracle's
decode-numerics family (`gate_decode`, `down_decode`, `select_topk`) against what the
reference's kernels actually compute."""

import pytest
import torch

from oracle import build_ref
from oracle import ref_path as R

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
H, I_LOC, E, TOPK, Q, ROW_BM = 3072, 192, 256, 8, 8, 16
NPAIR = Q * TOPK


@pytest.fixture(scope="module")
def ref():
    if not build_ref.available():
        pytest.skip("reference kernel modules not built (python -m oracle.build_ref)")
    if torch.cuda.get_device_capability() != (10, 0):
        pytest.skip("the reference's kernels are built for compute capability 10.0")
    return {n: build_ref.load(n) for n in build_ref.UNITS}


@pytest.fixture(scope="module")
def bank():
    from iquestrt_b200 import synth
    return synth.make_layer(synth.REFERENCE_Q1, tp=8, rank=3, device="cuda", seed=9)


def _routes(rows, seed):
    g = torch.Generator().manual_seed(seed)
    sel = torch.zeros(Q, TOPK, dtype=torch.int32)
    for r in range(Q):
        sel[r] = torch.sort(torch.randperm(E, generator=g)[:TOPK]).values.to(torch.int32)
    if rows >= 2:
        sel[1, :4] = sel[0, :4]                    # rows that share experts
        sel[1] = torch.sort(sel[1]).values
        if len(set(sel[1].tolist())) < TOPK:       # keep the row's ids distinct
            sel[1] = torch.sort(torch.randperm(E, generator=g)[:TOPK]).values.to(torch.int32)
    wt = torch.softmax(torch.randn(Q, TOPK, generator=g), -1)
    return sel, wt


def _x(rows, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.zeros(ROW_BM, H)
    x[:Q] = torch.randn(Q, H, generator=g)
    return x.bfloat16()


@pytest.mark.parametrize("rows", [1, 4, 6])
def test_gate_and_down_against_the_reference_kernels(ref, bank, rows):
    from iquestrt_b200 import ops
    scratch = ops.Scratch("cuda")
    sel, wt = _routes(rows, 31 + rows)
    x = _x(rows, 77 + rows)
    x8 = R.to_e4m3_sat(x).cuda()                                   # unscaled, as the reference casts
    sel_d, wt_d = sel.flatten().cuda(), wt.flatten().contiguous().cuda()
    fc, fcs, proj, pjs = bank["fc"], bank["fc_scale"], bank["proj"], bank["proj_scale"]

    # ---- Gate
    act_ref = torch.zeros(NPAIR, ROW_BM, I_LOC, dtype=E4M3, device="cuda")
    ref["iquestrt_moe_gate"].moe_gate_launch(x8.data_ptr(), fc.data_ptr(), fcs.data_ptr(),
                                             sel_d.data_ptr(), act_ref.data_ptr(), rows)
    act = torch.zeros(rows * TOPK, I_LOC, dtype=E4M3, device="cuda")
    ops.moe_gate(x8[:rows], sel_d[:rows * TOPK], fc, fcs, act, m=rows, top_k=TOPK,
                 scratch=scratch)
    assert scratch.status() == 0
    pairs = torch.arange(rows * TOPK, device="cuda")
    theirs = act_ref[pairs, pairs // TOPK]                          # [pairs, I_LOC]
    a, b = act.float().cpu(), theirs.float().cpu()
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    same = (act.view(torch.uint8) == theirs.view(torch.uint8)).float().mean().item()
    assert R.rel_fro(a, b) <= 2e-2
    assert same >= 0.97, f"only {same:.3f} of the e4m3 codes agree"
    # the oracle's restatement of the Gate against the reference's kernel
    want = R.to_e4m3_sat(R.gate_decode(x8[:rows].cpu(), sel[:rows], fc.cpu(), fcs.cpu()))
    want = want.view(rows * TOPK, I_LOC)
    agree = (want.view(torch.uint8) == theirs.cpu().view(torch.uint8)).float().mean().item()
    assert agree >= 0.97 and R.rel_fro(want.float(), b) <= 2e-2

    # ---- Down on the reference Gate's activations
    out_ref = torch.zeros(ROW_BM, H, dtype=torch.bfloat16, device="cuda")
    ref["iquestrt_moe_down"].moe_down_launch(act_ref.data_ptr(), proj.data_ptr(), pjs.data_ptr(),
                                             sel_d.data_ptr(), wt_d.data_ptr(),
                                             out_ref.data_ptr(), rows)
    out = torch.zeros(ROW_BM, H, dtype=torch.bfloat16, device="cuda")
    ops.moe_down(theirs.contiguous(), sel_d[:rows * TOPK], wt_d[:rows * TOPK], proj, pjs, out,
                 m=rows, top_k=TOPK, scratch=scratch)
    assert scratch.status() == 0
    got, base = out[:rows].float().cpu(), out_ref[:rows].float().cpu()
    assert R.rel_fro(got, base) <= 4e-3
    bound = 3 * torch.maximum(got.abs(), base.abs()) * 2.0 ** -8 + 1e-2 * base.abs().mean()
    assert ((got - base).abs() <= bound).all()
    want = R.down_decode(theirs.cpu().view(rows, TOPK, I_LOC), sel[:rows], wt[:rows], proj.cpu(),
                         pjs.cpu())
    assert R.rel_fro(want.float(), base) <= 4e-3


def test_router_against_the_reference_kernel(ref):
    from iquestrt_b200 import ops
    scratch = ops.Scratch("cuda")
    g = torch.Generator().manual_seed(123)
    w = (torch.randn(E, H, generator=g) * 0.02).bfloat16().cuda()
    parts = torch.full((12, ROW_BM, E), float("nan"), dtype=torch.float32, device="cuda")
    sel_ref = torch.zeros(NPAIR, dtype=torch.int32, device="cuda")
    wt_ref = torch.zeros(NPAIR, dtype=torch.float32, device="cuda")
    dev = torch.cuda.current_device()
    for call in range(2):                          # the second call finds the partials re-armed
        x = _x(Q, 500 + call).cuda()
        ref["iquestrt_router_q8_sm100"].router_q8_launch(
            x.data_ptr(), w.data_ptr(), parts.data_ptr(), sel_ref.data_ptr(), wt_ref.data_ptr(),
            dev)
        sel, wt, logits = ops.router(x[:Q], w, top_k=TOPK, scratch=scratch,
                                     score=ops.ROUTE_SOFTMAX)
        assert scratch.status() == 0
        rl = R.router_logits(x[:Q].cpu(), w.cpu())
        osel, owt, margin = R.select_topk(rl, TOPK, "softmax")
        s_ref, w_ref = sel_ref.cpu().view(Q, TOPK), wt_ref.cpu().view(Q, TOPK)
        s_own, w_own = sel.cpu().view(Q, TOPK), wt.cpu().view(Q, TOPK)
        checked = 0
        for r in range(Q):
            if margin[r] > 1e-3:
                checked += 1
                assert torch.equal(s_own[r], s_ref[r]), (r, s_own[r], s_ref[r])
                assert torch.equal(osel[r], s_ref[r])               # the oracle, pinned
                assert torch.allclose(w_own[r], w_ref[r], rtol=2e-3, atol=1e-6)
                assert torch.allclose(owt[r], w_ref[r], rtol=2e-3, atol=1e-6)
        assert checked >= Q // 2
