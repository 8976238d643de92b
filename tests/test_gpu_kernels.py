"""GPU parity of every kernel of the path, through the C ABI, against the CPU oracle.

Tolerances: the kernels and the oracle compute the same algebra with different fp32
summation orders, so results agree to bf16 rounding: relative Frobenius error <= 4e-3
per kernel (one bf16 ulp is 2^-8 = 3.9e-3 relative; the Frobenius mean is well below
it) and no element further than 3 bf16 ulps.  Against the reference's bf16 activation
path the bar is the path's stated 2e-2.  Router indices must match bit-exactly wherever
the top-k margin exceeds 1e-3."""

import pytest
import torch

from oracle import ref_path as R

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
KERNEL_TOL = 4e-3
PATH_TOL = 2e-2


def _ops():
    from iquestrt_b200 import ops
    return ops


def _synth():
    from iquestrt_b200 import synth
    return synth


def _scratch_clean(scratch):
    """Status word, tickets and tile counters are zero again after a launch (the fp32
    partials area behind them is overwritten before every use and never cleared; the
    launch counter at byte 128, which tags hand-off words, and the Gate's count of finished
    CTAs at byte 136 only ever grow)."""
    head = scratch.buf[:256 + 4 * 16384].clone().view(torch.int32)
    head[128 // 4] = 0
    head[136 // 4] = 0
    return int(head.abs().sum()) == 0


def _close(got, want, tol=KERNEL_TOL, ulps=3):
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all()
    err = R.rel_fro(got, want)
    assert err <= tol, f"rel fro {err:.3e} > {tol}"
    # element-wise: within `ulps` bf16 ulps of the larger magnitude, with an absolute
    # floor for cancellation
    scale = torch.maximum(got.abs(), want.abs())
    bound = ulps * scale * 2.0 ** -8 + 1e-2 * want.abs().mean()
    assert ((got - want).abs() <= bound).all(), \
        f"max abs diff {(got - want).abs().max():.4e}"
    return err


LINEAR_SHAPES = [
    # n, k, m            geometry exercised
    (6144, 6144, 1),   # benchmark configuration 0, Geo<1,8,2>, stream-K splits
    (256, 1024, 1),    # fewer items than SMs
    (512, 2048, 4),
    (3072, 768, 8),    # the reference's o_proj shard, Geo<2,4,3>
    (1024, 512, 3),    # Geo<2,4,2>
    (128, 256, 2),     # Geo<4,2,2>
    (256, 128, 5),     # Geo<8,1,2>
    (6144, 1024, 1),   # configuration 1's TP=8 shard
    (6144, 8192, 4),   # configuration 1 at TP=1
]


@pytest.mark.parametrize("n,k,m", LINEAR_SHAPES)
def test_linear_group_quantised(scratch, n, k, m):
    """bf16 activations quantised per 1x128 group in the kernel == the oracle's
    quantise -> dequantise -> fp32 linear."""
    ops, synth = _ops(), _synth()
    x, w, s = synth.make_linear_case(n, k, m, device="cuda", seed=n + k + m)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear(x, w, s, scratch=scratch, out=out)
    assert scratch.status() == 0
    xq, xs = R.quant_act_group(x.cpu())
    want = R.linear_a8(xq, xs, w.cpu(), s.cpu())
    _close(out, want)
    # the same product from pre-quantised activations
    out2 = torch.full_like(out, float("nan"))
    ops.linear(xq.cuda(), w, s, x_scale=xs.cuda(), scratch=scratch, out=out2)
    assert scratch.status() == 0
    assert torch.equal(out2.cpu().view(torch.int16), out.cpu().view(torch.int16))


@pytest.mark.parametrize("n,k,m", [(6144, 6144, 1), (3072, 768, 4), (512, 2048, 2)])
def test_linear_w8a16(scratch, n, k, m):
    """Two-term activations reproduce the reference's bf16-activation `linear`
    (iquestrt/model/reference.py:23-27) far inside the path tolerance."""
    ops, synth = _ops(), _synth()
    x, w, s = synth.make_linear_case(n, k, m, device="cuda", seed=3 * n + k + m)
    out = ops.linear(x, w, s, scratch=scratch, x_kind=ops.X_BF16_SPLIT2)
    assert scratch.status() == 0
    want = R.linear(x.cpu(), w.cpu(), s.cpu())
    err = R.rel_fro(out.cpu(), want)
    assert err <= 6e-3, err
    # and the single-term format stays inside the path tolerance's order of magnitude
    out1 = ops.linear(x, w, s, scratch=scratch)
    assert R.rel_fro(out1.cpu(), want) <= 5e-2


@pytest.mark.parametrize("n,k,m", [(768, 3072, 8), (256, 192, 1), (3072, 192, 8), (256, 64, 2)])
def test_linear_unscaled_e4m3(scratch, n, k, m):
    ops, synth = _ops(), _synth()
    x, w, s = synth.make_linear_case(n, k, m, device="cuda", seed=11)
    xq = R.to_e4m3_sat(x.cpu())
    if k % 128:      # whole 128-blocks do not tile K: scale tables at grain 64
        s = torch.exp2(-12 + 6 * torch.rand(n // 64, k // 64, device="cuda"))
        block = (64, 64)
    else:
        block = (128, 128)
    out = ops.linear(xq.cuda(), w, s, scratch=scratch, block=block)
    assert scratch.status() == 0
    want = R.linear(xq.float().bfloat16(), w.cpu(), s.cpu(), block)
    _close(out, want)


def test_linear_scale_grain_64(scratch):
    """Scale tables at grain 64 along rows and along K (expert-bank layout)."""
    ops, synth = _ops(), _synth()
    n, k, m = 512, 1024, 2
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(m, k, generator=g, device="cuda").bfloat16()
    w = synth.fp8_weight(n, k, g, "cuda")
    s = torch.exp2(-12 + 6 * torch.rand(n // 64, k // 64, generator=g, device="cuda"))
    out = ops.linear(x, w, s, scratch=scratch, block=(64, 64))
    assert scratch.status() == 0
    xq, xs = R.quant_act_group(x.cpu())
    want = R.linear_a8(xq, xs, w.cpu(), s.cpu(), block=(64, 64))
    _close(out, want)


def test_linear_repeatable_and_leaves_scratch_clean(scratch):
    ops, synth = _ops(), _synth()
    x, w, s = synth.make_linear_case(6144, 6144, 1, device="cuda", seed=1)
    a = ops.linear(x, w, s, scratch=scratch).clone()
    b = ops.linear(x, w, s, scratch=scratch).clone()
    assert scratch.status() == 0
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert _scratch_clean(scratch)


def test_linear_rejects_bad_arguments(scratch):
    ops, synth = _ops(), _synth()
    from iquestrt_b200._lib import IqError
    x, w, s = synth.make_linear_case(256, 1024, 1, device="cuda")
    with pytest.raises(ValueError):
        ops.linear(x.float(), w, s, scratch=scratch)
    with pytest.raises(ValueError):
        ops.linear(x, w, s[:1], scratch=scratch)
    x9 = torch.zeros(9, 1024, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(IqError):
        ops.linear(x9, w, s, scratch=scratch)


# ------------------------------------------------------------------------------ tails

def _tail_case(m, h, seed, fp32_residual=False):
    g = torch.Generator().manual_seed(seed)
    partial = (torch.randn(m, h, generator=g) * 3).bfloat16()
    residual = torch.randn(m, h, generator=g)
    residual = residual if fp32_residual else residual.bfloat16()
    w1 = 0.5 + torch.rand(h, generator=g)
    w2 = 0.5 + torch.rand(h, generator=g)
    return partial, residual, w1, w2


@pytest.mark.parametrize("m,h", [(1, 6144), (4, 6144), (8, 3072), (3, 1024)])
def test_tail_attention_world1(scratch, m, h):
    ops = _ops()
    partial, residual, w1, w2 = _tail_case(m, h, 7 * m + h)
    d = "cuda"
    h_out = torch.empty(m, h, dtype=torch.bfloat16, device=d)
    hn = torch.empty_like(h_out)
    hn8 = torch.empty(m, h, dtype=E4M3, device=d)
    inv = torch.empty(m, dtype=torch.float32, device=d)
    spec = ops.TailSpec(kind=ops.TAIL_ATTN, partial=partial.to(d), residual=residual.to(d),
                        w_first=w1.to(d), w_norm=w2.to(d), h_out=h_out, norm_out=hn,
                        norm_fp8=hn8, inv_out=inv, scale=0.75, eps=1e-6)
    ops.tail(spec, scratch)
    assert scratch.status() == 0
    rh, rhn, rhn8, rinv = R.attention_tail([partial], residual, w1, w2, 0.75, 1e-6)
    _close(h_out, rh, ulps=1)
    _close(hn, rhn, ulps=2)
    assert torch.allclose(inv.cpu(), rinv, rtol=1e-5)
    # e4m3 of a value one bf16 ulp apart may land on the neighbouring code
    assert R.rel_fro(hn8.float().cpu(), rhn8.float()) <= 2e-2
    # and the prefill algebra (iquestrt/model/reference.py:134-137) within path tolerance
    ph, phn = R.layer_residual_algebra([partial], residual, w1, w2, 0.75, 1e-6)
    assert R.rel_fro(h_out.cpu(), ph) <= PATH_TOL
    assert R.rel_fro(hn.cpu(), phn) <= PATH_TOL


@pytest.mark.parametrize("m,h", [(1, 6144), (4, 6144), (8, 3072)])
def test_tail_mlp_world1_with_group_scales(scratch, m, h):
    ops = _ops()
    partial, residual, _, w2 = _tail_case(m, h, 13 * m + h)
    d = "cuda"
    out = torch.empty(m, h, dtype=torch.bfloat16, device=d)
    nrm = torch.empty_like(out)
    n8 = torch.empty(m, h, dtype=E4M3, device=d)
    n8s = torch.empty(m, h // 128, dtype=torch.float32, device=d)
    spec = ops.TailSpec(kind=ops.TAIL_MLP, partial=partial.to(d), residual=residual.to(d),
                        w_norm=w2.to(d), h_out=out, norm_out=nrm, norm_fp8=n8,
                        norm_fp8_scale=n8s, scale=1.25, eps=1e-6)
    ops.tail(spec, scratch)
    assert scratch.status() == 0
    rout, rnorm = R.mlp_tail([partial], residual, 1.25, w2, 1e-6)
    _close(out, rout, ulps=1)
    _close(nrm, rnorm, ulps=2)
    # the group-quantised copy dequantises back to the bf16 row within e4m3 precision
    deq = R.dequant_act_group(n8.cpu(), n8s.cpu())
    assert R.rel_fro(deq, nrm.float().cpu()) <= 4e-2
    q, s = R.quant_act_group(nrm.cpu())
    assert torch.allclose(n8s.cpu(), s, rtol=1e-6)


def test_tail_fp32_residual(scratch):
    ops = _ops()
    m, h = 2, 3072
    partial, residual, w1, w2 = _tail_case(m, h, 99, fp32_residual=True)
    d = "cuda"
    h32 = torch.empty(m, h, dtype=torch.float32, device=d)
    hn = torch.empty(m, h, dtype=torch.bfloat16, device=d)
    spec = ops.TailSpec(kind=ops.TAIL_ATTN, partial=partial.to(d), residual=residual.to(d),
                        w_first=w1.to(d), w_norm=w2.to(d), h_out=h32, norm_out=hn, scale=1.0)
    ops.tail(spec, scratch)
    assert scratch.status() == 0
    rh, rhn, _, _ = R.attention_tail([partial], residual, w1, w2, 1.0, 1e-6)
    assert torch.allclose(h32.cpu(), rh, rtol=1e-5, atol=1e-5)
    _close(hn, rhn, ulps=2)


def test_linear_fused_tail_world1(scratch):
    """o_proj + epilogue in one launch == GEMV then the standalone epilogue == oracle."""
    ops, synth = _ops(), _synth()
    n, k, m = 6144, 8192, 1
    x, w, s = synth.make_linear_case(n, k, m, device="cuda", seed=21)
    g = torch.Generator().manual_seed(4)
    residual = torch.randn(m, n, generator=g).bfloat16().cuda()
    gamma = (0.5 + torch.rand(n, generator=g)).cuda()
    part = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    h_out, nrm = torch.empty_like(part), torch.empty_like(part)
    spec = ops.TailSpec(kind=ops.TAIL_MLP, partial=part, residual=residual, w_norm=gamma,
                        h_out=h_out, norm_out=nrm, scale=1.0, eps=1e-6)
    ops.linear(x, w, s, scratch=scratch, out=part, tail=spec)
    assert scratch.status() == 0
    xq, xs = R.quant_act_group(x.cpu())
    ref_part = R.linear_a8(xq, xs, w.cpu(), s.cpu())
    _close(part, ref_part)
    rout, rnorm = R.mlp_tail([part.cpu()], residual.cpu(), 1.0, gamma.cpu(), 1e-6)
    _close(h_out, rout, ulps=1)
    _close(nrm, rnorm, ulps=2)
    assert _scratch_clean(scratch)


@pytest.mark.parametrize("m,kind", [(4, "attn"), (8, "mlp"), (3, "attn")])
def test_linear_fused_tail_rows_on_their_own_ctas(scratch, m, kind):
    """Several rows: each row of the fused tail is finished by its own CTA of the GEMV
    launch (polling the landing zone the epilogue fills).  Same bits as the GEMV followed
    by the tail as a separate launch, and both against the oracle; three calls in a row
    (the hand-off words carry a new tag each call)."""
    ops, synth = _ops(), _synth()
    n, k = 6144, 1024
    g = torch.Generator().manual_seed(40 + m)
    residual = torch.randn(m, n, generator=g).bfloat16().cuda()
    w1 = (0.5 + torch.rand(n, generator=g)).cuda()
    w2 = (0.5 + torch.rand(n, generator=g)).cuda()
    attn = kind == "attn"

    def spec_for(part, h_out, nrm, n8=None, n8s=None):
        return ops.TailSpec(kind=ops.TAIL_ATTN if attn else ops.TAIL_MLP, partial=part,
                            residual=residual, w_first=w1 if attn else None, w_norm=w2,
                            h_out=h_out, norm_out=nrm, norm_fp8=n8, norm_fp8_scale=n8s,
                            scale=0.8, eps=1e-6)

    for call in range(3):
        x, w, s = synth.make_linear_case(n, k, m, device="cuda", seed=60 + call)
        part = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        h_out, nrm = torch.empty_like(part), torch.empty_like(part)
        n8 = torch.empty(m, n, dtype=E4M3, device="cuda")
        n8s = torch.empty(m, n // 128, dtype=torch.float32, device="cuda")
        ops.linear(x, w, s, scratch=scratch, out=part, tail=spec_for(part, h_out, nrm, n8, n8s))
        assert scratch.status() == 0
        part2 = torch.empty_like(part)
        h2, nrm2 = torch.empty_like(part), torch.empty_like(part)
        ops.linear(x, w, s, scratch=scratch, out=part2)
        ops.tail(spec_for(part2, h2, nrm2), scratch)
        assert scratch.status() == 0
        for a, b in ((part, part2), (h_out, h2), (nrm, nrm2)):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))
        xq, xs = R.quant_act_group(x.cpu())
        ref_part = R.linear_a8(xq, xs, w.cpu(), s.cpu())
        _close(part, ref_part)
        if attn:
            rh, rn, _, _ = R.attention_tail([part.cpu()], residual.cpu(), w1.cpu(), w2.cpu(),
                                            0.8, 1e-6)
        else:
            rh, rn = R.mlp_tail([part.cpu()], residual.cpu(), 0.8, w2.cpu(), 1e-6)
        _close(h_out, rh, ulps=1)
        _close(nrm, rn, ulps=2)
        q, sq = R.quant_act_group(nrm.cpu())
        assert torch.allclose(n8s.cpu(), sq, rtol=1e-6)
    assert _scratch_clean(scratch)


class _RanksOnOneGpu:
    """Eight "ranks" whose landing zones are ONE buffer on this GPU: every rank's peer
    table points at it, so rank r's GEMV stores its tagged rows into zone[r] (eight times
    over), and a tail that polls eight sources finds them all locally."""

    def __init__(self, world, h):
        self.world, self.h = world, h
        self.zone = torch.zeros(world * 8 * h, dtype=torch.int32, device="cuda")
        self.ctrl = torch.zeros(64, dtype=torch.int32, device="cuda")
        self.peers = torch.tensor([self.zone.data_ptr()] * world, dtype=torch.int64, device="cuda")

    def rank(self, r):
        owner = self

        class Slot:
            world, protocol = owner.world, "push"

            def push_args(self):
                from iquestrt_b200 import _lib
                a = _lib.PushArgs()
                a.world, a.rank, a.rows, a.h = owner.world, r, 8, owner.h
                a.recv = owner.zone.data_ptr()
                a.recv_mc = None
                a.peer_recv = owner.peers.data_ptr()
                a.epoch = owner.ctrl.data_ptr()
                a.ticket = owner.ctrl.data_ptr() + 4
                self._keep = a
                return a

            def fill(self, a, partial):
                import ctypes as C
                a.world, a.rank = owner.world, r
                a.push = C.pointer(self.push_args())
        return Slot()


@pytest.mark.parametrize("m,kind", [(1, "attn"), (4, "mlp")])
def test_fused_tail_adds_eight_sources(scratch, m, kind):
    """World 8 on one GPU: seven ranks' GEMVs send their rows, the eighth runs the fused
    tail, whose CTAs take the eight sources in rounds of what their shared memory holds
    (four at a time beside a half-SM stream).  Rank-order fp32 sum, one bf16 rounding."""
    ops, synth = _ops(), _synth()
    n, k, world = 6144, 1024, 8
    ranks = _RanksOnOneGpu(world, n)
    g = torch.Generator().manual_seed(90 + m)
    residual = torch.randn(m, n, generator=g).bfloat16().cuda()
    w1 = (0.5 + torch.rand(n, generator=g)).cuda()
    w2 = (0.5 + torch.rand(n, generator=g)).cuda()
    attn = kind == "attn"
    for call in range(2):                              # a new tag on the second call
        parts = []
        for r in range(world):
            x, w, s = synth.make_linear_case(n, k, m, device="cuda", seed=700 + 10 * call + r)
            part = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            if r < world - 1:
                ops.linear(x, w, s, scratch=scratch, out=part, push=ranks.rank(r))
            else:
                h_out, nrm = torch.empty_like(part), torch.empty_like(part)
                spec = ops.TailSpec(kind=ops.TAIL_ATTN if attn else ops.TAIL_MLP, partial=part,
                                    residual=residual, w_first=w1 if attn else None, w_norm=w2,
                                    h_out=h_out, norm_out=nrm, scale=0.8, eps=1e-6,
                                    comm=ranks.rank(r), timeout_ms=200)
                ops.linear(x, w, s, scratch=scratch, out=part, tail=spec)
            parts.append(part)
        assert scratch.status() == 0
        assert int(ranks.ctrl[0]) == call + 1          # the tail closed the call
        cpu_parts = [p.cpu() for p in parts]
        if attn:
            rh, rn, _, _ = R.attention_tail(cpu_parts, residual.cpu(), w1.cpu(), w2.cpu(), 0.8, 1e-6)
        else:
            rh, rn = R.mlp_tail(cpu_parts, residual.cpu(), 0.8, w2.cpu(), 1e-6)
        _close(h_out, rh, ulps=1)
        _close(nrm, rn, ulps=2)


# ------------------------------------------------------------------------------ router

@pytest.mark.parametrize("m,h,e,score", [(1, 6144, 256, "sigmoid"), (4, 6144, 256, "softmax"),
                                         (8, 3072, 256, "softmax"), (2, 1024, 64, "sigmoid")])
def test_router(scratch, m, h, e, score):
    ops = _ops()
    g = torch.Generator().manual_seed(m * 31 + h + e)
    x = torch.randn(m, h, generator=g).bfloat16()
    w = (torch.randn(e, h, generator=g) * 0.02).bfloat16()
    mode = ops.ROUTE_SOFTMAX if score == "softmax" else ops.ROUTE_SIGMOID
    sel, wt, logits = ops.router(x.cuda(), w.cuda(), top_k=8, scratch=scratch, score=mode)
    assert scratch.status() == 0
    ref_logits = R.router_logits(x, w)
    assert torch.allclose(logits.cpu(), ref_logits, rtol=1e-4, atol=1e-4)
    rsel, rwt, margin = R.select_topk(ref_logits, 8, score)
    sel, wt = sel.cpu().view(m, 8), wt.cpu().view(m, 8)
    for r in range(m):
        assert sorted(sel[r].tolist()) == sel[r].tolist()
        if margin[r] > 1e-3:
            assert torch.equal(sel[r], rsel[r]), (r, sel[r], rsel[r])
            assert torch.allclose(wt[r], rwt[r], rtol=2e-3, atol=1e-6)
    # selection from the kernel's own logits is exact, ties included
    ksel, kwt, _ = R.select_topk(logits.cpu(), 8, score)
    assert torch.equal(sel, ksel)
    assert torch.allclose(wt, kwt, rtol=1e-5, atol=1e-7)
    assert torch.allclose(wt.sum(-1), torch.ones(m), atol=1e-5)


def test_router_ties_take_lower_id(scratch):
    ops = _ops()
    m, h, e = 2, 512, 64
    x = torch.zeros(m, h, dtype=torch.bfloat16)
    x[:, 0] = 1.0
    w = torch.zeros(e, h, dtype=torch.bfloat16)
    w[:, 0] = 0.25                      # every logit equal: the eight lowest ids win
    w[40, 0] = 0.5
    w[5, 0] = -0.0
    sel, wt, _ = ops.router(x.cuda(), w.cuda(), top_k=8, scratch=scratch)
    assert scratch.status() == 0
    assert sel.cpu().view(m, 8)[0].tolist() == [0, 1, 2, 3, 4, 6, 7, 40]


# ------------------------------------------------------------------------------ MoE

def _moe_case(m, h, inter, tp, e, seed, n_shared, dev="cuda"):
    """Rank 1 (or 0) shard of a synthetic MoE layer plus routes in which odd rows share
    half of their experts with the row before."""
    synth = _synth()
    shape = synth.LayerShape(hidden=h, q_dim=1024, n_experts=e, top_k=8, inter=inter,
                             n_shared=n_shared)
    lw = synth.make_layer(shape, tp=tp, rank=min(1, tp - 1), device=dev, seed=seed)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, h, generator=g).bfloat16()
    rows = []
    for r in range(m):
        perm = [int(v) for v in torch.randperm(e, generator=g)]
        if r % 2 == 1:
            prev = rows[r - 1][:4].tolist()
            ids = prev + [v for v in perm if v not in prev][:4]
        else:
            ids = perm[:8]
        rows.append(torch.tensor(sorted(ids)))
    sel = torch.stack(rows).to(torch.int32)
    wt = torch.softmax(torch.randn(m, 8, generator=g), -1)
    return lw, x, sel, wt


@pytest.mark.parametrize("m,h,inter,tp,n_shared,mode", [
    (1, 6144, 2048, 8, 1, "group"),     # configuration 2's TP=8 shard, benchmark formats
    (4, 6144, 2048, 8, 1, "group"),
    (1, 3072, 1536, 8, 0, "unscaled"),  # the reference's shard (I_loc 192) and formats
    (8, 3072, 1536, 8, 0, "unscaled"),
    (2, 1024, 2048, 1, 1, "group"),     # deep Down contraction (TP=1 width)
    (1, 6144, 2048, 4, 1, "group"),     # the TP=4 shard (I_loc 512): widest direct Down
    (4, 6144, 2048, 4, 1, "group"),
    (3, 3072, 2048, 4, 0, "unscaled"),
])
def test_moe_gate_down(scratch, m, h, inter, tp, n_shared, mode):
    ops = _ops()
    e = 32
    il = inter // tp
    lw, x, sel, wt = _moe_case(m, h, inter, tp, e, 17 * m + il, n_shared)
    d = "cuda"
    slots = 8 + n_shared
    if mode == "group":
        xq, xs = R.quant_act_group(x)
        act = torch.full((m * slots, il), float("nan"), dtype=torch.bfloat16, device=d)
    else:
        xq, xs = R.to_e4m3_sat(x), None
        act = torch.zeros(m * slots, il, dtype=E4M3, device=d)
    ops.moe_gate(xq.cuda(), sel.cuda().flatten(), lw["fc"], lw["fc_scale"], act, m=m, top_k=8,
                 scratch=scratch, x_scale=None if xs is None else xs.cuda(),
                 shared_fc=lw.get("shared_fc"), shared_fc_scale=lw.get("shared_fc_scale"))
    assert scratch.status() == 0
    # oracle Gate on the routed pairs (+ shared expert as a ninth slot)
    fc, fcs = lw["fc"].cpu(), lw["fc_scale"].cpu()
    ref_act = R.gate_decode(xq, sel, fc, fcs, xs)                       # [m, 8, il]
    if n_shared:
        sh = R.gate_decode(xq, torch.zeros(m, 1, dtype=torch.int32), lw["shared_fc"].cpu(),
                           lw["shared_fc_scale"].cpu(), xs)
        ref_act = torch.cat([ref_act, sh], 1)
    got_act = act.float().cpu().view(m, slots, il)
    if mode == "group":
        _close(got_act, ref_act.bfloat16(), ulps=2)
    else:
        assert R.rel_fro(got_act, R.to_e4m3_sat(ref_act).float()) <= 2e-2

    # Down on the kernel's own activations
    out = torch.full((m, h), float("nan"), dtype=torch.bfloat16, device=d)
    ops.moe_down(act, sel.cuda().flatten(), wt.cuda().flatten(), lw["proj"], lw["proj_scale"],
                 out, m=m, top_k=8, scratch=scratch, shared_proj=lw.get("shared_proj"),
                 shared_proj_scale=lw.get("shared_proj_scale"))
    assert scratch.status() == 0
    a = act.cpu().view(m, slots, il)
    if mode == "group":
        aq, a_s = R.quant_act_group(a.reshape(m * slots, il))
        aq, a_s = aq.view(m, slots, il), a_s.view(m, slots, il // 128)
    else:
        aq, a_s = a, None
    sel_all, wt_all = sel, wt
    proj, pjs = lw["proj"].cpu(), lw["proj_scale"].cpu()
    if n_shared:
        proj = torch.cat([proj, lw["shared_proj"].cpu()], 0)
        pjs = torch.cat([pjs, lw["shared_proj_scale"].cpu()], 0)
        sel_all = torch.cat([sel, torch.full((m, 1), e, dtype=torch.int32)], 1)
        wt_all = torch.cat([wt, torch.ones(m, 1)], 1)
    want = R.down_decode(aq, sel_all, wt_all, proj, pjs, a_s)
    _close(out, want)
    assert _scratch_clean(scratch)


def test_moe_route_out_of_range_sets_status(scratch):
    ops = _ops()
    m, h, il, e = 1, 1024, 128, 16
    lw, x, sel, wt = _moe_case(m, h, il, 1, e, 3, 0)
    sel = sel.clone()
    sel[0, 3] = 99
    act = torch.zeros(m * 8, il, dtype=E4M3, device="cuda")
    ops.moe_gate(R.to_e4m3_sat(x).cuda(), sel.cuda().flatten(), lw["fc"], lw["fc_scale"], act,
                 m=m, top_k=8, scratch=scratch)
    assert scratch.status() == 5        # IQ_ERR_ROUTE, and the context stays usable
    assert scratch.status() == 0
