"""The reference-shaped holders called the way the reference's `Engine._layer` calls them
(iquestrt/engine.py:387-450): two-call forms (GEMV, then the all-reduce tail as its own
launch), the MoE-layer attention tail with its extra outputs, the MLP tail, the dense
MLP.  One GPU, through the C ABI, against the CPU oracle."""

import pytest
import torch

from oracle import ref_path as R

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
KERNEL_TOL = 4e-3
PATH_TOL = 2e-2


def _holders(hidden, q_dim, q, i_loc=256, experts=16):
    from iquestrt_b200 import ops
    from iquestrt_b200.kernels import (MoeDecodeKernels, MultimemARTail, MultimemMLPTail,
                                       OProjGemv, TailKernels)
    from iquestrt_b200.workspace import Workspace
    ws = Workspace(device="cuda")
    scratch = ops.Scratch("cuda")
    tail = TailKernels(hidden, 1e-6, ws=ws, q_len=q)
    oproj = OProjGemv(q_dim, hidden, ws=ws, q_len=q, scratch=scratch)
    moe = MoeDecodeKernels(experts, 8, hidden, i_loc, ws=ws, q_len=q, n_shared=0,
                           act_format="bf16", scratch=scratch)
    norm_out = ws.slot(("layer", "norm_out"), (q, hidden), torch.bfloat16)
    ar = MultimemARTail(oproj.outputs, tail=tail, scratch=scratch)
    mlp = MultimemMLPTail(moe.outputs, tail=tail, norm_out=norm_out, scratch=scratch)
    ws.freeze()
    return ws, scratch, tail, oproj, moe, ar, mlp


@pytest.mark.parametrize("q", [1, 4])
def test_oproj_then_attention_tail_as_two_calls(q):
    """`oproj_fn(ao, w, s)` then `ar_tail_fn(ao_out, residual, w_ao, w_ffn, a, f)` ->
    `(tail.h, tail.hn)`, twice (the two output slots alternate)."""
    from iquestrt_b200 import synth
    hidden, q_dim = 6144, 1024
    ws, scratch, tail, oproj, moe, ar, mlp = _holders(hidden, q_dim, q)
    g = torch.Generator().manual_seed(q)
    w_ao = (0.5 + torch.rand(hidden, generator=g)).cuda()
    w_ffn = (0.5 + torch.rand(hidden, generator=g)).cuda()
    for call in range(2):
        x, w, s = synth.make_linear_case(hidden, q_dim, q, device="cuda", seed=7 + call)
        res = torch.randn(q, hidden, generator=g).bfloat16().cuda()
        part = oproj(x, w, s)
        h, hn = ar(part, res, w_ao, w_ffn, 0.9, 1.1)
        assert scratch.status() == 0
        assert h.data_ptr() == tail.h.data_ptr() and hn.data_ptr() == tail.hn.data_ptr()
        xq, xs = R.quant_act_group(x.cpu())
        ref_part = R.linear_a8(xq, xs, w.cpu(), s.cpu())
        assert R.rel_fro(part.cpu(), ref_part) <= KERNEL_TOL
        rh, rhn, _, _ = R.attention_tail([part.cpu()], res.cpu(), w_ao.cpu(), w_ffn.cpu(), 0.9,
                                         1e-6)
        assert R.rel_fro(h.cpu(), rh) <= KERNEL_TOL and R.rel_fro(hn.cpu(), rhn) <= KERNEL_TOL
        ph, phn = R.layer_residual_algebra([R.linear(x.cpu(), w.cpu(), s.cpu())], res.cpu(),
                                           w_ao.cpu(), w_ffn.cpu(), 0.9, 1e-6)
        assert R.rel_fro(h.cpu(), ph) <= PATH_TOL and R.rel_fro(hn.cpu(), phn) <= PATH_TOL


@pytest.mark.parametrize("fp32_residual", [False, True])
def test_attention_tail_for_moe_layers(fp32_residual):
    """`.h_inv_xpad_fp8_pdl_overlap_local`: h, the second norm's inverse RMS, the router
    input `x_pad` (bf16) and the MoE input `x_pad_fp8` (unscaled e4m3, the reference's
    format; and with 1x128 group scales when a scale buffer is given)."""
    q, hidden, q_dim = 3, 3072, 768
    ws, scratch, tail, oproj, moe, ar, mlp = _holders(hidden, q_dim, q)
    g = torch.Generator().manual_seed(11)
    part = (torch.randn(q, hidden, generator=g) * 2).bfloat16()
    res = torch.randn(q, hidden, generator=g)
    res = res if fp32_residual else res.bfloat16()
    w_ao = 0.5 + torch.rand(hidden, generator=g)
    w_ffn = 0.5 + torch.rand(hidden, generator=g)
    buf = oproj.next_out()
    buf[:q].copy_(part.cuda())
    inv = torch.empty(q, dtype=torch.float32, device="cuda")
    h = ar.h_inv_xpad_fp8_pdl_overlap_local(buf[:q], res.cuda(), w_ao.cuda(), w_ffn.cuda(), inv,
                                            moe.x_pad, moe.x_pad_fp8, 0.7, 1.0,
                                            fp32_residual=fp32_residual)
    assert scratch.status() == 0
    rh, rhn, rhn8, rinv = R.attention_tail([part], res, w_ao, w_ffn, 0.7, 1e-6)
    if fp32_residual:
        assert h.dtype == torch.float32 and torch.allclose(h.cpu(), rh, rtol=1e-5, atol=1e-5)
    else:
        assert R.rel_fro(h.cpu(), rh) <= KERNEL_TOL
    assert R.rel_fro(moe.x_pad[:q].cpu(), rhn) <= KERNEL_TOL
    assert torch.allclose(inv.cpu(), rinv, rtol=1e-5)
    assert R.rel_fro(moe.x_pad_fp8[:q].float().cpu(), rhn8.float()) <= 2e-2
    with pytest.raises(ValueError):
        ar.h_inv_xpad_fp8_pdl_overlap_local(buf[:q], res.cuda(), w_ao.cuda(), w_ffn.cuda(), inv,
                                            moe.x_pad, moe.x_pad_fp8, 0.7, 1.0,
                                            fp32_residual=not fp32_residual)
    # benchmark format: group scales beside the e4m3 rows
    if not fp32_residual:
        ar.h_inv_xpad_fp8_pdl_overlap_local(buf[:q], res.cuda(), w_ao.cuda(), w_ffn.cuda(), inv,
                                            moe.x_pad, moe.x_pad_fp8, 0.7, 1.0,
                                            x_pad_scale=moe.x_pad_scale)
        assert scratch.status() == 0
        deq = R.dequant_act_group(moe.x_pad_fp8[:q].cpu(), moe.x_pad_scale[:q].cpu())
        assert R.rel_fro(deq, moe.x_pad[:q].float().cpu()) <= 4e-2


def test_mlp_tail_as_its_own_call():
    """`mlp_ar_tail_fn(mlp_out, residual, f_scale, w_norm)` -> `(tail.out, norm_out)` on
    both rotating MoE output slots."""
    q, hidden = 4, 6144
    ws, scratch, tail, oproj, moe, ar, mlp = _holders(hidden, 1024, q)
    g = torch.Generator().manual_seed(5)
    w_norm = 0.5 + torch.rand(hidden, generator=g)
    for call in range(2):
        part = (torch.randn(q, hidden, generator=g) * 2).bfloat16()
        res = torch.randn(q, hidden, generator=g).bfloat16()
        buf = moe.next_out()
        buf[:q].copy_(part.cuda())
        out, norm = mlp(buf[:q], res.cuda(), 1.2, w_norm.cuda())
        assert scratch.status() == 0
        assert out.data_ptr() == tail.out.data_ptr()
        rout, rnorm = R.mlp_tail([part], res, 1.2, w_norm, 1e-6)
        assert R.rel_fro(out.cpu(), rout) <= KERNEL_TOL
        assert R.rel_fro(norm.cpu(), rnorm) <= KERNEL_TOL
    with pytest.raises(ValueError):
        mlp(torch.zeros(q, hidden, dtype=torch.bfloat16, device="cuda"), res.cuda(), 1.2,
            w_norm.cuda())                        # not one of the registered buffers


@pytest.mark.parametrize("q,grain", [(1, 128), (4, 64)])
def test_dense_mlp_with_the_reference_signature(q, grain):
    """`DenseMlp(hidden, inter, ws=, q_len=)(hn, w_gate_up, gate_up_scale, w_down,
    down_scale, out)` against `reference.dense_mlp` (iquestrt/model/reference.py:70-74)
    with bf16 activations; scale tables at the checkpoint's 128 grain or at 64."""
    from iquestrt_b200 import ops, synth
    from iquestrt_b200.kernels import DenseMlp
    from iquestrt_b200.workspace import Workspace
    hidden, inter = 2048, 512
    ws = Workspace(device="cuda")
    scratch = ops.Scratch("cuda")
    dense = DenseMlp(hidden, inter, ws=ws, q_len=q, scratch=scratch)
    out = ws.slot(("dense", "out"), (16, hidden), torch.bfloat16, symm=True)
    ws.freeze()
    g = synth._gen("cuda", 77, q)
    gu = synth.fp8_weight(2 * inter, hidden, g, "cuda")
    dn = synth.fp8_weight(hidden, inter, g, "cuda")
    if grain == 128:
        gus, dns = synth.block_scales(2 * inter, hidden, g, "cuda"), \
            synth.block_scales(hidden, inter, g, "cuda")
        blk_gu = blk_dn = (128, 128)
    else:
        gus = torch.exp2(-12 + 6 * torch.rand(2 * inter // 64, hidden // 128, generator=g,
                                              device="cuda"))
        dns = torch.exp2(-12 + 6 * torch.rand(hidden // 128, inter // 64, generator=g,
                                              device="cuda"))
        blk_gu, blk_dn = (64, 128), (128, 64)
    hn = torch.randn(q, hidden, generator=g, device="cuda").bfloat16()
    for _ in range(2):                              # the widened tables are reused
        got = dense(hn, gu, gus, dn, dns, out).clone()
    assert scratch.status() == 0
    x = hn.cpu()
    # the kernels' own numerics (1x128-group e4m3 activations into both products)
    gus64 = gus.cpu() if grain == 64 else gus.cpu().repeat_interleave(2, 0)
    dns64 = dns.cpu() if grain == 64 else dns.cpu().repeat_interleave(2, 1)
    xq, xs = R.quant_act_group(x)
    sel0 = torch.zeros(q, 1, dtype=torch.int32)
    act = R.gate_decode(xq, sel0, gu.cpu()[None], gus64[None], xs).bfloat16()     # [q,1,I]
    aq, a_s = R.quant_act_group(act.reshape(q, inter))
    want = R.down_decode(aq.view(q, 1, inter), sel0, torch.ones(q, 1), dn.cpu()[None],
                         dns64[None], a_s.view(q, 1, inter // 128))
    assert got.shape == (q, hidden)
    assert R.rel_fro(got.cpu(), want) <= KERNEL_TOL
    # the reference's bf16-activation algebra (iquestrt/model/reference.py:70-74): two
    # single-term e4m3 activation casts sit between the two, about 2.6e-2 each
    ref = R.dense_mlp(x, gu.cpu(), gus.cpu(), dn.cpu(), dns.cpu(), blk_gu) if grain == 128 else None
    w_gu = R.dequant(gu.cpu(), gus.cpu(), blk_gu, torch.float32)
    pre = torch.nn.functional.linear(x.float(), w_gu).bfloat16()
    mid = torch.nn.functional.silu(pre[:, :inter]) * pre[:, inter:]
    w_dn = R.dequant(dn.cpu(), dns.cpu(), blk_dn, torch.float32)
    algebra = torch.nn.functional.linear(mid.float(), w_dn).bfloat16()
    if ref is not None:
        assert torch.equal(ref.view(torch.int16), algebra.view(torch.int16))
    assert R.rel_fro(got.cpu(), algebra) <= 6e-2
    # the pre-quantised form stays available as a keyword
    got8 = dense(xq.cuda(), gu, gus, dn, dns, out, x_scale=xs.cuda())
    assert scratch.status() == 0
    assert torch.equal(got8.view(torch.int16), got.view(torch.int16))
