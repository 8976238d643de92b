"""Child of tests/test_multi_gpu.py: one process per GPU under torchrun.

    torchrun --nproc-per-node N tests/mp_worker.py --mode parity|timeout [--no-multicast]

parity : the decode layer at TP = N with both all-reduce protocols (push: tiles stored
         into every rank's landing zone from the GEMV epilogue; pull: signal, wait,
         switch read), against the CPU oracle computed from all ranks' shards; identical
         outputs on every rank; the pull all-reduce alone against NCCL's all_reduce of
         the same bf16 partials (untimed cross-check).
timeout: a rank that does not launch its all-reduce (host-side fault), for both
         protocols: the peers' wait runs out, they return IQ_ERR_PEER_TIMEOUT with the
         context still usable, the late rank catches up and the next call is correct
         again."""

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from iquestrt_b200 import ops, synth  # noqa: E402
from iquestrt_b200.layer import DecodeLayer  # noqa: E402
from iquestrt_b200.workspace import Workspace  # noqa: E402
from oracle import ref_path as R  # noqa: E402


def oracle_layer(shape, lws, aos, res, m, a_scale, f_scale):
    """Decode numerics over all ranks' shards (benchmark formats)."""
    parts = []
    for lw, ao in zip(lws, aos):
        aq, a_s = R.quant_act_group(ao)
        parts.append(R.linear_a8(aq, a_s, lw["o_proj"], lw["o_scale"]))
    lw0 = lws[0]
    h, hn, _, _ = R.attention_tail(parts, res, lw0["attn_out_norm"], lw0["feed_forward_norm"],
                                   a_scale, shape.eps)
    return parts, h, hn


def oracle_moe(shape, lws, hn, sel, wt):
    m = hn.shape[0]
    outs = []
    for lw in lws:
        il = lw["proj"].shape[2]
        xq, xs = R.quant_act_group(hn)
        act = R.gate_decode(xq, sel, lw["fc"], lw["fc_scale"], xs)
        sh = R.gate_decode(xq, torch.zeros(m, 1, dtype=torch.int32), lw["shared_fc"],
                           lw["shared_fc_scale"], xs)
        act = torch.cat([act, sh], 1).bfloat16()
        slots = act.shape[1]
        aq, a_s = R.quant_act_group(act.reshape(m * slots, il))
        proj = torch.cat([lw["proj"], lw["shared_proj"]], 0)
        pjs = torch.cat([lw["proj_scale"], lw["shared_proj_scale"]], 0)
        sel_all = torch.cat([sel, torch.full((m, 1), shape.n_experts, dtype=torch.int32)], 1)
        wt_all = torch.cat([wt, torch.ones(m, 1)], 1)
        outs.append(R.down_decode(aq.view(m, slots, il), sel_all, wt_all, proj, pjs,
                                  a_s.view(m, slots, il // 128)))
    return outs


def run_parity(rank, world, dev, group, multicast):
    shape = synth.LayerShape(n_experts=16)
    a_scale, f_scale = 0.9, 1.1
    for m, protocol in ((1, "push"), (4, "push"), (1, "pull"), (4, "pull")):
        layer = DecodeLayer(shape, q_len=m, tp=world, group=group, device=dev,
                            formats="benchmark", a_scale=a_scale, f_scale=f_scale,
                            use_multicast=multicast, protocol=protocol)
        slot = layer.ws._symm[("oproj", "out")]
        if rank == 0:
            print(f"[tp={world} m={m} {protocol}] multicast="
                  f"{'yes' if slot.has_multicast else 'no'}", flush=True)
        lws = [synth.make_layer(shape, tp=world, rank=r, device=dev, seed=2) for r in range(world)]
        ins = [synth.make_step_inputs(shape, m, tp=world, rank=r, device=dev, seed=2)
               for r in range(world)]
        ao, res = ins[rank]
        for rep in range(3):                      # both alternating slots, repeated epochs
            out, norm_out = layer.step(ao, res, lws[rank])
        layer.check()
        out, norm_out = out.clone(), norm_out.clone()
        # the two tails as launches of their own: same protocol, same bits
        for rep in range(2):
            out2, norm2 = layer.step(ao, res, lws[rank], fused=False)
        layer.check()
        assert torch.equal(out2.view(torch.int16), out.view(torch.int16)), "unfused: out"
        assert torch.equal(norm2.view(torch.int16), norm_out.view(torch.int16)), "unfused: norm"
        # identical on every rank
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        for g in gathered:
            assert torch.equal(g.view(torch.int16), out.view(torch.int16)), "ranks disagree"
        # oracle from all shards
        cl = [{k: v.cpu() for k, v in lw.items()} for lw in lws]
        parts, h, hn = oracle_layer(shape, cl, [i[0].cpu() for i in ins], res.cpu(), m,
                                    a_scale, f_scale)
        assert R.rel_fro(layer.tail.h[:m].cpu(), h) <= 4e-3
        assert R.rel_fro(layer.moe.x_pad[:m].cpu(), hn) <= 4e-3
        sel = layer.router.sel.cpu().view(m, shape.top_k)
        wt = layer.router.wt.cpu().view(m, shape.top_k)
        mparts = oracle_moe(shape, cl, layer.moe.x_pad[:m].cpu(), sel, wt)
        want_out, want_norm = R.mlp_tail(mparts, layer.tail.h[:m].cpu(), f_scale,
                                         cl[0]["next_attention_norm"], shape.eps)
        e1, e2 = R.rel_fro(out.cpu(), want_out), R.rel_fro(norm_out.cpu(), want_norm)
        assert e1 <= 4e-3 and e2 <= 4e-3, (e1, e2)
        if rank == 0:
            print(f"[tp={world} m={m} {protocol}] layer vs oracle: out {e1:.2e} norm {e2:.2e}",
                  flush=True)
        del layer, lws

    # the pull all-reduce alone against NCCL and the oracle's fp32-accumulate sum
    ws = Workspace(device=dev, symm_group=group, use_multicast=multicast, protocol="pull")
    bufs = [ws.slot(("t", i), (16, 6144), torch.bfloat16, symm=True) for i in range(2)]
    ws.freeze()
    scratch = ops.Scratch(dev)
    from iquestrt_b200 import parallel
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    zero = torch.zeros(4, 6144, dtype=torch.bfloat16, device=dev)
    ones = torch.ones(6144, dtype=torch.float32, device=dev)
    for call in range(4):
        buf = bufs[call % 2]
        part = (torch.randn(4, 6144, generator=g, device=dev) * 3).bfloat16()
        buf[:4].copy_(part)
        got = torch.empty(4, 6144, dtype=torch.bfloat16, device=dev)
        nrm = torch.empty_like(got)
        spec = ops.TailSpec(kind=ops.TAIL_MLP, partial=buf[:4], residual=zero, w_norm=ones,
                            h_out=got, norm_out=nrm, scale=1.0, eps=1e-6,
                            comm=parallel.slot_of(buf))
        ops.tail(spec, scratch)
        assert scratch.status() == 0
        ref = part.clone()
        dist.all_reduce(ref)                                  # NCCL, untimed cross-check
        allp = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(allp, part)
        exact = R.all_reduce_bf16([p.cpu() for p in allp])
        mag = torch.stack([p.cpu().float().abs() for p in allp]).sum(0)   # sum of |terms|
        # fp32 accumulation in another order: one bf16 ulp of the result plus the fp32
        # rounding of the terms (matters only where the terms cancel)
        d_exact = (got.cpu().float() - exact.float()).abs()
        assert (d_exact <= exact.float().abs() * 2.0 ** -7 + mag * 2.0 ** -20).all(), \
            f"vs fp32-accumulate sum: {float(d_exact.max())}"
        # NCCL rounds to bf16 after every partial sum: a bf16 ulp of the terms per step
        d_nccl = (got.cpu().float() - ref.cpu().float()).abs()
        assert (d_nccl <= mag * 2.0 ** -6).all(), f"vs NCCL all_reduce: {float(d_nccl.max())}"
    if rank == 0:
        print(f"[tp={world}] all-reduce matches NCCL and the fp32-accumulate sum", flush=True)


def run_timeout(rank, world, dev, group):
    """Host-side fault: the last rank skips one call.  Both protocols, no multicast."""
    from iquestrt_b200 import parallel
    late = world - 1
    zero = torch.zeros(1, 1024, dtype=torch.bfloat16, device=dev)
    ones = torch.ones(1024, dtype=torch.float32, device=dev)
    got = torch.empty(1, 1024, dtype=torch.bfloat16, device=dev)
    nrm = torch.empty_like(got)
    # a GEMV whose output row is `value` in every column: x = value in element 0, weight
    # column 0 all ones, unit scales
    w = torch.zeros(1024, 256, dtype=torch.float32, device=dev)
    w[:, 0] = 1.0
    w = w.to(torch.float8_e4m3fn)
    w_scale = torch.ones(1024 // 128, 256 // 128, dtype=torch.float32, device=dev)
    for protocol in ("pull", "push"):
        ws = Workspace(device=dev, symm_group=group, use_multicast=False, protocol=protocol)
        buf = ws.slot(("t", protocol), (16, 1024), torch.bfloat16, symm=True)
        ws.freeze()
        scratch = ops.Scratch(dev)

        def call(value, timeout_ms):
            spec = ops.TailSpec(kind=ops.TAIL_MLP, partial=buf[:1], residual=zero, w_norm=ones,
                                h_out=got, norm_out=nrm, scale=1.0, eps=1e-6,
                                comm=parallel.slot_of(buf), timeout_ms=timeout_ms)
            if protocol == "pull":
                buf[:1].fill_(value)
                ops.tail(spec, scratch)
            else:
                x = torch.zeros(1, 256, dtype=torch.bfloat16, device=dev)
                x[0, 0] = value
                ops.linear(x, w, w_scale, scratch=scratch, out=buf[:1], tail=spec)
            return scratch.status()

        assert call(1.0, 2000) == 0 and float(got[0, 0]) == world          # a normal call
        dist.barrier()
        if rank != late:
            code = call(2.0, 300)                                           # the peer is absent
            assert code == 4, f"{protocol}: expected IQ_ERR_PEER_TIMEOUT, got {code}"
        dist.barrier()
        if rank == late:
            assert call(2.0, 2000) == 0                                     # catches up at once
        dist.barrier()
        assert call(3.0, 2000) == 0                                         # healthy again
        assert float(got[0, 0]) == 3.0 * world, float(got[0, 0])
        dist.barrier()
        if rank == 0:
            print(f"[tp={world} {protocol}] peer timeout reported, context usable, next call "
                  "correct", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="parity")
    ap.add_argument("--no-multicast", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD.group_name
    try:
        if args.mode == "parity":
            run_parity(rank, world, dev, group, not args.no_multicast)
        else:
            run_timeout(rank, world, dev, group)
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
