#!/usr/bin/env python
"""Benchmark of the block-FP8 tensor-parallel decode layer (the path's headline metric).

    python bench.py --gpus N --steps K --warmup W            # this build's CUDA path
    python bench.py --impl reference --gpus N ...            # the reference's CPU algebra

N is the tensor-parallel degree (one process per GPU; under torchrun for N > 1).  A step
is one pass of the hot path of ONE decode layer at batch 1 over one synthetic input:
o_proj + attention all-reduce tail, router top-k, expert Gate+SiLU, expert Down + MLP
all-reduce tail (four launches), at the benchmark configuration's shapes (hidden 6144,
o_proj K 8192, 256 experts top-8 + 1 shared, expert intermediate 2048, all sharded over
N).  Total work is fixed as N grows ("strong" scaling).  Weights rotate over several
distinct layers so every step streams from HBM, not L2.

Prints ONE JSON line: `value` = microseconds per layer with inputs resident in HBM (K
steps replayed from CUDA graphs, device-timed, max over ranks); `e2e` = the same through
the public holder API from pinned HOST buffers (input copy in, result copy out, every
step); `roofline` = the dominant kernel (expert Gate) against the measured HBM peak;
`cpu_baseline` = the reference's torch algebra on this box's host cores."""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "us per TP FP8 MoE decode layer at bs=1 (fused AR)"
UNIT = "us/layer"
WORKLOAD = ("cfg2 MoE decode layer + cfg1 o_proj, hidden 6144, o_proj K 8192, 256 experts top-8 "
            "+ 1 shared, inter 2048, block-FP8 e4m3 128x128 scales, 1x128 activation groups")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--rows", type=int, default=1, help="tokens per step (1, or 4 for MTP verify)")
    ap.add_argument("--layers", type=int, default=0, help="distinct weight sets to rotate over")
    ap.add_argument("--experts", type=int, default=256,
                    help="routed experts in the bank (smaller banks keep profiler captures "
                         "small; a step still streams top-k routed + the shared expert)")
    ap.add_argument("--launches", type=int, default=4, choices=(1, 4),
                    help="kernel launches per layer: the four fused kernels, or the one-launch "
                         "cooperative layer (same results bit for bit)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-multicast", action="store_true",
                    help="all-reduce over plain peer loads instead of NVLS multimem")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:                                   # noqa: BLE001 - clocks are optional
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:                           # noqa: BLE001 - older NVML name
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:                               # noqa: BLE001
                break
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def layer_bytes(shape, tp, rows, distinct_routed):
    """Algorithmic bytes one rank streams per layer step (each weight, scale and activation
    byte counted once)."""
    h, ql, il = shape.hidden, shape.q_dim // tp, shape.inter // tp
    m = rows
    oproj = h * ql + 4 * (h // 128) * (ql // 128) + m * ql * 2 + m * h * 2 * 4 + 2 * h * 4
    router = shape.n_experts * h * 2 + m * h * 2
    groups = distinct_routed + shape.n_shared
    gate = groups * (2 * il * h + 4 * (2 * il // 64) * (h // 128)) + m * h
    down = groups * (h * il + 4 * (h // 128) * (il // 64)) + m * h * 2 * 3 + h * 4
    return {"oproj_tail": oproj, "router": router, "gate": gate, "down_tail": down,
            "total": oproj + router + gate + down}


# ------------------------------------------------------------------------------ CPU arm

def cpu_layer_time(rows, budget_s=20.0, max_steps=8, threads=None):
    """Times the reference's torch algebra for the same layer on the host cores.  The
    expert bank is cut to 16 experts (routing picks 8 of them, plus the shared expert, so
    the work per layer is unchanged) to keep generation short."""
    import torch
    from iquestrt_b200 import synth
    from oracle.cpu_layer import layer_cpu
    if threads:
        torch.set_num_threads(threads)
    shape = synth.LayerShape(n_experts=16)
    lw = synth.make_layer(shape, tp=1, rank=0, device="cpu", seed=0)
    times = []
    t_all = time.time()
    for step in range(max_steps + 1):
        ao, res = synth.make_step_inputs(shape, rows, device="cpu", step=step)
        t0 = time.time()
        layer_cpu([lw], [ao], res, top_k=shape.top_k, n_shared=shape.n_shared, eps=shape.eps,
                  score="sigmoid")
        dt = time.time() - t0
        if step > 0:                                        # first pass warms allocators
            times.append(dt)
        if time.time() - t_all > budget_s and times:
            break
    return times, torch.get_num_threads()


def run_reference(args):
    """`--impl reference`: the reference's CPU algebra (oracle port: the reference is
    Python and is not present on the GPU box), rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    # a step is one full layer (~1-2 s on a few cores); bound the run to a few minutes
    max_steps = min(steps + args.warmup, 60)
    times, cores = cpu_layer_time(args.rows, budget_s=150.0, max_steps=max_steps)
    timed = times[min(args.warmup, max(0, len(times) - 1)):] or times
    us = statistics.median(timed) * 1e6
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(timed), "warmup": len(times) - len(timed), "ms_per_step": us / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 dequantise-and-matmul (bf16 activations)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": args.rows, "tp": args.gpus,
                   "note": "whole layer (all TP shards) on host cores; expert bank cut to 16 "
                           "experts, same work per layer"},
        "cpu_baseline": {"value": us, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{len(timed)} full layer steps, median"},
        "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------ GPU arm

def run_ours(args):
    import torch
    import torch.distributed as dist
    from iquestrt_b200 import _build, ops, synth
    from iquestrt_b200.layer import DecodeLayer

    tp = args.gpus
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != tp:
        raise SystemExit(f"--gpus {tp} needs WORLD_SIZE={tp} (launch with torchrun), got {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if tp > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD.group_name
    _build.build()                                          # no-op when the .so is current
    shape = synth.BASELINE if args.experts == 256 else synth.LayerShape(n_experts=args.experts)
    rows = args.rows
    bank_bytes = 37.75e6 * (args.experts + 1) / tp
    n_layers = args.layers or max(2, min(4, int(24e9 // bank_bytes)))
    layer = DecodeLayer(shape, q_len=rows, tp=tp, group=group, device=dev,
                        formats="benchmark", use_multicast=not args.no_multicast)
    weights = [synth.make_layer(shape, tp=tp, rank=rank, device=dev, seed=0, layer=i)
               for i in range(n_layers)]
    n_inputs = 8
    inputs = [synth.make_step_inputs(shape, rows, tp=tp, rank=rank, device=dev, seed=0, step=i)
              for i in range(n_inputs)]
    K, W = max(1, args.steps), max(3, args.warmup)

    one_launch = args.launches == 1

    def call(i, **kw):
        ao, res = inputs[i % n_inputs]
        return layer.step(ao, res, weights[i % n_layers], one_launch=one_launch, **kw)

    def barrier():
        if tp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream(device=dev)
    chunk = 128
    with torch.cuda.stream(stream):
        for i in range(W):                                  # warm-up, eager
            call(i)
        stream.synchronize()
        layer.check()
        # Exactly K steps: a graph of `chunk` steps replayed K // chunk times plus a graph of
        # the remainder.  `chunk` is even, so the alternating output slots keep alternating
        # across replays.
        def capture(n):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(n):
                    call(i)
            return g

        graphs = []
        if K >= chunk:
            g_chunk = capture(chunk)
            graphs += [(g_chunk, chunk)] * (K // chunk)
        if K % chunk:
            graphs.append((capture(K % chunk), K % chunk))
        graphs[0][0].replay()                               # one untimed replay
        stream.synchronize()
        barrier()
        # one event per graph boundary: the total is first-to-last, the per-chunk times give
        # the spread
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(len(graphs) + 1)]
        with ClockSampler(local_rank) as clocks:
            marks[0].record(stream)
            for j, (g, _) in enumerate(graphs):
                g.replay()
                marks[j + 1].record(stream)
            stream.synchronize()
        barrier()
        ms = marks[0].elapsed_time(marks[-1])
        per_step_us = sorted(marks[j].elapsed_time(marks[j + 1]) * 1e3 / n
                             for j, (_, n) in enumerate(graphs))
        layer.check()

        # ---- per-kernel pass: each of the four kernels on its own, `n_probe` launches of
        # it captured in one graph (same arguments as in the layer, weights rotating over the
        # layers so that every launch streams from HBM, PDL on) and replayed; the kernel's
        # time is the replay's device time / n_probe.  Events inside the layer's own graph
        # would break the launch overlap being measured.
        q = rows
        moe = layer.moe
        n_probe = 32
        sel, wt = layer.router.sel, layer.router.wt

        def k_oproj(i):
            ao, res = inputs[i % n_inputs]
            lw = weights[i % n_layers]
            out = layer.oproj.outputs[i % 2]
            spec = layer.ar_tail.spec(out[:q], res, lw["attn_out_norm"], lw["feed_forward_norm"],
                                      1.0, 1.0, norm_out=moe.x_pad, norm_fp8=moe.x_pad_fp8,
                                      norm_fp8_scale=moe.x_pad_scale, inv_out=layer.ar_tail.inv)
            ops.linear(ao, lw["o_proj"], lw["o_scale"], scratch=layer.scratch, out=out[:q],
                       tail=spec, pdl=True)

        def k_router(i):
            layer.router(moe.x_pad, weights[i % n_layers]["router"], pdl=True)

        def k_gate(i):
            lw = weights[i % n_layers]
            ops.moe_gate(moe.x_pad_fp8, sel, lw["fc"], lw["fc_scale"], moe.act, m=q,
                         top_k=shape.top_k, scratch=layer.scratch, x_scale=moe.x_pad_scale,
                         shared_fc=lw["shared_fc"], shared_fc_scale=lw["shared_fc_scale"],
                         pdl=True)

        def k_down(i):
            lw = weights[i % n_layers]
            out = moe.outputs[i % 2]
            mspec = layer.mlp_tail.spec(out[:q], layer.tail.h[:q], 1.0, lw["next_attention_norm"])
            ops.moe_down(moe.act, sel, wt, lw["proj"], lw["proj_scale"], out, m=q,
                         top_k=shape.top_k, scratch=layer.scratch,
                         shared_proj=lw["shared_proj"],
                         shared_proj_scale=lw["shared_proj_scale"], tail=mspec, pdl=True)

        kern_ms = {}
        for name, fn in (("oproj_tail", k_oproj), ("router", k_router), ("gate", k_gate),
                         ("down_tail", k_down)):
            for i in range(2):
                fn(i)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(n_probe):
                    fn(i)
            g.replay()
            stream.synchronize()
            barrier()
            samples = []
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                stream.synchronize()
                samples.append(a.elapsed_time(b) / n_probe)
            kern_ms[name] = samples
            layer.check()

        # distinct routed experts per step (1 row -> top_k)
        distinct = shape.top_k if rows == 1 else len(set(layer.router.sel.cpu().tolist()))

        # ---- end to end from HOST buffers: `HostStep` (one graph launch per step holding
        # the H2D copies of the step's inputs, the layer, and the D2H copy of its output),
        # one synchronise per step, weights rotating over the layers as above.
        from iquestrt_b200.layer import HostStep
        h_in = [(ao.cpu(), res.cpu()) for ao, res in inputs]
        host_steps = [HostStep(layer, weights[j], one_launch=one_launch) for j in range(n_layers)]
        n_e2e = min(K, 256)
        for i in range(4):
            host_steps[i % n_layers](*h_in[i % n_inputs])
        barrier()
        t_e2e = time.perf_counter()
        for i in range(n_e2e):
            host_steps[i % n_layers](*h_in[i % n_inputs])
        e2e_ms = (time.perf_counter() - t_e2e) * 1e3
        h2d_bytes, d2h_bytes = host_steps[0].h2d_bytes, host_steps[0].d2h_bytes
        layer.check()

    def max_over_ranks(v):
        if tp == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = max_over_ranks(ms)
    e2e_ms = max_over_ranks(e2e_ms)
    med = {k: max_over_ranks(statistics.median(v)) for k, v in kern_ms.items()}
    if rank == 0:
        us = ms * 1e3 / K
        peak, peak_kind = measured_peak()
        by = layer_bytes(shape, tp, rows, distinct)
        gate_s = med["gate"] * 1e-3
        achieved = by["gate"] / gate_s / 1e9
        cpu = None
        if not args.no_cpu_baseline and tp == 1:
            times, cores = cpu_layer_time(rows, budget_s=20.0, max_steps=8)
            cpu = {"value": statistics.median(times) * 1e6, "unit": UNIT, "cores": cores,
                   "kind": "port",
                   "sample": f"{len(times)} full layer steps of the reference's torch algebra "
                             "(expert bank cut to 16 experts, same work per layer), median"}
        line = {
            "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": tp, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows": rows, "tp": tp, "launches_per_step": args.launches,
                       "experts_in_bank": args.experts,
                       "l2": f"weights rotate over {n_layers} distinct layers "
                             f"({by['total'] * n_layers / 1e6:.0f} MB touched per cycle, L2 is 126 MB)",
                       "all_reduce": "none (TP=1)" if tp == 1 else
                                     ("peer loads" if args.no_multicast else "NVLS multimem")},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_ms * 1e3 / n_e2e, "unit": UNIT, "steps": n_e2e,
                    "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": int(d2h_bytes)},
            "gpu_launches": args.launches * K,
            "roofline": {"bound": "hbm", "kernel": "gate_kernel (expert Gate/Up + SiLU)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": by["gate"],
                         "launch_us": med["gate"] * 1e3,
                         # dram__bytes_read + dram__bytes_write of one launch, from the ncu
                         # capture summarised in profiles/gate_kernel_tp1_m1.md
                         "traffic": 230.82e6 if (tp == 1 and rows == 1) else None,
                         "layer_frac": by["total"] / (us * 1e-6) / 1e9 / peak},
            "kernel_us": {k: v * 1e3 for k, v in med.items()},
            "layer_bytes": by["total"],
            "tokens_per_s_per_layer": rows / (us * 1e-6),
            "spread_us": {"chunks": len(per_step_us), "min": per_step_us[0],
                          "median": per_step_us[len(per_step_us) // 2], "max": per_step_us[-1]},
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if tp > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
