"""One decode layer of the hot path, wired in the reference's order.

`Engine._layer` of the reference (iquestrt/engine.py:387-450) runs, per MoE layer,

    o_proj -> attention all-reduce tail -> router -> expert Gate+SiLU -> expert Down
    -> (at the start of the next layer) MLP all-reduce tail + next attention norm

as ten kernels chained by programmatic dependent launch.  Here the same step is FOUR
launches: o_proj with the attention tail in its epilogue, the router, the expert Gate,
and the expert Down with the MLP tail in its epilogue.  Attention itself, QKV and the
KV cache are outside this path: `step` takes the attention output `ao` as its input.

`formats="benchmark"`: activations carry 1x128 group scales, router scores are
renormalised sigmoids, one shared expert (the benchmark configurations).
`formats="reference"`: unscaled e4m3 MoE activations, W8A16 o_proj, softmax-of-top-k
router weights, no shared expert (the reference model's own numerics)."""

from __future__ import annotations

import torch

from . import ops
from .kernels import (MoeDecodeKernels, MultimemARTail, MultimemMLPTail, OProjGemv,
                      RouterSelect, TailKernels)
from .synth import LayerShape
from .workspace import Workspace


class DecodeLayer:
    """Holders and buffers of one TP rank for `q_len` live rows of a `LayerShape`."""

    def __init__(self, shape: LayerShape, *, q_len: int = 1, tp: int = 1, group=None,
                 device="cuda", formats: str = "benchmark", a_scale: float = 1.0,
                 f_scale: float = 1.0, use_multicast: bool = True, timeout_ms: int = 2000):
        if formats not in ("benchmark", "reference"):
            raise ValueError(f"formats must be 'benchmark' or 'reference', got {formats!r}")
        self.shape, self.q_len, self.tp, self.formats = shape, q_len, tp, formats
        self.a_scale, self.f_scale = float(a_scale), float(f_scale)
        bench = formats == "benchmark"
        q_loc, i_loc = shape.local(tp)
        self.q_loc, self.i_loc = q_loc, i_loc
        h = shape.hidden
        self.ws = Workspace(device=device, symm_group=group if tp > 1 else None,
                            use_multicast=use_multicast)
        ws = self.ws
        self.scratch = ops.Scratch(device)
        self.tail = TailKernels(h, shape.eps, ws=ws, q_len=q_len)
        self.oproj = OProjGemv(q_loc, h, ws=ws, q_len=q_len, scratch=self.scratch,
                               activation="group" if bench or q_len > 4 else "w8a16")
        self.router = RouterSelect(shape.n_experts, shape.top_k, h, device=device, ws=ws,
                                   q_len=q_len, score="sigmoid" if bench else "softmax",
                                   scratch=self.scratch)
        self.moe = MoeDecodeKernels(shape.n_experts, shape.top_k, h, i_loc, ws=ws, q_len=q_len,
                                    n_shared=shape.n_shared,
                                    act_format="bf16" if bench else "e4m3",
                                    scratch=self.scratch)
        self.norm_out = ws.slot(("layer", "norm_out"), (q_len, h), torch.bfloat16)
        self.ar_tail = MultimemARTail(self.oproj.outputs, group=group, tail=self.tail,
                                      scratch=self.scratch, timeout_ms=timeout_ms)
        self.mlp_tail = MultimemMLPTail(self.moe.outputs, group=group, tail=self.tail,
                                        norm_out=self.norm_out, scratch=self.scratch,
                                        timeout_ms=timeout_ms)
        ws.freeze()

    def step(self, ao, residual, lw, *, fused: bool = True, pdl: bool = True,
             one_launch: bool = False):
        """One layer for the first `q_len` rows.

        `ao [q, q_dim/tp]` bf16 is this rank's attention output, `residual [q, hidden]`
        bf16 the residual base, `lw` the rank-local weights (`synth.make_layer`).  Returns
        `(out, norm_out)`: the layer output (next residual) and its RMSNorm under the next
        layer's attention norm.  `fused=False` runs the two all-reduce tails as their own
        launches (the reference's kernel boundaries).  `one_launch=True` runs the four
        fused launches as a single cooperative launch (`iq_decode_layer`), same results."""
        if one_launch:
            if not fused:
                raise ValueError("one_launch needs the fused tails")
            with ops.one_launch(pdl=pdl):
                return self.step(ao, residual, lw, fused=True, pdl=pdl)
        q = self.q_len
        moe = self.moe
        bench = self.formats == "benchmark"
        x_scale = moe.x_pad_scale if bench else None
        spec = self.ar_tail.spec(
            self.oproj.outputs[self.oproj._next_output][:q], residual, lw["attn_out_norm"],
            lw["feed_forward_norm"], self.a_scale, self.f_scale, norm_out=moe.x_pad,
            norm_fp8=moe.x_pad_fp8, norm_fp8_scale=x_scale, inv_out=self.ar_tail.inv)
        if fused:
            self.oproj(ao, lw["o_proj"], lw["o_scale"], tail=spec, pdl=pdl)
        else:
            self.oproj(ao, lw["o_proj"], lw["o_scale"], pdl=pdl)
            ops.tail(spec, self.scratch, pdl=pdl)
        h = spec.h_out
        sel, wt = self.router(moe.x_pad, lw["router"], pdl=pdl)
        shared = None
        if self.shape.n_shared:
            shared = (lw["shared_fc"], lw["shared_fc_scale"], lw["shared_proj"],
                      lw["shared_proj_scale"])
        out_buf = moe.outputs[moe._out_index]
        mspec = self.mlp_tail.spec(out_buf[:q], h, self.f_scale, lw["next_attention_norm"])
        # Level 2: the Gate's activations (written by the attention tail) and the Down's
        # routes (written by the router) are each two launches old when those kernels
        # start, so they may be read before the kernels' dependency wait.
        level = 2 if pdl else 0
        if fused:
            moe(sel, wt, lw["fc"], lw["fc_scale"], lw["proj"], lw["proj_scale"], x_scale=x_scale,
                shared=shared, tail=mspec, pdl=level)
        else:
            moe(sel, wt, lw["fc"], lw["fc_scale"], lw["proj"], lw["proj_scale"], x_scale=x_scale,
                shared=shared, pdl=level)
            ops.tail(mspec, self.scratch, pdl=pdl)
        return mspec.h_out, mspec.norm_out

    def check(self) -> None:
        """Synchronises and raises if any launch recorded a device-side error."""
        self.scratch.raise_on_error("decode layer")


class CapturedSteps:
    """`n` consecutive `DecodeLayer.step` calls recorded into one CUDA graph (the
    reference captures its whole step the same way, iquestrt/engine.py:677-772)."""

    def __init__(self, layer: DecodeLayer, calls, *, fused=True, pdl=True, warmup=2):
        """`calls` is a list of `(ao, residual, lw)` whose tensors stay alive and in place."""
        self.layer, self.calls = layer, list(calls)
        self.stream = torch.cuda.Stream(device=layer.norm_out.device)
        self.results = []
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                for ao, res, lw in self.calls:
                    layer.step(ao, res, lw, fused=fused, pdl=pdl)
            self.stream.synchronize()
            layer.check()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                for ao, res, lw in self.calls:
                    self.results.append(layer.step(ao, res, lw, fused=fused, pdl=pdl))
        self.stream.synchronize()

    def replay(self):
        self.graph.replay()


class HostStep:
    """One `DecodeLayer.step` from HOST buffers as a single CUDA-graph launch: the graph
    holds the host-to-device copies of the step's inputs (from this object's pinned
    buffers), the layer's launches, and the device-to-host copy of the layer output.

        hs = HostStep(layer, lw)
        out = hs(ao_host, residual_host)        # host bf16 tensors in, pinned host tensor out

    `__call__` copies its arguments into the pinned input buffers, launches the graph and
    waits for it; `out` is overwritten by the next call."""

    def __init__(self, layer: DecodeLayer, lw, *, one_launch: bool = False, pdl: bool = True):
        dev = layer.norm_out.device
        q, shape = layer.q_len, layer.shape
        self.layer = layer
        self.stream = torch.cuda.Stream(device=dev)
        self.ao_pin = torch.empty(q, layer.q_loc, dtype=torch.bfloat16).pin_memory()
        self.res_pin = torch.empty(q, shape.hidden, dtype=torch.bfloat16).pin_memory()
        self.out_pin = torch.empty(q, shape.hidden, dtype=torch.bfloat16).pin_memory()
        self.ao_dev = torch.empty(q, layer.q_loc, dtype=torch.bfloat16, device=dev)
        self.res_dev = torch.empty(q, shape.hidden, dtype=torch.bfloat16, device=dev)
        self.ao_pin.zero_()
        self.res_pin.zero_()

        def body():
            self.ao_dev.copy_(self.ao_pin, non_blocking=True)
            self.res_dev.copy_(self.res_pin, non_blocking=True)
            out, _ = layer.step(self.ao_dev, self.res_dev, lw, one_launch=one_launch, pdl=pdl)
            self.out_pin.copy_(out, non_blocking=True)

        with torch.cuda.stream(self.stream):
            for _ in range(2):                    # both output slots warm before the capture
                body()
            self.stream.synchronize()
            layer.check()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                body()
        self.stream.synchronize()
        self.h2d_bytes = 2 * (self.ao_pin.numel() + self.res_pin.numel())
        self.d2h_bytes = 2 * self.out_pin.numel()

    def __call__(self, ao_host, residual_host):
        self.ao_pin.copy_(ao_host)
        self.res_pin.copy_(residual_host)
        with torch.cuda.stream(self.stream):
            self.graph.replay()
        self.stream.synchronize()
        return self.out_pin
