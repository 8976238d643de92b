"""One decode layer of the hot path, wired in the reference's order.

`Engine._layer` of the reference (iquestrt/engine.py:387-450) runs, per MoE layer,

    o_proj -> attention all-reduce tail -> router -> expert Gate+SiLU -> expert Down
    -> (at the start of the next layer) MLP all-reduce tail + next attention norm

as ten kernels chained by programmatic dependent launch.  Here the same step is FOUR
launches: o_proj with the attention tail in the same launch, the router, the expert Gate,
and the expert Down with the MLP tail in the same launch.  Attention itself, QKV and the
KV cache are outside this path: `step` takes the attention output `ao` as its input.

`formats="benchmark"`: activations carry 1x128 group scales, router scores are
renormalised sigmoids, one shared expert (the benchmark configurations).
`formats="reference"`: unscaled e4m3 MoE activations, W8A16 o_proj, softmax-of-top-k
router weights, no shared expert (the reference model's own numerics).

`protocol` picks the all-reduce of the two tails (see `parallel`): "push" (default: tiles
stored into every rank's landing zone from the GEMV epilogue, rows finished by dedicated
CTAs of the same launch) or "pull" (signal, wait, `multimem.ld_reduce` on the last CTA)."""

from __future__ import annotations

import torch

from . import ops
from .kernels import (MoeDecodeKernels, MultimemARTail, MultimemMLPTail, OProjGemv,
                      PrologueKernels, RouterSelect, TailKernels)
from .synth import HEADS, HeadShape, LayerShape, rope_tables
from .workspace import Workspace


class DecodeLayer:
    """Holders and buffers of one TP rank for `q_len` live rows of a `LayerShape`."""

    def __init__(self, shape: LayerShape, *, q_len: int = 1, tp: int = 1, group=None,
                 device="cuda", formats: str = "benchmark", a_scale: float = 1.0,
                 f_scale: float = 1.0, use_multicast: bool = True, timeout_ms: int = 2000,
                 protocol: str = "push", oproj_activation: str | None = None):
        if formats not in ("benchmark", "reference"):
            raise ValueError(f"formats must be 'benchmark' or 'reference', got {formats!r}")
        self.shape, self.q_len, self.tp, self.formats = shape, q_len, tp, formats
        self.a_scale, self.f_scale = float(a_scale), float(f_scale)
        bench = formats == "benchmark"
        q_loc, i_loc = shape.local(tp)
        self.q_loc, self.i_loc = q_loc, i_loc
        h = shape.hidden
        self.ws = Workspace(device=device, symm_group=group if tp > 1 else None,
                            use_multicast=use_multicast, protocol=protocol)
        ws = self.ws
        self.scratch = ops.Scratch(device)
        self.tail = TailKernels(h, shape.eps, ws=ws, q_len=q_len)
        if oproj_activation is None:
            oproj_activation = "group" if bench or q_len > 4 else "w8a16"
        self.oproj = OProjGemv(q_loc, h, ws=ws, q_len=q_len, scratch=self.scratch,
                               activation=oproj_activation)
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

    # ------------------------------------------------------------------ the four launches
    def _attn_spec(self, out_buf, residual, lw):
        moe = self.moe
        x_scale = moe.x_pad_scale if self.formats == "benchmark" else None
        return self.ar_tail.spec(
            out_buf[:self.q_len], residual, lw["attn_out_norm"], lw["feed_forward_norm"],
            self.a_scale, self.f_scale, norm_out=moe.x_pad, norm_fp8=moe.x_pad_fp8,
            norm_fp8_scale=x_scale, inv_out=self.ar_tail.inv)

    def _shared(self, lw):
        if not self.shape.n_shared:
            return None
        return (lw["shared_fc"], lw["shared_fc_scale"], lw["shared_proj"],
                lw["shared_proj_scale"])

    def step(self, ao, residual, lw, *, fused: bool = True, pdl: bool = True):
        """One layer for the first `q_len` rows.

        `ao [q, q_dim/tp]` bf16 is this rank's attention output, `residual [q, hidden]`
        bf16 the residual base, `lw` the rank-local weights (`synth.make_layer`).  Returns
        `(out, norm_out)`: the layer output (next residual) and its RMSNorm under the next
        layer's attention norm.  `fused=False` runs the two all-reduce tails as their own
        launches (the reference's kernel boundaries)."""
        q = self.q_len
        moe = self.moe
        x_scale = moe.x_pad_scale if self.formats == "benchmark" else None
        out_buf = self.oproj.outputs[self.oproj._next_output]
        spec = self._attn_spec(out_buf, residual, lw)
        if fused:
            self.oproj(ao, lw["o_proj"], lw["o_scale"], tail=spec, pdl=pdl)
        else:
            self.oproj(ao, lw["o_proj"], lw["o_scale"], push=spec.comm, pdl=pdl)
            ops.tail(spec, self.scratch, pdl=pdl)
        h = spec.h_out
        sel, wt = self.router(moe.x_pad, lw["router"], pdl=pdl)
        mlp_buf = moe.outputs[moe._out_index]
        mspec = self.mlp_tail.spec(mlp_buf[:q], h, self.f_scale, lw["next_attention_norm"])
        # Level 2: the Gate's activations (written by the attention tail) and the Down's
        # routes (written by the router) are each two launches old when those kernels
        # start, so they may be read before the kernels' dependency wait.
        level = 2 if pdl else 0
        if fused:
            moe(sel, wt, lw["fc"], lw["fc_scale"], lw["proj"], lw["proj_scale"], x_scale=x_scale,
                shared=self._shared(lw), tail=mspec, pdl=level)
        else:
            moe(sel, wt, lw["fc"], lw["fc_scale"], lw["proj"], lw["proj_scale"], x_scale=x_scale,
                shared=self._shared(lw), push=mspec.comm, pdl=level)
            ops.tail(mspec, self.scratch, pdl=pdl)
        return mspec.h_out, mspec.norm_out

    def kernel_probes(self, inputs, weights):
        """`{name: fn(i)}`: each of the layer's four launches on its own, with the layer's
        arguments (input set `i % len(inputs)`, weight set `i % len(weights)`), for timing
        one kernel in isolation."""
        q, moe, shape = self.q_len, self.moe, self.shape
        sel, wt = self.router.sel, self.router.wt
        x_scale = moe.x_pad_scale if self.formats == "benchmark" else None

        def oproj_tail(i):
            ao, res = inputs[i % len(inputs)]
            lw = weights[i % len(weights)]
            out = self.oproj.outputs[i % 2]
            ops.linear(ao, lw["o_proj"], lw["o_scale"], scratch=self.scratch, out=out[:q],
                       x_kind=self.oproj.x_kind, tail=self._attn_spec(out, res, lw), pdl=True)

        def router(i):
            self.router(moe.x_pad, weights[i % len(weights)]["router"], pdl=True)

        def gate(i):
            lw = weights[i % len(weights)]
            sh = self._shared(lw)
            ops.moe_gate(moe.x_pad_fp8, sel, lw["fc"], lw["fc_scale"], moe.act, m=q,
                         top_k=shape.top_k, scratch=self.scratch, x_scale=x_scale,
                         shared_fc=sh[0] if sh else None, shared_fc_scale=sh[1] if sh else None,
                         pdl=True)

        def down_tail(i):
            lw = weights[i % len(weights)]
            sh = self._shared(lw)
            out = moe.outputs[i % 2]
            mspec = self.mlp_tail.spec(out[:q], self.tail.h[:q], self.f_scale,
                                       lw["next_attention_norm"])
            ops.moe_down(moe.act, sel, wt, lw["proj"], lw["proj_scale"], out, m=q,
                         top_k=shape.top_k, scratch=self.scratch,
                         shared_proj=sh[2] if sh else None,
                         shared_proj_scale=sh[3] if sh else None, tail=mspec, pdl=True)

        return {"oproj_tail": oproj_tail, "router": router, "gate": gate, "down_tail": down_tail}

    def check(self) -> None:
        """Synchronises and raises if any launch recorded a device-side error."""
        self.scratch.raise_on_error("decode layer")


class DecodeSlice:
    """Consecutive decoder layers of one TP rank as one chain of launches: per layer the
    attention prologue (column-parallel QKV product, q/k norm, rotary embedding, KV-cache
    write), then the `DecodeLayer` (o_proj + attention tail, router, expert Gate, expert
    Down + MLP tail).  The attention core between the two is not part of this library: the
    layer's `ao` is a stand-in the caller supplies per layer, and the prologue's q and the
    cache rows it writes are outputs nobody consumes here.  Everything else is chained as in
    the model: layer i's output is layer i+1's residual, and its norm (under layer i+1's
    attention norm) is what layer i+1's QKV product reads.

    `layers` is a list of `(lw, pw)`: `synth.make_layer` and `synth.make_prologue` dicts.  An
    even number of layers keeps the alternating all-reduce outputs in step with a captured
    graph."""

    def __init__(self, shape: LayerShape, layers, *, heads: HeadShape = HEADS, q_len: int = 1,
                 tp: int = 1, group=None, device="cuda", cache_rows: int = 4096,
                 positions=None, **layer_kwargs):
        self.layers = list(layers)
        self.layer = DecodeLayer(shape, q_len=q_len, tp=tp, group=group, device=device,
                                 formats="benchmark", **layer_kwargs)
        qh, kh = heads.local(tp)
        self.heads, self.q_heads, self.kv_heads = heads, qh, kh
        self._ws = Workspace(device=device)
        self.prologue = PrologueKernels(shape.hidden, qh, kh, heads.head_dim, heads.rotary_dim,
                                        shape.eps, ws=self._ws, q_len=q_len,
                                        scratch=self.layer.scratch)
        self._ws.freeze()
        if positions is None:
            positions = [32000 + r for r in range(q_len)]
        self.cos, self.sin = rope_tables(positions, heads, device=device)
        self.slot = torch.arange(100, 100 + q_len, dtype=torch.int64, device=device)
        e4m3 = torch.float8_e4m3fn
        self.k_cache = [torch.zeros(cache_rows, kh, heads.head_dim, dtype=e4m3, device=device)
                        for _ in self.layers]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]

    def prologue_step(self, i, xn, *, pdl=True):
        """Layer `i`'s prologue on `xn [q, hidden]`: returns q `[q, q_heads, D]` (one buffer,
        overwritten by the next layer); k and v go into the layer's cache rows."""
        pw = self.layers[i][1]
        _, q = self.prologue.call_prenorm(xn, pw["w_qkv"], pw["w_qkv_scale"], pw["w_qn"],
                                          pw["w_kn"], self.cos, self.sin, self.slot,
                                          self.k_cache[i], self.v_cache[i], pdl=pdl)
        return q

    def step(self, residual, xn, aos, *, pdl=True, visit=None):
        """One token step through every layer.  `residual`, `xn` `[q, hidden]` bf16: the
        stream entering layer 0 and its norm; `aos[i]` the stand-in attention output of
        layer i (`[q, q_dim/tp]` bf16).  Returns the last layer's `(out, norm_out)`.
        `visit(i, q, out, norm_out)` is called after each layer's launches are enqueued."""
        for i, (lw, _) in enumerate(self.layers):
            q = self.prologue_step(i, xn, pdl=pdl)
            residual, xn = self.layer.step(aos[i], residual, lw, pdl=pdl)
            if visit is not None:
                visit(i, q, residual, xn)
        return residual, xn

    @property
    def launches_per_layer(self):
        return 6

    def check(self) -> None:
        self.layer.check()


class HostSliceStep:
    """One `DecodeSlice.step` from HOST buffers as a single CUDA-graph launch: the copies of
    the stream entering layer 0 and its norm from pinned host memory, every layer's
    launches, and the copy of the last layer's output back to pinned host memory (`HostStep`
    for the slice).  The stand-in attention outputs `aos` stay on the device, where an
    attention kernel would have written them.  Captures the slice's CURRENT `layers`."""

    def __init__(self, sl: DecodeSlice, aos, *, pdl: bool = True):
        layer = sl.layer
        dev = layer.norm_out.device
        q, h = layer.q_len, layer.shape.hidden
        self.stream = torch.cuda.Stream(device=dev)
        self.res_pin = torch.zeros(q, h, dtype=torch.bfloat16).pin_memory()
        self.xn_pin = torch.zeros(q, h, dtype=torch.bfloat16).pin_memory()
        self.out_pin = torch.empty(q, h, dtype=torch.bfloat16).pin_memory()
        self.res_dev = torch.empty(q, h, dtype=torch.bfloat16, device=dev)
        self.xn_dev = torch.empty(q, h, dtype=torch.bfloat16, device=dev)

        def body():
            self.res_dev.copy_(self.res_pin, non_blocking=True)
            self.xn_dev.copy_(self.xn_pin, non_blocking=True)
            out, _ = sl.step(self.res_dev, self.xn_dev, aos, pdl=pdl)
            self.out_pin.copy_(out, non_blocking=True)

        with torch.cuda.stream(self.stream):
            body()
            self.stream.synchronize()
            sl.check()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                body()
        self.stream.synchronize()
        self.h2d_bytes = 2 * (self.res_pin.numel() + self.xn_pin.numel())
        self.d2h_bytes = 2 * self.out_pin.numel()

    def __call__(self, residual_host, xn_host):
        self.res_pin.copy_(residual_host)
        self.xn_pin.copy_(xn_host)
        with torch.cuda.stream(self.stream):
            self.graph.replay()
        self.stream.synchronize()
        return self.out_pin


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

    def __init__(self, layer: DecodeLayer, lw, *, pdl: bool = True):
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
            out, _ = layer.step(self.ao_dev, self.res_dev, lw, pdl=pdl)
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
