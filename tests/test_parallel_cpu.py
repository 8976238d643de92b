"""Host-side logic of the tensor-parallel path on CPU: two gloo ranks.

Covers what needs no GPU: every rank derives its shard from the same seeded global
tensors, the rank-local scale tables follow the reference's `shard_scale` rule, and the
sum over ranks of the row-parallel partial products (the all-reduce, here gloo's) equals
the unsharded product -- for o_proj and for the expert Down; the column-parallel QKV
shards of the attention prologue, gathered, equal the unsharded product."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_path as R


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from iquestrt_b200 import synth
        torch.set_num_threads(2)
        shape = synth.LayerShape(hidden=1024, q_dim=1024, n_experts=4, top_k=2, inter=512,
                                 n_shared=1)
        m = 2
        lw = synth.make_layer(shape, tp=world, rank=rank, device="cpu", seed=7)
        full = synth.make_layer(shape, tp=1, rank=0, device="cpu", seed=7)
        ao, res = synth.make_step_inputs(shape, m, tp=world, rank=rank, device="cpu", seed=7)
        ao_full, res_full = synth.make_step_inputs(shape, m, device="cpu", seed=7)
        assert torch.equal(res, res_full)
        ql = shape.q_dim // world
        assert torch.equal(ao, ao_full[:, rank * ql:(rank + 1) * ql])
        # o_proj: fp32 partials summed over ranks == the unsharded fp32 product
        part = torch.nn.functional.linear(
            ao.float(), R.dequant(lw["o_proj"], lw["o_scale"], dtype=torch.float32))
        dist.all_reduce(part)
        want = torch.nn.functional.linear(
            ao_full.float(), R.dequant(full["o_proj"], full["o_scale"], dtype=torch.float32))
        assert torch.allclose(part, want, rtol=1e-4, atol=1e-5)
        # router replicated
        assert torch.equal(lw["router"], full["router"])
        # expert Down: shard on the intermediate dim, scale tables at grain 64
        il = shape.inter // world
        e = 1
        w_loc = R.dequant(lw["proj"][e], lw["proj_scale"][e], (128, 64), dtype=torch.float32)
        w_all = R.dequant(full["proj"][e], full["proj_scale"][e], (128, 64), dtype=torch.float32)
        assert torch.equal(w_loc, w_all[:, rank * il:(rank + 1) * il])
        g_loc = R.dequant(lw["fc"][e], lw["fc_scale"][e], (64, 128), dtype=torch.float32)
        g_all = R.dequant(full["fc"][e], full["fc_scale"][e], (64, 128), dtype=torch.float32)
        assert torch.equal(g_loc[:il], g_all[rank * il:(rank + 1) * il])
        assert torch.equal(g_loc[il:], g_all[shape.inter + rank * il:shape.inter + (rank + 1) * il])
        act = torch.randn(m, shape.inter, generator=torch.Generator().manual_seed(3))
        d = act[:, rank * il:(rank + 1) * il] @ w_loc.t()
        dist.all_reduce(d)
        assert torch.allclose(d, act @ w_all.t(), rtol=1e-4, atol=1e-6)
        # attention prologue: column-parallel QKV (no reduction): the ranks' head shards,
        # gathered, are the unsharded [q | k | v] product and its heads
        heads = synth.HeadShape(q_heads=4, kv_heads=2)
        pw = synth.make_prologue(shape, heads, tp=world, rank=rank, device="cpu", seed=7)
        pf = synth.make_prologue(shape, heads, tp=1, rank=0, device="cpu", seed=7)
        assert torch.equal(pw["w_qn"], pf["w_qn"]) and torch.equal(pw["w_kn"], pf["w_kn"])
        xn = res_full
        mine = R.linear(xn, pw["w_qkv"], pw["w_qkv_scale"])
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        whole = R.linear(xn, pf["w_qkv"], pf["w_qkv_scale"])
        qh, kh = heads.local(world)
        d_ = heads.head_dim
        q_all = torch.cat([b[:, :qh * d_] for b in both], 1)
        k_all = torch.cat([b[:, qh * d_:(qh + kh) * d_] for b in both], 1)
        v_all = torch.cat([b[:, (qh + kh) * d_:] for b in both], 1)
        nq, nk = heads.q_heads * d_, heads.kv_heads * d_
        assert torch.equal(q_all, whole[:, :nq])
        assert torch.equal(k_all, whole[:, nq:nq + nk])
        assert torch.equal(v_all, whole[:, nq + nk:])
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_reduce_consistently():
    world = 2
    port = 29900 + (os.getpid() % 90)
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}


def test_symm_slot_single_rank_layout():
    """World-size-1 slots (no process group): plain memory with the same layout -- rows,
    control words, landing zone."""
    from iquestrt_b200.parallel import CTRL_BYTES, ZONE_ROWS, SymmSlot
    s = SymmSlot((16, 1024), torch.bfloat16, device="cpu")
    assert s.world == 1 and not s.has_multicast and s.protocol == "push"
    assert (s.zone_rows, s.zone_h) == (ZONE_ROWS, 1024)
    assert s.buf.numel() == 16 * 1024 * 2 + CTRL_BYTES + 4 * ZONE_ROWS * 1024
    assert s.data.shape == (16, 1024) and int(s.buf.sum()) == 0
    p = s.push_args()
    assert (p.world, p.rank, p.rows, p.h) == (1, 0, ZONE_ROWS, 1024)
    assert p.recv == s.base_ptr + s.zone_off and p.recv % 16 == 0
    assert p.epoch == s.base_ptr + s.data_bytes + 64 and p.ticket == p.epoch + 4
    assert not p.recv_mc and not p.peer_recv

    class A:
        pass
    a = A()
    s.fill(a, s.data[:4])
    assert (a.world, a.rank) == (1, 0)
    with pytest.raises(ValueError):
        s.fill(a, torch.zeros(4, 1024, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        SymmSlot((16, 1024), torch.bfloat16, device="cpu", protocol="ring")
    flat = SymmSlot((64,), torch.int32, device="cpu")        # no rows: no landing zone
    assert flat.zone_bytes == 0
    with pytest.raises(ValueError):
        flat.push_args()


def test_workspace_hands_out_fixed_aligned_views():
    """Slots are real views of one buffer from the first request; `freeze()` closes the
    arena; a key cannot be re-registered with another shape."""
    from iquestrt_b200.workspace import ALIGN, Workspace
    ws = Workspace(device="cpu", capacity=1 << 16)
    a = ws.slot("a", (3, 5), torch.bfloat16)
    b = ws.slot(("b", 1), (7,), torch.float32)
    assert a.data_ptr() % ALIGN == 0 and b.data_ptr() % ALIGN == 0
    assert b.data_ptr() >= a.data_ptr() + 30
    a.fill_(1.5)
    assert ws.slot("a", (3, 5), torch.bfloat16) is a and float(a[2, 4]) == 1.5
    with pytest.raises(ValueError):
        ws.slot("a", (3, 6), torch.bfloat16)
    with pytest.raises(MemoryError):
        ws.slot("big", (1 << 20,), torch.float32)
    s = ws.slot("sym", (16, 256), torch.bfloat16, symm=True)
    assert ws.symm_slot_of(s) is not None and ws.symm_slot_of(a) is None
    before = a.data_ptr()
    assert ws.freeze() is ws
    assert ws.slot("a", (3, 5), torch.bfloat16).data_ptr() == before
    with pytest.raises(RuntimeError):
        ws.slot("late", (4,), torch.float32)
    with pytest.raises(ValueError):
        Workspace(device="cpu", align=1000)


def test_block_fp8_helpers_match_the_reference_fixtures():
    """`iquestrt_b200.blockfp8` (the package's mirror of the reference's module) against
    outputs of the reference's own functions, bit for bit, and its error behaviour."""
    from iquestrt_b200 import blockfp8, synth
    gold = torch.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.pt"),
                      weights_only=False)
    d = gold["dequant"]
    assert torch.equal(blockfp8.dequant(d["q"], d["s"]), d["f64"])
    assert torch.equal(blockfp8.dequant(d["q"], d["s"], dtype=torch.float32), d["f32"])
    d = gold["dequant_64x128"]
    assert torch.equal(blockfp8.dequant(d["q"], d["s"], d["block"], torch.float32), d["f32"])
    batch = blockfp8.dequant(torch.stack([d["q"], d["q"]]), torch.stack([d["s"], d["s"]]),
                             d["block"], torch.float32)
    assert torch.equal(batch[1], d["f32"])
    with pytest.raises(ValueError):
        blockfp8.dequant(torch.zeros(256, 256).to(torch.float8_e4m3fn), torch.ones(2, 3))
    for c in gold["shard_scale"]:
        got = blockfp8.shard_scale(c["table"], c["dim"], c["start"], c["length"], c["grain"])
        assert torch.equal(got, c["out"])
    with pytest.raises(ValueError):
        blockfp8.shard_scale(gold["shard_scale"][0]["table"], 0, 32, 64, 64)
    with pytest.raises(ValueError):
        blockfp8.shard_scale(gold["shard_scale"][0]["table"], 0, 0, 96, 96)
    assert synth.shard_scale is blockfp8.shard_scale


def test_holders_keep_the_reference_call_signatures():
    """Constructor and call parameters of the reference's holders (names and order as in
    iquestrt/kernels/{oproj,router,moe_gemv,ar_tail,tail}.py and iquestrt/workspace.py),
    followed only by keyword-only extensions."""
    import inspect
    from iquestrt_b200 import blockfp8, kernels
    from iquestrt_b200.workspace import Workspace

    def head(fn, n):
        names = [p.name for p in inspect.signature(fn).parameters.values()
                 if p.name != "self"]
        return names[:n]

    def keyword_only(fn, names):
        params = inspect.signature(fn).parameters
        return all(params[n].kind is inspect.Parameter.KEYWORD_ONLY for n in names)

    assert head(blockfp8.dequant, 4) == ["q", "scale", "block", "dtype"]
    assert head(blockfp8.shard_scale, 5) == ["scale", "dim", "start", "length", "grain"]
    assert head(kernels.OProjGemv.__init__, 4) == ["q_dim", "hidden", "ws", "q_len"]
    assert keyword_only(kernels.OProjGemv.__init__, ["ws", "q_len"])
    assert head(kernels.OProjGemv.__call__, 3) == ["ao", "w_o", "w_scale"]
    assert head(kernels.DenseMlp.__init__, 4) == ["hidden", "inter", "ws", "q_len"]
    assert head(kernels.DenseMlp.__call__, 6) == ["hn", "w_gate_up", "gate_up_scale", "w_down",
                                                  "down_scale", "out"]
    assert head(kernels.RouterSelect.__init__, 6) == ["n_experts", "top_k", "hidden", "device",
                                                      "ws", "q_len"]
    assert keyword_only(kernels.RouterSelect.__init__, ["device", "ws", "q_len"])
    assert head(kernels.RouterSelect.__call__, 2) == ["x_pad", "weight"]
    assert head(kernels.MoeDecodeKernels.__init__, 7) == ["experts", "topk", "hidden", "i_loc",
                                                          "ws", "q_len", "live_rows"]
    assert head(kernels.MoeDecodeKernels.__call__, 7) == ["sel", "wt", "fc", "fc_scale", "proj",
                                                          "proj_scale", "rows"]
    assert keyword_only(kernels.MoeDecodeKernels.__call__, ["rows"])
    for name in ("next_out",):
        assert callable(getattr(kernels.MoeDecodeKernels, name))
    assert head(kernels.MultimemARTail.__init__, 3) == ["ao_buffers", "group", "tail"]
    assert head(kernels.MultimemARTail.__call__, 6) == ["ao", "residual", "w_ao", "w_ffn",
                                                        "a_scale", "f_scale"]
    assert head(kernels.MultimemARTail.h_inv_xpad_fp8_pdl_overlap_local, 10) == [
        "ao", "residual", "w_ao", "w_ffn", "inv_out", "x_pad", "x_pad_fp8", "a_scale", "f_scale",
        "fp32_residual"]
    assert keyword_only(kernels.MultimemARTail.h_inv_xpad_fp8_pdl_overlap_local,
                        ["fp32_residual"])
    assert head(kernels.MultimemMLPTail.__init__, 4) == ["mlp_buffers", "group", "tail",
                                                         "norm_out"]
    assert head(kernels.MultimemMLPTail.__call__, 4) == ["mlp_out", "residual", "f_scale",
                                                         "w_norm"]
    assert head(kernels.TailKernels.__init__, 4) == ["hidden", "eps", "ws", "q_len"]
    assert head(Workspace.__init__, 3) == ["device", "align", "symm_group"]
    assert head(Workspace.slot, 4) == ["key", "shape", "dtype", "symm"]
    assert inspect.signature(Workspace.slot).parameters["symm"].default is False


def test_abi_library_exports_every_declared_symbol():
    """The C-ABI library loads and exports everything `include/iqb200.h` declares (no
    compute without a GPU)."""
    import re
    from iquestrt_b200 import _build, _lib
    _build.build()
    lib = _lib.load()
    header = open(os.path.join(os.path.dirname(_build.HERE), "include", "iqb200.h")).read()
    declared = set(re.findall(r"^\s*(?:int|size_t)\s+(iq_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.iq_scratch_bytes() > 65536
    # argument checks run on the host before any CUDA call
    import ctypes as C
    assert lib.iq_linear(None, None) == _lib.IQ_ERR_ARG
    a = _lib.RouterArgs()
    assert lib.iq_router(C.byref(a), None) == _lib.IQ_ERR_ARG


def test_abi_rejects_null_arguments_without_a_gpu():
    """Argument checks come before any CUDA call: every entry point returns IQ_ERR_ARG for a
    null argument block, and the scratch size covers the one-launch layer's own area."""
    import ctypes as C
    from iquestrt_b200 import _lib
    _lib.load()                                   # raises if the library is not built
    lib = C.CDLL(_lib.lib_path())                 # a handle of its own: argtypes set here stay here
    lib.iq_scratch_bytes.restype = C.c_size_t
    lib.iq_status_read.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    null = C.c_void_p(None)
    for name in ("iq_linear", "iq_linear_static", "iq_router", "iq_moe_gate", "iq_moe_down"):
        fn = getattr(lib, name)
        fn.argtypes = [C.c_void_p, C.c_void_p]
        assert fn(null, null) == _lib.IQ_ERR_ARG, name
    lib.iq_tail.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    assert lib.iq_tail(null, null, 0) == _lib.IQ_ERR_ARG
    lib.iq_linear_static_status.argtypes = [C.c_void_p, C.c_void_p]
    assert lib.iq_linear_static_status(null, null) == _lib.IQ_ERR_ARG
    assert lib.iq_status_read(null, null, 0, null) == _lib.IQ_ERR_ARG
    assert lib.iq_scratch_bytes() >= 4 * 1024 * 1024


def test_slice_checker_accepts_the_oracle_chain_and_rejects_a_wrong_layer():
    """`bench.slice_check` (the parity gate of `--workload slice4`) on fabricated kernel
    outputs: the oracle's own four-layer chain over two simulated ranks passes with zero
    error; the same chain with one layer's output disturbed by 5 % fails at that layer."""
    import bench
    from iquestrt_b200 import synth
    from oracle.cpu_layer import layer_cpu
    torch.set_num_threads(4)
    shape = synth.LayerShape(hidden=1024, q_dim=1024, n_experts=16, inter=256)
    heads = synth.HeadShape(q_heads=8, kv_heads=2)
    tp, rows, n_layers = 2, 2, 4
    lws = [[synth.make_layer(shape, tp=tp, rank=r, device="cpu", layer=i) for r in range(tp)]
           for i in range(n_layers)]
    pws = [synth.make_prologue(shape, heads, tp=tp, rank=0, device="cpu", layer=i)
           for i in range(n_layers)]
    ins = [bench.slice_inputs(synth, shape, rows, tp, r, "cpu", n_layers) for r in range(tp)]
    cos, sin = synth.rope_tables([5, 6], heads, device="cpu")
    res, xn = ins[0][1], ins[0][2]
    seen = []
    qh, kh = heads.local(tp)
    for i in range(n_layers):
        aos = [ins[r][0][i] for r in range(tp)]
        out, norm, sel, wt = layer_cpu(lws[i], aos, res, top_k=shape.top_k, n_shared=1,
                                       eps=shape.eps, score="sigmoid")
        parts = [R.linear(a, lw["o_proj"], lw["o_scale"]) for a, lw in zip(aos, lws[i])]
        _, hn = R.layer_residual_algebra(parts, res, lws[i][0]["attn_out_norm"],
                                         lws[i][0]["feed_forward_norm"], 1.0, shape.eps)
        qkv = R.linear(xn, pws[i]["w_qkv"], pws[i]["w_qkv_scale"])
        q, k, v = R.heads_prefill(qkv, qh, kh, heads.head_dim, pws[i]["w_qn"], pws[i]["w_kn"],
                                  cos, sin, heads.rotary_dim, shape.eps)
        seen.append({"q": q, "out": out, "norm": norm, "sel": sel.int().flatten(),
                     "wt": wt.flatten(), "x_pad": hn, "k": R.to_e4m3_sat(k),
                     "v": R.to_e4m3_sat(v)})
        res, xn = out, norm
    case = bench.slice_check(rows, tp, shape, heads, seen, lws, pws, ins, cos, sin, True, 2e-2)
    assert case["ok"] and all(l["rel_fro_out"] == 0.0 and l["rel_fro_q"] == 0.0
                              for l in case["layers"])
    seen[2]["out"] = (seen[2]["out"].float() * 1.05).bfloat16()
    case = bench.slice_check(rows, tp, shape, heads, seen, lws, pws, ins, cos, sin, True, 2e-2)
    assert not case["ok"]
    assert [l["ok"] for l in case["layers"]][:3] == [True, True, False]
