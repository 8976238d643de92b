"""Host-side logic of the tensor-parallel path on CPU: two gloo ranks.

Covers what needs no GPU: every rank derives its shard from the same seeded global
tensors, the rank-local scale tables follow the reference's `shard_scale` rule, and the
sum over ranks of the row-parallel partial products (the all-reduce, here gloo's) equals
the unsharded product -- for o_proj and for the expert Down."""

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
    """World-size-1 slots (no process group): plain memory with the same layout."""
    from iquestrt_b200.parallel import CTRL_BYTES, SymmSlot
    s = SymmSlot((16, 1024), torch.bfloat16, device="cpu")
    assert s.world == 1 and not s.has_multicast
    assert s.buf.numel() == 16 * 1024 * 2 + CTRL_BYTES
    assert s.data.shape == (16, 1024) and int(s.buf.sum()) == 0

    class A:
        pass
    a = A()
    s.fill(a, s.data[:4])
    assert (a.world, a.rank) == (1, 0)
    with pytest.raises(ValueError):
        s.fill(a, torch.zeros(4, 1024, dtype=torch.bfloat16))


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


def test_one_launch_context_checks_its_calls():
    """`ops.one_launch` records the four calls of a layer and launches once on exit; on the
    host it refuses nesting, a call recorded twice, and an exit with a part missing -- all
    before anything reaches the library."""
    from iquestrt_b200 import _lib, ops
    with pytest.raises(RuntimeError, match="do not nest"):
        with ops.one_launch():
            with ops.one_launch():
                pass
    assert ops.one_launch._active is None
    with pytest.raises(RuntimeError, match="called twice"):
        with ops.one_launch() as ctx:
            ctx.record("router", _lib.RouterArgs())
            ctx.record("router", _lib.RouterArgs())
    assert ops.one_launch._active is None
    with pytest.raises(RuntimeError, match="no call recorded"):
        with ops.one_launch() as ctx:
            ctx.record("oproj", _lib.LinearArgs())
    assert ops.one_launch._active is None
    # an exception inside the context propagates and leaves no context open
    with pytest.raises(ValueError):
        with ops.one_launch():
            raise ValueError("inside")
    assert ops.one_launch._active is None


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
    lib.iq_decode_layer.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    assert lib.iq_decode_layer(null, null, 0) == _lib.IQ_ERR_ARG
    assert lib.iq_status_read(null, null, 0, null) == _lib.IQ_ERR_ARG
    assert lib.iq_scratch_bytes() >= 7 * 1024 * 1024
