"""Builds the reference's own single-GPU SM100 kernels into `oracle/_ref/`.  TEST
INFRASTRUCTURE ONLY (see `oracle/__init__.py`).

    python -m oracle.build_ref [/path/to/IQuestRT]

The reference keeps its expert Gate, expert Down and router kernels as CUDA source strings
that it compiles at start-up with `torch.utils.cpp_extension.load_inline`
(iquestrt/kernels/sm100_moe_fp8.py:28-346 `GATE_CUDA` / `DOWN_CUDA` and launchers,
iquestrt/kernels/router.py:416-613 `_CUDA` / `router_q8_launch`).  This recipe imports those
modules from the reference checkout, hands the UNMODIFIED strings to the same
`load_inline` call the reference makes (same function lists, same flags, architecture
10.0), and keeps only the resulting extension modules:

    oracle/_ref/iquestrt_moe_gate.so   oracle/_ref/iquestrt_moe_down.so
    oracle/_ref/iquestrt_router_q8_sm100.so

Nothing of the reference's source is written into the repository: the build directory
(which holds generated copies of the strings) is deleted after each build, and
`oracle/_ref/` is git-ignored.  The modules are what `tests/test_gpu_reference_kernels.py`
and `bench.py --impl reference-gpu` load to run the reference's kernels beside this
build's on the same GPU.  They need no GPU to build (nvcc cross-compiles), one GPU of
compute capability 10.0 to run, and the same torch as the one that built them.

The reference's TileLang kernels (o_proj, dense MLP, QKV) need tilelang 0.1.15 and CUDA
13.2 and cannot be built here; its all-reduce tails need eight ranks and wait on peers
without a bound, so they are not built either."""

from __future__ import annotations

import importlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REFERENCE = "/root/reference"

# (module file inside the reference, extension name)
UNITS = ("iquestrt_moe_gate", "iquestrt_moe_down", "iquestrt_router_q8_sm100")


def module_path(name: str) -> str:
    return os.path.join(OUT, name + ".so")


def available() -> bool:
    """True when every reference extension has been built."""
    return all(os.path.exists(module_path(n)) for n in UNITS)


def _sources(reference: str):
    """(name, cpp declaration, CUDA source, exported function, flags) for each unit, read
    from the reference's modules."""
    if reference not in sys.path:
        sys.path.insert(0, reference)
    moe = importlib.import_module("iquestrt.kernels.sm100_moe_fp8")
    router = importlib.import_module("iquestrt.kernels.router")
    return (
        ("iquestrt_moe_gate", moe._GATE_CPP, moe.GATE_CUDA, "moe_gate_launch", ["-O3"]),
        ("iquestrt_moe_down", moe._DOWN_CPP, moe.DOWN_CUDA, "moe_down_launch", ["-O3"]),
        ("iquestrt_router_q8_sm100", router._CPP, router._CUDA, "router_q8_launch",
         ["-O3", "-lineinfo"]),
    )


def _stale(name: str, reference: str) -> bool:
    path = module_path(name)
    if not os.path.exists(path):
        return True
    built = os.path.getmtime(path)
    deps = [os.path.join(reference, "iquestrt", "kernels", f)
            for f in ("sm100_moe_fp8.py", "router.py", "arch.py")]
    return any(os.path.getmtime(d) > built for d in deps)


def build(reference: str = DEFAULT_REFERENCE, force: bool = False, verbose: bool = False):
    """Build whatever is missing or older than the reference's files; returns the paths."""
    if not os.path.isdir(reference):
        raise RuntimeError(f"reference checkout not found at {reference}")
    os.makedirs(OUT, exist_ok=True)
    todo = [n for n in UNITS if force or _stale(n, reference)]
    if not todo:
        return [module_path(n) for n in UNITS]
    from torch.utils.cpp_extension import load_inline
    previous = os.environ.get("TORCH_CUDA_ARCH_LIST")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"          # what the reference's arch pin sets
    try:
        for name, cpp, cuda, function, flags in _sources(reference):
            if name not in todo:
                continue
            work = os.path.join(OUT, "build_" + name)
            shutil.rmtree(work, ignore_errors=True)
            os.makedirs(work)
            load_inline(name=name, cpp_sources=cpp, cuda_sources=cuda, functions=[function],
                        extra_cuda_cflags=flags, build_directory=work, verbose=verbose)
            shutil.copyfile(os.path.join(work, name + ".so"), module_path(name))
            shutil.rmtree(work, ignore_errors=True)
            print(f"built {module_path(name)}", flush=True)
    finally:
        if previous is None:
            os.environ.pop("TORCH_CUDA_ARCH_LIST", None)
        else:
            os.environ["TORCH_CUDA_ARCH_LIST"] = previous
    return [module_path(n) for n in UNITS]


def load(name: str):
    """Import a built reference extension (torch must already be imported: the module
    links against it)."""
    import importlib.util

    import torch  # noqa: F401
    path = module_path(name)
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: run `python -m oracle.build_ref` where the "
                           "reference checkout is available")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE
    for p in build(ref, verbose="-v" in sys.argv):
        print(p)
