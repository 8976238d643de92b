"""CPU oracle for the block-FP8 TP decode path.  TEST INFRASTRUCTURE ONLY.

Everything under this package is a checker: a torch-on-CPU restatement of the
reference's algebra for the path, pinned against fixtures that were produced by
importing the reference's own Python modules (`tests/golden/make_golden.py`).
Only `tests/`, `__graft_entry__.smoke()` and the CPU-baseline / reference legs of
`bench.py` may import it.  The product package never does: its operators fail
loudly when the CUDA library is missing.
"""
