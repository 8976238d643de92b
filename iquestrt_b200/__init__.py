"""B200-native block-FP8 tensor-parallel decode path (drop-in for IQuestRT's hot path).

`iquestrt_b200.blockfp8` and `iquestrt_b200.kernels.*` mirror the reference's call
signatures; `iquestrt_b200.ops` is the tensor-level binding of the C ABI in
`include/iqb200.h`, implemented by `csrc/` as hand-written sm_100a CUDA."""

__version__ = "0.1.0"
