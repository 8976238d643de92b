"""Symmetric buffers of the tensor-parallel all-reduce.

One process per GPU.  `torch.distributed` and torch's symmetric memory are used for
set-up only: allocating a buffer that every rank can address, exchanging its peer and
multicast (NVLS) addresses, and agreeing on errors.  The all-reduce itself is issued by
the kernels (`multimem.red` to signal, `multimem.ld_reduce` to read the switch-reduced
rows; plain peer loads when the GPUs expose no multicast).  No NCCL call is made on the
decode path.

Layout of a slot (bytes): `[rows | pad to 256 | arrive u32 @ +0 | epoch u32 @ +128]`.
`arrive` counts ranks that have published their rows (every rank adds one to every
rank's counter per call); `epoch` is local and counts completed calls, so waits need no
reset and survive CUDA-graph replay."""

from __future__ import annotations

import math

import torch

CTRL_BYTES = 256


def world_info():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class SymmSlot:
    """A `[*shape]` tensor every TP rank can address, plus its arrival counter."""

    def __init__(self, shape, dtype, *, device="cuda", group=None, use_multicast=True):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        nbytes = math.prod(self.shape) * torch.empty((), dtype=dtype).element_size()
        self.data_bytes = -(-nbytes // 256) * 256
        total = self.data_bytes + CTRL_BYTES
        self.world, self.rank = world_info() if group is not None else (1, 0)
        self.multicast_ptr = 0
        self.peer_ptrs = None
        self._handle = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self._handle = symm_mem.rendezvous(self.buf, group)
            self.peer_ptrs = [int(p) for p in self._handle.buffer_ptrs]
            if use_multicast:
                self.multicast_ptr = int(getattr(self._handle, "multicast_ptr", 0) or 0)
            base = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=device)
            self._peer_data = base
            self._peer_arrive = base + self.data_bytes
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=device)
        self.data = self.buf[:nbytes].view(dtype).view(self.shape)
        self.base_ptr = self.buf.data_ptr()
        self._peer_cache = {}

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0

    def fill(self, a, partial: torch.Tensor) -> None:
        """Writes the communication fields of a C `iq_tail_args` for `partial`, a view
        into this slot's rows."""
        off = partial.data_ptr() - self.base_ptr
        if off < 0 or off >= self.data_bytes:
            raise ValueError("partial is not a view into this symmetric slot")
        a.world, a.rank = self.world, self.rank
        if self.world == 1:
            return
        a.arrive = self.base_ptr + self.data_bytes
        a.epoch = self.base_ptr + self.data_bytes + 128
        if self.multicast_ptr:
            a.partial_mc = self.multicast_ptr + off
            a.arrive_mc = self.multicast_ptr + self.data_bytes
        if off not in self._peer_cache:
            self._peer_cache[off] = self._peer_data + off
        a.peer_partials = self._peer_cache[off].data_ptr()
        a.peer_arrive = self._peer_arrive.data_ptr()


# Slots by the address of their first row, so that a holder handed `slot.data[:q]` finds
# the slot's communication state (the reference keeps the same kind of table,
# iquestrt/kernels/ar_tail.py:1394-1402).
_BY_PTR: dict[int, SymmSlot] = {}


def register(slot: SymmSlot) -> SymmSlot:
    _BY_PTR[slot.data.data_ptr()] = slot
    return slot


def slot_of(tensor: torch.Tensor) -> SymmSlot | None:
    return _BY_PTR.get(tensor.data_ptr())
