"""Symmetric buffers of the tensor-parallel all-reduce.

One process per GPU.  `torch.distributed` and torch's symmetric memory are used for
set-up only: allocating a buffer that every rank can address, exchanging its peer and
multicast (NVLS) addresses, and agreeing on errors.  The all-reduce itself is issued by
the kernels.  No NCCL call is made on the decode path.  Two protocols share a slot:

push   the producing GEMV stores every finished tile of its rows, as 32-bit words
       (bf16 value + 16-bit tag of the call), from its epilogue into the landing zone
       `[source rank][row][feature]` of EVERY rank (`multimem.st`, or one store per peer
       when the GPUs expose no multicast); the tail polls its own zone, adds the sources
       in rank order in fp32 and rounds once.  Default.
pull   every rank signals every rank's `arrive` counter (`multimem.red`), waits for its
       own counter, and reads the switch-reduced rows with `multimem.ld_reduce` (or sums
       peer loads).

Layout of a slot (bytes): `[rows | pad to 256 | control 256 | landing zone]`.  Control:
`arrive` u32 @0 (pull: ranks that have published their rows), push epoch u32 @64 and
push ticket u32 @68 (local), pull epoch u32 @128 (local).  The epochs count completed
calls on the slot, so waits need no reset and survive CUDA-graph replay."""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib

CTRL_BYTES = 256
ZONE_ROWS = 8            # rows per call the landing zone is laid out for
PROTOCOLS = ("push", "pull")


def world_info():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class SymmSlot:
    """A `[*shape]` tensor every TP rank can address, with the control words and the landing
    zone of its all-reduce."""

    def __init__(self, shape, dtype, *, device="cuda", group=None, use_multicast=True,
                 protocol="push"):
        if protocol not in PROTOCOLS:
            raise ValueError(f"protocol must be one of {PROTOCOLS}, got {protocol!r}")
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        self.protocol = protocol
        nbytes = math.prod(self.shape) * torch.empty((), dtype=dtype).element_size()
        self.data_bytes = -(-nbytes // 256) * 256
        self.world, self.rank = world_info() if group is not None else (1, 0)
        # the landing zone exists for 2-D bf16 slots (rows of an all-reduce)
        self.zone_rows = self.zone_h = 0
        if dtype == torch.bfloat16 and len(self.shape) == 2:
            self.zone_rows, self.zone_h = min(self.shape[0], ZONE_ROWS), self.shape[1]
        self.zone_off = self.data_bytes + CTRL_BYTES
        self.zone_bytes = 4 * self.world * self.zone_rows * self.zone_h
        total = self.zone_off + self.zone_bytes
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
            self._peer_zone = base + self.zone_off
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=device)
        self.data = self.buf[:nbytes].view(dtype).view(self.shape)
        self.base_ptr = self.buf.data_ptr()
        self._peer_cache = {}
        self._push = None

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0

    def push_args(self) -> _lib.PushArgs:
        """The C description of this slot's landing zone (`iq_push_args`)."""
        if not self.zone_bytes:
            raise ValueError("this slot has no landing zone (it is not a 2-D bf16 slot)")
        if self._push is None:
            a = _lib.PushArgs()
            a.world, a.rank = self.world, self.rank
            a.rows, a.h = self.zone_rows, self.zone_h
            a.recv = self.base_ptr + self.zone_off
            a.recv_mc = self.multicast_ptr + self.zone_off if self.multicast_ptr else None
            a.peer_recv = self._peer_zone.data_ptr() if self.world > 1 else None
            a.epoch = self.base_ptr + self.data_bytes + 64
            a.ticket = self.base_ptr + self.data_bytes + 68
            self._push = a
        return self._push

    def fill(self, a, partial: torch.Tensor) -> None:
        """Writes the communication fields of a C `iq_tail_args` for `partial`, a view
        into this slot's rows."""
        off = partial.data_ptr() - self.base_ptr
        if off < 0 or off >= self.data_bytes:
            raise ValueError("partial is not a view into this symmetric slot")
        a.world, a.rank = self.world, self.rank
        if self.world == 1:
            return                      # no peers: the kernels use a zone inside their scratch
        if self.protocol == "push":
            if off != 0:
                raise ValueError("the push protocol takes the slot's rows from row 0")
            a.push = C.pointer(self.push_args())
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
