"""Fixed-address arena for the decode buffers.

Same interface as the reference's `iquestrt/workspace.py` (L16-119): opaque keys,
`slot(key, shape, dtype, symm=False)`, `freeze()`, 1024-byte aligned slots.  The design is
a bump allocator over ONE buffer that exists from construction: a slot is a real view of
the arena the moment it is requested, so an address never changes between the request
and a later CUDA-graph capture, and `freeze()` only closes the arena to new requests.
Symmetric slots are `parallel.SymmSlot`s (their own symmetric-memory allocations),
registered by the data pointer of their tensor so that the all-reduce holders can find
the communication state of a buffer they are handed (the reference looks its multicast
pointers up the same way, iquestrt/kernels/ar_tail.py:1394-1402)."""

from __future__ import annotations

import math

import torch

from .parallel import SymmSlot, register

ALIGN = 1024
DEFAULT_CAPACITY = 32 << 20      # bytes; the holders of one decode layer use about 1.5 MB


class Workspace:
    """Hands out stable, `align`-aligned views of one pre-sized device buffer."""

    def __init__(self, *, device="cuda", align: int = ALIGN, symm_group=None,
                 use_multicast: bool = True, protocol: str = "push",
                 capacity: int = DEFAULT_CAPACITY):
        if align <= 0 or align & (align - 1):
            raise ValueError(f"align must be a power of two, got {align}")
        self.device = torch.device(device)
        self.align = align
        self.symm_group = symm_group
        self.use_multicast = use_multicast
        self.protocol = protocol
        self.capacity = int(capacity)
        # One allocation, made now.  `_top` is the first free byte; the arena's own base
        # address may be less aligned than `align`, so offsets are rounded on addresses.
        self._arena = torch.zeros(self.capacity + align, dtype=torch.uint8, device=self.device)
        self._base = self._arena.data_ptr()
        self._top = 0
        self._closed = False
        self._local: dict[object, torch.Tensor] = {}
        self._symm: dict[object, SymmSlot] = {}
        self._symm_by_ptr: dict[int, SymmSlot] = {}

    @staticmethod
    def _same(t: torch.Tensor, shape, dtype) -> bool:
        return tuple(t.shape) == shape and t.dtype == dtype

    def slot(self, key, shape, dtype: torch.dtype, symm: bool = False) -> torch.Tensor:
        """The tensor registered under `key`, carved from the arena on first request."""
        shape = tuple(int(s) for s in shape)
        known = (self._symm[key].data if key in self._symm else None) if symm \
            else self._local.get(key)
        if known is not None:
            if not self._same(known, shape, dtype):
                raise ValueError(f"slot {key!r} exists as {tuple(known.shape)}/{known.dtype}; a "
                                 f"second request as {shape}/{dtype} would alias it")
            return known
        if symm:
            s = SymmSlot(shape, dtype, device=self.device, group=self.symm_group,
                         use_multicast=self.use_multicast, protocol=self.protocol)
            self._symm[key] = register(s)
            self._symm_by_ptr[s.data.data_ptr()] = s
            return s.data
        if self._closed:
            raise RuntimeError(f"slot {key!r} requested after freeze(): the arena is closed so "
                               "that captured graphs keep valid addresses")
        try:
            size = math.prod(shape) * dtype.itemsize
        except AttributeError as exc:
            raise ValueError(f"unsupported dtype {dtype}") from exc
        start = -(-(self._base + self._top) // self.align) * self.align - self._base
        if start + size > self._arena.numel():
            raise MemoryError(f"workspace arena of {self.capacity} bytes is full at slot {key!r} "
                              f"({size} bytes); construct Workspace(capacity=...) larger")
        view = self._arena.narrow(0, start, size).view(dtype).view(shape)
        self._top = start + size
        self._local[key] = view
        return view

    def symm_slot_of(self, tensor: torch.Tensor) -> SymmSlot | None:
        """The symmetric slot whose rows start at `tensor`'s address, if any."""
        return self._symm_by_ptr.get(tensor.data_ptr())

    def freeze(self) -> "Workspace":
        """Close the arena: later `slot` calls may only look existing slots up."""
        self._closed = True
        return self

    @property
    def used_bytes(self) -> int:
        return self._top
