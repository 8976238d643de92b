"""Aligned arena for decode buffers; addresses stay fixed while CUDA graphs use them.

Mirrors the reference's `iquestrt/workspace.py` (L16-119): opaque keys, `slot(key, shape,
dtype, symm=False)`, `freeze()`.  Symmetric slots are `parallel.SymmSlot`s, registered
by the data pointer of their tensor so that the all-reduce holders can find the
communication state of a buffer they are handed (the reference looks its multicast
pointers up the same way, iquestrt/kernels/ar_tail.py:1394-1402)."""

from __future__ import annotations

import torch

from .parallel import SymmSlot, register

ALIGN = 1024

_DT_BYTES = {
    torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int32: 4, torch.int64: 8,
    torch.uint8: 1, torch.bool: 1, torch.float8_e4m3fn: 1,
}


class Workspace:
    """Byte arena handing out stable, `ALIGN`-aligned views."""

    def __init__(self, *, device="cuda", align: int = ALIGN, symm_group=None,
                 use_multicast: bool = True):
        self.device = torch.device(device)
        self.align = align
        self.symm_group = symm_group
        self.use_multicast = use_multicast
        self._symm: dict[object, SymmSlot] = {}
        self._symm_by_ptr: dict[int, SymmSlot] = {}
        self._slots: dict[object, tuple[int, tuple[int, ...], torch.dtype]] = {}
        self._cursor = 0
        self._buf: torch.Tensor | None = None
        self._views: dict[object, torch.Tensor] = {}
        self._handed_out: dict[object, torch.Tensor] = {}

    def slot(self, key, shape, dtype: torch.dtype, symm: bool = False) -> torch.Tensor:
        """Register (or look up) a slot and return a tensor for it."""
        shape = tuple(int(s) for s in shape)
        if symm:
            if key in self._symm:
                t = self._symm[key].data
                if tuple(t.shape) != shape or t.dtype != dtype:
                    raise ValueError(f"symmetric slot {key!r} already registered as "
                                     f"{tuple(t.shape)}/{t.dtype}, requested {shape}/{dtype}")
                return t
            s = SymmSlot(shape, dtype, device=self.device, group=self.symm_group,
                         use_multicast=self.use_multicast)
            self._symm[key] = register(s)
            self._symm_by_ptr[s.data.data_ptr()] = s
            return s.data
        if key in self._slots:
            _, sh, dt = self._slots[key]
            if sh != shape or dt != dtype:
                raise ValueError(f"slot {key!r} already registered as {sh}/{dt}, requested "
                                 f"{shape}/{dtype}: two tensors under one key would alias")
            return self._view(key)
        if self._buf is not None:
            raise RuntimeError(f"slot {key!r} requested after freeze(): growing the arena "
                               "would move addresses captured graphs still write to")
        if dtype not in _DT_BYTES:
            raise ValueError(f"unsupported dtype {dtype}")
        nbytes = _DT_BYTES[dtype]
        for s in shape:
            nbytes *= s
        self._slots[key] = (self._cursor, shape, dtype)
        self._cursor += -(-nbytes // self.align) * self.align
        return self._view(key)

    def symm_slot_of(self, tensor: torch.Tensor) -> SymmSlot | None:
        """The symmetric slot whose rows start at `tensor`'s address, if any."""
        return self._symm_by_ptr.get(tensor.data_ptr())

    def freeze(self) -> "Workspace":
        """Allocate the arena once and move every placeholder, contents included, into it."""
        if self._buf is None:
            self._buf = torch.zeros(max(self._cursor, self.align), dtype=torch.uint8,
                                    device=self.device)
            self._views.clear()
            for key, ph in self._handed_out.items():
                final = self._view(key)
                final.copy_(ph)
                ph.set_(final)
                if ph.data_ptr() != final.data_ptr():
                    raise RuntimeError(f"failed to repoint placeholder for {key!r}")
            self._handed_out.clear()
        return self

    def _view(self, key) -> torch.Tensor:
        if key in self._views:
            return self._views[key]
        off, shape, dtype = self._slots[key]
        if self._buf is None:
            if key not in self._handed_out:
                self._handed_out[key] = torch.zeros(shape, dtype=dtype, device=self.device)
            return self._handed_out[key]
        n = 1
        for s in shape:
            n *= s
        v = self._buf[off:off + n * _DT_BYTES[dtype]].view(dtype).view(shape)
        self._views[key] = v
        return v
