"""Device buffers that grow without copying (``gca_vmem_*`` in the C ABI).

``VirtualBuffer`` reserves one range of virtual addresses per sequence, large enough for the longest
context the caller wants to support, and maps physical memory behind the front of every range in
2 MB steps as the cache fills.  The tensor over the whole reservation never moves, so the chunk
cache of a growing context is appended to in place for its whole life: no ``torch.cat`` re-copy per
append as in the reference (``model/DRT.py:87-133``), no doubling copy, no moment at which the old
and the new buffer exist side by side.  Only the mapped front of a range may be touched; the chunk
cache hands out views of exactly that part.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import torch

from . import _lib


class _Span:
    """Lets ``torch.as_tensor`` wrap raw device memory without copying (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class VirtualBuffer:
    def __init__(self, device: torch.device, ranges: int, range_bytes: int):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("VirtualBuffer maps device memory (there is no CPU path)")
        lib = _lib.lib()
        self.index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(self.index):
            self.gran = int(lib.gca_vmem_granularity(self.index))
            if self.gran <= 0:
                raise RuntimeError("the driver offers no virtual memory management on this device")
            self.ranges = int(ranges)
            self.range_bytes = -(-int(range_bytes) // self.gran) * self.gran
            va = C.c_void_p()
            _lib.call("gca_vmem_reserve", self.ranges * self.range_bytes, self.gran, C.byref(va))
        self.va = va.value
        self.mapped = 0                                   # bytes mapped at the front of EVERY range
        self._handles: List[Tuple[int, int, int]] = []    # (address, bytes, handle)
        self._flat = torch.as_tensor(_Span(self.va, self.ranges * self.range_bytes), device=self.device)

    def ensure(self, bytes_per_range: int) -> int:
        """Map memory so that the first ``bytes_per_range`` bytes of every range are usable.  Returns the
        number of usable bytes per range (a multiple of the granularity)."""
        need = -(-int(bytes_per_range) // self.gran) * self.gran
        if need > self.range_bytes:
            raise ValueError(f"the reservation holds {self.range_bytes} bytes per range, {need} requested")
        if need > self.mapped:
            with torch.cuda.device(self.index):
                for r in range(self.ranges):
                    addr = self.va + r * self.range_bytes + self.mapped
                    h = C.c_ulonglong()
                    _lib.call("gca_vmem_map", addr, need - self.mapped, self.index, C.byref(h))
                    self._handles.append((addr, need - self.mapped, h.value))
            self.mapped = need
        return self.mapped

    def view(self, dtype: torch.dtype, row_shape: Tuple[int, ...]) -> torch.Tensor:
        """A (ranges, rows, *row_shape) tensor over the whole reservation, rows = what a range can hold.
        Only rows inside the mapped front may be accessed."""
        item = torch.empty((), dtype=dtype).element_size()
        row = item
        for d in row_shape:
            row *= d
        rows = self.range_bytes // row
        flat = self._flat.view(dtype)
        strides = [self.range_bytes // item, row // item]
        acc = row // item
        for d in row_shape:
            acc //= d
            strides.append(acc)
        return flat.as_strided((self.ranges, rows) + tuple(row_shape), strides[:2 + len(row_shape)])

    def close(self) -> None:
        if self.va is None:
            return
        torch.cuda.synchronize(self.device)
        lib = _lib.lib()
        for addr, nbytes, h in self._handles:
            lib.gca_vmem_unmap(addr, nbytes, h)
        lib.gca_vmem_free(self.va, self.ranges * self.range_bytes)
        self._handles, self.va, self.mapped, self._flat = [], None, 0, None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
