"""Exchange memory of a tensor-parallel world of one process per GPU.

Every rank makes ONE allocation (``Arena``) and carves its exchange buffers out of it in a fixed order, so that a buffer
sits at the same offset on every rank; the ranks swap the allocation's 64-byte handle (``connect``), map each other's
arenas, and a peer's buffer is then ``peer base + the same offset``. Plays the part of the reference's ``Symmetric``
buffers (``sm103/buffers.py:42-120``, made there with torch's symmetric-memory rendezvous); here the handles are plain
CUDA IPC handles from the C ABI (``mk_symm_alloc`` / ``mk_symm_open``) and no multicast object is bound to the memory.

``LocalArena`` has the same interface over ordinary torch allocations for a world whose ranks all live in one process
(the single-GPU emulation used by the parity tests).
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

ALIGN = 256


def _nbytes(shape, dtype) -> int:
    return math.prod(shape) * torch.empty((), dtype=dtype).element_size()


class _Raw:
    """A device pointer dressed as a CUDA array, so that torch can view it without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class Layout:
    """Names -> (offset, shape, dtype), carved in call order with 256-byte alignment."""

    def __init__(self):
        self.items: dict[str, tuple[int, tuple, torch.dtype]] = {}
        self.nbytes = 0

    def add(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> None:
        if name in self.items:
            raise ValueError(f"{name} carved twice")
        self.items[name] = (self.nbytes, tuple(shape), dtype)
        self.nbytes += (_nbytes(shape, dtype) + ALIGN - 1) // ALIGN * ALIGN

    def offset(self, name: str) -> int:
        return self.items[name][0]

    def signature(self) -> tuple:
        """What two ranks must agree on before they exchange pointers."""
        return tuple((k, o, s, str(d)) for k, (o, s, d) in self.items.items()) + (self.nbytes,)


class Arena:
    """This rank's allocation: zeroed device memory that peer processes can map."""

    def __init__(self, lib, layout: Layout, device):
        self.lib, self.layout, self.device = lib, layout, torch.device(device)
        with torch.cuda.device(self.device):
            self.base, self.handle = lib.symm_alloc(max(layout.nbytes, ALIGN))
        self._raw = _Raw(self.base, max(layout.nbytes, ALIGN))
        self._bytes = torch.as_tensor(self._raw, device=self.device)
        self._views: dict[str, torch.Tensor] = {}

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self._views:
            off, shape, dtype = self.layout.items[name]
            self._views[name] = self._bytes[off : off + _nbytes(shape, dtype)].view(dtype).view(shape)
        return self._views[name]

    def ptr(self, name: str) -> int:
        return self.base + self.layout.offset(name)

    def close(self) -> None:
        self._views.clear()
        self._bytes = None
        if self.base:
            self.lib.symm_free(self.base)
            self.base = 0


class LocalArena:
    """Same interface over torch allocations (a world in one process: peers are addressed by their tensors)."""

    def __init__(self, layout: Layout, device):
        self.layout, self.device = layout, torch.device(device)
        self._views = {
            k: torch.zeros(shape, dtype=dtype, device=self.device) for k, (_, shape, dtype) in layout.items.items()
        }
        self.handle = b""

    def tensor(self, name: str) -> torch.Tensor:
        return self._views[name]

    def ptr(self, name: str) -> int:
        return self._views[name].data_ptr()

    def close(self) -> None:
        self._views.clear()


class PeerArena:
    """Another rank's arena mapped into this process: pointers only."""

    def __init__(self, lib, handle: bytes, layout: Layout):
        self.lib, self.layout = lib, layout
        self.base = lib.symm_open(handle)

    def ptr(self, name: str) -> int:
        return self.base + self.layout.offset(name)

    def close(self) -> None:
        if self.base:
            self.lib.symm_close(self.base)
            self.base = 0


def connect(arena, rank: int, world: int, group=None, lib=None) -> list:
    """All-gathers the arenas' handles over ``torch.distributed`` and maps the peers -> [arena or PeerArena] by rank.
    Raises when two ranks carved different layouts (their offsets would not line up)."""
    import torch.distributed as dist

    mine = (rank, arena.handle, arena.layout.signature())
    got: list = [None] * world
    dist.all_gather_object(got, mine, group=group)
    out: list = [None] * world
    for r, handle, sig in got:
        if sig != mine[2]:
            raise RuntimeError(f"rank {r} carved a different exchange layout than rank {rank}")
        out[r] = arena if r == rank else PeerArena(lib or arena.lib, handle, arena.layout)
    return out
