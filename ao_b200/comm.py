"""Peer-mapped buffers for the fused output exchange of row-sharded linears (one process per GPU, one node).

Every rank allocates one device buffer, exports its CUDA IPC handle, and maps the buffers of all other ranks, so that a
kernel on this GPU can store into them over NVLink.  The buffer is carved into call sites (one per sharded layer and
batch size, the same carving on every rank); a site holds
    [0, 16)                       the site's counters {pushed CTAs, pushes so far, CTAs done waiting, waits so far}
    [256, 256 + 2 W M N)          this rank's gathered output, bf16 [W][M][N]
    [.., + 8 W M N)               the landing area the peers' kernels store into: two buffers (used alternately by the
                                  parity of the call number) of [W][M][N/2] words {two bf16 rows, call number}
torch.distributed is used only to exchange the handles.

Lifetime rules a caller has to know: the gathered output of a site is a view of the buffer and is overwritten by the
next call of the same site (like the static outputs of a CUDA graph): consume or copy it before calling the same site
again.  Different layers must use different sites (RowShardedLinear reserves its own).  Every rank must make the same
calls in the same order.
"""
import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi

_HEADER = 256


class PeerExchange:
    def __init__(self, payload_bytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerExchange supports up to 8 ranks (one node)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.payload_bytes = (int(payload_bytes) + 255) // 256 * 256
        # at least 2 MiB so that the caching allocator gives the buffer a block of its own
        self.buf = torch.zeros(max(_HEADER + self.payload_bytes, 2 << 20), dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize(self.device)
        lib = _cabi.lib()
        handle = (ctypes.c_ubyte * 64)()
        offset = ctypes.c_int64(0)
        with torch.cuda.device(self.device):
            _cabi.check(lib.ao_comm_export(ctypes.c_void_p(self.buf.data_ptr()), handle, ctypes.byref(offset)),
                        "ao_comm_export")
        mine = (bytes(handle), int(offset.value))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self._mapped = []
        self.base = []
        with torch.cuda.device(self.device):
            for r, (h, off) in enumerate(everyone):
                if r == self.rank:
                    self.base.append(self.buf.data_ptr())
                    continue
                hbuf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                out = ctypes.c_void_p()
                _cabi.check(lib.ao_comm_import(hbuf, ctypes.byref(out)), "ao_comm_import")
                self._mapped.append(out.value)
                self.base.append(out.value + off)
        dist.barrier(group=group)
        self._next = 0          # bump pointer of reserve()
        self._sites = {}

    def payload(self, offset_bytes: int, shape, dtype) -> torch.Tensor:
        """A view of this rank's payload region."""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if offset_bytes % 16 or offset_bytes + nbytes > self.payload_bytes:
            raise ValueError("payload slice out of range or not 16-byte aligned")
        return self.buf[_HEADER + offset_bytes:_HEADER + offset_bytes + nbytes].view(dtype).view(*shape)

    def peer_pointers(self, offset_bytes: int):
        """ctypes array with the address of payload offset `offset_bytes` in every rank's buffer."""
        ptr_array = ctypes.c_void_p * self.world
        return ptr_array(*[b + _HEADER + offset_bytes for b in self.base])

    @staticmethod
    def site_bytes(world: int, M: int, N: int) -> int:
        """Payload bytes of one call site (counters, gathered output, double-buffered landing area)."""
        return 256 + (10 * world * M * N + 255) // 256 * 256

    def site(self, offset_bytes: int, M: int, N: int) -> "GatherSite":
        """The call site at payload offset `offset_bytes` (a multiple of 256) for outputs [world][M][N]."""
        key = (offset_bytes, M, N)
        st = self._sites.get(key)
        if st is None:
            if offset_bytes % 256 or offset_bytes + self.site_bytes(self.world, M, N) > self.payload_bytes:
                raise ValueError("exchange payload too small for this call site (or offset not a multiple of 256)")
            st = GatherSite(self, offset_bytes, M, N)
            self._sites[key] = st
        return st

    def reserve(self, M: int, N: int) -> "GatherSite":
        """A fresh call site behind the ones reserved so far; every rank must reserve in the same order."""
        st = self.site(self._next, M, N)
        self._next += self.site_bytes(self.world, M, N)
        return st

    def close(self):
        """Unmaps the peers' buffers; call on every rank after the last kernel that uses them has finished."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        lib = _cabi.lib()
        with torch.cuda.device(self.device):
            for p in self._mapped:
                lib.ao_comm_close(ctypes.c_void_p(p))
        self._mapped = []


class GatherSite:
    """One call site of the fused exchange: addresses of its counters, gathered output and landing areas."""

    def __init__(self, exchange: PeerExchange, offset_bytes: int, M: int, N: int):
        self.exchange, self.M, self.N = exchange, M, N
        world = exchange.world
        self.y = exchange.payload(offset_bytes + 256, (world, M, N), torch.bfloat16)
        landing_off = offset_bytes + 256 + 2 * world * M * N
        if landing_off % 16:
            raise ValueError("landing area not 16-byte aligned")
        self.peer_landing = exchange.peer_pointers(landing_off)
        self.own_landing = ctypes.c_void_p(exchange.base[exchange.rank] + _HEADER + landing_off)
        self.state = ctypes.c_void_p(exchange.base[exchange.rank] + _HEADER + offset_bytes)
        self.y_ptr = ctypes.c_void_p(self.y.data_ptr())
