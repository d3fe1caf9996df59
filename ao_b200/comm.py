"""Peer-mapped buffers for the fused output exchange of row-sharded linears (one process per GPU, one node).

Every rank allocates one device buffer, exports its CUDA IPC handle, and maps the buffers of all other ranks, so that a
kernel on this GPU can store into them over NVLink.  Layout of each rank's buffer:
    [64, 72)   this rank's {finished-CTA counter, calls so far} (used by the kernels)
    [256, ...) payload: gathered outputs and landing areas, carved by the caller
torch.distributed is used only to exchange the handles.
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
        self.local_state = ctypes.c_void_p(self.base[self.rank] + 64)

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

    def close(self):
        """Unmaps the peers' buffers; call on every rank after the last kernel that uses them has finished."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        lib = _cabi.lib()
        with torch.cuda.device(self.device):
            for p in self._mapped:
                lib.ao_comm_close(ctypes.c_void_p(p))
        self._mapped = []
