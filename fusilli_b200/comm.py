"""Multi-GPU exchange over the C ABI's fb_comm_* entry points: one `Comm` per rank (one
process per GPU, one Handle per device as in the reference, include/fusilli/backend/handle.h:74-112).

The reference has no multi-device code; this is the piece the sharded benchmark needs beyond
per-device Handles: the cross-rank sum of the convolution weight gradient (fused peer-memory
kernel or NCCL all-reduce + cast) and the output all-gather. Bootstrap bytes travel through a
caller-supplied all-gather (torch.distributed in bench.py; anything that moves bytes will do)."""
from __future__ import annotations

import ctypes
from typing import Callable, List, Optional

from .graph import DataType, ErrorCode, FusilliError
from .runtime import Buffer, Handle, _check, lib

HANDLE_BYTES = 256
_VP = ctypes.c_void_p


class Comm:
    def __init__(self, ptr, handle: Handle):
        self._ptr = ptr
        self._handle = handle

    @staticmethod
    def create(handle: Handle, rank: int, world: int, buffer_bytes: int,
               allgather_bytes: Optional[Callable[[bytes], List[bytes]]] = None) -> "Comm":
        """Collective over all ranks. `allgather_bytes(b)` returns every rank's `b` in rank order;
        it may be omitted when world == 1."""
        buffer_bytes = (int(buffer_bytes) + 255) // 256 * 256
        out = _VP()
        _check(lib().fb_comm_create(handle._ptr, int(rank), int(world), buffer_bytes, ctypes.byref(out)))
        comm = Comm(out, handle)
        if world > 1:
            if allgather_bytes is None:
                raise FusilliError(ErrorCode.InvalidArgument, "Comm.create: world > 1 needs an all-gather of bytes")
            block = ctypes.create_string_buffer(HANDLE_BYTES)
            _check(lib().fb_comm_local_handle(comm._ptr, block))
            blocks = allgather_bytes(block.raw)
            if len(blocks) != world or any(len(b) != HANDLE_BYTES for b in blocks):
                raise FusilliError(ErrorCode.InvalidArgument, "Comm.create: all-gather returned malformed blocks")
            _check(lib().fb_comm_connect(comm._ptr, b"".join(blocks)))
        return comm

    def rank(self) -> int:
        return lib().fb_comm_rank(self._ptr)

    def world(self) -> int:
        return lib().fb_comm_world(self._ptr)

    def bufferPtr(self) -> int:
        return lib().fb_comm_buffer(self._ptr) or 0

    def bufferBytes(self) -> int:
        return lib().fb_comm_buffer_bytes(self._ptr)

    def view(self, offset: int, nbytes: int) -> Buffer:
        """A Buffer over [offset, offset + nbytes) of this rank's exchange buffer: bind a weight
        gradient output to it, or read a summed result from it."""
        if offset < 0 or nbytes <= 0 or offset + nbytes > self.bufferBytes():
            raise FusilliError(ErrorCode.InvalidArgument, "Comm.view: range outside the exchange buffer")
        return Buffer.importPointer(self._handle, self.bufferPtr() + offset, nbytes)

    def sumFused(self, in_offset: int, count: int, out_offset: int, out_dtype: DataType) -> None:
        _check(lib().fb_comm_sum_fused(self._ptr, int(in_offset), int(count), int(out_offset), int(out_dtype)))

    def sumNccl(self, inout_ptr: int, count: int, out_ptr: int, out_dtype: DataType) -> None:
        _check(lib().fb_comm_sum_nccl(self._ptr, _VP(inout_ptr), int(count), _VP(out_ptr), int(out_dtype)))

    def allGather(self, send_ptr: int, recv_ptr: int, bytes_per_rank: int) -> None:
        _check(lib().fb_comm_allgather(self._ptr, _VP(send_ptr), _VP(recv_ptr), int(bytes_per_rank)))

    def close(self) -> None:
        if self._ptr:
            lib().fb_comm_close(self._ptr)
            self._ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def torch_allgather_bytes(group=None) -> Callable[[bytes], List[bytes]]:
    """All-gather of small byte strings over an initialised torch.distributed group."""
    import torch.distributed as dist

    def gather(b: bytes) -> List[bytes]:
        out: List[Optional[bytes]] = [None] * dist.get_world_size(group)
        dist.all_gather_object(out, b, group=group)
        return [bytes(x) for x in out]
    return gather
