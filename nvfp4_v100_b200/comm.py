"""Peer-memory communication buffers for the one-shot all-reduce (csrc/comm.cu).

One buffer per rank, allocated with the library's own ``gpu_malloc`` (plain cudaMalloc memory, so
it can be exported through CUDA IPC), handles exchanged once through torch.distributed, peers'
buffers mapped into this process.  torch.distributed is only the rendezvous; the data path is the
library's kernel over NVLink peer loads and stores.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib

vp = ctypes.c_void_p


class PeerComm:
    def __init__(self, n: int, rank: int, world: int):
        lib = _lib.load()
        self.lib, self.n, self.rank, self.world = lib, n, rank, world
        nbytes = lib.nvfp4_comm_buffer_bytes(n)
        if nbytes < 0:
            raise ValueError("vector length must be a positive multiple of 8")
        self.own = lib.gpu_malloc(nbytes)
        if not self.own or lib.nvfp4_comm_init(vp(self.own), n) != 0:
            raise RuntimeError("communication buffer allocation failed")
        hdl = ctypes.create_string_buffer(64)
        if lib.nvfp4_ipc_get_handle(vp(self.own), hdl) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        handles = [None] * world
        dist.all_gather_object(handles, hdl.raw)
        ptrs = []
        for r, raw in enumerate(handles):
            if r == rank:
                ptrs.append(self.own)
                continue
            p = lib.nvfp4_ipc_open_handle(ctypes.create_string_buffer(raw, 64))
            if not p:
                raise RuntimeError(f"cannot map rank {r}'s communication buffer")
            ptrs.append(p)
        self.ptrs = (vp * world)(*ptrs)
        # where the producing GEMV writes its partial vector, per parity
        self.slot = [self.own + lib.nvfp4_comm_data_offset(n, p) for p in (0, 1)]
        self.calls = 0
        dist.barrier()

    def next_slot(self) -> tuple[int, int]:
        """(device address for the next partial vector, its parity); call once per all-reduce."""
        parity = self.calls & 1
        self.calls += 1
        return self.slot[parity], parity

    def allreduce_residual(self, h: torch.Tensor, parity: int, stream) -> None:
        rc = self.lib.launch_allreduce_residual(vp(h.data_ptr()), self.ptrs, self.rank, self.world,
                                                self.n, parity, stream)
        if rc != 0:
            raise RuntimeError(f"launch_allreduce_residual rc={rc}")

    def status(self) -> int:
        torch.cuda.synchronize()
        return self.lib.nvfp4_comm_status(vp(self.own))

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's.  Every rank must have finished using
        the buffers (the barrier), and no kernel may still be running on this GPU."""
        if self.own is None:
            return
        torch.cuda.synchronize()
        dist.barrier()
        for r in range(self.world):
            if r != self.rank and self.ptrs[r]:
                self.lib.nvfp4_ipc_close_handle(vp(self.ptrs[r]))
        self.lib.gpu_free(vp(self.own))
        self.own = None
