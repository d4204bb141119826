"""Peer-mapped receive areas for the in-kernel all-reduce of the tensor-parallel decode.

Every rank allocates one receive area with ``leankv_ipc_alloc`` (plain ``cudaMalloc`` memory
exported over CUDA IPC), the 64-byte handles travel through the process group's control plane
(``all_gather_object``), and each rank maps its peers' areas. The resulting
``leankv_xchg_t`` is what ``leankv_sparse_gemv_allreduce_f16`` takes. With ``world == 1`` nothing
is exported: the rank exchanges with itself (useful on a single GPU to exercise the code path).
"""

from __future__ import annotations

import ctypes

import torch

from . import _native


class PeerExchange:
    def __init__(self, device, rank: int = 0, world: int = 1, group=None, n_slots: int = 64,
                 max_cols: int = 4096, max_wait_iters: int = 1 << 22):
        if not 1 <= world <= _native.MAX_RANKS:
            raise ValueError(f"world must be in 1..{_native.MAX_RANKS}")
        self.lib = _native.lib()
        self.dev = torch.device(device)
        self.rank, self.world, self.group = rank, world, group
        max_cols = (max_cols + 255) // 256 * 256
        self.n_slots, self.max_cols = n_slots, max_cols
        self._mine, self._opened = [], []
        with torch.cuda.device(self.dev):
            nbytes = self.lib.leankv_xchg_recv_bytes(world, n_slots, max_cols)
            p = ctypes.c_void_p()
            h = ctypes.create_string_buffer(64)
            _native.check(self.lib.leankv_ipc_alloc(nbytes, ctypes.byref(p), h), "ipc_alloc")
            self._mine.append(p.value)
            recv = [None] * world
            recv[rank] = p.value
            if world > 1:
                import torch.distributed as dist

                gathered = [None] * world
                dist.all_gather_object(gathered, h.raw, group=group)
                for r in range(world):
                    if r == rank:
                        continue
                    q = ctypes.c_void_p()
                    _native.check(self.lib.leankv_ipc_open(gathered[r], ctypes.byref(q)), "ipc_open")
                    self._opened.append(q.value)
                    recv[r] = q.value
                dist.barrier(group=group)      # every area is zeroed and mapped before anyone writes
            self.epoch = torch.ones(1, dtype=torch.int32, device=self.dev)
            self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
            x = _native.Xchg()
            x.world, x.rank, x.n_slots, x.max_cols, x.max_wait_iters = world, rank, n_slots, max_cols, max_wait_iters
            for r in range(world):
                x.recv[r] = recv[r]
            x.epoch, x.status = self.epoch.data_ptr(), self.status.data_ptr()
            self.c = x

    def advance(self, stream: int) -> None:
        """Move to the next epoch (once per decode step, same on every rank)."""
        _native.check(self.lib.leankv_xchg_advance(self.epoch.data_ptr(), stream), "xchg_advance")

    def timed_out(self) -> bool:
        """True once any wait inside an exchanging kernel has run out."""
        return bool(int(self.status.item()))

    def close(self) -> None:
        if self.world > 1 and torch.distributed.is_initialized():
            torch.cuda.synchronize(self.dev)
            torch.distributed.barrier(group=self.group)     # nobody unmaps memory a peer may still write
        with torch.cuda.device(self.dev):
            for p in self._opened:
                self.lib.leankv_ipc_close(p)
            for p in self._mine:
                self.lib.leankv_ipc_free(p)
        self._opened, self._mine = [], []
