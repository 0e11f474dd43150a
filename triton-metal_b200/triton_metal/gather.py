"""Host side of the row-sharded matmul whose epilogue replicates C (one process per GPU).

Every rank owns a copy of the whole C and a flag array, both plain device memory.  At set-up
the ranks trade the 64-byte tokens of those two buffers (`exchange` - any all-gather of bytes:
`torch.distributed.all_gather_object`, a file, a socket) and map each other's buffers; from then
on `launch` enqueues this rank's rows and the kernel itself writes them into every copy and
raises the flags.  This class keeps what the protocol needs on the host: which handle is whose,
and the epoch of each flag slot, which must grow by one per launch on all ranks alike.

The reference has no counterpart (one device: Sources/TritonMetalCore/Runtime.swift:10-11); the
unfused baseline is an NCCL all-gather behind an ordinary launch.
"""

from . import cuda as _cuda


class ReplicatedC:
    def __init__(self, M, N, rank, world, exchange, element_bytes=2, backend=_cuda):
        if not 0 <= rank < world <= 8:
            raise ValueError("1...8 ranks, this rank among them")
        self.M, self.N, self.rank, self.world, self.backend = M, N, rank, world, backend
        self.nbytes = M * N * element_bytes
        self.flag_bytes = backend.gather_flag_bytes()
        self.c = backend.alloc_device_buffer(self.nbytes)
        self.flags = backend.alloc_device_buffer(self.flag_bytes)
        mine = backend.ipc_export(self.c) + backend.ipc_export(self.flags) if world > 1 else b""
        tokens = exchange(mine) if world > 1 else [mine]
        if len(tokens) != world:
            raise RuntimeError(f"the exchange returned {len(tokens)} tokens for {world} ranks")
        if world > 1 and tokens[rank] != mine:
            raise RuntimeError("the exchange did not return this rank's token at its own index")
        self.replicas, self.flag_buffers, self.imported = [], [], []
        for r in range(world):
            if r == rank:
                self.replicas.append(self.c)
                self.flag_buffers.append(self.flags)
                continue
            if len(tokens[r]) != 128:
                raise RuntimeError(f"rank {r} sent {len(tokens[r])} bytes, expected two 64-byte tokens")
            c_r = backend.ipc_import(tokens[r][:64], self.nbytes)
            f_r = backend.ipc_import(tokens[r][64:], self.flag_bytes)
            self.imported += [c_r, f_r]
            self.replicas.append(c_r)
            self.flag_buffers.append(f_r)
        self.epochs = {}

    def next_epoch(self, slot):
        self.epochs[slot] = self.epochs.get(slot, 0) + 1
        return self.epochs[slot]

    def launch(self, kernel_handle, a, b, row0, rows, K, slot=0, wait=True):
        """Enqueue C[row0:row0+rows] = A @ B into every copy; returns the epoch used."""
        if row0 < 0 or rows <= 0 or row0 + rows > self.M:
            raise ValueError("rows outside C")
        epoch = self.next_epoch(slot)
        self.backend.matmul_gathered(kernel_handle, a, b, self.replicas, self.flag_buffers, self.rank,
                                     row0, rows, self.N, K, slot, epoch, wait)
        return epoch

    def close(self, free=None):
        """Unmap the peers' buffers and free this rank's.  Every rank must have finished its
        launches first (a barrier): a peer may still be storing into this rank's copy."""
        from . import _core
        free = free or _core.free_buffer
        for handle in self.imported + [self.c, self.flags]:
            free(handle)
        self.imported, self.replicas, self.flag_buffers = [], [], []
