"""The row-sharded matmul whose epilogue replicates C.

Host side (world_size 2, gloo, CPU): the set-up of `triton_metal.gather.ReplicatedC` - trading
the tokens of each rank's copy of C and of its flag array, mapping the peers' buffers, the order
of the handle lists the kernel receives, the epoch of every flag slot - against a stand-in for
the device calls.  On two GPUs (skipped with fewer): two processes run the real thing through
the C ABI and each checks its whole copy of C - its own rows and the peer's - against the
oracle, on several launches in a row.
"""

import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

import tmtest  # noqa: F401  (puts the package on the path)
from triton_metal.gather import ReplicatedC

ROOT = Path(__file__).resolve().parents[1]


class FakeDevice:
    """Stands in for triton_metal.cuda: buffers are counters, a token names (rank, buffer)."""

    def __init__(self, rank):
        self.rank, self.next, self.calls, self.freed = rank, 100 * (rank + 1), [], []

    def gather_flag_bytes(self):
        return 2048

    def alloc_device_buffer(self, nbytes):
        self.next += 1
        return self.next

    def ipc_export(self, handle):
        return bytes([self.rank]) + handle.to_bytes(8, "little") + bytes(55)

    def ipc_import(self, token, nbytes):
        assert len(token) == 64
        owner, theirs = token[0], int.from_bytes(token[1:9], "little")
        self.next += 1
        self.calls.append(("import", owner, theirs, nbytes, self.next))
        return self.next

    def matmul_gathered(self, kernel, a, b, replicas, flags, rank, row0, rows, N, K, slot, epoch, wait):
        self.calls.append(("launch", tuple(replicas), tuple(flags), rank, row0, rows, N, K, slot, epoch, wait))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _host_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def exchange(mine):
            out = [None] * world
            dist.all_gather_object(out, mine)
            return out

        dev = FakeDevice(rank)
        M, N, K = 512, 256, 128
        rep = ReplicatedC(M, N, rank, world, exchange, backend=dev)
        rows = M // world
        e1 = rep.launch(7, 1, 2, rank * rows, rows, K)
        e2 = rep.launch(7, 1, 2, rank * rows, rows, K)
        e_other_slot = rep.launch(7, 1, 2, rank * rows, rows, K, slot=3, wait=False)
        freed = []
        rep.close(free=freed.append)
        results[rank] = dict(c=rep.c, flags=rep.flags, calls=dev.calls, epochs=(e1, e2, e_other_slot), freed=freed)
    finally:
        dist.destroy_process_group()


def test_two_rank_setup_and_epochs_on_the_host():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_host_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        r, peer = results[rank], results[1 - rank]
        imports = [c for c in r["calls"] if c[0] == "import"]
        launches = [c for c in r["calls"] if c[0] == "launch"]
        # the peer's copy of C and its flag array were mapped, with the right sizes
        assert [(c[1], c[2], c[3]) for c in imports] == [(1 - rank, peer["c"], 512 * 256 * 2),
                                                         (1 - rank, peer["flags"], 2048)]
        mapped_c, mapped_flags = imports[0][4], imports[1][4]
        want_c = [r["c"], mapped_c] if rank == 0 else [mapped_c, r["c"]]
        want_f = [r["flags"], mapped_flags] if rank == 0 else [mapped_flags, r["flags"]]
        for call in launches:
            assert list(call[1]) == want_c and list(call[2]) == want_f      # index = rank, own buffer at own index
            assert call[3] == rank and call[4] == rank * 256 and call[5] == 256
        # epochs grow per slot, the same on both ranks
        assert r["epochs"] == (1, 2, 1) == peer["epochs"]
        assert [(c[8], c[9], c[10]) for c in launches] == [(0, 1, True), (0, 2, True), (3, 1, False)]
        assert r["freed"] == [mapped_c, mapped_flags, r["c"], r["flags"]]


def test_setup_refuses_a_broken_exchange():
    dev = FakeDevice(0)
    with pytest.raises(RuntimeError, match="returned 1 tokens for 2 ranks"):
        ReplicatedC(64, 64, 0, 2, lambda mine: [mine], backend=dev)
    with pytest.raises(RuntimeError, match="its own index"):
        ReplicatedC(64, 64, 0, 2, lambda mine: [bytes(128), mine], backend=dev)
    with pytest.raises(ValueError):
        ReplicatedC(64, 64, 2, 2, lambda mine: [mine, mine], backend=dev)


# ----------------------------------------------------------------------------- two GPUs

GPU_WORKER = r'''
import os, sys
import numpy as np
import torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
sys.path[:0] = [os.environ["TM_ROOT"], os.path.join(os.environ["TM_ROOT"], "triton-metal_b200")]
from triton_metal import _core, cuda, kernels
from triton_metal.gather import ReplicatedC
from triton_metal.synthetic import from_bf16_bits, gemm_inputs_bf16
from oracle import reference_math as ref
cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
def exchange(mine):
    out = [None] * world
    dist.all_gather_object(out, mine)
    return out
M, N, K = 1024, 768, 512
rows = M // world
rep = ReplicatedC(M, N, rank, world, exchange)
mm = kernels.Matmul("bf16", (128, 256, 64))
b_bits = gemm_inputs_bf16(M, N, K, 5, 0, 1)[1]
b = _core.alloc_buffer(b_bits.nbytes); _core.buffer_write(b, 0, b_bits.ctypes.data, b_bits.nbytes)
a = _core.alloc_buffer(rows * K * 2)
worst = 0.0
for step in range(3):
    parts = [gemm_inputs_bf16(M, N, K, 5 + step, r * rows, rows)[0] for r in range(world)]
    _core.buffer_write(a, 0, parts[rank].ctypes.data, parts[rank].nbytes)
    dist.barrier()                      # every rank is done reading the previous C
    rep.launch(mm.handle, a, b, rank * rows, rows, K)
    cuda.synchronize()                  # own rows stored everywhere, peers' rows arrived here
    got = np.empty((M, N), dtype=np.uint16)
    _core.buffer_read(rep.c, 0, got.ctypes.data, got.nbytes)
    want = np.concatenate([ref.matmul(from_bf16_bits(p), from_bf16_bits(b_bits)) for p in parts])
    worst = max(worst, ref.relative_error(from_bf16_bits(got), want))
dist.barrier()
rep.close(); mm.release(); _core.free_buffer(a); _core.free_buffer(b)
assert _core.live_handle_count() == 0
print(f"rank {rank} worst {worst:.3e}")
assert worst <= 2e-2, worst
dist.destroy_process_group()
'''


@pytest.mark.gpu
def test_two_gpus_replicate_c_from_the_epilogue(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(GPU_WORKER)
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TM_ROOT=str(ROOT))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outputs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, f"rank {rank}:\n{out}"
        assert "worst" in out
