"""Multi-rank host logic on CPU (gloo, world_size 2): the partition of (batch, head)
slices and of GEMM row blocks, the max-over-ranks timing reduction and the
all-gather that assembles the replicated C.  No GPU and no libtmcuda compute."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_shard_partitions_exactly():
    for total in (0, 1, 7, 128, 8192, 8193):
        for world in (1, 2, 3, 4, 8):
            parts = [bench.shard(total, r, world) for r in range(world)]
            assert parts[0][0] == 0
            assert sum(n for _, n in parts) == total
            for (a0, an), (b0, _) in zip(parts, parts[1:]):
                assert a0 + an == b0
            assert max(n for _, n in parts) - min(n for _, n in parts) <= 1


def test_flop_accounting_matches_the_reference():
    assert bench.flops(bench.WORKLOADS["gemm_bf16_8192"]) == 2 * 8192 ** 3
    fwd = bench.WORKLOADS["attn_fwd_bf16_s4096_full"]
    assert bench.flops(fwd) == 4 * 4096 ** 2 * 128 * 128
    assert bench.flops(bench.WORKLOADS["attn_fwd_bf16_s4096"]) == bench.flops(fwd) / 2
    bwd = bench.WORKLOADS["attn_bwd_bf16_s4096_d128"]
    assert bench.flops(bwd) == 10 * 4096 ** 2 * 128 * 128 / 2


def test_gemm_row_blocks_tile_the_rows():
    assert bench.gemm_chunks(4096) == 4 and bench.gemm_chunks(1024) == 2 and bench.gemm_chunks(8192) == 4
    assert bench.gemm_chunks(1536) == 3 and bench.gemm_chunks(1100) == 2 and bench.gemm_chunks(100) == 1
    for M, world in ((8192, 1), (8192, 2), (8192, 4), (8192, 8), (16384, 8), (3072, 2)):
        owned = [bench.gemm_row_blocks(M, r, world) for r in range(world)]
        chunks = len(owned[0])
        assert all(len(o) == chunks for o in owned)
        covered = sorted(b for o in owned for b in o)
        assert covered[0][0] == 0 and sum(n for _, n in covered) == M
        for (r0, n), (r1, _) in zip(covered, covered[1:]):
            assert r0 + n == r1
        # chunk c of ranks 0..world-1 is one contiguous slab, in rank order
        for c in range(chunks):
            starts = [owned[r][c][0] for r in range(world)]
            assert starts == [starts[0] + r * owned[0][c][1] for r in range(world)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triton_metal.synthetic import from_bf16_bits, gemm_inputs_bf16
        M, N, K = 64, 48, 32
        row0, rows = bench.shard(M, rank, world)
        a, b = gemm_inputs_bf16(M, N, K, 0, row0, rows)
        c_local = torch.from_numpy(from_bf16_bits(a) @ from_bf16_bits(b))
        # the exchange step of the row-sharded GEMM: all-gather of the C row blocks
        gathered = [torch.empty_like(c_local) for _ in range(world)]
        dist.all_gather(gathered, c_local)
        c_full = torch.cat(gathered, dim=0)
        # the benchmark's layout: block-cyclic row blocks, one all-gather per chunk into its
        # contiguous slab of the replicated C
        Mc = 4096
        mine = bench.gemm_row_blocks(Mc, rank, world)
        full = torch.zeros(Mc, 3)
        per_chunk = world * mine[0][1]
        for c, (r0, n) in enumerate(mine):
            local = torch.arange(r0, r0 + n, dtype=torch.float32).repeat(3, 1).T.contiguous()
            dist.all_gather_into_tensor(full[c * per_chunk:(c + 1) * per_chunk], local)
        cyclic_ok = bool(torch.equal(full[:, 0], torch.arange(Mc, dtype=torch.float32)))
        # every rank derives the same B and its own rows of A: rebuild the whole product
        blocks = []
        for r in range(world):
            r0, n = bench.shard(M, r, world)
            ar, br = gemm_inputs_bf16(M, N, K, 0, r0, n)
            blocks.append(from_bf16_bits(ar) @ from_bf16_bits(br))
        want = np.concatenate(blocks, axis=0)
        ok = np.allclose(c_full.numpy(), want)
        # timing is reported as the max over ranks
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # attention shards are disjoint contiguous slabs of batch*heads
        bh0, bh = bench.shard(128, rank, world)
        spans = [None] * world
        dist.all_gather_object(spans, (bh0, bh))
        results[rank] = (ok and cyclic_ok, float(t.item()), spans)
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_and_reduction():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        ok, tmax, spans = results[rank]
        assert ok
        assert tmax == float(world)
        assert spans == [(0, 64), (64, 64)]
