#!/usr/bin/env python
"""Benchmark of the matmul / FlashAttention-2 hot path through libtmcuda's C ABI.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

Headline workload (default): bf16 GEMM 8192^3, fp32 accumulate, inputs
N(0,1)/sqrt(K) rounded to bf16; row blocks of M sharded over the ranks with an
all-gather of C.  One step = one pass of the kernel over the whole problem.
Other workloads: gemm_skinny, attn_fwd (batch 4, heads 32, d 128, seq 4096,
causal), attn_bwd (batch 8, heads 16, seq 4096, d 128, causal); attention is
sharded by (batch, head) with no collective.  With `--also` (default at N=1)
the attention workloads are measured too and reported under "also".

One JSON line on stdout (rank 0).  Everything else goes to stderr.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

if "reference" in sys.argv[1:]:
    # The CPU arm uses every host core.  A launcher that starts one process per GPU sets
    # OMP_NUM_THREADS=1 for its children; the BLAS thread count is fixed here, before numpy
    # (and with it the BLAS library) is loaded, so the arm measures the same thing under it.
    for _var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_var] = str(os.cpu_count() or 1)

import numpy as np

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "triton-metal_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def log(*a, every_rank=False):
    """Progress lines on stderr, from rank 0 unless told otherwise (one write per line, so that the
    ranks' lines do not run into each other)."""
    if every_rank or os.environ.get("RANK", "0") == "0":
        sys.stderr.write(" ".join(str(x) for x in a) + "\n")
        sys.stderr.flush()


# --------------------------------------------------------------------------- #
# Workload definitions
# --------------------------------------------------------------------------- #

WORKLOADS = {
    "gemm_bf16_8192": dict(kind="gemm", M=8192, N=8192, K=8192, element="bf16"),
    "gemm_bf16_skinny": dict(kind="gemm", M=16384, N=4096, K=14336, element="bf16"),
    "attn_fwd_bf16_s4096": dict(kind="attn_fwd", batch=4, heads=32, seq=4096, d=128, causal=True,
                                element="bf16"),
    "attn_fwd_bf16_s4096_full": dict(kind="attn_fwd", batch=4, heads=32, seq=4096, d=128,
                                     causal=False, element="bf16"),
    "attn_fwd_bf16_s16384": dict(kind="attn_fwd", batch=4, heads=32, seq=16384, d=128, causal=True,
                                 element="bf16"),
    "attn_bwd_bf16_s4096_d128": dict(kind="attn_bwd", batch=8, heads=16, seq=4096, d=128,
                                     causal=True, element="bf16"),
    "attn_bwd_bf16_s4096_d64": dict(kind="attn_bwd", batch=8, heads=16, seq=4096, d=64,
                                    causal=True, element="bf16"),
}
HEADLINE = "gemm_bf16_8192"
ALSO = ["gemm_bf16_skinny", "attn_fwd_bf16_s4096", "attn_fwd_bf16_s4096_full", "attn_fwd_bf16_s16384",
        "attn_bwd_bf16_s4096_d128", "attn_bwd_bf16_s4096_d64"]


def flops(w):
    """The reference's accounting: GEMM 2MNK (GEMMBenchmark.swift:449-451);
    forward 4 S^2 D per head (AttentionBenchmark.swift:66-68); backward
    10 S^2 D per head, five GEMMs credited (AttentionBackwardBenchmark.swift:46-49);
    a causal mask halves the credited work."""
    if w["kind"] == "gemm":
        return 2.0 * w["M"] * w["N"] * w["K"]
    per_head = (4.0 if w["kind"] == "attn_fwd" else 10.0) * w["seq"] ** 2 * w["d"]
    total = per_head * w["batch"] * w["heads"]
    return total / 2 if w["causal"] else total


def config_of(name, dist=None):
    """The `config` object both arms print."""
    w = WORKLOADS[name]
    out = {"workload": name}
    out.update({k: v for k, v in w.items() if k != "kind"})
    out["sharding"] = "rows of M + all-gather of C" if w["kind"] == "gemm" else "(batch, head)"
    if dist is not None and dist.world > 1 and w["kind"] == "gemm":
        out["gather"] = ("peer stores from the GEMM epilogue" if dist.gather_mode == "fused"
                         else "NCCL all-gather behind each launch")
        if getattr(dist, "gather_note", None):
            out["gather_note"] = dist.gather_note
    out["l2"] = "inputs larger than L2, no flush"
    return out


#: dram__bytes_read.sum + dram__bytes_write.sum per step (all kernels of the step), from the ncu
#: captures summarised under profiles/ (same workload sizes as the benchmark, one GPU).
NCU_TRAFFIC_BYTES = {
    "gemm_bf16_8192": {"bytes": 1075.6e6, "source": "profiles/gemm_tc_bf16_8192.md"},
    "attn_fwd_bf16_s4096": {"bytes": 520.0e6, "source": "profiles/attn_fwd_tc_bf16_s4096_causal.md"},
    "attn_fwd_bf16_s4096_full": {"bytes": 517.7e6, "source": "profiles/attn_fwd_tc_bf16_s4096_causal.md"},
    # dq 662.9 MB + dkdv 775.9 MB + preprocess 273.9 MB
    "attn_bwd_bf16_s4096_d128": {"bytes": 1712.7e6, "source": "profiles/attn_bwd_tc_bf16_s4096_d128_causal.md"},
    # dq 329.8 MB + dkdv 377.6 MB; the preprocess pass (O and dO once: 134 MB) was not captured at D=64
    "attn_bwd_bf16_s4096_d64": {"bytes": 707.4e6 + 134.2e6,
                                "source": "profiles/attn_bwd_tc_bf16_s4096_d64_causal.md (preprocess pass counted "
                                          "at its algorithmic bytes)"},
}


def shard(total, rank, world):
    """Contiguous block partition of `total` units: (first, count)."""
    base, extra = divmod(total, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(source="measured", hbm_gbs=p["hbm_gbs"], tf_burst=p["bf16_tflops"],
                    tf_sustained=p["bf16_tflops_sustained"])
    return dict(source="fallback", hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0)


# --------------------------------------------------------------------------- #
# Clock sampling during the timed region
# --------------------------------------------------------------------------- #

class ClockSampler:
    """nvidia-smi polled in the background.  Every line is stamped with the host time at which
    it arrived, and `stop(window)` keeps only the samples that arrived while the GPU was inside
    the timed region [window[0], window[1]] - samples from the idle time before and after say
    nothing about the clock the kernels ran at."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device, period_ms=20):
        self.device, self.period_ms, self.proc, self.lines = device, period_ms, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, window):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        return self.summarise(self.lines, window)

    @classmethod
    def summarise(cls, stamped_lines, window):
        sm, mx, power, reasons, total = [], [], [], set(), 0
        for stamp, line in stamped_lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clock, top = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            total += 1
            # a sample describes the interval that ended when it arrived
            if not (window[0] <= stamp <= window[1] + 0.005):
                continue
            sm.append(clock)
            mx.append(top)
            try:
                power.append(float(parts[3]))
            except ValueError:
                pass
            for name, flag in zip(cls.NAMES, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples_in_window": 0, "samples": total,
                    "window_s": window[1] - window[0], "reasons": []}
        return {"sm_mhz": float(np.median(sm)), "sm_min_mhz": min(sm), "sm_max_mhz": max(mx),
                "power_w": float(np.median(power)) if power else None, "samples_in_window": len(sm),
                "samples": total, "window_s": window[1] - window[0], "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- #
# GPU arm
# --------------------------------------------------------------------------- #

class Dist:
    """torch.distributed plumbing: barrier, max over ranks, all-gather of C."""

    def __init__(self, gpus):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.torch = None
        self.gather_mode = "nccl"
        if self.world > 1:
            import torch
            import torch.distributed as dist
            self.torch, self.dist = torch, dist
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        elif gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max(self, value):
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, value):
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return type(value)(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


class DeviceView:
    """Lets torch alias a libtmcuda buffer (for the NCCL all-gather of C)."""

    def __init__(self, address, shape, typestr):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr,
                                         "data": (address, False), "version": 3}


def pinned(array_like_bytes):
    """A pinned host staging buffer of the given size (torch is the allocator)."""
    import torch
    return torch.empty(array_like_bytes, dtype=torch.uint8, pin_memory=True)


def gemm_chunks(rows_per_rank):
    """How many row blocks each rank's share of M is cut into so that the all-gather of one
    block overlaps the GEMM of the next (at least 512 rows per block: a block should still
    fill the 148 SMs with 128 x 256 tiles)."""
    chunks = max(1, min(4, rows_per_rank // 512))
    while rows_per_rank % chunks:
        chunks -= 1
    return chunks


def gemm_row_blocks(M, rank, world):
    """(first row, rows) of every row block of C that `rank` computes: the M rows are cut into
    world * chunks equal blocks dealt round-robin, so chunk c of every rank - blocks
    c*world ... c*world + world-1 - is one contiguous slab of C and one all-gather fills it."""
    rows = M // world
    chunks = gemm_chunks(rows) if world > 1 else 1
    block = rows // chunks
    return [((c * world + rank) * block, block) for c in range(chunks)]


class Job:
    """Buffers and kernels of one workload; `close()` gives them back."""

    def track(self, handle):
        self.__dict__.setdefault("_buffers", []).append(handle)
        return handle

    def close(self):
        from triton_metal import _core
        for kern in self.all_kernels():
            kern.release()
        for handle in self.__dict__.get("_buffers", []):
            _core.free_buffer(handle)
        self._buffers = []


class GemmJob(Job):
    """C = A @ B with row blocks of M dealt to the ranks block-cyclically: with `chunks`
    blocks per rank, global block g = c * world + rank belongs to chunk c of `rank`.  Each
    chunk is one kernel launch; with more than one rank its C block is all-gathered (NCCL,
    enqueued in order on the library's stream) while the next chunk computes, and chunk c
    of every rank lands contiguously in the replicated C."""

    def __init__(self, w, dist, seed=0):
        from triton_metal.synthetic import gemm_inputs_bf16
        from triton_metal import _core, cuda, kernels
        self.w, self.dist, self.core, self.seed = w, dist, _core, seed
        M, N, K = w["M"], w["N"], w["K"]
        if M % dist.world:
            raise SystemExit("M must be a multiple of the number of ranks")
        self.rows = M // dist.world
        # fused gather: one launch per step computes the rank's whole share of rows and stores
        # it into every rank's copy of C; NCCL gather: block-cyclic row blocks, one launch and
        # one all-gather per block
        self.fused = dist.world > 1 and dist.gather_mode == "fused"
        blocks = [(dist.rank * self.rows, self.rows)] if self.fused else gemm_row_blocks(M, dist.rank, dist.world)
        self.row0 = blocks[0][0]
        self.chunks, self.block = len(blocks), blocks[0][1]
        self.a_host, self.b_host = [], None
        for row0, _ in blocks:
            a, b = gemm_inputs_bf16(M, N, K, seed, row0, self.block)
            self.a_host.append(a)
            self.b_host = b
        self.b = self.track(_core.alloc_buffer(self.b_host.nbytes))
        _core.buffer_write(self.b, 0, self.b_host.ctypes.data, self.b_host.nbytes)
        self.a, self.c_local = [], []
        for a in self.a_host:
            handle = self.track(_core.alloc_buffer(a.nbytes))
            _core.buffer_write(handle, 0, a.ctypes.data, a.nbytes)
            self.a.append(handle)
            # C lives in plain device memory: with more than one rank it is handed to NCCL
            self.c_local.append(self.track(cuda.alloc_device_buffer(self.block * N * 2)))
        self.kernel = kernels.Matmul("bf16", (128, 256, 64))
        self.launches_per_step = self.chunks

    def prepare(self):
        from triton_metal import cuda
        w = self.w
        self.args = [self.kernel.arguments(a, self.b, c, self.block, w["N"], w["K"])
                     for a, c in zip(self.a, self.c_local)]
        if self.dist.world > 1:
            torch = self.dist.torch
            self.stream = torch.cuda.ExternalStream(cuda.stream_handle())
        if self.fused:
            from triton_metal.gather import ReplicatedC

            def exchange(mine):
                out = [None] * self.dist.world
                self.dist.dist.all_gather_object(out, mine)
                return out

            self.replicated = ReplicatedC(w["M"], w["N"], self.dist.rank, self.dist.world, exchange)
            self.c_full = self.replicated.c
        elif self.dist.world > 1:
            torch = self.dist.torch
            self.c_full = self.track(cuda.alloc_device_buffer(w["M"] * w["N"] * 2))
            full = torch.as_tensor(DeviceView(cuda.device_pointer(self.c_full), (w["M"] * w["N"],), "<i2"),
                                   device="cuda").view(torch.bfloat16)
            per_chunk = self.dist.world * self.block * w["N"]
            self.t_out = [full[c * per_chunk:(c + 1) * per_chunk] for c in range(self.chunks)]
            self.t_local = [torch.as_tensor(DeviceView(cuda.device_pointer(h), (self.block * w["N"],), "<i2"),
                                            device="cuda").view(torch.bfloat16) for h in self.c_local]

    def step(self):
        if self.dist.world == 1:
            self.kernel.launch_async(*self.args[0])
            return
        if self.fused:
            self.replicated.launch(self.kernel.handle, self.a[0], self.b, self.row0, self.rows, self.w["K"])
            return
        torch, works = self.dist.torch, []
        with torch.cuda.stream(self.stream):
            for c in range(self.chunks):
                self.kernel.launch_async(*self.args[c])
                works.append(self.dist.dist.all_gather_into_tensor(self.t_out[c], self.t_local[c],
                                                                   async_op=True))
            for work in works:
                work.wait()      # the library's stream waits; the host does not

    def e2e_setup(self):
        """Pinned host copies of A (in row pieces), B and C, and per-piece device buffers: a piece's
        C is read back on the library's side stream while the next piece's A goes up and its GEMM
        runs, so the two PCIe directions and the tensor cores work at the same time.  With more
        than one rank each uploads only its K/world rows of B and the ranks all-gather B over
        NVLink, so the job as a whole moves A and B across PCIe once per step, as at one GPU."""
        from triton_metal import cuda
        w, b, world = self.w, self.b_host, self.dist.world
        self.pieces = []
        # plain device memory for everything the copies touch (managed memory copies slower)
        self.b_e2e = self.track(cuda.alloc_device_buffer(b.nbytes))
        sub = max(1, min(8, self.block // 1024))       # pieces per row block
        rows = self.block // sub
        for a in self.a_host:
            for i in range(sub):
                part = a[i * rows:(i + 1) * rows] if i + 1 < sub else a[i * rows:]
                pin_a = pinned(part.nbytes)
                pin_a.numpy()[:] = np.ascontiguousarray(part).reshape(-1).view(np.uint8)
                n_rows = part.shape[0]
                a_buf = self.track(cuda.alloc_device_buffer(part.nbytes))
                c_buf = self.track(cuda.alloc_device_buffer(n_rows * w["N"] * 2))
                args = self.kernel.arguments(a_buf, self.b_e2e, c_buf, n_rows, w["N"], w["K"])
                self.pieces.append((pin_a, a_buf, c_buf, pinned(n_rows * w["N"] * 2), args))
        k0, k_rows = shard(w["K"], self.dist.rank, world)
        mine = np.ascontiguousarray(b[k0:k0 + k_rows])
        self.pin_b = pinned(mine.nbytes)
        self.pin_b.numpy()[:] = mine.reshape(-1).view(np.uint8)
        if world > 1:
            if w["K"] % world:
                raise SystemExit("K must be a multiple of the number of ranks")
            torch = self.dist.torch
            self.b_part = self.track(cuda.alloc_device_buffer(mine.nbytes))
            self.t_b_part = torch.as_tensor(DeviceView(cuda.device_pointer(self.b_part), (mine.size,), "<i2"),
                                            device="cuda").view(torch.bfloat16)
            self.t_b_full = torch.as_tensor(DeviceView(cuda.device_pointer(self.b_e2e), (b.size,), "<i2"),
                                            device="cuda").view(torch.bfloat16)
        return sum(a.nbytes for a in self.a_host) + mine.nbytes, self.rows * w["N"] * 2

    def e2e_step(self):
        from triton_metal import cuda
        if self.dist.world == 1:
            cuda.write_async(self.b_e2e, 0, self.pin_b.data_ptr(), self.pin_b.numel())
        else:
            torch = self.dist.torch
            cuda.write_async(self.b_part, 0, self.pin_b.data_ptr(), self.pin_b.numel())
            with torch.cuda.stream(self.stream):
                self.dist.dist.all_gather_into_tensor(self.t_b_full, self.t_b_part)
        for pin_a, a_buf, c_buf, pin_c, args in self.pieces:
            cuda.write_async(a_buf, 0, pin_a.data_ptr(), pin_a.numel())
            self.kernel.launch_async(*args)
            cuda.read_async(c_buf, 0, pin_c.data_ptr(), pin_c.numel())
        cuda.synchronize()           # every piece of C is in host memory

    def e2e_verify(self):
        """What the end-to-end steps left in pinned host memory against what the device-resident
        steps left on the device (already checked against the oracle): the first rows of the first
        piece and the last rows of the last one, which the kernels produce bit for bit alike."""
        from triton_metal.synthetic import from_bf16_bits
        N, rows = self.w["N"], 48
        dev = np.empty((rows, N), dtype=np.uint16)
        worst = 0.0
        for piece, first in ((self.pieces[0], True), (self.pieces[-1], False)):
            pin_c = piece[3].numpy().view(np.uint16).reshape(-1, N)
            host = pin_c[:rows] if first else pin_c[-rows:]
            row = 0 if first else self.chunks * self.block - rows       # row of this rank's share
            if self.fused:
                self.core.buffer_read(self.c_full, (self.row0 + row) * N * 2, dev.ctypes.data, dev.nbytes)
            else:
                chunk, r = divmod(row, self.block)
                self.core.buffer_read(self.c_local[chunk], r * N * 2, dev.ctypes.data, dev.nbytes)
            worst = max(worst, float(np.max(np.abs(from_bf16_bits(host.copy()) - from_bf16_bits(dev)))))
        return worst

    def verify(self):
        """Relative error (the reference's `relative_error`) of sampled rows of C against the
        numpy oracle, after a step: rows of this rank's own first block and, with more than one
        rank, rows of another rank's last block read from this rank's gathered copy of C."""
        from oracle import reference_math as ref
        from triton_metal.synthetic import from_bf16_bits, gemm_inputs_bf16
        w, world, rank = self.w, self.dist.world, self.dist.rank
        N, rows = w["N"], 48
        b = from_bf16_bits(self.b_host)
        got = np.empty((rows, N), dtype=np.uint16)
        if self.fused:
            self.core.buffer_read(self.c_full, self.row0 * N * 2, got.ctypes.data, got.nbytes)
        else:
            self.core.buffer_read(self.c_local[0], 0, got.ctypes.data, got.nbytes)
        worst = ref.relative_error(from_bf16_bits(got), ref.matmul(from_bf16_bits(self.a_host[0][:rows]), b))
        if world > 1:
            other, chunk = (rank + 1) % world, self.chunks - 1
            # first row of that block in C
            row0 = other * self.rows if self.fused else (chunk * world + other) * self.block
            tail = row0 + self.block - rows
            a_other, _ = gemm_inputs_bf16(w["M"], N, w["K"], self.seed, row0, self.block)
            self.core.buffer_read(self.c_full, tail * N * 2, got.ctypes.data, got.nbytes)
            worst = max(worst, ref.relative_error(from_bf16_bits(got),
                                                  ref.matmul(from_bf16_bits(a_other[-rows:]), b)))
        return worst

    def algorithmic_bytes(self):
        w = self.w
        return 2.0 * (self.block * w["K"] + w["K"] * w["N"] + self.block * w["N"])

    def all_kernels(self):
        return [self.kernel]

    def close(self):
        if self.fused:
            self.dist.barrier()          # no rank is still storing into another's copy
            if getattr(self, "replicated", None) is not None:
                self.replicated.close()
        super().close()

    def path(self):
        return self.kernel.last_path()


class AttnJob(Job):
    def __init__(self, w, dist, seed=0):
        from triton_metal.synthetic import attention_inputs_bf16
        from triton_metal import _core, kernels
        self.w, self.dist, self.core = w, dist, _core
        bh_total = w["batch"] * w["heads"]
        self.bh0, self.bh = shard(bh_total, dist.rank, dist.world)
        S, D = w["seq"], w["d"]
        self.backward = w["kind"] == "attn_bwd"
        names = ["q", "k", "v"] + (["do"] if self.backward else [])
        self.host = attention_inputs_bf16(self.bh, S, D, seed + self.bh0, len(names))
        self.buf = {}
        nbytes = max(1, self.bh) * S * D * 2
        for name, arr in zip(names, self.host):
            self.buf[name] = self.track(_core.alloc_buffer(nbytes))
            if self.bh:
                _core.buffer_write(self.buf[name], 0, arr.ctypes.data, arr.nbytes)
        outs = ["o"] + (["dq", "dk", "dv"] if self.backward else [])
        for name in outs:
            self.buf[name] = self.track(_core.alloc_buffer(nbytes))
        for name in ("lse", "delta"):
            self.buf[name] = self.track(_core.alloc_buffer(max(1, self.bh) * S * 4))
        self.scale = kernels.default_scale(D)
        self.fwd = kernels.AttnFwd("bf16", D, (128, 128), w["causal"])
        self.kernels = [self.fwd]
        if self.backward:
            self.pre = kernels.AttnBwdPreprocess("bf16", D, 128)
            self.dq = kernels.AttnBwdDq("bf16", D, (128, 128), w["causal"])
            self.dkdv = kernels.AttnBwdDkdv("bf16", D, (128, 128), w["causal"])
            self.kernels += [self.pre, self.dq, self.dkdv]
        self.launches_per_step = 3 if self.backward else 1

    def prepare(self):
        b, S = self.buf, self.w["seq"]
        self.fwd_args = self.fwd.arguments(b["q"], b["k"], b["v"], b["o"], b["lse"], self.scale,
                                           self.bh, S)
        if self.backward:
            # the backward consumes the forward's O and L: run the forward once, untimed
            if self.bh:
                self.fwd.launch(*self.fwd_args)
            self.pre_args = self.pre.arguments(b["o"], b["do"], b["delta"], self.bh, S)
            self.dq_args = self.dq.arguments(b["q"], b["k"], b["v"], b["do"], b["dq"], b["lse"],
                                             b["delta"], self.scale, self.bh, S)
            self.dkdv_args = self.dkdv.arguments(b["q"], b["k"], b["v"], b["do"], b["dk"], b["dv"],
                                                 b["lse"], b["delta"], self.scale, self.bh, S)

    def step(self):
        if not self.bh:
            return
        if self.backward:
            self.pre.launch_async(*self.pre_args)
            self.dq.launch_async(*self.dq_args)
            self.dkdv.launch_async(*self.dkdv_args)
        else:
            self.fwd.launch_async(*self.fwd_args)

    def e2e_setup(self):
        """Pinned host copies of the inputs and outputs, and per-piece device buffers: the heads
        are cut into up to eight pieces, and a piece's outputs are read back on the library's side
        stream while the next piece's inputs go up and its kernels run."""
        from triton_metal import cuda
        S, D = self.w["seq"], self.w["d"]
        self.pins = {}
        ins = ["q", "k", "v"] + (["do"] if self.backward else [])
        h2d = 0
        for name, arr in zip(ins, self.host):
            p = pinned(arr.nbytes)
            p.numpy()[:] = arr.reshape(-1).view(np.uint8)
            self.pins[name] = p
            h2d += arr.nbytes
        outs = ["dq", "dk", "dv"] if self.backward else ["o"]
        self.pin_out = {name: pinned(max(1, self.bh) * S * D * 2) for name in outs}
        self.pieces = []
        n_pieces = max(1, min(8, self.bh // 8)) if self.bh else 0
        for i in range(n_pieces):
            h0, hn = shard(self.bh, i, n_pieces)
            nbytes, offset = hn * S * D * 2, h0 * S * D * 2
            buf = {name: self.track(cuda.alloc_device_buffer(nbytes)) for name in set(ins + outs + ["o"])}
            for name in ("lse", "delta"):
                buf[name] = self.track(cuda.alloc_device_buffer(hn * S * 4))
            launches = []
            fwd_args = self.fwd.arguments(buf["q"], buf["k"], buf["v"], buf["o"], buf["lse"], self.scale, hn, S)
            if self.backward:
                # the backward consumes the forward's O and L of the same heads: once, untimed
                for name in ("q", "k", "v"):
                    self.core.buffer_write(buf[name], 0, self.pins[name].data_ptr() + offset, nbytes)
                self.fwd.launch(*fwd_args)
                launches = [
                    (self.pre, self.pre.arguments(buf["o"], buf["do"], buf["delta"], hn, S)),
                    (self.dq, self.dq.arguments(buf["q"], buf["k"], buf["v"], buf["do"], buf["dq"], buf["lse"],
                                                buf["delta"], self.scale, hn, S)),
                    (self.dkdv, self.dkdv.arguments(buf["q"], buf["k"], buf["v"], buf["do"], buf["dk"], buf["dv"],
                                                    buf["lse"], buf["delta"], self.scale, hn, S))]
            else:
                launches = [(self.fwd, fwd_args)]
            self.pieces.append((buf, launches, offset, nbytes))
        self.e2e_in, self.e2e_out = ins, outs
        return h2d, sum(p.numel() for p in self.pin_out.values()) if self.bh else 0

    def e2e_step(self):
        from triton_metal import cuda
        for buf, launches, offset, nbytes in self.pieces:
            for name in self.e2e_in:
                cuda.write_async(buf[name], 0, self.pins[name].data_ptr() + offset, nbytes)
            for kernel, args in launches:
                kernel.launch_async(*args)
            for name in self.e2e_out:
                cuda.read_async(buf[name], 0, self.pin_out[name].data_ptr() + offset, nbytes)
        cuda.synchronize()           # every output is in host memory

    def e2e_verify(self):
        """The end-to-end outputs in pinned host memory against the device-resident ones (checked
        against the oracle by `verify`): first and last 128 rows of this rank's last head."""
        from triton_metal.synthetic import from_bf16_bits
        if not self.bh:
            return 0.0
        S, D, head = self.w["seq"], self.w["d"], self.bh - 1
        worst = 0.0
        for name in self.e2e_out:
            host = self.pin_out[name].numpy().view(np.uint16).reshape(self.bh, S, D)[head]
            for r0, r1 in ((0, 128), (S - 128, S)):
                dev = self.read_rows(name, head, r0, r1)
                worst = max(worst, float(np.max(np.abs(from_bf16_bits(host[r0:r1].copy()) - from_bf16_bits(dev)))))
        return worst

    def read_rows(self, name, head, r0, r1):
        """Rows [r0, r1) of one (batch, head) slice of a tensor of this rank's slab, as bf16 words."""
        S, D = self.w["seq"], self.w["d"]
        got = np.empty((r1 - r0, D), dtype=np.uint16)
        self.core.buffer_read(self.buf[name], (head * S + r0) * D * 2, got.ctypes.data, got.nbytes)
        return got

    def verify(self):
        """Relative error of the last (batch, head) slice of this rank's slab against the numpy
        oracle, after a step.  Up to seq 4096 the whole slice is evaluated; above that (the oracle
        is quadratic) the first and the last block of query rows."""
        from oracle import reference_math as ref
        from triton_metal.synthetic import from_bf16_bits
        if not self.bh:
            return 0.0
        w, S, D = self.w, self.w["seq"], self.w["d"]
        head, scale = self.bh - 1, 1.0 / np.sqrt(D)
        tensors = [from_bf16_bits(t[head]) for t in self.host]
        q, k, v = tensors[:3]
        if not self.backward:
            blocks = [(0, S)] if S <= 4096 else [(0, 128), (S - 256, S)]
            worst = 0.0
            for r0, r1 in blocks:
                keys = r1 if w["causal"] else S
                want, _ = ref.attention_forward(q[r0:r1], k[:keys], v[:keys], scale, w["causal"], row0=r0)
                worst = max(worst, ref.relative_error(from_bf16_bits(self.read_rows("o", head, r0, r1)), want))
            return worst
        _, weights = ref.attention_forward(q, k, v, scale, w["causal"])
        grads = ref.attention_backward(q, k, v, weights, tensors[3], scale)
        return max(ref.relative_error(from_bf16_bits(self.read_rows(n, head, 0, S)), g)
                   for n, g in zip(("dq", "dk", "dv"), grads))

    def all_kernels(self):
        return self.kernels

    def algorithmic_bytes(self):
        S, D = self.w["seq"], self.w["d"]
        tensors = 8 if self.backward else 4      # q,k,v,do + dq,dk,dv (+o read) / q,k,v + o
        return float(tensors * self.bh * S * D * 2)

    def path(self):
        return max(k.last_path() for k in self.kernels[1:] or self.kernels)


def timed_steps(job, dist, steps):
    """`steps` steps between two events on the library's stream, bracketed by a barrier and a
    synchronisation on both sides.  Returns (milliseconds, max over ranks; host-time window of
    the region; kernels launched)."""
    from triton_metal import cuda
    before = cuda.launch_count()
    dist.barrier()
    cuda.synchronize()
    t0 = time.time()
    cuda.timer_begin()
    for _ in range(steps):
        job.step()
    ms = cuda.timer_end()
    t1 = time.time()
    dist.barrier()
    return dist.max(ms), (t0, t1), cuda.launch_count() - before


def run_workload(name, args, dist, headline):
    from triton_metal import cuda
    w = WORKLOADS[name]
    pk = peaks()
    job = (GemmJob if w["kind"] == "gemm" else AttnJob)(w, dist)
    if w["kind"] == "gemm" and dist.world > 1 and dist.gather_mode == "fused":
        # The fused gather needs every rank's C mapped into every other process (CUDA IPC over
        # NVLink).  Set it up and run one step under a guard; the ranks then agree on the outcome
        # and, if any of them failed, all rebuild the job on the NCCL all-gather and say so.
        why = ""
        try:
            job.prepare()
            job.step()
            cuda.synchronize()
        except Exception as exc:      # noqa: BLE001 - reported in the JSON line
            why = f"{type(exc).__name__}: {exc}"
        if dist.max(1.0 if why else 0.0) > 0.0:
            log(f"[{name}] fused gather unavailable on rank {dist.rank}: {why or 'another rank failed'}",
                every_rank=True)
            try:
                job.close()
            except Exception:         # noqa: BLE001
                pass
            dist.gather_mode = "nccl"
            dist.gather_note = "fused gather could not be set up on every rank; NCCL all-gather used"
            job = GemmJob(w, dist)
            job.prepare()
    else:
        job.prepare()
    for _ in range(max(args.warmup, 3)):
        job.step()
    cuda.synchronize()
    sampler = ClockSampler(dist.local) if headline else None
    if sampler:
        sampler.start()
        time.sleep(0.1)
    ms, window, launches = timed_steps(job, dist, args.steps)
    total_flops = flops(w)
    tflops = total_flops / (ms / args.steps) / 1e9
    sustained = None
    if headline and not args.no_sustained:
        # the same step back to back for at least two seconds: the clock the power limit allows
        n = int(np.ceil(2100.0 / (ms / args.steps)))
        s_ms, s_window, _ = timed_steps(job, dist, n)
        lines = list(sampler.lines) if sampler.proc else []
        s_tflops = total_flops / (s_ms / n) / 1e9
        sustained = {"value": s_tflops, "unit": "TFLOP/s", "steps": n, "seconds": s_ms / 1e3,
                     "ms_per_step": s_ms / n, "peak": pk["tf_sustained"],
                     "frac": s_tflops / dist.world / pk["tf_sustained"],
                     "peak_source": f"{pk['source']} cuBLAS bf16 sustained",
                     "clocks": ClockSampler.summarise(lines, s_window) if lines else None}
    clocks = None
    if sampler:
        time.sleep(0.05)
        clocks = sampler.stop(window)
        clocks["window"] = "timed region"
        if not clocks.get("samples_in_window") and sustained and sustained["clocks"]:
            # the timed region was shorter than the sampling period: report the clocks of the
            # sustained run that followed it, and say so
            clocks = dict(sustained["clocks"], window="sustained run (the timed region of "
                          f"{ms:.1f} ms held no sample)")
    # parity of what the timed steps left in memory, on every rank
    parity = dist.max(job.verify())
    # end to end through the asynchronous tmx_* calls with pinned host buffers
    h2d, d2h = job.e2e_setup()
    for _ in range(2):
        job.e2e_step()
    e2e_steps = max(3, min(args.steps, 10))
    dist.barrier()
    cuda.synchronize()
    cuda.timer_begin()
    for _ in range(e2e_steps):
        job.e2e_step()
    e2e_ms = dist.max(cuda.timer_end())
    # the end-to-end outputs (host memory) against the device-resident ones verified above
    parity = max(parity, dist.max(job.e2e_verify()))
    h2d, d2h = dist.sum(h2d), dist.sum(d2h)
    per_gpu = tflops / dist.world
    long_region = ms > 1000.0
    peak = pk["tf_sustained"] if long_region else pk["tf_burst"]
    traffic = NCU_TRAFFIC_BYTES.get(name)
    roofline = {
        "bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
        "peak_source": f"{pk['source']} cuBLAS bf16 {'sustained' if long_region else 'burst'}",
        "traffic": traffic["bytes"] if traffic else None,
        "traffic_source": traffic["source"] if traffic else None,
        "algorithmic_bytes_per_launch": job.algorithmic_bytes(),
        "algorithmic_flops_per_step": total_flops,
    }
    result = dict(
        name=name, ms_per_step=ms / args.steps, tflops=tflops, per_gpu=per_gpu,
        e2e_tflops=total_flops / (e2e_ms / e2e_steps) / 1e9, e2e_ms_per_step=e2e_ms / e2e_steps,
        h2d=h2d, d2h=d2h, launches=launches, clocks=clocks, path=job.path(), roofline=roofline,
        timed_ms=ms, parity=parity, sustained=sustained, cpu=None)
    if not args.no_cpu_baseline and dist.world == 1:
        result["cpu"] = cpu_baseline(name)
    log(f"[{name}] {tflops:.1f} TFLOP/s  {ms / args.steps:.3f} ms/step  frac {per_gpu / peak:.3f}  "
        f"e2e {result['e2e_tflops']:.2f} TFLOP/s  parity {parity:.2e}  path {result['path']}  cpu {result['cpu']}")
    job.close()
    return result


def load_synthetic():
    """triton_metal/synthetic.py as a stand-alone module: importing it through its package
    would load libtmcuda, which the CPU legs have no use for."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "tm_synthetic", str(ROOT / "triton-metal_b200" / "triton_metal" / "synthetic.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def cpu_baseline(name, budget_s=12.0):
    """The reference's CPU path for the workload (its numpy oracles, restated in
    oracle/reference_math.py), timed on this machine's host cores on a bounded sample of the
    same problem."""
    from oracle import reference_math as ref
    syn = load_synthetic()
    w = WORKLOADS[name]
    cores = os.cpu_count() or 1
    if w["kind"] == "gemm":
        rows = min(w["M"], 2048)
        a_bits, b_bits = syn.gemm_inputs_bf16(w["M"], w["N"], w["K"], 0, 0, rows)
        a, b = syn.from_bf16_bits(a_bits), syn.from_bf16_bits(b_bits)
        best, spent = float("inf"), 0.0
        while spent < budget_s:
            t0 = time.perf_counter()
            ref.matmul(a, b)
            dt = time.perf_counter() - t0
            best, spent = min(best, dt), spent + dt
        value = 2.0 * rows * w["N"] * w["K"] / best / 1e12
        return dict(value=value, unit="TFLOP/s", cores=cores, kind="port",
                    sample=f"numpy float32 a@b on {rows} of {w['M']} rows of A (bf16-rounded "
                           f"inputs), best time within {budget_s:.0f} s")
    S, D = w["seq"], w["d"]
    scale = 1.0 / np.sqrt(D)
    seq = min(S, 2048)
    tensors = [syn.from_bf16_bits(a) for a in syn.attention_inputs_bf16(1, seq, D, 0, 4)]
    q, k, v = tensors[:3]
    t0 = time.perf_counter()
    _, weights = ref.attention_forward(q, k, v, scale, w["causal"])
    t_fwd = time.perf_counter() - t0
    halve = 2 if w["causal"] else 1
    if w["kind"] == "attn_fwd":
        return dict(value=4.0 * seq * seq * D / halve / t_fwd / 1e12, unit="TFLOP/s", cores=cores,
                    kind="port",
                    sample=f"numpy attention forward, 1 (batch, head) slice at seq {seq} of {S}")
    t0 = time.perf_counter()
    ref.attention_backward(q, k, v, weights, tensors[3], scale)
    t_bwd = time.perf_counter() - t0
    return dict(value=10.0 * seq * seq * D / halve / t_bwd / 1e12, unit="TFLOP/s", cores=cores,
                kind="port",
                sample=f"numpy attention backward, 1 (batch, head) slice at seq {seq} of {S}")


def reference_arm(args):
    """`--impl reference`: the reference's CPU implementation of the headline workload (numpy
    float32 matmul on bf16-rounded inputs: python/examples/matmul.py:71) on every host core.  One
    step is the whole 8192^3 product; rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import reference_math as ref
    syn = load_synthetic()
    name = args.workload or HEADLINE
    w = WORKLOADS[name]
    cores = os.cpu_count() or 1
    threads = os.environ.get("OPENBLAS_NUM_THREADS")
    if w["kind"] != "gemm":
        base = cpu_baseline(name)
        value, ms, sample = base["value"], None, base["sample"]
    else:
        a, b = syn.gemm_inputs_bf16(w["M"], w["N"], w["K"], 0)
        a, b = syn.from_bf16_bits(a), syn.from_bf16_bits(b)
        for _ in range(max(1, min(args.warmup, 3))):
            ref.matmul(a, b)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ref.matmul(a, b)
        dt = (time.perf_counter() - t0) / args.steps
        value = flops(w) / dt / 1e12
        ms = dt * 1e3
        sample = (f"each step = numpy float32 a@b on the whole {w['M']}x{w['N']}x{w['K']} problem "
                  f"(bf16-rounded inputs), BLAS threads {threads}")
    line = {
        "impl": "reference", "metric": "bf16_gemm_fa2_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config_of(name),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="tmcuda", choices=["tmcuda", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--also", default=None, help="comma-separated extra workloads ('none' for none)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="how the row-sharded GEMM replicates C: peer stores from the kernel's "
                         "epilogue, or an NCCL all-gather behind each launch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 20 if args.impl == "reference" else 100

    if args.impl == "reference":
        reference_arm(args)
        return

    local = int(os.environ.get("LOCAL_RANK", "0"))
    from triton_metal import _core, cuda
    cuda.set_device(local)
    if not _core.is_usable():
        raise SystemExit("libtmcuda cannot run here: " + str(_core.unusable_reason()))
    dist = Dist(args.gpus)
    dist.gather_mode = args.gather
    name = args.workload or HEADLINE
    head = run_workload(name, args, dist, True)
    also = {}
    extra = ALSO if args.also is None else [x for x in args.also.split(",") if x and x != "none"]
    if args.workload:
        extra = [] if args.also is None else extra
    for other in extra:
        r = run_workload(other, args, dist, False)
        also[other] = {"tflops": r["tflops"], "ms_per_step": r["ms_per_step"],
                       "per_gpu_tflops": r["per_gpu"], "frac_of_bf16_peak": r["roofline"]["frac"],
                       "roofline": r["roofline"], "parity_error": r["parity"],
                       "e2e_tflops": r["e2e_tflops"], "gpu_launches": r["launches"],
                       "cpu_baseline": r["cpu"], "path": r["path"]}
    if dist.rank == 0:
        pk = peaks()
        line = {
            "metric": "bf16_gemm_fa2_tflops", "value": head["tflops"], "unit": "TFLOP/s",
            "n_gpus": dist.world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_of(name, dist),
            "per_gpu_tflops": head["per_gpu"],
            "frac_of_bf16_peak": head["per_gpu"] / pk["tf_burst"],
            "roofline": head["roofline"],
            "parity_error": head["parity"],
            "sustained": head["sustained"],
            "e2e": {"value": head["e2e_tflops"], "unit": "TFLOP/s",
                    "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": head["d2h"],
                    "ms_per_step": head["e2e_ms_per_step"]},
            "gpu_launches": head["launches"],
            "kernel_path": {1: "simt", 2: "tcgen05"}.get(head["path"], "none"),
            "clocks": head["clocks"],
            "also": also,
        }
        if head["cpu"] is not None:
            line["cpu_baseline"] = head["cpu"]
        print(json.dumps(line), flush=True)
    dist.close()


if __name__ == "__main__":
    main()
