"""The benchmark CLI (csrc/tmbench.cpp), the counterpart of the reference's `tmbench`
(Sources/tmbench/main.swift:62-176): it verifies every result against a CPU reference before it
prints a number (Sources/TritonMetalBench/GEMMBenchmark.swift:325-375,
AttentionBenchmark.swift:223-291, AttentionBackwardBenchmark.swift:263-414) and exits non-zero
when the verification fails."""

import subprocess
from pathlib import Path

import pytest

import tmtest

TMBENCH = Path(__file__).resolve().parents[1] / "triton-metal_b200" / "lib" / "tmbench"


def run(*args, timeout=300):
    return subprocess.run([str(TMBENCH), *args], capture_output=True, text=True, timeout=timeout)


def test_probe_and_flag_parsing_need_no_gpu():
    out = run("--probe")
    assert out.returncode == 0 and out.stdout.startswith("device: ")
    assert ("usable" in out.stdout)
    assert run("--help").returncode == 0
    bad = run("--no-such-flag")
    assert bad.returncode == 1 and "unknown argument" in bad.stderr
    assert run("--attn-shapes", "1,2,3").returncode == 1


@pytest.mark.gpu
def test_gemm_sweep_verifies_before_it_prints():
    tmtest.require_gpu()
    out = run("--sizes", "256,512", "--element", "f32")
    assert out.returncode == 0, out.stderr
    rows = [l for l in out.stdout.splitlines() if l.split() and l.split()[0] in ("256", "512")]
    assert len(rows) == 2 and all("verified (max error" in r for r in rows), out.stdout
    out = run("--sizes", "1024", "--element", "bf16", "--config", "128,256,64,4;128,128,64,4", "--peak", "1603")
    assert out.returncode == 0, out.stderr
    assert "verified (max error" in out.stdout and "%" in out.stdout
    unverified = run("--sizes", "256", "--no-verify")
    assert unverified.returncode == 0 and "not verified" in unverified.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("flags", [("--attn",), ("--attn", "--causal"), ("--attn-bwd",), ("--attn-bwd", "--causal")])
def test_attention_benchmarks_verify_before_they_print(flags):
    tmtest.require_gpu()
    out = run(*flags, "--attn-shapes", "1,2,512,64;1,2,384,128", "--attn-element", "bf16")
    assert out.returncode == 0, out.stderr
    rows = [l for l in out.stdout.splitlines() if l.startswith("b1 h2")]
    assert len(rows) == 2 and all("verified (max error" in r for r in rows), out.stdout
    out = run(*flags, "--attn-shapes", "1,2,96,64", "--attn-element", "f32")
    assert out.returncode == 0, out.stderr
    assert "verified (max error" in out.stdout
