"""The per-CTA work lists of the persistent attention kernels (csrc/attn_schedule.h), on the host.

Two schedules are built for every shape - equal-cost units dealt in rounds, and list scheduling
onto the least-loaded CTA - and the one that finishes earlier by the cost model is used, rounds
winning near-ties.  Every item is dealt out exactly once; a CTA's modelled load is what its
items add up to; the whole job on one GPU goes in rounds (long block paired with short one); a
shard of a job spread over eight GPUs - 16 (batch, head) slices, about as many items as SMs -
goes by the list and still keeps every SM busy."""

import numpy as np
import pytest

from triton_metal import cuda

SHAPES = [
    # kind, bh, rows, n_ctx, causal
    ("fwd", 128, 4096, 4096, True), ("fwd", 16, 4096, 4096, True), ("fwd", 16, 4096, 4096, False),
    ("fwd", 16, 16384, 16384, True), ("fwd", 3, 1000, 1000, True), ("fwd", 1, 128, 128, True),
    ("fwd", 5, 384, 1024, False),
    ("dq", 128, 4096, 4096, True), ("dq", 16, 4096, 4096, True), ("dq", 2, 1000, 1000, False),
    ("dkdv", 128, 4096, 4096, True), ("dkdv", 16, 4096, 4096, True), ("dkdv", 7, 640, 640, True),
]


def cost_of(kind, block, n_ctx, causal):
    all_blocks = -(-n_ctx // 128)
    if not causal:
        return all_blocks
    if kind == "fwd":
        return min(all_blocks, -(-min(n_ctx, (block + 1) * 256) // 128))
    return min(all_blocks, block + 1) if kind == "dq" else max(1, all_blocks - block)


@pytest.mark.parametrize("kind,bh,rows,n_ctx,causal", SHAPES)
def test_every_item_once_and_loads_level(kind, bh, rows, n_ctx, causal):
    ctas = 148
    lists, loads = cuda.attention_schedule(kind, bh, rows, n_ctx, causal, ctas)
    block_rows = 256 if kind == "fwd" else 128
    blocks = -(-rows // block_rows)
    seen = sorted(item for lst in lists for item in lst)
    assert seen == [(h, b) for h in range(bh) for b in range(blocks)]
    assert len(lists) == min(ctas, bh * blocks) and all(lists)
    overhead = 3 if kind == "fwd" else 2
    costs = [cost_of(kind, b, n_ctx, causal) + overhead for b in range(blocks)]
    # the model's loads are what the items add up to
    for lst, load in zip(lists, loads):
        assert load == sum(costs[b] for _, b in lst)
    # either the rounds (unit u = long block k + short block n-1-k of a head, to CTA u mod ctas) ...
    varying = costs[0] != costs[-1]
    units = (blocks + 1) // 2 if varying else blocks
    long_last = costs[-1] > costs[0]
    rounds = [[] for _ in lists]
    u = 0
    for h in range(bh):
        for k in range(units):
            far = blocks - 1 - k
            pair = [k] if not varying else ([far, k] if long_last else [k, far])
            if len(pair) == 2 and pair[0] == pair[1]:
                pair = pair[:1]
            rounds[u % len(lists)] += [(h, b) for b in pair]
            u += 1
    if lists == rounds:
        return
    # ... or the list: no CTA more than one item behind, and every CTA meets its items in dispatch
    # order - head-major with the long blocks of a head first before the tail (the last whole heads
    # holding at most three items per CTA), by decreasing cost inside it
    round_loads = [sum(costs[b] for _, b in lst) for lst in rounds]
    assert max(round_loads) * 100 > max(loads) * 105          # the list was taken because it is shorter
    assert max(loads) - min(loads) <= max(costs)
    tail_heads = max(1, min(bh, (3 * len(lists)) // blocks))
    for lst in lists:
        body = [(h, b) for h, b in lst if h < bh - tail_heads]
        tail = [(h, b) for h, b in lst if h >= bh - tail_heads]
        assert lst == body + tail
        assert [h for h, _ in body] == sorted(h for h, _ in body)
        for (h0, b0), (h1, b1) in zip(body, body[1:]):
            if h0 == h1:
                assert costs[b0] >= costs[b1]
        assert [costs[b] for _, b in tail] == sorted((costs[b] for _, b in tail), reverse=True)


def test_an_eighth_of_the_job_keeps_the_sms_busy():
    """16 of 128 (batch, head) slices at seq 4096, causal: the busiest CTA's load over the mean
    bounds the loss against perfect division of the work."""
    for kind, bound in (("fwd", 1.10), ("dq", 1.05), ("dkdv", 1.05)):
        _, loads = cuda.attention_schedule(kind, 16, 4096, 4096, True, 148)
        assert len(loads) == 148
        assert max(loads) / np.mean(loads) <= bound, (kind, max(loads), np.mean(loads))
    # the whole job on one GPU: within a few per cent of perfect
    for kind in ("fwd", "dq", "dkdv"):
        _, loads = cuda.attention_schedule(kind, 128, 4096, 4096, True, 148)
        assert max(loads) / np.mean(loads) <= 1.03, kind
