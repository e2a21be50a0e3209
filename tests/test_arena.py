"""The activation planner (rt_arena_plan) against a Python restatement of the reference's
BufferAllocator::greedy_by_size (crates/ratchet-core/src/gpu/buffer_allocator/allocator.rs:209-271) and against
the properties any placement must have.  Host only."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from ratchet_b200 import _lib


def plan(records, alignment=256):
    lib = _lib.load()
    n = len(records)
    rec = (_lib.rt_usage_record * max(n, 1))()
    for i, (size, prod, last) in enumerate(records):
        rec[i].size, rec[i].producer, rec[i].last_consumer = size, prod, last
    objs = (ctypes.c_int32 * max(n, 1))()
    offs = (ctypes.c_uint64 * max(n, 1))()
    n_obj, total = ctypes.c_int32(), ctypes.c_uint64()
    _lib.check(lib.rt_arena_plan(rec, n, alignment, objs, offs, ctypes.byref(n_obj), ctypes.byref(total)))
    return [int(objs[i]) for i in range(n)], [int(offs[i]) for i in range(n)], int(n_obj.value), int(total.value)


def greedy_by_size_restated(records):
    """allocator.rs:209-271 line by line: records by size descending (stable), the last suitable shared object
    wins, a new object has the record's size."""
    order = sorted(range(len(records)), key=lambda i: -records[i][0])
    assigned = {}
    objects = []  # sizes
    for r in order:
        _, prod, last = records[r]
        best = None
        for obj in range(len(objects)):
            suitable = True
            for o, (_, p2, l2) in enumerate(records):
                if max(prod, p2) <= min(last, l2) and assigned.get(o) == obj:
                    suitable = False
                    break
            if suitable:
                best = obj
        if best is None:
            objects.append(records[r][0])
            best = len(objects) - 1
        assigned[r] = best
    return [assigned[i] for i in range(len(records))], objects


def alive_together(a, b):
    return max(a[1], b[1]) <= min(a[2], b[2])


def check_valid(records, offs, total):
    for i, a in enumerate(records):
        assert offs[i] + a[0] <= total
        for j in range(i + 1, len(records)):
            b = records[j]
            if alive_together(a, b) and a[0] and b[0]:
                assert offs[i] + a[0] <= offs[j] or offs[j] + b[0] <= offs[i], (i, j, a, b, offs[i], offs[j])


def peak_live_bytes(records):
    steps = max((r[2] for r in records), default=-1) + 1
    return max((sum(r[0] for r in records if r[1] <= t <= r[2]) for t in range(steps)), default=0)


def test_random_graphs_match_the_restatement_and_never_overlap_live_tensors():
    rng = np.random.default_rng(7)
    for case in range(200):
        n = int(rng.integers(1, 40))
        steps = int(rng.integers(1, 30))
        records = []
        for _ in range(n):
            prod = int(rng.integers(0, steps))
            last = int(rng.integers(prod, steps))
            size = int(rng.integers(1, 64)) * int(rng.choice([1, 256, 4096, 1000]))
            records.append((size, prod, last))
        objs, offs, n_obj, total = plan(records, alignment=int(rng.choice([1, 16, 256])))
        want_objs, want_sizes = greedy_by_size_restated(records)
        assert objs == want_objs, case
        assert n_obj == len(want_sizes)
        check_valid(records, offs, total)
        assert total >= peak_live_bytes(records)
        # records of one object start at one offset; an object is as large as its first (largest) tenant
        for o in range(n_obj):
            mine = [i for i in range(n) if objs[i] == o]
            assert len({offs[i] for i in mine}) == 1
            assert max(records[i][0] for i in mine) == want_sizes[o]


def test_the_last_suitable_object_is_taken_not_the_first():
    # two objects exist (100 and 90 bytes, alive together); a later 10-byte record fits either: the reference's
    # loop keeps the last one it finds
    records = [(100, 0, 1), (90, 0, 1), (10, 3, 4)]
    objs, offs, n_obj, total = plan(records, alignment=1)
    assert objs == [0, 1, 1] and n_obj == 2 and total == 190 and offs == [0, 100, 100]


def test_decoder_layers_of_mlp_blocks_ping_pong_between_two_objects():
    """The node list of a decode step: x -> fc1 -> h -> fc2 -> y -> fc1 -> ... (phi2/mlp.rs:13-15 repeated): every
    tensor dies at its consumer, so two objects hold all of them: the largest hidden and the largest model-width
    tensor."""
    records = []
    for layer in range(32):
        records.append((10240 * 2, 2 * layer, 2 * layer + 1))      # hidden: fc1 -> fc2
        records.append((2560 * 2, 2 * layer + 1, 2 * layer + 2))   # layer output: fc2 -> next fc1
    objs, offs, n_obj, total = plan(records)
    assert n_obj == 2
    assert total == 10240 * 2 + 2560 * 2
    assert total <= sum(sorted((r[0] for r in records), reverse=True)[:2])
    check_valid(records, offs, total)


def test_phi3_block_with_node_scratch():
    """gate_up (paired output scratch alive during node 0 only) -> hidden -> down: the scratch and the hidden are
    alive together at node 0; nothing of node 0's scratch survives into node 1, so node 1's scratch reuses it."""
    records = [(8192 * 2, 0, 1),        # hidden
               (16384 * 2, 0, 0),       # node 0: plain gate|up row before the fold
               (3072 * 8192 * 2, 1, 1)]  # node 1: dequantised weights
    objs, offs, n_obj, total = plan(records)
    assert objs[1] == objs[2] != objs[0]
    assert total == 3072 * 8192 * 2 + 8192 * 2
    check_valid(records, offs, total)


def test_alignment_and_empty_and_bad_arguments():
    objs, offs, n_obj, total = plan([], alignment=256)
    assert (n_obj, total) == (0, 0)
    objs, offs, n_obj, total = plan([(1, 0, 0), (1, 0, 0), (1, 0, 0)], alignment=256)
    assert offs == [0, 256, 512] and total == 768
    lib = _lib.load()
    rec = (_lib.rt_usage_record * 1)()
    rec[0].size, rec[0].producer, rec[0].last_consumer = 8, 3, 2
    assert lib.rt_arena_plan(rec, 1, 256, None, None, None, None) == _lib.RT_ERR_ARG
    rec[0].last_consumer = 3
    assert lib.rt_arena_plan(rec, 1, 48, None, None, None, None) == _lib.RT_ERR_ARG
    assert lib.rt_arena_plan(rec, 1, 256, None, None, None, None) == _lib.RT_OK
