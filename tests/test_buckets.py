"""Bucket scheduling and the partition hand-off between ranks (CPU: gloo, world size 2)."""
import os
import tempfile

import pytest
import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torchbiggraph_b200.buckets import (OverlappedRing, assign_round, average_relation_parameters, partition_bounds,
                                        partition_of, ring_exchange, round_robin_rounds)


@pytest.mark.parametrize("P", [1, 2, 3, 4, 7, 16])
def test_rounds_cover_every_bucket_once_without_sharing_partitions(P):
    rounds = round_robin_rounds(P)
    seen = [b for r in rounds for b in r]
    assert sorted(seen) == sorted((a, b) for a in range(P) for b in range(P))
    for r in rounds[1:]:
        parts = [p for b in r for p in b]
        assert len(parts) == len(set(parts)), "two buckets of a round share a partition"


def test_partition_bounds_follow_the_ceil_split():
    b = partition_bounds(4_847_571, 16)
    assert b[0] == 0 and b[-1] == 4_847_571 and len(b) == 17
    sizes = [b[i + 1] - b[i] for i in range(16)]
    assert max(sizes) - min(sizes) <= 1
    ids = torch.tensor([0, b[1] - 1, b[1], 4_847_570])
    part, off = partition_of(ids, b)
    assert part.tolist() == [0, 0, 1, 15] and off.tolist() == [0, b[1] - 1, 0, 4_847_570 - b[15]]


def test_partition_bounds_reproduce_the_reference_float_rounding():
    """part_start is math.ceil(part / num_parts * size) in floating point (dictionary.py:28-29): where
    part * size / num_parts is an exact integer the float product can round up past it."""
    import math
    assert partition_bounds(97078560, 100)[55] == 53393209          # exact ceiling: 53393208
    rng = np.random.default_rng(0)
    for _ in range(2000):
        N, P = int(rng.integers(1, 10**9)), int(rng.integers(1, 300))
        b = partition_bounds(N, P)
        assert b[0] == 0 and b[P] == N and all(b[i] <= b[i + 1] for i in range(P))
        p = int(rng.integers(0, P + 1))
        assert b[p] == math.ceil(p / P * N)


def test_assign_round_deals_buckets_to_ranks():
    rnd = [(0, 1), (2, 3), (4, 5), (6, 7)]
    assert assign_round(rnd, 2) == [[(0, 1), (4, 5)], [(2, 3), (6, 7)]]


def _worker(rank, world, initfile, out):
    dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    emb = torch.full((4, 3), float(rank + 1))
    state = torch.full((4,), float(10 * (rank + 1)))
    r_emb, r_state = torch.empty_like(emb), torch.empty_like(state)
    ring_exchange([emb, state], [r_emb, r_state])
    theta = torch.full((2, 3), float(rank))
    average_relation_parameters([theta])
    out.put((rank, r_emb[0, 0].item(), r_state[0].item(), theta[0, 0].item()))
    dist.barrier()
    dist.destroy_process_group()


def test_ring_exchange_and_parameter_average_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        init = os.path.join(d, "init")
        procs = [ctx.Process(target=_worker, args=(r, 2, init, q)) for r in range(2)]
        for p in procs:
            p.start()
        res = sorted(q.get(timeout=120) for _ in range(2))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    # rank 0 received rank 1's partition and vice versa; the shared table is the mean of 0 and 1
    assert res == [(0, 2.0, 20.0, 0.5), (1, 1.0, 10.0, 0.5)]


def _overlap_worker(rank, world, initfile, out):
    """Three buckets in a row: the rhs partition travels in two halves; half h leaves as soon as
    'training' on it (here: adding the rank's mark) is done and must have arrived, unchanged,
    before the next bucket trains on it."""
    dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    ring = OverlappedRing()
    rows = 6
    cur = torch.full((rows, 2), float(100 * (rank + 1)))
    other = torch.zeros_like(cur)
    halves = [slice(0, 3), slice(3, 6)]
    pend = [None, None]
    seen = []
    for step in range(3):
        for h in (0, 1):
            OverlappedRing.finish(pend[h])            # the half about to be trained on has arrived
            cur[halves[h]] += 1.0                     # "train" on the half
            seen.append(cur[halves[h]][0, 0].item())
            pend[h] = ring.start([cur[halves[h]]], [other[halves[h]]])
        cur, other = other, cur
    for h in (0, 1):
        OverlappedRing.finish(pend[h])
    out.put((rank, seen, cur[0, 0].item(), cur[5, 0].item()))
    dist.barrier()
    dist.destroy_process_group()


def test_overlapped_ring_hands_halves_on_in_order_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        init = os.path.join(d, "init")
        procs = [ctx.Process(target=_overlap_worker, args=(r, 2, init, q)) for r in range(2)]
        for p in procs:
            p.start()
        res = sorted(q.get(timeout=120) for _ in range(2))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    # every bucket adds 1 to both halves; partitions alternate between the two ranks
    assert res[0] == (0, [101.0, 101.0, 202.0, 202.0, 103.0, 103.0], 203.0, 203.0)
    assert res[1] == (1, [201.0, 201.0, 102.0, 102.0, 203.0, 203.0], 103.0, 103.0)


# ---------------------------------------------------------------- a whole epoch on several ranks
@pytest.mark.parametrize("P", [2, 4, 8, 16, 32])
def test_epoch_schedule_trains_every_bucket_once_with_two_partitions_per_slot(P):
    from torchbiggraph_b200.buckets import epoch_schedule, partition_moves
    steps = epoch_schedule(P)
    seen = [b for st in steps for bs in st.buckets for b in bs]
    assert sorted(seen) == sorted((a, b) for a in range(P) for b in range(P))
    for st in steps:
        assert sorted(p for h in st.holds for p in h) == list(range(P))          # every partition in exactly one slot
        for h, bs in zip(st.holds, st.buckets):
            assert all(set(b) <= set(h) for b in bs)                             # a slot trains over its own two partitions
    # inside a level a slot passes on one partition per step; the stationary one stays
    for a, b in zip(steps, steps[1:]):
        if a.level == b.level:
            assert [h[0] for h in a.holds] == [h[0] for h in b.holds]
            assert len(partition_moves(a, b, P // 2)) == P // 2
    # a change of level is a swap between two slots: with one slot per rank every rank gives one partition away and
    # takes one in at EVERY transition, and the placement an epoch ends with starts the next one (nothing moves)
    from torchbiggraph_b200.buckets import next_epoch_start
    for a, b in zip(steps, steps[1:]):
        moves = partition_moves(a, b, P // 2)
        assert sorted(src for _, src, _ in moves) == sorted(dst for _, _, dst in moves) == list(range(P // 2))
    again = epoch_schedule(P, next_epoch_start(steps))
    assert partition_moves(steps[-1], again[0], P // 2) == []
    assert sorted(b for st in again for bs in st.buckets for b in bs) == sorted((a, b) for a in range(P) for b in range(P))
    with pytest.raises(ValueError):
        epoch_schedule(12)
    with pytest.raises(ValueError):
        epoch_schedule(4, [(0, 1), (1, 2)])


def _epoch_worker(rank, world, initfile, P, epochs, out):
    from torchbiggraph_b200.buckets import EpochDriver, PartitionBuffer
    if world > 1:
        dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    rows, cut = 10, 6
    drv = EpochDriver(P, lambda: PartitionBuffer(torch.zeros(rows, 2), torch.zeros(rows)), cut)
    for buf in drv.resident():
        buf.emb.fill_(float(buf.partition))
    log = []

    def train(bucket, lhs, rhs, sub):
        # the tensors handed over are those of the bucket's partitions (whole, or the half the sub-bucket names)
        assert float(lhs[0][0, 0]) == bucket[0] and float(rhs[0][0, 0]) == bucket[1], (bucket, sub)
        want_l = rows if sub is None or sub[0] != "lhs" else (cut if sub[1] == 0 else rows - cut)
        want_r = rows if sub is None or sub[0] != "rhs" else (cut if sub[1] == 0 else rows - cut)
        assert lhs[0].shape[0] == want_l and rhs[0].shape[0] == want_r
        # "training" marks the rows it touched, one mark per bucket and side (the side that is whole in a half
        # sub-bucket gets half a mark from each of the two); the marks travel with the partition
        lhs[1].add_(1.0 if sub is None or sub[0] == "lhs" else 0.5)
        rhs[1].add_(1.0 if sub is None or sub[0] == "rhs" else 0.5)
        log.append((bucket, None if sub is None else sub[:2]))

    steps_per_epoch = len(drv.steps)
    for _ in range(epochs * steps_per_epoch):
        told = drv.calls_of(drv.step_index)              # what the driver says it will hand to train_fn ...
        before = len(log)
        drv.run_step(train)
        got = log[before:]                               # ... is what it hands over: split buckets once per half
        want = sorted([(bk, (side, h)) for _, bk, side in told if side is not None for h in (0, 1)] +
                      [(bk, None) for _, bk, side in told if side is None], key=repr)
        assert sorted(got, key=repr) == want, (rank, drv.step_index, told, got)
    state = {buf.partition: buf.state.clone() for buf in drv.resident()}
    out.put((rank, log, {p: (float(s.min()), float(s.max())) for p, s in state.items()}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_epoch_driver_on_one_rank_trains_whole_buckets_unless_told_to_split():
    """One rank owns every slot: partitions only change labels, buckets are trained whole; `always_split` keeps the
    half sub-buckets (the no-exchange reference point of the scaling measurements)."""
    from torchbiggraph_b200.buckets import EpochDriver, PartitionBuffer
    P, rows, cut = 8, 10, 6
    for always in (False, True):
        drv = EpochDriver(P, lambda: PartitionBuffer(torch.zeros(rows, 2), torch.zeros(rows)), cut, always_split=always)
        for buf in drv.resident():
            buf.emb.fill_(float(buf.partition))
        seen = {}

        def train(bucket, lhs, rhs, sub):
            assert float(lhs[0][0, 0]) == bucket[0] and float(rhs[0][0, 0]) == bucket[1]
            seen[bucket] = seen.get(bucket, 0.0) + (1.0 if sub is None else 0.5)
            if not always:
                assert sub is None

        n = len(drv.steps)
        split_calls = 0
        for g in range(n):
            split_calls += sum(1 for _, _, side in drv.calls_of(g) if side is not None)
            drv.run_step(train)
        assert seen == {(a, b): 1.0 for a in range(P) for b in range(P)}
        # the last step of an epoch hands nothing on (the next epoch starts from the same placement): never split
        assert (split_calls > 0) == always
        assert all(side is None for _, _, side in drv.calls_of(n - 1))


@pytest.mark.parametrize("world,P", [(1, 8), (2, 8), (2, 16), (4, 8), (8, 16)])
def test_epoch_driver_visits_every_bucket_once_per_epoch_and_marks_travel_with_partitions(world, P):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    epochs = 2
    with tempfile.TemporaryDirectory() as d:
        init = os.path.join(d, "init")
        procs = [ctx.Process(target=_epoch_worker, args=(r, world, init, P, epochs, q)) for r in range(world)]
        for p in procs:
            p.start()
        res = [q.get(timeout=180) for _ in range(world)]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    whole = {}
    marks = {}
    for rank, log, state in res:
        for bucket, sub in log:
            whole[bucket] = whole.get(bucket, 0.0) + (1.0 if sub is None else 0.5)       # two half sub-buckets make one bucket
        marks.update(state)
    assert whole == {(a, b): float(epochs) for a in range(P) for b in range(P)}
    # every row of every partition was touched by its 2P - 1 buckets (the diagonal one on both sides), each epoch
    assert marks == {p: (2.0 * P * epochs, 2.0 * P * epochs) for p in range(P)}
