"""Partition and bucket bookkeeping for several GPUs of one box.

Entities of a partitioned type are cut into `num_partitions` contiguous id ranges (the split of
torchbiggraph/converters/dictionary.py:28-43); edges fall into (lhs partition, rhs partition)
buckets.  Buckets that share no partition are independent and train concurrently, one per GPU
(docs/source/distributed_training.rst:64-68; the lock server enforces the same rule,
torchbiggraph/bucket_scheduling.py:477-540).  `round_robin_rounds` lays an epoch out as rounds of
pairwise-disjoint buckets; `ring_exchange` moves a partition (embedding rows + RowAdagrad state) to
the next GPU between rounds with torch.distributed point-to-point calls -- NCCL over NVLink on
GPUs, gloo on CPU for the tests.  The receiving GPU reads the partition only from its own memory.
"""
import math
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_bounds(num_entities: int, num_partitions: int) -> List[int]:
    """Partition p owns ids [bounds[p], bounds[p+1]).  bounds[p] = ceil(p / P * N) evaluated in double
    precision exactly as the reference does (part_start, torchbiggraph/converters/dictionary.py:28-29):
    where p * N / P is an integer the floating-point product can land just above it, and data
    partitioned by the reference then has that bound one row higher than the exact ceiling."""
    return [math.ceil(p / num_partitions * num_entities) for p in range(num_partitions + 1)]


def partition_of(ids: torch.Tensor, bounds: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """(partition, offset inside the partition) of global entity ids."""
    b = torch.as_tensor(list(bounds), device=ids.device, dtype=ids.dtype)
    part = torch.searchsorted(b, ids, right=True) - 1
    return part, ids - b[part]


def round_robin_rounds(num_partitions: int) -> List[List[Tuple[int, int]]]:
    """An epoch as rounds of buckets in which no partition appears twice.

    Off-diagonal buckets follow the circle method of round-robin tournaments: with P partitions
    (P even) there are P-1 pairings of P/2 disjoint pairs; every pair {a, b} gives the two buckets
    (a, b) and (b, a), scheduled in separate sweeps.  Diagonal buckets (p, p) come first, P per
    round.  Every one of the P*P buckets appears exactly once."""
    P = num_partitions
    rounds: List[List[Tuple[int, int]]] = [[(p, p) for p in range(P)]]
    if P == 1:
        return rounds
    n = P if P % 2 == 0 else P + 1              # odd P: one partition sits out each pairing
    ring = list(range(n))
    pairings = []
    for _ in range(n - 1):
        pairs = [(ring[i], ring[n - 1 - i]) for i in range(n // 2)]
        pairings.append([(a, b) for a, b in pairs if a < P and b < P])
        ring = [ring[0]] + [ring[-1]] + ring[1:-1]
    for pairs in pairings:
        rounds.append([(a, b) for a, b in pairs])
    for pairs in pairings:
        rounds.append([(b, a) for a, b in pairs])
    return rounds


def assign_round(round_buckets: Sequence[Tuple[int, int]], world_size: int) -> List[List[Tuple[int, int]]]:
    """Buckets of one round dealt to ranks (rank r trains assign_round(...)[r] in order)."""
    out: List[List[Tuple[int, int]]] = [[] for _ in range(world_size)]
    for i, b in enumerate(round_buckets):
        out[i % world_size].append(b)
    return out


def ring_exchange(send: Sequence[torch.Tensor], recv: Sequence[torch.Tensor], group=None) -> None:
    """Sends `send` tensors to rank+1 and fills `recv` from rank-1 (same shapes).  All ranks call
    it between rounds, when none of their kernels touches the tensors."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world == 1:
        for s, r in zip(send, recv):
            r.copy_(s)
        return
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    ops = []
    for s, r in zip(send, recv):
        ops.append(dist.P2POp(dist.isend, s, nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, prv, group))
    for req in dist.batch_isend_irecv(ops):
        req.wait()


class OverlappedRing:
    """Partition hand-off that runs beside training instead of between buckets.

    A bucket (lhs partition A, rhs partition B) is trained as two sub-buckets (A, B[:h]) and
    (A, B[h:]), edges grouped by the half their rhs row falls in -- the reference's GPU trainer
    cuts buckets into sub-partition jobs in the same way (torchbiggraph/train_gpu.py:77-100,
    243-266).  As soon as the kernels of a sub-bucket are enqueued, `start` sends that half (rows +
    RowAdagrad state) to the next rank and receives the previous rank's half into the spare
    buffer, on a side stream; the other half trains meanwhile.  `finish` makes the current stream
    wait for a transfer before the half it brought is trained on.  With the NCCL backend the
    copies travel over NVLink into the receiver's own memory; with gloo (CPU tests) the calls are
    the same without streams.  Every rank must call start/finish in the same order."""

    def __init__(self, device=None, group=None):
        self.group = group
        self.cuda = device is not None and torch.device(device).type == "cuda"
        self.stream = torch.cuda.Stream(device) if self.cuda else None

    def start(self, send: Sequence[torch.Tensor], recv: Sequence[torch.Tensor]):
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        ops = []
        for s_, r_ in zip(send, recv):
            ops.append(dist.P2POp(dist.isend, s_, nxt, self.group))
            ops.append(dist.P2POp(dist.irecv, r_, prv, self.group))
        if not self.cuda:
            return dist.batch_isend_irecv(ops)
        done = torch.cuda.Event()
        done.record()                                # everything enqueued so far has written `send`
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(done)
            return dist.batch_isend_irecv(ops)

    @staticmethod
    def finish(handle) -> None:
        if handle is None:
            return
        for req in handle:
            req.wait()


def average_relation_parameters(tensors: Sequence[torch.Tensor], group=None) -> None:
    """Shared operator tables and their AsyncAdagrad accumulators are averaged over the GPUs at
    round boundaries (one all-reduce each).  The reference's parameter server instead adds every
    trainer's delta (torchbiggraph/parameter_sharing.py:662-672); averaging keeps the step size of
    a single trainer."""
    world = dist.get_world_size(group)
    if world == 1:
        return
    for t in tensors:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        t.div_(world)
