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
from typing import List, NamedTuple, Sequence, Tuple

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

    def start_to(self, send: Sequence[torch.Tensor], to_rank: int, recv: Sequence[torch.Tensor], from_rank: int):
        """As `start`, with explicit peers: `send` goes to `to_rank`, `recv` is filled by `from_rank`."""
        ops = []
        for s_ in send:
            ops.append(dist.P2POp(dist.isend, s_, to_rank, self.group))
        for r_ in recv:
            ops.append(dist.P2POp(dist.irecv, r_, from_rank, self.group))
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


def sum_relation_parameter_deltas(tensors: Sequence[torch.Tensor], before: Sequence[torch.Tensor], group=None) -> None:
    """The reference's reconciliation (torchbiggraph/parameter_sharing.py:662-672): every trainer's change since the
    last exchange is added to the shared value, theta = before + sum over ranks of (theta_rank - before); the
    AsyncAdagrad accumulators (sums of squared gradients) add up the same way.  `before` holds the values all ranks
    agreed on at the last exchange."""
    world = dist.get_world_size(group)
    if world == 1:
        return
    for t, b in zip(tensors, before):
        delta = t - b
        dist.all_reduce(delta, op=dist.ReduceOp.SUM, group=group)
        t.copy_(b + delta)


# ---------------------------------------------------------------------------------------------------
# A whole epoch on several GPUs: every bucket once, no partition in two places, hand-offs beside training
# ---------------------------------------------------------------------------------------------------
class EpochStep(NamedTuple):
    """One step of an epoch.  `holds[s]` = (stationary partition, circulating partition) resident in slot s;
    `buckets[s]` = the buckets slot s trains in this step, all over its two partitions."""
    holds: List[Tuple[int, int]]
    buckets: List[List[Tuple[int, int]]]
    level: int


def epoch_schedule(num_partitions: int) -> List[EpochStep]:
    """All P x P buckets of an epoch for P/2 slots (P a power of two, P >= 2), every slot holding two
    partitions at a time and training only buckets over those two -- the lock server's rule that buckets
    in flight share no partition (torchbiggraph/bucket_scheduling.py:477-540), laid out ahead of time as the
    reference's GPU trainer lays out its sub-partition jobs (torchbiggraph/train_gpu.py:354-387).

    Level 0 splits the partitions into a stationary half A and a circulating half B: in step s slot i holds
    (A[i], B[(i + s) mod |B|]) and trains (a, b) and (b, a); after |B| steps every A x B and B x A bucket is
    done and B has gone once round the ring of slots.  What is left are the buckets inside A and inside B:
    the next level does the same for each half on half of the slots, and so on; at the last level a slot
    holds the only two partitions of its group and also trains their diagonal buckets.  For P = 16:
    8 + 4 + 2 + 1 = 15 steps, 256 buckets, and between two steps of a level a slot passes exactly one
    partition to its ring neighbour."""
    P = num_partitions
    if P < 2 or P & (P - 1):
        raise ValueError("epoch_schedule needs a power-of-two number of partitions >= 2")
    steps: List[EpochStep] = []
    groups = [list(range(P))]            # each group owns len(group) / 2 consecutive slots
    level = 0
    while len(groups[0]) >= 2:
        g = len(groups[0])
        half = g // 2
        last = g == 2
        for s in range(half):
            holds, buckets = [], []
            for grp in groups:
                A, B = grp[:half], grp[half:]
                for i in range(half):
                    a, b = A[i], B[(i + s) % half]
                    holds.append((a, b))
                    bs = [(a, b), (b, a)]
                    if last:
                        bs += [(a, a), (b, b)]
                    buckets.append(bs)
            steps.append(EpochStep(holds, buckets, level))
        groups = [h for grp in groups for h in (grp[:half], grp[half:])]
        level += 1
    return steps


def slot_rank(slot: int, num_slots: int, world_size: int) -> int:
    """Slots are dealt to ranks in consecutive blocks, so that the rings of the deeper levels (which span
    fewer and fewer neighbouring slots) stay inside one GPU as far as possible."""
    if num_slots % world_size:
        raise ValueError("the number of slots (partitions / 2) must be a multiple of the world size")
    return slot // (num_slots // world_size)


def partition_moves(prev: EpochStep, nxt: EpochStep, world_size: int) -> List[Tuple[int, int, int]]:
    """(partition, from rank, to rank) for every partition that changes GPU between two steps."""
    S = len(prev.holds)
    where = {}
    for s, (a, b) in enumerate(prev.holds):
        where[a] = where[b] = slot_rank(s, S, world_size)
    moves = []
    for s, (a, b) in enumerate(nxt.holds):
        r = slot_rank(s, S, world_size)
        for p in (a, b):
            if where[p] != r:
                moves.append((p, where[p], r))
    return moves


class PartitionBuffer:
    """Embedding rows and RowAdagrad state of one partition in this GPU's memory (all buffers of a driver
    have the same shape, so that any partition fits any buffer)."""

    def __init__(self, emb: torch.Tensor, state: torch.Tensor):
        self.emb, self.state = emb, state
        self.partition = -1

    def half(self, h: int, cut: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return (self.emb[:cut], self.state[:cut]) if h == 0 else (self.emb[cut:], self.state[cut:])

    def tensors(self) -> List[torch.Tensor]:
        return [self.emb, self.state]


class EpochDriver:
    """Runs `epoch_schedule` on the ranks of a process group: every rank owns the slots `slot_rank` gives it,
    trains their buckets step by step, and passes partitions on as the schedule says.

    Inside a level the circulating partition b of a slot leaves for the ring neighbour in two halves (rows
    [0, cut) and [cut, rows)): the step trains, for h = 0, 1, the sub-buckets (b[h], a) -- edges of bucket
    (b, a) whose lhs row lies in half h -- and (a, b[h]); as soon as those of half h are enqueued the half is
    sent (and the half arriving from the other neighbour received into the spare buffer) on a side stream,
    beside the training of the other half: the hand-off is off the critical path, as the reference overlaps
    partition swaps with training through its sub-partition jobs (torchbiggraph/train_gpu.py:456-652).  A
    neighbour on the same GPU gets the buffer itself.  Between levels (three times per epoch of 16
    partitions, and at the epoch's end) partitions are re-dealt with one blocking exchange.

    train_fn(bucket, lhs, rhs, sub) does the training: lhs / rhs are (emb, state) tensors -- whole partitions
    or halves -- and sub is None for a whole bucket or ("lhs" | "rhs", h, cut) for a half sub-bucket.
    after_step(step) runs once per step on every rank (e.g. the all-reduce of shared relation parameters).
    """

    def __init__(self, num_partitions: int, alloc, cut: int, group=None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.steps = epoch_schedule(num_partitions)
        self.S = num_partitions // 2
        self.local_slots = [s for s in range(self.S) if slot_rank(s, self.S, self.world) == self.rank]
        self.cut = cut
        self.alloc = alloc
        self.ring = OverlappedRing(device, group) if self.world > 1 else None
        self.stat = {s: alloc() for s in self.local_slots}
        self.circ = {s: alloc() for s in self.local_slots}
        self.spare = alloc() if self.world > 1 else None
        self.pending = [None, None]          # hand-off of half h started in the previous step
        self.step_index = 0
        self._pool: List[PartitionBuffer] = []
        for s in self.local_slots:
            a, b = self.steps[0].holds[s]
            self.stat[s].partition, self.circ[s].partition = a, b

    def resident(self) -> List[PartitionBuffer]:
        """Buffers that hold a partition right now (for initialisation and checkpointing)."""
        return [self.stat[s] for s in self.local_slots] + [self.circ[s] for s in self.local_slots]

    # ---- one step -------------------------------------------------------------------------------
    def _ring_of(self, step: EpochStep, slot: int) -> Tuple[int, int]:
        half = self.S >> step.level            # slots per ring at this level
        base = slot // half * half
        return base, half

    def run_step(self, train_fn, after_step=None) -> int:
        """Trains the current step of the schedule on this rank's slots, starts the hand-offs that lead to the
        next one, and returns the number of buckets (whole-bucket equivalents) trained here."""
        k = self.step_index % len(self.steps)
        st = self.steps[k]
        nxt = self.steps[(k + 1) % len(self.steps)]
        same_level = nxt.level == st.level and k + 1 < len(self.steps)
        last_level = len(st.buckets[0]) == 4
        cut = self.cut
        base, half = self._ring_of(st, self.local_slots[0])
        # the one ring that spans ranks (if any): its lowest local slot sends off-rank, its highest receives
        spans = same_level and half > len(self.local_slots)
        send_slot = self.local_slots[0] if spans else None
        recv_slot = self.local_slots[-1] if spans else None
        done = 0
        for h in (0, 1):
            if self.pending[h] is not None:          # the half about to be trained on has arrived, the old one has left
                OverlappedRing.finish(self.pending[h])
                self.pending[h] = None
            for s in self.local_slots:
                a, b = st.holds[s]
                A, B = self.stat[s], self.circ[s]
                assert A.partition == a and B.partition == b, (self.rank, k, s, A.partition, B.partition, a, b)
                train_fn((b, a), B.half(h, cut), (A.emb, A.state), ("lhs", h, cut))
                train_fn((a, b), (A.emb, A.state), B.half(h, cut), ("rhs", h, cut))
                if s == send_slot:
                    nb_rank = slot_rank(base + (s - base - 1) % half, self.S, self.world)
                    from_rank = slot_rank(base + (recv_slot - base + 1) % half, self.S, self.world)
                    self.pending[h] = self.ring.start_to(list(B.half(h, cut)), nb_rank, list(self.spare.half(h, cut)), from_rank)
        for s in self.local_slots:
            done += 2
            if last_level:
                a, b = st.holds[s]
                A, B = self.stat[s], self.circ[s]
                train_fn((a, a), (A.emb, A.state), (A.emb, A.state), None)
                train_fn((b, b), (B.emb, B.state), (B.emb, B.state), None)
                done += 2
        if after_step is not None:
            after_step(st)
        # ---- where the partitions are in the next step ----
        if same_level:
            self._rotate(st, nxt, spans, send_slot, recv_slot)
        else:
            for h in (0, 1):
                OverlappedRing.finish(self.pending[h])
                self.pending[h] = None
            self._redeal(st, nxt)
        self.step_index += 1
        return done

    def _rotate(self, st: EpochStep, nxt: EpochStep, spans: bool, send_slot, recv_slot) -> None:
        """Inside a level: slot s's circulating partition becomes that of slot s - 1 of its ring."""
        old = {s: self.circ[s] for s in self.local_slots}
        for s in self.local_slots:
            base, half = self._ring_of(st, s)
            src = base + (s - base + 1) % half               # the slot whose partition comes here
            if src in old and not (spans and s == recv_slot):
                self.circ[s] = old[src]
        if spans:
            incoming = self.spare                             # being filled by the transfers started in this step
            incoming.partition = nxt.holds[recv_slot][1]
            self.spare = old[send_slot]                       # leaves with the same transfers; free once they finish
            self.spare.partition = -1
            self.circ[recv_slot] = incoming
        for s in self.local_slots:
            assert self.circ[s].partition == nxt.holds[s][1], (self.rank, s, self.circ[s].partition, nxt.holds[s])

    def _redeal(self, st: EpochStep, nxt: EpochStep) -> None:
        """Between levels and at the end of an epoch: every partition goes where the next step wants it, in
        one blocking exchange (buffers that stay on the GPU are only re-labelled)."""
        have = {}
        for s in self.local_slots:
            have[self.stat[s].partition] = self.stat[s]
            have[self.circ[s].partition] = self.circ[s]
        want = [(s, role, p) for s in self.local_slots for role, p in zip(("stat", "circ"), nxt.holds[s])]
        moves = partition_moves(st, nxt, self.world)
        outgoing = [(p, dst) for p, src, dst in moves if src == self.rank]
        incoming = [(p, src) for p, src, dst in moves if dst == self.rank]
        recv_buf = {}
        ops = []
        for p, src in sorted(incoming):
            buf = self._pool.pop() if self._pool else self.alloc()
            buf.partition = p
            recv_buf[p] = buf
        # one group; sends and receives between a pair of ranks are matched in partition order on both sides
        for p, dst in sorted(outgoing):
            ops += [dist.P2POp(dist.isend, t, dst, self.group) for t in have[p].tensors()]
        for p, src in sorted(incoming):
            ops += [dist.P2POp(dist.irecv, t, src, self.group) for t in recv_buf[p].tensors()]
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        for p, _ in outgoing:
            buf = have.pop(p)
            buf.partition = -1
            self._pool.append(buf)
        have.update(recv_buf)
        for s, role, p in want:
            (self.stat if role == "stat" else self.circ)[s] = have[p]
