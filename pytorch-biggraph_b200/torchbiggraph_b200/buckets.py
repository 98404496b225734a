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
from typing import List, NamedTuple, Sequence, Tuple, Optional

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

    def start_many(self, sends: Sequence[Tuple[torch.Tensor, int]], recvs: Sequence[Tuple[torch.Tensor, int]]):
        """As `start_to`, with a peer per tensor: (tensor, to rank) and (tensor, from rank) pairs, one group."""
        ops = [dist.P2POp(dist.isend, t, peer, self.group) for t, peer in sends]
        ops += [dist.P2POp(dist.irecv, t, peer, self.group) for t, peer in recvs]
        if not ops:
            return None
        if not self.cuda:
            return dist.batch_isend_irecv(ops)
        done = torch.cuda.Event()
        done.record()                                # everything enqueued so far has written the tensors that leave
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


def epoch_schedule(num_partitions: int, start: Optional[Sequence[Tuple[int, int]]] = None) -> List[EpochStep]:
    """All P x P buckets of an epoch for P/2 slots (P a power of two, P >= 2), every slot holding two
    partitions at a time and training only buckets over those two -- the lock server's rule that buckets
    in flight share no partition (torchbiggraph/bucket_scheduling.py:477-540), laid out ahead of time as the
    reference's GPU trainer lays out its sub-partition jobs (torchbiggraph/train_gpu.py:354-387).

    `start[s]` = (stationary, circulating) partition of slot s when the epoch begins; any placement of the P
    partitions will do (default: slot s holds s and P/2 + s).  Level 0 is one ring over all slots: for as many
    steps as there are slots every slot trains (a, b) and (b, a) over its two partitions, then the circulating
    ones move one slot on -- after which every stationary x circulating bucket is done.  What is left are the
    buckets inside the stationary set and inside the circulating set.  The ring is cut in two: slot j of the
    lower half keeps its stationary partition and takes that of slot j of the upper half as its circulating
    one; the upper slot keeps the circulating partition it has, now as its stationary one, and takes the lower
    slot's circulating partition.  So a change of level is one swap between two slots -- one partition out and
    one in per slot -- and the next level runs the same scheme in rings of half the size, down to rings of one
    slot, which also train the diagonal buckets of their two partitions.  For P = 16: 8 + 4 + 2 + 1 = 15 steps,
    256 buckets.  The placement the epoch ends with is a valid `start` for the next one: nothing moves between
    epochs."""
    P = num_partitions
    if P < 2 or P & (P - 1):
        raise ValueError("epoch_schedule needs a power-of-two number of partitions >= 2")
    S = P // 2
    holds = [(s, S + s) for s in range(S)] if start is None else [tuple(h) for h in start]
    if len(holds) != S or sorted(p for h in holds for p in h) != list(range(P)):
        raise ValueError("start must place every partition in exactly one of the P/2 slots")
    steps: List[EpochStep] = []
    g, level = S, 0                                   # slots per ring at this level
    while True:
        last = g == 1
        for s in range(g):
            buckets = [[(a, b), (b, a)] + ([(a, a), (b, b)] if last else []) for a, b in holds]
            steps.append(EpochStep(list(holds), buckets, level))
            if s < g - 1:                             # the circulating partitions move one slot down their ring
                holds = [(holds[i][0], holds[i // g * g + (i % g + 1) % g][1]) for i in range(S)]
        if last:
            break
        h = g // 2
        nxt = list(holds)
        for base in range(0, S, g):
            for j in range(h):
                lo, up = base + j, base + h + j
                nxt[lo] = (holds[lo][0], holds[up][0])
                nxt[up] = (holds[up][1], holds[lo][1])
        holds, g, level = nxt, h, level + 1
    return steps


def next_epoch_start(steps: Sequence[EpochStep]) -> List[Tuple[int, int]]:
    """The placement an epoch ends with, as the `start` of the next one."""
    return list(steps[-1].holds)


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
    """Runs `epoch_schedule` on the ranks of a process group, epoch after epoch: every rank owns the slots
    `slot_rank` gives it, trains their buckets step by step, and passes partitions on as the schedule says.

    Between two steps a slot gives away at most one of its two partitions and takes one in.  The one that leaves
    -- the circulating partition inside a level; at a change of level the circulating one in the lower half of a
    ring and the stationary one in the upper half -- travels in two halves (rows [0, cut) and [cut, rows)): the
    step trains, for h = 0, 1, the two sub-buckets over half h of it (the edges whose row on that side lies in
    half h), and as soon as those are enqueued half h is sent, and half h of the arriving partition received into
    a spare buffer, on a side stream beside the training of the other half: the hand-off is off the critical
    path, as the reference overlaps partition swaps with training through its sub-partition jobs
    (torchbiggraph/train_gpu.py:456-652).  A partition that only changes slots on one GPU changes labels, and
    its buckets are trained whole (unless `always_split`); nothing moves between epochs.  A partition that
    arrives is the circulating one of its new slot; a step that needs it whole from the start (the one step of
    the last level, and the upper half's last step of a level) first waits for both of its halves.

    train_fn(bucket, lhs, rhs, sub) does the training: lhs / rhs are (emb, state) tensors -- whole partitions
    or halves -- and sub is None for a whole bucket or ("lhs" | "rhs", h, cut) for a half sub-bucket.
    after_step(step) runs once per step on every rank (e.g. the all-reduce of shared relation parameters).
    `calls_of(g)` lists what step g will hand to train_fn, for callers that prepare sub-bucket edge lists.
    """

    def __init__(self, num_partitions: int, alloc, cut: int, group=None, device=None, always_split: bool = False):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.P = num_partitions
        self._epochs = {0: epoch_schedule(num_partitions)}
        self.steps = self._epochs[0]                  # the first epoch's steps (every epoch has as many)
        self.S = num_partitions // 2
        self.local_slots = [s for s in range(self.S) if slot_rank(s, self.S, self.world) == self.rank]
        self.cut = cut
        self.always_split = always_split
        self.ring = OverlappedRing(device, group) if self.world > 1 else None
        self.stat = {s: alloc() for s in self.local_slots}
        self.circ = {s: alloc() for s in self.local_slots}
        self.pending = [None, None]          # transfers of half h started in the previous step
        self.step_index = 0
        for s in self.local_slots:
            a, b = self.steps[0].holds[s]
            self.stat[s].partition, self.circ[s].partition = a, b
        self._spares: List[PartitionBuffer] = []
        if self.world > 1:
            # Everything a hand-off needs exists before the first step: spare buffers for the largest number of
            # partitions that ever arrive from other ranks at once (the placements of later epochs differ, the
            # counts do not), and an open connection to every rank (NCCL sets a pair's connection up at their
            # first exchange, which takes on the order of a second; a level's ring only ever talks to two
            # neighbours, so without this the first change of level would pay for all the others).
            n = len(self.steps)
            two = self._epochs[0] + epoch_schedule(num_partitions, next_epoch_start(self._epochs[0]))
            most = max(sum(1 for _, src, dst in partition_moves(x, y, self.world) if dst == self.rank) for x, y in zip(two, two[1:]))
            self._spares = [alloc() for _ in range(most)]
            self._connect_all(self.stat[self.local_slots[0]].state)

    def _connect_all(self, like: torch.Tensor) -> None:
        out = torch.zeros(1, dtype=like.dtype, device=like.device)
        into = [torch.zeros(1, dtype=like.dtype, device=like.device) for _ in range(self.world)]
        ops = []
        for peer in range(self.world):
            if peer != self.rank:
                ops.append(dist.P2POp(dist.isend, out, peer, self.group))
                ops.append(dist.P2POp(dist.irecv, into[peer], peer, self.group))
        for req in dist.batch_isend_irecv(ops):
            req.wait()

    def step_at(self, g: int) -> EpochStep:
        """Step g of the job (epochs follow one another; each starts from the placement the one before ended with)."""
        n = len(self.steps)
        e, k = divmod(g, n)
        if e not in self._epochs:
            if e < min(self._epochs):                         # asked for the past: lay it out again from the start
                self._epochs = {0: epoch_schedule(self.P)}
            for x in range(max(self._epochs) + 1, e + 1):
                self._epochs[x] = epoch_schedule(self.P, next_epoch_start(self._epochs[x - 1]))
            for x in [x for x in self._epochs if x < self.step_index // n - 1]:       # epochs the job has left behind
                del self._epochs[x]
        return self._epochs[e][k]

    def resident(self) -> List[PartitionBuffer]:
        """Buffers that hold a partition right now (for initialisation and checkpointing)."""
        return [self.stat[s] for s in self.local_slots] + [self.circ[s] for s in self.local_slots]

    # ---- what a step does -----------------------------------------------------------------------
    def _plan(self, g: int):
        """Per local slot of step g: (slot, role of the partition that leaves -- "circ", "stat" or None --, whether its
        buckets are trained as half sub-buckets, slot it goes to, partition that arrives, slot it comes from)."""
        st, nxt = self.step_at(g), self.step_at(g + 1)
        where_next = {p: t for t, h in enumerate(nxt.holds) for p in h}
        where_now = {p: t for t, h in enumerate(st.holds) for p in h}
        fresh = self._fresh(g)
        plan = []
        for s in self.local_slots:
            a, b = st.holds[s]
            gone = [p for p in (a, b) if p not in nxt.holds[s]]
            come = [p for p in nxt.holds[s] if p not in (a, b)]
            assert len(gone) <= 1 and len(gone) == len(come), (g, s, st.holds[s], nxt.holds[s])
            if not gone:
                plan.append((s, None, False, None, None, None))
                continue
            role = "circ" if gone[0] == b else "stat"
            to_slot, from_slot = where_next[gone[0]], where_now[come[0]]
            crosses = slot_rank(to_slot, self.S, self.world) != self.rank
            # a circulating partition whose second half is still on its way here is read half by half as well
            plan.append((s, role, crosses or self.always_split or (role == "circ" and s in fresh), to_slot, come[0], from_slot))
        return st, nxt, plan

    def _fresh(self, g: int) -> set:
        """Local slots whose circulating partition of step g came from another rank during step g - 1."""
        if g == 0 or self.world == 1:
            return set()
        prev, st = self.step_at(g - 1), self.step_at(g)
        where_prev = {p: t for t, h in enumerate(prev.holds) for p in h}
        return {s for s in self.local_slots for p in st.holds[s]
                if p not in prev.holds[s] and slot_rank(where_prev[p], self.S, self.world) != self.rank}

    def calls_of(self, g: int) -> List[Tuple[int, Tuple[int, int], Optional[str]]]:
        """(slot, bucket, side split in halves or None) for every bucket this rank trains in step g."""
        st, _, plan = self._plan(g)
        out = []
        for s, role, split, *_ in plan:
            a, b = st.holds[s]
            if split:
                first, second = ((b, a), (a, b)) if role == "circ" else ((a, b), (b, a))
                out += [(s, first, "lhs"), (s, second, "rhs")]           # the leaving partition is first's lhs and second's rhs
            else:
                out += [(s, (a, b), None), (s, (b, a), None)]
            out += [(s, bk, None) for bk in st.buckets[s][2:]]
        return out

    def run_step(self, train_fn, after_step=None) -> int:
        """Trains the current step of the schedule on this rank's slots, starts the hand-offs that lead to the
        next one, and returns the number of buckets (whole-bucket equivalents) trained here."""
        g = self.step_index
        st, nxt, plan = self._plan(g)
        cut = self.cut
        # a partition that arrived last step is the circulating one of its slot; unless every slot reads it half by
        # half (it is the one that is split), both halves must be here before anything is trained
        fresh = self._fresh(g)
        if any(s in fresh and not (split and role == "circ") for s, role, split, *_ in plan):
            for h in (0, 1):
                OverlappedRing.finish(self.pending[h])
                self.pending[h] = None
        # cross-rank traffic of this step, in partition order (both ends of a pair of ranks sort alike)
        outgoing = sorted((self.stat[s] if role == "stat" else self.circ[s]).partition for s, role, split, to, _, _ in plan
                          if role is not None and slot_rank(to, self.S, self.world) != self.rank)
        incoming = sorted(come for s, role, split, to, come, frm in plan
                          if role is not None and slot_rank(frm, self.S, self.world) != self.rank)
        peer_out = {(self.stat[s] if role == "stat" else self.circ[s]).partition: slot_rank(to, self.S, self.world)
                    for s, role, split, to, _, _ in plan if role is not None}
        peer_in = {come: slot_rank(frm, self.S, self.world) for s, role, split, to, come, frm in plan if role is not None}
        landing = {}
        for p in incoming:
            buf = self._spares.pop()
            buf.partition = p
            landing[p] = buf
        leaving_buf = {}
        for s, role, split, to, _, _ in plan:
            if role is not None:
                buf = self.stat[s] if role == "stat" else self.circ[s]
                leaving_buf[buf.partition] = buf
        done = 0
        for h in (0, 1):
            if self.pending[h] is not None:          # the half about to be trained on has arrived, the old one has left
                OverlappedRing.finish(self.pending[h])
                self.pending[h] = None
            for s, role, split, *_ in plan:
                A, B = self.stat[s], self.circ[s]
                a, b = st.holds[s]
                assert A.partition == a and B.partition == b, (self.rank, g, s, A.partition, B.partition, a, b)
                if not split:
                    if h == 0:
                        train_fn((a, b), (A.emb, A.state), (B.emb, B.state), None)
                        train_fn((b, a), (B.emb, B.state), (A.emb, A.state), None)
                elif role == "circ":
                    train_fn((b, a), B.half(h, cut), (A.emb, A.state), ("lhs", h, cut))
                    train_fn((a, b), (A.emb, A.state), B.half(h, cut), ("rhs", h, cut))
                else:
                    train_fn((a, b), A.half(h, cut), (B.emb, B.state), ("lhs", h, cut))
                    train_fn((b, a), (B.emb, B.state), A.half(h, cut), ("rhs", h, cut))
            if outgoing or incoming:
                sends = [(t, peer_out[p]) for p in outgoing for t in leaving_buf[p].half(h, cut)]
                recvs = [(t, peer_in[p]) for p in incoming for t in landing[p].half(h, cut)]
                self.pending[h] = self.ring.start_many(sends, recvs)
        for s, role, split, *_ in plan:
            done += 2
            A, B = self.stat[s], self.circ[s]
            for bk in st.buckets[s][2:]:
                src = {A.partition: A, B.partition: B}
                L, R = src[bk[0]], src[bk[1]]
                train_fn(bk, (L.emb, L.state), (R.emb, R.state), None)
                done += 1
        if after_step is not None:
            after_step(st)
        # ---- where the partitions are in the next step ----
        have = {}
        for s in self.local_slots:
            have[self.stat[s].partition] = self.stat[s]
            have[self.circ[s].partition] = self.circ[s]
        for p in outgoing:                              # leaves with the transfers just started; a spare once they finish
            buf = have.pop(p)
            buf.partition = -1
            self._spares.append(buf)
        have.update(landing)
        for s in self.local_slots:
            a2, b2 = nxt.holds[s]
            self.stat[s], self.circ[s] = have[a2], have[b2]
        self.step_index += 1
        return done
