"""Shared relation parameters on several trainers: end-to-end quality of the two ways to reconcile them.

The reference's parameter server adds up every trainer's delta (torchbiggraph/parameter_sharing.py:662-672);
torchbiggraph_b200.buckets offers the mean of the trainers' copies (`average_relation_parameters`) and the sum
of their deltas (`sum_relation_parameter_deltas`).  Here the planted dynamic-relation graph of tests/mrr_util.py
is trained over four partitions with the epoch driver -- once by a single trainer, once by two gloo ranks that
reconcile after every step of the schedule -- with the CPU oracle as the training step (float64 NumPy), and the
held-out MRR of the runs is compared."""
import os
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mrr_util import CASES, COMMON, mrr_rhs, planted_graph

CASE = "dyn_complex_diagonal"
P = 4
EPOCHS = 4


def _worker(rank, world, initfile, mode, out):
    from oracle import pbg_step as O
    from torchbiggraph_b200.buckets import (EpochDriver, PartitionBuffer, average_relation_parameters,
                                            sum_relation_parameter_deltas)
    if world > 1:
        dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    torch.set_num_threads(1)
    c = CASES[CASE]
    (lhs, rhs, rel), _, W0 = planted_graph(CASE)
    N, D, R = c["N"], c["D"], c["R"]
    rows = N // P
    cut = -(-rows // 2)
    cfg = O.StepConfig(dim=D, operator=c["op"], comparator=COMMON["comp"], loss=COMMON["loss"], lr=COMMON["lr"],
                       num_batch_negs=COMMON["nb"], num_uniform_negs=COMMON["nu"], dynamic=True, num_rels=R)
    drv = EpochDriver(P, lambda: PartitionBuffer(torch.zeros(rows, D, dtype=torch.float64), torch.zeros(rows, dtype=torch.float64)), cut)
    for buf in drv.resident():
        buf.emb.copy_(torch.tensor(W0[buf.partition * rows:(buf.partition + 1) * rows], dtype=torch.float64))
    theta = [torch.tensor(O.operator_init(c["op"], D, R)) for _ in range(2)]          # rhs, lhs operator tables
    acc = [torch.zeros_like(t) for t in theta]
    shared = theta + acc
    before = [t.clone() for t in shared]
    # edges of every bucket, partition-local
    pl, ol, pr, orr = lhs // rows, lhs % rows, rhs // rows, rhs % rows
    bucket_edges = {(a, b): np.flatnonzero((pl == a) & (pr == b)) for a in range(P) for b in range(P)}
    state = {"epoch": 0}
    B = COMMON["batch"]

    def train(bucket, L, Rt, sub):
        idx = bucket_edges[bucket]
        l, r = ol[idx], orr[idx]
        if sub is not None:
            side, h, ct = sub
            key = l if side == "lhs" else r
            keep = key < ct if h == 0 else key >= ct
            idx, l, r = idx[keep], l[keep], r[keep]
            if side == "lhs":
                l = l - (0 if h == 0 else ct)
            else:
                r = r - (0 if h == 0 else ct)
        if len(idx) == 0:
            return
        rng = np.random.default_rng(hash((bucket, state["epoch"], None if sub is None else sub[:2])) % 2**32)
        order = rng.permutation(len(idx))
        same = L[0].data_ptr() == Rt[0].data_ptr()
        Wl, Gl = L[0].numpy(), L[1].numpy()
        Wr, Gr = (Wl, Gl) if same else (Rt[0].numpy(), Rt[1].numpy())
        st = O.BucketState(Wl, Gl, Wr, Gr, theta[0].numpy(), acc[0].numpy(), theta[1].numpy(), acc[1].numpy())
        for o in range(0, len(order), B):
            sel = order[o:o + B]
            n = len(sel)
            chunk = min(cfg.num_batch_negs, n)
            chunks = -(-n // chunk)
            ul = rng.integers(0, Wl.shape[0], (chunks, cfg.num_uniform_negs))
            ur = rng.integers(0, Wr.shape[0], (chunks, cfg.num_uniform_negs))
            O.train_batch(cfg, st, l[sel], r[sel], rel[idx][sel], ul, ur)

    def after_step(st):
        if world > 1:
            if mode == "average":
                average_relation_parameters(shared)
            else:
                sum_relation_parameter_deltas(shared, before)
        for b_, t_ in zip(before, shared):
            b_.copy_(t_)

    for ep in range(EPOCHS):
        state["epoch"] = ep
        for _ in range(len(drv.steps)):
            drv.run_step(train, after_step)
    parts = {buf.partition: buf.emb.numpy().copy() for buf in drv.resident()}
    out.put((rank, parts, theta[1].numpy().copy()))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _run(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, world, os.path.join(d, "init"), mode, q)) for r in range(world)]
        for p in procs:
            p.start()
        res = [q.get(timeout=900) for _ in range(world)]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    c = CASES[CASE]
    rows = c["N"] // P
    W = np.zeros((c["N"], c["D"]))
    for _, parts, _ in res:
        for p, w in parts.items():
            W[p * rows:(p + 1) * rows] = w
    thetas = [th for _, _, th in res]
    for th in thetas[1:]:
        np.testing.assert_allclose(th, thetas[0], rtol=1e-12, atol=1e-15)       # every rank holds the reconciled tables
    _, test, _ = planted_graph(CASE)
    return mrr_rhs(CASE, W, thetas[0], test)


def test_two_trainers_reach_the_quality_of_one_with_either_reconciliation():
    single = _run(1, "average")
    averaged = _run(2, "average")
    summed = _run(2, "sum_deltas")
    print(f"\nheld-out MRR: one trainer {single:.4f}; two trainers, averaged copies {averaged:.4f}; two trainers, summed deltas {summed:.4f}")
    assert single > 0.05                                  # the graph's structure was learnt (reference trainer: 0.104 after 6 epochs)
    assert averaged >= single - 0.01, (single, averaged)
    assert summed >= single - 0.01, (single, summed)
