#!/usr/bin/env python3
"""Benchmark of the per-bucket training step: edges/sec trained.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c3|c1|c2|c4|c5]

Workload (default): the social-graph-shaped configuration ("c3"): 4,847,571 entities in 16
partitions, dimension 1024, no operator / dot / softmax, batch 1000, 100 batch + 100 uniform
negatives, RowAdagrad lr 0.1.  The graph is synthetic: endpoints drawn from a Chung-Lu power law
(exponent 2.3) over seeded, randomly permuted entity ids; embeddings N(0, 1e-3).  A bucket of the
16 x 16 grid is 68,993,773 / 256 = 269,507 edges = 270 batches handed to the library in one call (what
process_in_batches does per bucket in the reference).  One *step* on one GPU is eight buckets (a region of a
few ten-millisecond buckets would be timed at burst clocks); on N > 1 GPUs (torchrun) it is one step of the
epoch schedule of torchbiggraph_b200.buckets: every GPU trains the buckets over the partitions it holds and
hands one partition per slot on to another GPU beside the training.

Prints ONE JSON line.  `value`: edges already in HBM, CUDA events around K steps.  `e2e`: the same
through the host-buffer path (edges in pinned host memory, host->device copy and the read-back of the step's
summed statistics inside the timed region).  `roofline`: the dominant kernel class, timed with CUDA events
on the library's stream in a separate short pass; its `traffic` comes from the ncu summary under profiles/
as long as that was captured on the kernel sources in the tree.  `sequential`: the same build with one batch
in flight.  `tiers`: the two-plane bf16 tier (rtol 1e-3) beside the headline tier (rtol 1e-4).
`cpu_baseline` / `--impl reference`: the PyTorch-CPU port of the reference trainer (oracle/pbg_step_torch.py),
one HOGWILD process per host core.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "pytorch-biggraph_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

WORKLOADS = {
    # name: entities, edges, partitions, dim, operator, comparator, loss, batch, batch negs, uniform negs, degree exponent
    "c3": dict(entities=4_847_571, edges=68_993_773, partitions=16, dim=1024, op="none", comp="dot", loss="softmax",
               batch=1000, nb=100, nu=100, gamma=2.3, precision="bf16x6", desc="social-graph shaped, Chung-Lu exponent 2.3"),
    "c4": dict(entities=41_652_230, edges=1_468_365_182, partitions=16, dim=100, op="translation", comp="cos",
               loss="ranking", batch=1000, nb=100, nu=100, gamma=2.0, precision="bf16x6", desc="follower-graph shaped, Chung-Lu exponent 2.0"),
    "c5": dict(entities=86_054_151, edges=338_586_276, partitions=16, dim=200, op="complex_diagonal", comp="l2",
               loss="logistic", batch=1000, nb=100, nu=100, gamma=None, rels=14_824, dynamic=True, rel_zipf=1.2, uniform_endpoints=True,
               desc="large multi-relation KG shaped, 14824 relations Zipf(1.2), per-relation operators (dynamic relations)"),
    "c2": dict(entities=14_951, edges=483_142, partitions=1, dim=400, op="complex_diagonal", comp="dot", loss="softmax",
               batch=5000, nb=1000, nu=0, gamma=None, rels=1345, dynamic=True, k=3,
               desc="15k-entity multi-relation KG shaped, 1345 relations Zipf(1.0), planted permutation maps + 20% noise, dynamic relations"),
    "c1": dict(entities=100_000, edges=1_000_000, partitions=1, dim=100, op="none", comp="dot", loss="ranking",
               batch=1000, nb=50, nu=50, gamma=None, precision="bf16x6", desc="plumbing graph, Zipf(1.1) endpoints"),
}
EDGES_PER_STEP_CAP = 269_507
# DRAM bytes per trained edge of each kernel class come from the ncu summaries under profiles/: the file
# of a (workload, precision) pair carries one line
#   traffic_per_edge_bytes: gather=... score=... grad=... update=... csrc_sha256=<digest>
# where the digest is csrc_digest() of the kernel sources the capture ran.  A summary whose digest is
# not that of the sources in the tree describes other kernels: its figures are then not used.
PROFILE_FILES = {("c3", "tf32x3"): "kernels_c3_tf32x3.md", ("c3", "bf16x6"): "kernels_c3_bf16x6.md",
                 ("c3", "bf16x3"): "kernels_c3_bf16x3.md"}


def csrc_digest():
    """sha256 over the CUDA sources of the library (names and contents, sorted by name)."""
    import glob
    import hashlib
    h = hashlib.sha256()
    for path in sorted(glob.glob(os.path.join(ROOT, "pytorch-biggraph_b200", "csrc", "*.cu*"))):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def ncu_traffic_per_edge(workload, precision):
    """(per-class DRAM bytes per trained edge, source note) from the profile summary of this pair, or
    (None, why) when there is none for the kernels in the tree."""
    name = PROFILE_FILES.get((workload, precision))
    path = os.path.join(ROOT, "profiles", name) if name else None
    if not path or not os.path.exists(path):
        return None, "no ncu summary for this workload and precision"
    with open(path) as f:
        lines = [l for l in f if l.startswith("traffic_per_edge_bytes:")]
    if not lines:
        return None, f"profiles/{name} carries no traffic line"
    kv = dict(t.split("=", 1) for t in lines[-1].split()[1:])
    if kv.get("csrc_sha256") != csrc_digest():
        return None, f"profiles/{name} was captured on other kernel sources ({kv.get('csrc_sha256')}, tree {csrc_digest()})"
    return {k: float(v) for k, v in kv.items() if k != "csrc_sha256"}, f"profiles/{name} (ncu, sources {kv['csrc_sha256']})"


PRECISION_NOTES = {
    "fp32": "fp32 FMA on the CUDA cores",
    "tf32x3": "tcgen05 kind::tf32, operands split hi + lo in shared memory, three MMAs per product, fp32 accumulation; parity tier rtol 1e-4",
    "bf16x6": "tcgen05 kind::f16 on three bf16 planes per fp32 operand value (24 mantissa bits), six plane products, fp32 accumulation; parity tier rtol 1e-4",
    "bf16x3": "tcgen05 kind::f16 on two bf16 planes per fp32 operand value (16 mantissa bits), three plane products (b0.b0 + b0.b1 + b1.b0), fp32 accumulation; parity tier rtol 1e-3 (two of the rtol 1e-4 comparisons fail in it)",
    "tf32": "tcgen05 kind::tf32, single pass; parity tier rtol 1e-3",
}
REF_BATCHES = 5          # batches per worker in one step of the CPU reference arm


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def algorithmic(w):
    """Per trained edge: flops = 12 D (P+U); bytes = (2 + 2U/P)(12 D + 8) + 24."""
    D, P, U = w["dim"], w["nb"], w["nu"]
    rho = U / P
    return dict(flops=12.0 * D * (P + U), bytes=(2 + 2 * rho) * (12 * D + 8) + 24,
                fwd_flops=4.0 * D * (P + U), bwd_flops=8.0 * D * (P + U),
                gather_bytes=(2 + 2 * rho) * 8 * D + 24, update_bytes=(2 + 2 * rho) * (12 * D + 8))


# ------------------------------------------------------------------------------------------------
# synthetic graph
# ------------------------------------------------------------------------------------------------
class Sampler:
    """Endpoint sampler of one partition: P(node) proportional to its Chung-Lu weight."""

    def __init__(self, weights):
        import torch
        c = torch.cumsum(weights.double(), 0)
        self.cdf = (c / c[-1]).float()
        self.n = weights.shape[0]
        self.weights = weights

    def part(self, lo, hi):
        """Sampler of the rows [lo, hi) of the partition; ids count from lo."""
        return Sampler(self.weights[lo:hi])

    def draw(self, n, gen):
        import torch
        u = torch.rand(n, device=self.cdf.device, generator=gen)
        return torch.searchsorted(self.cdf, u).clamp_(max=self.n - 1)


def make_samplers(w, device, seed):
    """Per-partition samplers after a seeded random permutation of entity ids."""
    import torch
    from torchbiggraph_b200.buckets import partition_bounds
    N, P = w["entities"], w["partitions"]
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    ranks = torch.arange(1, N + 1, device=device, dtype=torch.float32)
    expo = 1.1 if w["gamma"] is None else 1.0 / (w["gamma"] - 1.0)
    weight_by_rank = ranks.pow(-expo)
    perm = torch.randperm(N, device=device, generator=g)      # rank -> entity id
    weight_by_id = torch.empty_like(weight_by_rank)
    weight_by_id[perm] = weight_by_rank
    bounds = partition_bounds(N, P)
    return [Sampler(weight_by_id[bounds[p]:bounds[p + 1]]) for p in range(P)], bounds, g


def bucket_sequence(P):
    from torchbiggraph_b200.buckets import round_robin_rounds
    return [b for rnd in round_robin_rounds(P) for b in rnd]


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index
        self.t0 = self.t1 = None

    def start(self):
        """nvidia-smi takes a few hundred ms to come up (longer with eight ranks starting one each):
        it is started before the warm-up steps so that it is already sampling when the timed
        region begins."""
        if self.proc is not None:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def __enter__(self):
        self.start()
        self.t0 = time.time()
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def __exit__(self, *a):
        self.t1 = time.time()
        if self.proc:
            time.sleep(0.12)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        def ok(r):
            return r and r[0].replace(".", "").isdigit()
        inside = [r for t, r in self.rows if ok(r) and self.t0 is not None and self.t0 <= t <= (self.t1 or t) + 0.06]
        window = "timed region"
        if not inside:          # a timed region shorter than the sampling period: the warm-up steps ran the same load
            inside = [r for t, r in self.rows if ok(r)]
            window = "warm-up and timed region"
        sm = sorted(int(float(r[0])) for r in inside)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in inside)]
        mx = max(int(float(r[1])) for r in inside if len(r) > 1)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm), "window": window}


# ------------------------------------------------------------------------------------------------
# CPU baseline: the PyTorch-CPU port of the reference trainer, one HOGWILD process per core
# ------------------------------------------------------------------------------------------------
def _cpu_worker(i, w, W, G, theta, acc, cdf, cmd_q, start, finish):
    """One HOGWILD worker process: trains batches on the shared tables without locks, as the
    reference's worker pool does (torchbiggraph/train_cpu.py:861-884, util.py:294-314)."""
    import torch
    from oracle.pbg_step_torch import StepModel
    torch.set_num_threads(1)
    torch.manual_seed(1000 + i)
    m = StepModel(w["dim"], w["op"], w["comp"], w["loss"], 0.1, 0.1, None, w["nb"], w["nu"], False, 1)
    m.attach(W[0], G[0], W[1], G[1])
    if theta is not None:
        m.theta, m.acc = {"rhs": torch.nn.Parameter(theta)}, {"rhs": acc}
    rows, B = W[0].shape[0], w["batch"]
    while True:
        n = cmd_q.get()
        if n <= 0:
            return
        work = [(torch.searchsorted(cdf, torch.rand(B)).clamp_(max=rows - 1),
                 torch.searchsorted(cdf, torch.rand(B)).clamp_(max=rows - 1)) for _ in range(n)]
        start.wait()
        for lhs, rhs in work:
            m.train_batch(lhs, rhs, 0)
        finish.wait()


class CpuTrainer:
    """All host cores as HOGWILD worker processes (forked before CUDA is touched) over embedding
    tables in shared memory."""

    def __init__(self, w, rows, seed=7):
        import torch
        import torch.multiprocessing as mp
        torch.manual_seed(seed)
        self.w, self.rows = w, rows
        self.cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        D = w["dim"]
        self.shared = True
        W = [torch.randn(rows, D) * 1e-3 for _ in range(2)]
        G = [torch.zeros(rows) for _ in range(2)]
        try:
            for t in W + G:
                t.share_memory_()
        except Exception:
            self.shared = False        # no room in shared memory: forked workers update private copies
        theta = acc = None
        if w["op"] != "none":
            theta = torch.zeros(1, D)
            if w["op"] == "diagonal":
                theta.fill_(1.0)
            acc = torch.zeros(1, D)
            if self.shared:
                theta.share_memory_(); acc.share_memory_()
        ranks = torch.arange(1, rows + 1, dtype=torch.float32)
        expo = 1.1 if w["gamma"] is None else 1.0 / (w["gamma"] - 1.0)
        c = torch.cumsum(ranks.pow(-expo)[torch.randperm(rows)].double(), 0)
        cdf = (c / c[-1]).float()
        ctx = mp.get_context("fork")
        self.start, self.finish = ctx.Barrier(self.cores + 1), ctx.Barrier(self.cores + 1)
        self.queues = [ctx.Queue() for _ in range(self.cores)]
        self.procs = [ctx.Process(target=_cpu_worker, daemon=True,
                                  args=(i, w, W, G, theta, acc, cdf, self.queues[i], self.start, self.finish))
                      for i in range(self.cores)]
        for p in self.procs:
            p.start()

    def run(self, batches_per_worker):
        """Every worker trains `batches_per_worker` batches concurrently; returns (edges, seconds)."""
        for q in self.queues:
            q.put(batches_per_worker)
        self.start.wait(timeout=600)
        t0 = time.perf_counter()
        self.finish.wait(timeout=3600)
        dt = time.perf_counter() - t0
        return self.cores * batches_per_worker * self.w["batch"], dt

    def close(self):
        for q in self.queues:
            q.put(0)
        for p in self.procs:
            p.join(timeout=10)


def cpu_baseline(w, budget_s=15.0):
    rows = min(-(-w["entities"] // w["partitions"]), 400_000)
    tr = CpuTrainer(w, rows)
    tr.run(1)                                    # warm-up: allocator, autograd, thread start
    e1, t1 = tr.run(1)
    n = max(1, min(50, int(budget_s / max(t1, 1e-3))))
    edges, dt = tr.run(n)
    tr.close()
    return {"value": edges / dt, "unit": "edges/sec", "cores": tr.cores, "kind": "port",
            "sample": f"{tr.cores} HOGWILD processes x {n} batches of {w['batch']} edges on one bucket "
                      f"({rows} rows per side, dim {w['dim']}); fp32 PyTorch-CPU port of the reference trainer"}


def run_reference(args, w):
    """`--impl reference`: K timed steps of the CPU port; a step = REF_BATCHES batches per host core."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = min(-(-w["entities"] // w["partitions"]), 400_000)
    tr = CpuTrainer(w, rows)
    for _ in range(max(args.warmup, 1)):
        tr.run(1)
    edges = 0
    total = 0.0
    for _ in range(args.steps):
        e, t = tr.run(REF_BATCHES)
        edges += e
        total += t
    tr.close()
    v = edges / total
    sample = (f"{tr.cores} HOGWILD processes x {REF_BATCHES} batches of {w['batch']} edges per step, one bucket of {rows} rows "
              f"per side; fp32 PyTorch-CPU port of the reference trainer")
    line = {"impl": "reference", "metric": "edges/sec trained", "value": v, "unit": "edges/sec", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": reference_config(args, w, step_edges=tr.cores * w["batch"] * REF_BATCHES, cores=tr.cores),
            "cpu_baseline": {"value": v, "unit": "edges/sec", "cores": tr.cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "edges/sec", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args, w, step_edges, halves=False):
    cfg = _workload_config(args, w, step_edges)
    if halves:
        cfg["step"] += " as two sub-buckets (rhs partition cut in two row ranges)"
        cfg["hand_off"] = ("rhs partition travels to the next GPU in two halves over NCCL send/recv (NVLink), each half "
                           "beside the training of the other; inside the timed region")
    return cfg


def reference_config(args, w, step_edges, cores):
    """The CPU arm's own description: same workload string, its own step and arithmetic."""
    return {"workload": _workload_config(args, w, step_edges)["workload"],
            "step": f"{REF_BATCHES} batches of {w['batch']} edges on each of {cores} HOGWILD processes: {step_edges} edges",
            "l2": "inputs_larger_than_l2", "precision": "fp32",
            "arithmetic": "fp32 PyTorch CPU kernels (the reference's ATen call sequence), one thread per process"}


def _workload_config(args, w, step_edges):
    return {"workload": f"{args.workload}: {w['desc']}; {w['entities']} entities, {w['partitions']} partitions, dim {w['dim']}, "
                        f"{w['op']}/{w['comp']}/{w['loss']}, batch {w['batch']}, {w['nb']} batch + {w['nu']} uniform negs",
            "step": f"one bucket: {step_edges} edges", "l2": "inputs_larger_than_l2",
            "batches_in_flight": args.k, "precision": args.precision,
            "arithmetic": PRECISION_NOTES.get(args.precision, args.precision)}


# ------------------------------------------------------------------------------------------------
# the B200 arm
# ------------------------------------------------------------------------------------------------
class EdgeDrawer:
    """Synthetic edges of one bucket, as partition-local offsets (lhs, rhs, rel or None)."""

    def __init__(self, w, samplers, bounds, dev, gen):
        import torch
        self.w, self.samplers, self.bounds, self.dev, self.gen = w, samplers, bounds, dev, gen
        self.dyn = bool(w.get("dynamic"))
        if self.dyn:
            rw = torch.arange(1, w["rels"] + 1, device=dev, dtype=torch.float64).pow(-float(w.get("rel_zipf", 1.0)))
            self.rel_cdf = (torch.cumsum(rw, 0) / rw.sum()).float()
            n = w["entities"]
            self.rel_a = torch.randint(1, n, (w["rels"],), device=dev, generator=gen)     # planted maps v = a_r u + b_r mod N
            self.rel_b = torch.randint(0, n, (w["rels"],), device=dev, generator=gen)

    def __call__(self, bk, count):
        import torch
        pl, pr = bk
        w, dev, gen = self.w, self.dev, self.gen
        if not self.dyn:
            return self.samplers[pl].draw(count, gen), self.samplers[pr].draw(count, gen), None
        rel = torch.searchsorted(self.rel_cdf, torch.rand(count, device=dev, generator=gen)).clamp_(max=w["rels"] - 1)
        if w["partitions"] > 1:
            # partitioned multi-relation graph: endpoints uniform inside the bucket's two partitions (the planted
            # structure decides which bucket an edge falls in, not how a bucket trains)
            nl, nr = self.bounds[pl + 1] - self.bounds[pl], self.bounds[pr + 1] - self.bounds[pr]
            return (torch.randint(0, nl, (count,), device=dev, generator=gen),
                    torch.randint(0, nr, (count,), device=dev, generator=gen), rel)
        n = w["entities"]
        u = torch.randint(0, n, (count,), device=dev, generator=gen)
        v = (self.rel_a[rel] * u + self.rel_b[rel]) % n
        noisy = torch.rand(count, device=dev, generator=gen) < 0.2
        v = torch.where(noisy, torch.randint(0, n, (count,), device=dev, generator=gen), v)
        return u, v, rel


def build_trainer(args, w, dev):
    import torchbiggraph_b200 as T
    dyn = bool(w.get("dynamic"))
    cfg = T.ConfigSchema(entities={"e": T.EntitySchema(num_partitions=w["partitions"])},
                         relations=[T.RelationSchema("r", "e", "e", operator=w["op"])], dimension=w["dim"],
                         comparator=w["comp"], loss_fn=w["loss"], margin=0.1, lr=0.1, batch_size=w["batch"],
                         num_batch_negs=w["nb"], num_uniform_negs=w["nu"], precision=args.precision,
                         batches_in_flight=args.k, dynamic_relations=dyn, num_dynamic_rels=w.get("rels", 0) if dyn else 0)
    model = T.make_model(cfg, dev)
    trainer = T.B200Trainer(T.make_optimizer(cfg, model.parameters(), False),
                            T.LOSS_FUNCTIONS.get_class(w["loss"])(margin=0.1), [1.0])
    return cfg, model, trainer


def run_b200_epoch(args, w, world, rank, dev):
    """Several GPUs, partitioned workload: K steps of the epoch schedule (torchbiggraph_b200.buckets.epoch_schedule --
    every bucket of the P x P grid once per epoch, each GPU training the buckets over the two partitions it holds,
    partitions handed on over NCCL in halves beside training, relation parameters all-reduced after every step).
    A step is one step of that schedule: two buckets per GPU (four in the last step of an epoch)."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    import torchbiggraph_b200 as T
    from torchbiggraph_b200 import _C as native, _lib
    from torchbiggraph_b200.buckets import EpochDriver, PartitionBuffer, average_relation_parameters

    P, D, B = w["partitions"], w["dim"], w["batch"]
    bucket_edges = min(EDGES_PER_STEP_CAP, max(B, w["edges"] // (P * P)))
    samplers, bounds, gen = make_samplers(w, dev, seed=3)
    max_rows = max(bounds[p + 1] - bounds[p] for p in range(P))
    cut = -(-max_rows // 2)                                   # sub-partition size of a two-way split (util.cpp:296-315)
    cfg, model, trainer = build_trainer(args, w, dev)
    dyn = bool(w.get("dynamic"))
    draw = EdgeDrawer(w, samplers, bounds, dev, gen)
    drv = EpochDriver(P, lambda: PartitionBuffer(torch.empty(max_rows, D, device=dev), torch.empty(max_rows, device=dev)), cut, device=dev,
                      always_split=(world == 1))      # one GPU: the sub-bucket split without any exchange
    for buf in drv.resident():
        buf.emb.copy_(torch.randn(max_rows, D, device=dev, generator=gen) * 1e-3)
        buf.state.zero_()
    ident = torch.arange(max_rows, device=dev)
    nsteps_epoch = len(drv.steps)
    total_steps = args.warmup + args.steps
    local_slots = drv.local_slots

    def batches_of(n):
        return [(o, min(B, n - o), 0) for o in range(0, n, B)]

    def split(bucket, edges, which):
        """The two half sub-buckets of a bucket, by the rows of its circulating side (device sub_bucket)."""
        l, r, rl = edges
        n = l.shape[0]
        rel_in = rl if rl is not None else torch.zeros(n, dtype=torch.long, device=dev)
        out = [torch.empty(n, dtype=torch.long, device=dev) for _ in range(3)]
        nl, nr = (2, 1) if which == "lhs" else (1, 2)
        res = native.sub_bucket(l, r, rel_in, [max_rows], [ident], [max_rows], [ident], out[0], out[1], out[2], nl, nr, 1, True)
        keys = [(0, 0), (1, 0)] if which == "lhs" else [(0, 0), (0, 1)]
        return [(res[k][0], res[k][1], res[k][2] if rl is not None else None) for k in keys]

    def plan_step(g):
        """Whole-bucket edges of every bucket this rank trains in step g of the job."""
        return {(s, bk): draw(bk, bucket_edges) for s, bk, _ in drv.calls_of(g)}

    def presplit(g, whole):
        """Step g's edge lists as the driver will ask for them: whole buckets, or the two half sub-buckets by the
        rows of the side whose partition is leaving."""
        return {bk: whole[(s, bk)] if side is None else split(bk, whole[(s, bk)], side) for s, bk, side in drv.calls_of(g)}

    def optimizer_for(table, state):
        o = T.RowAdagrad([table], lr=0.1)
        o.state[id(table)]["sum"] = state
        return o

    cur = {}

    def train_fn(bucket, lhs, rhs, sub):
        e = cur["edges"][bucket]
        l, r, rl = e if sub is None else e[sub[1]]
        if l.shape[0] == 0:
            return
        model.clear_all_embeddings()
        model.set_embeddings("e", T.Side.LHS, lhs[0])
        model.set_embeddings("e", T.Side.RHS, rhs[0])
        trainer.partitioned_optimizers.clear()
        trainer.partitioned_optimizers["e", bucket[0]] = optimizer_for(lhs[0], lhs[1])
        if rhs[0].data_ptr() != lhs[0].data_ptr():
            trainer.partitioned_optimizers["e", bucket[1]] = optimizer_for(rhs[0], rhs[1])
        trainer.train_batches(model, l, r, rl, batches_of(l.shape[0]), want_per_batch=False)
        cur["edges_done"] += l.shape[0]

    shared = [t for t in model.parameters()]
    shared_state = [trainer.model_optimizer.sum_for(t) for t in shared] if shared else []

    def after_step(st):
        if shared and world > 1:
            average_relation_parameters(shared + shared_state)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(x, op=None):
        if world > 1:
            dist.all_reduce(x, **({} if op is None else {"op": op}))
        return x

    # device-resident pass: edges drawn and split into sub-buckets ahead of the timed region
    whole = [plan_step(k) for k in range(total_steps)]
    pre = [presplit(k, whole[k]) for k in range(total_steps)]

    trace = []                                    # --trace: per step (schedule level, host ms to enqueue, device ms)

    def step_device(k):
        cur["edges"] = pre[k]
        if not args.trace:
            drv.run_step(train_fn, after_step)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        level = drv.step_at(drv.step_index).level
        t0 = time.perf_counter()
        a.record()
        drv.run_step(train_fn, after_step)
        b.record()
        trace.append((level, (time.perf_counter() - t0) * 1e3, a, b))

    clocks = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))).start()
    cur["edges_done"] = 0
    for k in range(args.warmup):
        step_device(k)
    barrier()
    nat = trainer._native
    launches0 = nat.lib.pbg_launch_count(nat.ctx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cur["edges_done"] = 0
    with clocks:
        barrier()
        e0.record()
        for k in range(args.warmup, total_steps):
            step_device(k)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    edges_rank = cur["edges_done"]
    if args.trace:
        print(f"rank {rank} steps (level, host ms, device ms): " +
              " ".join(f"({lv},{h:.1f},{a.elapsed_time(b):.1f})" for lv, h, a, b in trace[args.warmup:]), file=sys.stderr, flush=True)
    launches = nat.lib.pbg_launch_count(nat.ctx) - launches0
    trainer.read_stats()
    if args.trace:
        # two more steps with every kernel class of every wave between its own pair of events
        _lib.check(nat.lib.pbg_set_profiling(nat.ctx, 2), nat.ctx)
        done0 = cur["edges_done"]
        for _ in range(2):
            cur["edges"] = presplit(drv.step_index, plan_step(drv.step_index))
            drv.run_step(train_fn, after_step)
        msc, lc = (C.c_double * 7)(), (C.c_int64 * 7)()
        _lib.check(nat.lib.pbg_kernel_times(nat.ctx, msc, lc), nat.ctx)
        _lib.check(nat.lib.pbg_set_profiling(nat.ctx, 0), nat.ctx)
        ne = max(cur["edges_done"] - done0, 1)
        print(f"rank {rank} kernel classes, us per 1000 edges: " +
              " ".join(f"{n}={msc[i] * 1e6 / ne:.2f}" for i, n in enumerate(_lib.KERNEL_CLASSES)), file=sys.stderr, flush=True)
        cur["edges_done"] = done0
    t = torch.tensor([ms], device=dev)
    ms = float(over_ranks(t, dist.ReduceOp.MAX))
    te = torch.tensor([float(edges_rank)], device=dev, dtype=torch.float64)
    over_ranks(te)
    value = float(te) / (ms / 1e3)

    # end-to-end pass: whole-bucket edges in pinned host memory; copy, device sub_bucket, training and the read-back of
    # the step's summed Stats inside the timed region.  The job goes on where the first pass stopped.
    del whole, pre
    g0 = drv.step_index
    nwarm = min(args.warmup, 2)

    def pinned(e):
        return tuple(None if t is None else t.cpu().pin_memory() for t in e)

    host = [{key: pinned(e) for key, e in plan_step(g0 + i).items()} for i in range(nwarm + args.steps)]

    def step_host(i):
        assert drv.step_index == g0 + i
        up = {key: tuple(None if t is None else t.to(dev, non_blocking=True) for t in e) for key, e in host[i].items()}
        cur["edges"] = presplit(g0 + i, up)
        drv.run_step(train_fn, after_step)
        return trainer.read_stats()

    for i in range(nwarm):
        step_host(i)
    barrier()
    cur["edges_done"] = 0
    e0.record()
    last = None
    for i in range(nwarm, nwarm + args.steps):
        last = step_host(i)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    t = torch.tensor([ms_e2e], device=dev)
    over_ranks(t, dist.ReduceOp.MAX)
    te = torch.tensor([float(cur["edges_done"])], device=dev, dtype=torch.float64)
    over_ranks(te)
    e2e = {"value": float(te) / (float(t) / 1e3), "unit": "edges/sec",
           "h2d_bytes_per_step": int((3 if dyn else 2) * 8 * float(te) / args.steps), "d2h_bytes_per_step": 40 * world,
           "last_step_loss": last.metrics["loss"] if last is not None else None}

    if rank == 0:
        cfgd = _workload_config(args, w, bucket_edges)
        per = P // 2 // world
        cfgd["step"] = (f"one step of the epoch schedule: {2 * per} buckets of {bucket_edges} edges per GPU ({4 * per} in the last step of an "
                        f"epoch); a bucket over a partition that leaves for another GPU after the step is trained as two half sub-buckets")
        cfgd["schedule"] = (f"{nsteps_epoch} steps per epoch cover all {P * P} buckets; every slot holds two partitions at a time, {P // 2 // world} slots per GPU")
        cfgd["hand_off"] = ("between two steps a slot gives one partition away and takes one in; it travels in two halves over NCCL "
                            "send/recv (NVLink), each half beside the training of the other, inside a level and at a change of level "
                            "alike; nothing moves between epochs; all inside the timed region" + ("; shared relation parameters and their accumulators averaged with one "
                                                             "all-reduce per step" if shared else ""))
        line = {"metric": "edges/sec trained", "value": value, "unit": "edges/sec", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32" if args.precision == "fp32" else args.precision, "data": "synthetic",
                "config": cfgd, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary(),
                "algorithmic_per_edge": {"flops": algorithmic(w)["flops"], "bytes": algorithmic(w)["bytes"]}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_b200(args, w):
    import torch
    import torch.distributed as dist
    import torchbiggraph_b200 as T
    from torchbiggraph_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w)                    # before CUDA is initialised in this process
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    P, D, B = w["partitions"], w["dim"], w["batch"]
    if (world > 1 or args.epoch_path) and P > 1:
        return run_b200_epoch(args, w, world, rank, dev)
    step_edges = min(EDGES_PER_STEP_CAP if P > 1 else w["edges"], max(B, w["edges"] // (P * P)))
    if args.step_edges > 0:
        step_edges = args.step_edges
    samplers, bounds, gen = make_samplers(w, dev, seed=3)
    # resident partitions: all of them (one GPU).  A workload of one partition on several GPUs is N independent
    # replicas of the single-GPU run: nothing to exchange.
    mine = list(range(min(P, args.resident) if args.resident > 0 else P))
    tables, states = {}, {}
    for p in mine:
        rows = bounds[p + 1] - bounds[p]
        tables[p] = torch.randn(rows, D, device=dev, generator=gen) * 1e-3
        states[p] = torch.zeros(rows, device=dev)

    dyn = bool(w.get("dynamic"))
    cfg = T.ConfigSchema(entities={"e": T.EntitySchema(num_partitions=P)},
                         relations=[T.RelationSchema("r", "e", "e", operator=w["op"])], dimension=D,
                         comparator=w["comp"], loss_fn=w["loss"], margin=0.1, lr=0.1, batch_size=B,
                         num_batch_negs=w["nb"], num_uniform_negs=w["nu"], precision=args.precision,
                         batches_in_flight=args.k, dynamic_relations=dyn, num_dynamic_rels=w.get("rels", 0) if dyn else 0)
    model = T.make_model(cfg, dev)
    trainer = T.B200Trainer(T.make_optimizer(cfg, model.parameters(), False),
                            T.LOSS_FUNCTIONS.get_class(w["loss"])(margin=0.1), [1.0])
    def optimizer_for(table, state):
        o = T.RowAdagrad([table], lr=0.1)
        o.state[id(table)]["sum"] = state
        return o

    opts = {p: optimizer_for(tables[p], states[p]) for p in mine}

    seq = bucket_sequence(len(mine))
    total_steps = args.warmup + args.steps
    # Buckets per step.  A partitioned workload trains eight buckets per step (one library call each): a timed region
    # of K ten-millisecond buckets is a burst that ends before the board's power limit pulls the SM clock down
    # (1965 MHz sampled), where the steps of a long job -- and of the several-GPU runs, whose steps are eight
    # buckets per GPU and more -- run at the clock the limit allows (about 1750 MHz on this workload).
    bps = args.buckets_per_step if args.buckets_per_step > 0 else (8 if P > 1 and args.resident == 0 and args.step_edges == 0 else 1)
    nprof = 2 if bps == 1 else 1

    def buckets_for(step):
        return [seq[(step * bps + j) % len(seq)] for j in range(bps)]

    def bind(bk):
        pl, pr = bk
        model.clear_all_embeddings()
        model.set_embeddings("e", T.Side.LHS, tables[pl])
        model.set_embeddings("e", T.Side.RHS, tables[pr])
        trainer.partitioned_optimizers.clear()
        trainer.partitioned_optimizers["e", pl] = opts[pl]
        trainer.partitioned_optimizers["e", pr] = opts[pr]

    batches = [(o, min(B, step_edges - o), 0) for o in range(0, step_edges, B)]

    draw = EdgeDrawer(w, samplers, bounds, dev, gen)

    def draw_edges(bk):
        return draw(bk, step_edges)

    def train_bucket(edges, want_per_batch):
        l, r, rl = edges
        return trainer.train_batches(model, l, r, rl, batches, want_per_batch=want_per_batch)

    # ---- device-resident pass: `value` -------------------------------------------------------
    dev_edges = [[draw_edges(bk) for bk in buckets_for(s)] for s in range(total_steps + nprof)]

    def to_host(e):
        if isinstance(e, list):
            return [to_host(x) for x in e]
        return tuple(None if t is None else t.cpu().pin_memory() for t in e)

    host_edges = [to_host(e) for e in dev_edges[: total_steps]]

    def step_device(s):
        for bk, e in zip(buckets_for(s), dev_edges[s]):
            bind(bk)
            train_bucket(e, False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clocks = ClockSampler(local).start()
    for s in range(args.warmup):
        step_device(s)
    barrier()
    nat = trainer._native
    launches0 = nat.lib.pbg_launch_count(nat.ctx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clocks:
        barrier()
        e0.record()
        for s in range(args.warmup, total_steps):
            step_device(s)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    launches = nat.lib.pbg_launch_count(nat.ctx) - launches0
    trainer.read_stats()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    value = world * args.steps * bps * step_edges / (ms / 1e3)

    # ---- end-to-end pass: host edges, copies and stats read-back inside the timed region --------
    def step_host(s):
        # the step's result read back: the summed Stats of its batches (loss, violators, count), one
        # 40-byte device-to-host read that waits for the step
        for bk, e in zip(buckets_for(s), host_edges[s]):
            bind(bk)
            train_bucket(e, False)
        return trainer.read_stats()

    for s in range(min(args.warmup, 2)):
        step_host(s)
    barrier()
    e0.record()
    last = None
    for s in range(args.warmup, total_steps):
        last = step_host(s)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t)
    e2e = {"value": world * args.steps * bps * step_edges / (ms_e2e / 1e3), "unit": "edges/sec",
           "h2d_bytes_per_step": (3 if dyn else 2) * 8 * bps * step_edges, "d2h_bytes_per_step": 40,
           "last_step_loss": last.metrics["loss"] if last is not None else None}

    def other_setting(precision, k, nsteps, whole_steps):
        """The same workload through a second trainer with another precision tier or number of batches in flight:
        one untimed step, then `nsteps` timed ones (whole steps, or the first bucket of each)."""
        import dataclasses
        cfg1 = dataclasses.replace(cfg, batches_in_flight=k, precision=precision)
        model1 = T.make_model(cfg1, dev)
        trainer1 = T.B200Trainer(T.make_optimizer(cfg1, model1.parameters(), False),
                                 T.LOSS_FUNCTIONS.get_class(w["loss"])(margin=0.1), [1.0])

        def step1(s):
            n = 0
            for (pl, pr), (l, r, rl) in list(zip(buckets_for(s), dev_edges[s]))[: bps if whole_steps else 1]:
                model1.clear_all_embeddings()
                model1.set_embeddings("e", T.Side.LHS, tables[pl])
                model1.set_embeddings("e", T.Side.RHS, tables[pr])
                trainer1.partitioned_optimizers.clear()
                trainer1.partitioned_optimizers["e", pl] = opts[pl]
                trainer1.partitioned_optimizers["e", pr] = opts[pr]
                trainer1.train_batches(model1, l, r, rl, batches, want_per_batch=False)
                n += step_edges
            return n

        step1(0)
        torch.cuda.synchronize()
        e0.record()
        n = sum(step1(s) for s in range(1, 1 + nsteps))
        e1.record()
        torch.cuda.synchronize()
        trainer1.read_stats()
        return n / (e0.elapsed_time(e1) / 1e3)

    # ---- sequential batches (one batch in flight: the reference's own GPU semantics) ----------------
    sequential = None
    if world == 1 and args.k > 1 and not args.no_sequential:
        nseq = 2
        sequential = {"value": other_setting(args.precision, 1, nseq, False), "unit": "edges/sec", "batches_in_flight": 1,
                      "steps": nseq, "note": "same build and workload with one batch in flight: every batch reads the "
                                             "tables its predecessor updated, as the reference's GPU trainer does"}
    # ---- the two-plane tier beside the headline (rtol 1e-3 where the headline tier holds rtol 1e-4) --------
    tiers = None
    if world == 1 and args.precision in ("bf16x6", "tf32x3") and w["op"] not in ("linear", "affine") and not args.no_sequential:
        nt = min(args.steps, 10)
        tiers = {"bf16x3": {"value": other_setting("bf16x3", args.k, nt, True), "unit": "edges/sec", "steps": nt,
                            "parity": "rtol 1e-3", "note": PRECISION_NOTES.get("bf16x3")}}

    # ---- per-kernel-class timing pass ----------------------------------------------------------
    import ctypes as C
    check = _lib.check
    check(nat.lib.pbg_set_profiling(nat.ctx, 2), nat.ctx)     # halves of a wave one after the other: a pair brackets its kernels alone
    for s in range(total_steps, total_steps + nprof):
        step_device(s)
    msc = (C.c_double * 7)()
    lc = (C.c_int64 * 7)()
    check(nat.lib.pbg_kernel_times(nat.ctx, msc, lc), nat.ctx)
    check(nat.lib.pbg_set_profiling(nat.ctx, 0), nat.ctx)
    alg = algorithmic(w)
    pk = peaks()
    edges_prof = nprof * bps * step_edges
    per_class = {}
    model_bytes = {"gather": alg["gather_bytes"], "update": alg["update_bytes"]}
    model_flops = {"score": alg["fwd_flops"], "grad": alg["bwd_flops"]}
    for i, name in enumerate(_lib.KERNEL_CLASSES):
        t_ms = msc[i]
        ent = {"ms": round(t_ms, 3), "launches": int(lc[i]), "share": None}
        if t_ms > 0 and name in model_bytes:
            ent["GBps"] = round(model_bytes[name] * edges_prof / (t_ms / 1e3) / 1e9, 1)
        if t_ms > 0 and name in model_flops:
            ent["TFLOPs"] = round(model_flops[name] * edges_prof / (t_ms / 1e3) / 1e12, 2)
        per_class[name] = ent
    tot = sum(v["ms"] for v in per_class.values()) or 1.0
    for v in per_class.values():
        v["share"] = round(v["ms"] / tot, 3)
    dom = max((n for n in per_class if n in model_bytes or n in model_flops), key=lambda n: per_class[n]["ms"])
    launches_dom = max(per_class[dom]["launches"], 1)
    per_class_traffic, traffic_source = ncu_traffic_per_edge(args.workload, args.precision)
    per_edge = None if per_class_traffic is None else per_class_traffic.get(dom)
    # ncu's DRAM bytes of the dominant class, per launch of this run (edges of the timing pass / its launches)
    # (the update class is several kernels per wave, the tile kernel carries its traffic: one launch per wave, as the statistics kernel)
    dom_kernel_launches = max(per_class["stats"]["launches"], 1) if dom == "update" else launches_dom
    traffic = None if per_edge is None else per_edge * edges_prof / dom_kernel_launches
    if dom in model_flops:
        ach = per_class[dom]["TFLOPs"]
        per_product = {"tf32x3": 6.0, "tf32": 2.0, "bf16x6": 6.0, "bf16x3": 3.0}.get(args.precision)     # TF32 runs at half the bf16 rate; TF32X3 issues three MMAs per product, BF16X6 six bf16 ones
        roof = {"bound": "tensor", "kernel": dom, "achieved": ach, "peak": pk["tflops"], "unit": "TFLOP/s",
                "frac": round(ach / pk["tflops"], 4), "traffic": traffic, "traffic_source": traffic_source,
                "ceiling_for_precision": None if per_product is None else round(pk["tflops"] / per_product, 1),
                "frac_of_ceiling": None if per_product is None else round(ach * per_product / pk["tflops"], 4),
                "peak_source": pk["source"] + " (cuBLAS bf16, sustained); the contraction runs in " + args.precision}
    else:
        ach = per_class[dom]["GBps"]
        roof = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(ach / pk["hbm_gbs"], 4), "traffic": traffic, "traffic_source": traffic_source,
                "peak_source": pk["source"]}

    if rank == 0:
        line = {"metric": "edges/sec trained", "value": value, "unit": "edges/sec", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32" if args.precision == "fp32" else args.precision, "data": "synthetic",
                "config": dict(workload_config(args, w, step_edges),
                               **({"step": f"{bps} buckets of {step_edges} edges, one library call each"} if bps > 1 else {})),
                "e2e": e2e, "gpu_launches": int(launches),
                "clocks": clocks.summary(), "roofline": roof, "kernels": per_class,
                "algorithmic_per_edge": {"flops": alg["flops"], "bytes": alg["bytes"]},
                "edges_per_sec_hbm_bound": pk["hbm_gbs"] * 1e9 / alg["bytes"]}
        if sequential is not None:
            line["sequential"] = sequential
        if tiers is not None:
            line["tiers"] = tiers
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--k", type=int, default=None,
                    help="batches in flight (1 = sequential batches, the reference's GPU semantics).  Default: 14, and 3 on c2, "
                         "whose batches of 5000 edges are a twentieth of an epoch each (the held-out MRR of its shape stays within "
                         "0.01 of the sequential reference up to 3 batches in flight, tests/test_gpu_mrr.py)")
    ap.add_argument("--precision", default=None, choices=["fp32", "tf32x3", "tf32", "bf16x6", "bf16x3"],
                    help="arithmetic of the contractions.  tf32x3: tcgen05 TF32 with 3-term split, the rtol 1e-4 tier; "
                         "bf16x6: tcgen05 bf16 on three planes per fp32 operand (24 mantissa bits), six plane products, "
                         "the rtol 1e-4 tier; fp32: CUDA cores; tf32: single pass, the rtol 1e-3 tier.  Default: the faster "
                         "of the two rtol 1e-4 tensor-core tiers on the workload (c3, c1, c4: bf16x6; c2, c5: tf32x3)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--buckets-per-step", type=int, default=0,
                    help="one GPU: buckets (library calls) per step; default 8 on partitioned workloads, 1 otherwise")
    ap.add_argument("--step-edges", type=int, default=0,
                    help="one GPU, one bucket per step: edges per step (library call) instead of the workload's bucket size; "
                         "for measuring what a call costs beside its batches")
    ap.add_argument("--trace", action="store_true", help="epoch path: print every step's host enqueue time and device time to stderr")
    ap.add_argument("--epoch-path", action="store_true",
                    help="one GPU: run the steps of the multi-GPU epoch schedule (all slots on this GPU, nothing to hand on) "
                         "instead of one bucket per step; the no-exchange reference point of the scaling runs")
    ap.add_argument("--no-sequential", action="store_true", help="skip the two extra steps with one batch in flight")
    ap.add_argument("--resident", type=int, default=0,
                    help="partitions kept on the device at N=1 (0 = all); a small number keeps profiler captures small")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    w = WORKLOADS[args.workload]
    if args.precision is None:
        args.precision = w.get("precision", "tf32x3")
    if args.k is None:
        args.k = w.get("k", 14)
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_b200(args, w)


if __name__ == "__main__":
    main()
