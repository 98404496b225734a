#!/usr/bin/env python3
"""Records the held-out MRR the REFERENCE trainer reaches on the planted graphs of tests/mrr_util.py.

    python tests/golden/make_mrr_golden.py --reference /path/to/PyTorch-BigGraph

Trains with the reference's Trainer.process_one_batch (torchbiggraph/train_cpu.py:86-112), one
process, sequential batches, and writes tests/golden/mrr_planted.json.  The GPU end-to-end test
trains the same graphs from the same initial embeddings and must land within 0.01 of these."""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
from make_golden import _bootstrap  # noqa: E402
from mrr_util import CASES, COMMON, epoch_order, mrr_rhs, planted_graph, setting  # noqa: E402


def run(case, seed=0):
    import torch
    import torchbiggraph.model as M
    from torchbiggraph.config import ConfigSchema, EntitySchema, RelationSchema
    from torchbiggraph.edgelist import EdgeList
    from torchbiggraph.entitylist import EntityList
    from torchbiggraph.losses import LOSS_FUNCTIONS
    from torchbiggraph.model import make_model
    from torchbiggraph.train_cpu import Trainer, make_optimizer
    from torchbiggraph.types import Side
    c = CASES[case]
    torch.set_num_threads(8)
    torch.manual_seed(seed)      # seeds the reference's uniform-negative draws
    (lhs, rhs, rel), test, W0 = planted_graph(case)
    cfg = ConfigSchema(entities={"e": EntitySchema(num_partitions=1)},
                       relations=[RelationSchema(name="r", lhs="e", rhs="e", operator=c["op"])], dimension=c["D"],
                       entity_path="x", edge_paths=["y"], checkpoint_path="z", comparator=COMMON["comp"],
                       loss_fn=COMMON["loss"], global_emb=False, batch_size=setting(case, "batch"),
                       num_batch_negs=setting(case, "nb"), num_uniform_negs=setting(case, "nu"), lr=COMMON["lr"],
                       dynamic_relations=c["dyn"])
    if c["dyn"]:
        class RelCount:
            def __init__(self, path): pass
            def load_count(self): return c["R"]
        M.RELATION_TYPE_STORAGES.registry["x"] = RelCount
        M.RELATION_TYPE_STORAGES.registry[""] = RelCount
    model = make_model(cfg)
    trainer = Trainer(make_optimizer(cfg, model.parameters(), False), LOSS_FUNCTIONS.get_class(COMMON["loss"])(margin=0.1), [1.0])
    emb = torch.nn.Parameter(torch.tensor(W0))
    model.set_embeddings("e", Side.LHS, emb)
    model.set_embeddings("e", Side.RHS, emb)
    trainer.partitioned_optimizers["e", 0] = make_optimizer(cfg, [emb], True)
    B = setting(case, "batch")
    for ep in range(c["epochs"]):
        order = epoch_order(len(lhs), ep)
        for o in range(0, len(order), B):
            idx = order[o:o + B]
            r = torch.tensor(rel[idx]) if c["dyn"] else torch.tensor(0)
            trainer.process_one_batch(model, EdgeList(EntityList.from_tensor(torch.tensor(lhs[idx])),
                                                      EntityList.from_tensor(torch.tensor(rhs[idx])), r))
    op = (model.lhs_operators if c["dyn"] else model.rhs_operators)[0]
    if c["op"] == "translation":
        th = (op.translations if c["dyn"] else op.translation).detach().numpy().reshape(-1, c["D"])
    else:
        th = torch.cat([op.real, op.imag], -1).detach().numpy().reshape(-1, c["D"])
    return mrr_rhs(case, emb.detach().numpy(), th, test)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a PyTorch-BigGraph checkout")
    ap.add_argument("--only", nargs="*", default=None, help="record these cases only; the others keep their recorded values")
    args = ap.parse_args()
    _bootstrap(args.reference)
    out, runs = {}, {}
    path = os.path.join(HERE, "mrr_planted.json")
    if args.only and os.path.exists(path):
        with open(path) as f:
            old = json.load(f)
        out, runs = old["mrr"], old["runs"]
    for case in (args.only or CASES):
        runs[case] = [run(case, seed) for seed in (0, 1, 2)]      # spread over negative-sampling seeds
        out[case] = float(np.mean(runs[case]))
        print(case, out[case], runs[case], flush=True)
    with open(path, "w") as f:
        json.dump({"mrr": out, "runs": runs, "cases": CASES, "common": COMMON}, f, indent=1)


if __name__ == "__main__":
    main()
