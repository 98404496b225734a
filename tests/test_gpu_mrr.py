"""End-to-end quality: held-out MRR on planted-structure graphs after training on the GPU path is
within 0.01 of what the reference CPU trainer reaches (tests/golden/mrr_planted.json, recorded by
tests/golden/make_mrr_golden.py from the reference itself; mean over three negative-sampling
seeds, whose own spread is about +-0.005)."""
import json
import os

import numpy as np
import pytest
import torch

from golden_util import GOLDEN
from mrr_util import CASES, COMMON, epoch_order, mrr_rhs, planted_graph, setting

pytestmark = pytest.mark.gpu


# The two small graphs run in every tier, sequentially and with batches in flight; the two graphs at
# the shapes of the benchmark configurations (dim 400 with 1000-row chunks; power-law endpoints at
# dim 256) run in the arithmetic and with the batches in flight that bench.py uses on them: 14 on the
# power-law graph, 3 on the multi-relation one -- its batches of 5000 edges are a twentieth of an epoch each,
# and with 14 of them in flight the held-out MRR after 3 epochs falls to 0.159 against the reference's 0.193
# (measured; 0.188 / 0.190 / 0.183 with 2 / 3 / 4 in flight).
SMALL = ("std_translation", "dyn_complex_diagonal")
RUNS = [(case, k, prec) for case in SMALL
        for k, prec in ((1, "fp32"), (1, "tf32x3"), (16, "tf32x3"), (1, "bf16x6"), (14, "bf16x6"))]
RUNS += [(case, 14, "bf16x3") for case in SMALL]
RUNS += [("kg15k_shape", 1, "tf32x3"), ("kg15k_shape", 3, "bf16x6"), ("kg15k_shape", 3, "tf32x3"),
         ("powerlaw_hubs", 1, "bf16x6"), ("powerlaw_hubs", 14, "bf16x6"), ("powerlaw_hubs", 14, "tf32x3"),
         ("powerlaw_hubs", 14, "bf16x3")]


@pytest.mark.parametrize("case,k,precision", RUNS)
def test_held_out_mrr_matches_reference_trainer(case, k, precision):
    import torchbiggraph_b200 as T
    with open(os.path.join(GOLDEN, "mrr_planted.json")) as f:
        want = json.load(f)["mrr"][case]
    c = CASES[case]
    (lhs, rhs, rel), test, W0 = planted_graph(case)
    cfg = T.ConfigSchema(entities={"e": T.EntitySchema()}, relations=[T.RelationSchema("r", "e", "e", operator=c["op"])],
                         dimension=c["D"], comparator=COMMON["comp"], loss_fn=COMMON["loss"], lr=COMMON["lr"],
                         batch_size=setting(case, "batch"), num_batch_negs=setting(case, "nb"), num_uniform_negs=setting(case, "nu"),
                         dynamic_relations=c["dyn"], num_dynamic_rels=c["R"] if c["dyn"] else 0,
                         precision=precision, batches_in_flight=k)
    model = T.make_model(cfg, "cuda")
    trainer = T.B200Trainer(T.make_optimizer(cfg, model.parameters(), False),
                            T.LOSS_FUNCTIONS.get_class(COMMON["loss"])(margin=0.1), [1.0])
    W = torch.tensor(W0, device="cuda")
    model.set_embeddings("e", T.Side.LHS, W)
    model.set_embeddings("e", T.Side.RHS, W)
    trainer.partitioned_optimizers["e", 0] = T.make_optimizer(cfg, [W], True)
    trainer.seed = 17
    B = setting(case, "batch")
    for ep in range(c["epochs"]):
        order = epoch_order(len(lhs), ep)
        edges = T.EdgeList(T.EntityList.from_tensor(torch.tensor(lhs[order])), T.EntityList.from_tensor(torch.tensor(rhs[order])),
                           torch.tensor(rel[order]) if c["dyn"] else torch.tensor(0))
        stats = T.process_in_batches(B, model, trainer, edges.to("cuda"))
        assert stats.count == len(order) and np.isfinite(stats.metrics["loss"])
    th = (model.lhs_op_table if c["dyn"] else model.rhs_op_table).cpu().numpy()
    got = mrr_rhs(case, W.cpu().numpy(), th, test)
    print(f"\nMRR {case} k={k} {precision}: {got:.4f} (reference {want:.4f})")
    if k == 1:
        assert abs(got - want) <= 0.01, f"MRR {got:.4f} vs reference {want:.4f}"
    else:
        # batches in flight read tables that are up to k - 1 steps old; held to "not worse than the sequential
        # reference by more than 0.01" (on power-law graphs the run with batches in flight ends a little higher)
        assert got >= want - 0.01, f"MRR {got:.4f} vs reference {want:.4f}"
