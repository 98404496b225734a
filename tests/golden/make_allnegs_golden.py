#!/usr/bin/env python3
"""Records what the REFERENCE returns for relations with all_negs=True (every entity of a side's table is a
negative, the true entity ignored; torchbiggraph/model.py:582-617): the Scores of MultiRelationEmbedder.forward
and the Stats of RankingEvaluator._process_one_batch (torchbiggraph/eval.py:43-81).

    python tests/golden/make_allnegs_golden.py --reference /path/to/PyTorch-BigGraph

Writes tests/golden/allnegs_<case>.npz.  The CPU oracle (oracle/pbg_step.py: score_all_negs) and the device
evaluator are held to these."""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
from make_golden import _bootstrap  # noqa: E402

CASES = [
    dict(name="std_translation_dot_softmax", op="translation", comp="dot", loss="softmax", B=70, D=16, N=211),
    dict(name="std_complex_cos_ranking_two_tables", op="complex_diagonal", comp="cos", loss="ranking", B=64, D=16, N=150, N2=97, w_scale=1.0),
    dict(name="std_none_l2_logistic", op="none", comp="l2", loss="logistic", B=33, D=8, N=120),
    dict(name="dyn_diagonal_dot_softmax", op="diagonal", comp="dot", loss="softmax", B=90, D=16, N=211, dyn=True, R=6),
    dict(name="dyn_complex_sql2_ranking_two_tables", op="complex_diagonal", comp="squared_l2", loss="ranking", B=50, D=16, N=130, N2=77, dyn=True, R=4),
    dict(name="std_diagonal_dot_logistic_many_rows", op="diagonal", comp="dot", loss="logistic", B=300, D=32, N=3001),
]


def run_case(case):
    import torch
    import torchbiggraph.model as M
    from torchbiggraph.config import ConfigSchema, EntitySchema, RelationSchema
    from torchbiggraph.edgelist import EdgeList
    from torchbiggraph.entitylist import EntityList
    from torchbiggraph.eval import RankingEvaluator
    from torchbiggraph.losses import LOSS_FUNCTIONS
    from torchbiggraph.model import make_model
    from torchbiggraph.types import Side
    torch.set_num_threads(1)
    c = dict(dyn=False, R=1, N2=None, w_scale=0.3, margin=0.1)
    c.update(case)
    D, N, B, dyn = c["D"], c["N"], c["B"], c["dyn"]
    sep = c["N2"] is not None
    ents = {"e": EntitySchema(num_partitions=1)}
    rhs_ent = "e"
    if sep:
        ents["f"] = EntitySchema(num_partitions=1)
        rhs_ent = "f"
    rels = [RelationSchema(name="r0", lhs="e", rhs=rhs_ent, operator=c["op"], all_negs=True)]
    cfg = ConfigSchema(entities=ents, relations=rels, dimension=D, entity_path="x", edge_paths=["y"], checkpoint_path="z",
                       comparator=c["comp"], loss_fn=c["loss"], margin=c["margin"], global_emb=False, batch_size=1000,
                       num_batch_negs=50, num_uniform_negs=0, dynamic_relations=dyn)
    if dyn:
        class RelCount:
            def __init__(self, path): pass
            def load_count(self): return c["R"]
        M.RELATION_TYPE_STORAGES.registry["x"] = RelCount
        M.RELATION_TYPE_STORAGES.registry[""] = RelCount
    model = make_model(cfg)
    seed = sum(ord(ch) for ch in c["name"]) * 104729 % (2 ** 31)
    torch.manual_seed(seed)
    with torch.no_grad():
        for prm in model.parameters():
            prm.add_(torch.randn_like(prm) * 0.3)
    emb_l = torch.nn.Parameter(torch.randn(N, D) * c["w_scale"])
    model.set_embeddings("e", Side.LHS, emb_l)
    N2 = c["N2"] if sep else N
    emb_r = torch.nn.Parameter(torch.randn(N2, D) * c["w_scale"]) if sep else emb_l
    model.set_embeddings(rhs_ent, Side.RHS, emb_r)
    lhs = torch.randint(0, N, (B,))
    rhs = torch.randint(0, N2, (B,))
    rel = torch.randint(0, c["R"], (B,)) if dyn else torch.tensor(0)
    edges = EdgeList(EntityList.from_tensor(lhs), EntityList.from_tensor(rhs), rel)
    with torch.no_grad():
        scores, _ = model(edges)
    ev = RankingEvaluator(LOSS_FUNCTIONS.get_class(c["loss"])(margin=c["margin"]), [1.0])
    stats = ev.process_one_batch(model, edges)

    def table(ops):
        if c["op"] == "none" or all(o is None for o in ops):
            return np.zeros((0, D), np.float32)
        rows = []
        for o in ops:
            sd = {k: v.detach() for k, v in o.named_parameters()}
            t = torch.cat([sd["real"], sd["imag"]], -1) if c["op"] == "complex_diagonal" else next(iter(sd.values()))
            rows.append(t if t.dim() == 2 else t.unsqueeze(0))
        return torch.cat(rows, 0).numpy().copy()

    out = dict(op=c["op"], comp=c["comp"], loss=c["loss"], margin=c["margin"], dyn=dyn, R=c["R"], separate=sep,
               W_lhs=emb_l.detach().numpy(), W_rhs=emb_r.detach().numpy(), theta_rhs=table(model.rhs_operators),
               theta_lhs=table(model.lhs_operators) if dyn else np.zeros((0, D), np.float32),
               lhs=lhs.numpy(), rhs=rhs.numpy(), rel=rel.numpy(), lhs_pos=scores.lhs_pos.numpy(), rhs_pos=scores.rhs_pos.numpy(),
               lhs_neg=scores.lhs_neg.numpy(), rhs_neg=scores.rhs_neg.numpy())
    if N > 1000:        # keep the fixture small: the evaluator's Stats pin this case, not the full score matrices
        out["lhs_neg"], out["rhs_neg"] = out["lhs_neg"][:, :64].copy(), out["rhs_neg"][:, :64].copy()
    for k in ("loss", "pos_rank", "mrr", "r1", "r10", "r50", "auc"):
        out["stat_" + k] = float(stats.metrics[k])
    out["stat_count"] = int(stats.count)
    np.savez_compressed(os.path.join(HERE, f"allnegs_{c['name']}.npz"), **out)
    print(c["name"], {k: round(float(stats.metrics[k]), 4) for k in ("loss", "pos_rank", "mrr", "r10")}, scores.lhs_neg.shape, scores.rhs_neg.shape)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a PyTorch-BigGraph checkout")
    args = ap.parse_args()
    _bootstrap(args.reference)
    for case in CASES:
        run_case(case)


if __name__ == "__main__":
    main()
