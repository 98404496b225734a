#!/usr/bin/env python3
"""Generate the golden fixtures in this directory by EXECUTING the reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/PyTorch-BigGraph

Two fixture families are written next to this script:

* reference_unit_calls.json -- every call the reference's own known-answer tests
  (test/test_model.py operators + comparators, test/test_losses.py) make into an
  operator / comparator / loss function: inputs, parameters, the value the
  reference returned and the value its test asserted.  Captured by running those
  unittest classes with recording wrappers; nothing is transcribed by hand.
* step_*.npz -- composed training steps: initial tables, Adagrad state, relation
  parameters, edges, the uniform negatives the reference drew, and what
  Trainer.process_one_batch (torchbiggraph/train_cpu.py:86-112) left behind
  (loss, violator counts, updated tables, state and parameters), for a list of
  cases covering chunk padding, U == 0, uniform-only mode, separate tables,
  duplicate rows, every operator/comparator/loss, dynamic relations, disabled
  sides, relation weights and multi-batch sequences.

The reference imports h5py at module import time; a three-class stand-in is put
on sys.path for this script only.
"""
import argparse
import json
import os
import sys
import tempfile
import unittest
import warnings

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _bootstrap(ref_root: str):
    stub = tempfile.mkdtemp(prefix="h5stub_")
    os.makedirs(os.path.join(stub, "h5py"))
    with open(os.path.join(stub, "h5py", "__init__.py"), "w") as f:
        f.write("class File: pass\nclass Dataset: pass\nclass Group: pass\n")
    sys.path[:0] = [stub, ref_root]
    warnings.filterwarnings("ignore")


# --------------------------------------------------------------------------- #
# part 1: record the reference's own known-answer tests
# --------------------------------------------------------------------------- #
def record_unit_calls():
    import torch
    import test.test_losses as tl
    import test.test_model as tm
    from torchbiggraph import losses as L, model as M, operators as O

    records = []
    current = {"test": None}

    def tolist(x):
        if x is None:
            return None
        if torch.is_tensor(x):
            return {"shape": list(x.shape), "data": x.detach().double().flatten().tolist()}
        return x

    def wrap(cls, kind, name, param_names=()):
        orig = cls.forward

        def fwd(self, *args):
            out = orig(self, *args)
            rec = {"test": current["test"], "kind": kind, "name": name,
                   "inputs": [tolist(a) for a in args],
                   "params": {p: tolist(getattr(self, p)) for p in param_names},
                   "outputs": [tolist(o) for o in (out if isinstance(out, tuple) else (out,))],
                   "asserted": []}
            if kind == "loss" and hasattr(self, "margin"):
                rec["margin"] = float(self.margin)
            records.append(rec)
            return out

        cls.forward = fwd

    for name in ("dot", "cos", "l2", "squared_l2"):
        wrap(M.COMPARATORS.get_class(name), "comparator", name)
    pn = {"none": (), "diagonal": ("diagonal",), "translation": ("translation",),
          "linear": ("linear_transformation",), "affine": ("linear_transformation", "translation"),
          "complex_diagonal": ("real", "imag")}
    dpn = {"none": (), "diagonal": ("diagonals",), "translation": ("translations",),
           "linear": ("linear_transformations",), "affine": ("linear_transformations", "translations"),
           "complex_diagonal": ("real", "imag")}
    for name, p in pn.items():
        wrap(O.OPERATORS.get_class(name), "operator", name, p)
    for name, p in dpn.items():
        wrap(O.DYNAMIC_OPERATORS.get_class(name), "dynamic_operator", name, p)
    for name in ("logistic", "ranking", "softmax"):
        wrap(L.LOSS_FUNCTIONS.get_class(name), "loss", name)

    for mod in (tm, tl):
        orig_assert = mod.TensorTestCase.assertTensorEqual

        def rec_assert(self, actual, expected, _orig=orig_assert):
            _orig(self, actual, expected)
            if records and records[-1]["test"] == current["test"]:
                records[-1]["asserted"].append(tolist(expected))

        mod.TensorTestCase.assertTensorEqual = rec_assert

    class Tracker(unittest.TextTestResult):
        def startTest(self, test):
            current["test"] = test.id()
            super().startTest(test)

    wanted = [
        tm.TestIdentityOperator, tm.TestDiagonalOperator, tm.TestTranslationOperator, tm.TestLinearOperator,
        tm.TestAffineOperator, tm.TestComplexDiagonalOperator, tm.TestIdentityDynamicOperator,
        tm.TestDiagonalDynamicOperator, tm.TestTranslationDynamicOperator, tm.TestLinearDynamicOperator,
        tm.TestAffineDynamicOperator, tm.TestComplexDiagonalDynamicOperator, tm.TestDotComparator,
        tm.TestCosComparator, tm.TestL2Comparator, tm.TestSquaredL2Comparator,
        tl.TestLogisticLossFunction, tl.TestRankingLossFunction, tl.TestSoftmaxLossFunction,
    ]
    suite = unittest.TestSuite()
    for c in wanted:
        suite.addTests(unittest.defaultTestLoader.loadTestsFromTestCase(c))
    res = unittest.TextTestRunner(resultclass=Tracker, verbosity=0).run(suite)
    assert res.wasSuccessful(), "reference unit tests failed here; fixtures not written"
    with open(os.path.join(HERE, "reference_unit_calls.json"), "w") as f:
        json.dump({"tests_run": res.testsRun, "records": records}, f)
    print(f"reference_unit_calls.json: {len(records)} calls from {res.testsRun} reference tests")


# --------------------------------------------------------------------------- #
# part 2: composed training steps through the reference Trainer
# --------------------------------------------------------------------------- #
CASES = [
    # name, overrides
    dict(name="c1_none_dot_ranking_full", op="none", comp="dot", loss="ranking", B=100, nb=50, nu=20),
    dict(name="partial_last_chunk", op="none", comp="dot", loss="ranking", B=130, nb=50, nu=20),
    dict(name="batch_smaller_than_chunk", op="none", comp="dot", loss="softmax", B=30, nb=50, nu=10),
    dict(name="no_uniform_negs", op="none", comp="dot", loss="softmax", B=120, nb=40, nu=0),
    dict(name="uniform_only_mode", op="translation", comp="dot", loss="ranking", B=70, nb=0, nu=25),
    dict(name="separate_tables", op="diagonal", comp="dot", loss="logistic", B=130, nb=50, nu=20, separate=True),
    dict(name="heavy_duplicates", op="none", comp="dot", loss="softmax", B=130, nb=50, nu=20, id_range=9),
    dict(name="c3_none_dot_softmax", op="none", comp="dot", loss="softmax", B=230, nb=100, nu=100, D=32),
    dict(name="c4_translation_cos_ranking", op="translation", comp="cos", loss="ranking", B=130, nb=50, nu=20, w_scale=1.0),
    dict(name="std_complex_dot_softmax", op="complex_diagonal", comp="dot", loss="softmax", B=130, nb=50, nu=20),
    dict(name="std_complex_l2_logistic", op="complex_diagonal", comp="l2", loss="logistic", B=130, nb=50, nu=20),
    dict(name="std_diagonal_l2_softmax", op="diagonal", comp="l2", loss="softmax", B=130, nb=50, nu=20),
    dict(name="std_translation_sql2_ranking", op="translation", comp="squared_l2", loss="ranking", B=130, nb=50, nu=20),
    dict(name="std_linear_dot_ranking", op="linear", comp="dot", loss="ranking", B=90, nb=40, nu=10, D=8),
    dict(name="std_affine_cos_logistic", op="affine", comp="cos", loss="logistic", B=90, nb=40, nu=10, D=8, w_scale=1.0),
    dict(name="c2_dyn_complex_dot_softmax", op="complex_diagonal", comp="dot", loss="softmax", B=130, nb=50, nu=0, dyn=True, R=7),
    dict(name="c5_dyn_complex_l2_logistic", op="complex_diagonal", comp="l2", loss="logistic", B=130, nb=50, nu=20, dyn=True, R=7),
    dict(name="dyn_translation_cos_ranking", op="translation", comp="cos", loss="ranking", B=130, nb=50, nu=20, dyn=True, R=7, w_scale=1.0),
    dict(name="dyn_diagonal_dot_logistic_unseen_rels", op="diagonal", comp="dot", loss="logistic", B=60, nb=25, nu=5, dyn=True, R=40),
    dict(name="dyn_none_dot_ranking", op="none", comp="dot", loss="ranking", B=130, nb=50, nu=20, dyn=True, R=3),
    dict(name="dyn_separate_tables", op="translation", comp="dot", loss="softmax", B=130, nb=50, nu=20, dyn=True, R=5, separate=True),
    dict(name="disable_lhs_negs", op="translation", comp="dot", loss="logistic", B=130, nb=50, nu=20, disable_lhs=True),
    dict(name="disable_rhs_negs_dyn", op="diagonal", comp="dot", loss="softmax", B=130, nb=50, nu=20, dyn=True, R=4, disable_rhs=True),
    dict(name="relation_weight_two_relations", op="translation", comp="dot", loss="ranking", B=130, nb=50, nu=20, n_rel_std=2, rel_idx=1, rel_weight=2.5),
    dict(name="sequence_3_batches", op="complex_diagonal", comp="dot", loss="softmax", B=130, nb=50, nu=20, steps=3),
    dict(name="sequence_3_batches_dyn_cos", op="diagonal", comp="cos", loss="ranking", B=110, nb=50, nu=10, dyn=True, R=6, steps=3, w_scale=1.0),
    dict(name="single_edge", op="none", comp="dot", loss="logistic", B=1, nb=50, nu=4),
    # per-edge weights (EdgeList.weight; losses.py:65-78, 104-113, 145-157)
    dict(name="edge_weights_softmax", op="none", comp="dot", loss="softmax", B=130, nb=50, nu=20, edge_weight=True),
    dict(name="edge_weights_ranking_cos", op="translation", comp="cos", loss="ranking", B=130, nb=50, nu=20, w_scale=1.0, edge_weight=True, steps=2),
    # config.global_emb (the reference's default): one trained vector per entity type added to every row
    dict(name="global_emb_one_type", op="translation", comp="dot", loss="softmax", B=130, nb=50, nu=20, global_emb=True),
    dict(name="global_emb_two_types", op="diagonal", comp="cos", loss="ranking", B=130, nb=50, nu=20, w_scale=1.0, separate=True, global_emb=True),
    dict(name="global_emb_sequence", op="none", comp="dot", loss="logistic", B=110, nb=50, nu=10, steps=2, global_emb=True),
    dict(name="global_emb_complex_l2", op="complex_diagonal", comp="l2", loss="softmax", B=90, nb=40, nu=10, global_emb=True),
    # N3 regularizer (regularization_coef; regularizers.py:51-97)
    dict(name="n3_std_diagonal_dot_softmax", op="diagonal", comp="dot", loss="softmax", B=130, nb=50, nu=20, reg_coef=1e-2),
    dict(name="n3_dyn_complex_dot_softmax", op="complex_diagonal", comp="dot", loss="softmax", B=130, nb=50, nu=0, dyn=True, R=7, reg_coef=1e-2),
    dict(name="n3_std_translation_cos_ranking_weighted_rel", op="translation", comp="cos", loss="ranking", B=130, nb=50, nu=20, w_scale=1.0,
         n_rel_std=2, rel_idx=1, rel_weight=2.5, reg_coef=5e-2, steps=2),
    dict(name="n3_std_none_dot_logistic", op="none", comp="dot", loss="logistic", B=90, nb=40, nu=10, reg_coef=1e-2),
    dict(name="n3_std_translation_l2_softmax", op="translation", comp="l2", loss="softmax", B=90, nb=40, nu=10, reg_coef=1e-2),
    dict(name="n3_std_complex_dot_ranking_global", op="complex_diagonal", comp="dot", loss="ranking", B=90, nb=40, nu=10, reg_coef=1e-2, global_emb=True),
    # max_norm: looked-up rows longer than max_norm are rescaled in the table (F.embedding, model.py:57-61)
    dict(name="max_norm_std_translation_dot_softmax", op="translation", comp="dot", loss="softmax", B=130, nb=50, nu=20, max_norm=1.0, steps=2),
    dict(name="max_norm_dyn_complex_dot_logistic", op="complex_diagonal", comp="dot", loss="logistic", B=110, nb=50, nu=10, dyn=True, R=5, max_norm=1.2),
    dict(name="max_norm_separate_global", op="diagonal", comp="cos", loss="ranking", B=130, nb=50, nu=20, w_scale=1.0, separate=True, global_emb=True, max_norm=3.5),
    dict(name="edge_weights_logistic_dyn", op="diagonal", comp="dot", loss="logistic", B=110, nb=50, nu=10, dyn=True, R=5, edge_weight=True),
]


def run_case(case):
    import torch
    import torchbiggraph.model as M
    from torchbiggraph.config import ConfigSchema, EntitySchema, RelationSchema
    from torchbiggraph.edgelist import EdgeList
    from torchbiggraph.entitylist import EntityList
    from torchbiggraph.losses import LOSS_FUNCTIONS
    from torchbiggraph.model import make_model
    from torchbiggraph.train_cpu import Trainer, make_optimizer
    from torchbiggraph.types import Side

    torch.set_num_threads(1)
    c = dict(D=16, N=211, N2=157, dyn=False, R=1, separate=False, id_range=None, steps=1, w_scale=0.3,
             disable_lhs=False, disable_rhs=False, n_rel_std=1, rel_idx=0, rel_weight=1.0, margin=0.1,
             lr=0.1, relation_lr=0.05, edge_weight=False, global_emb=False, reg_coef=0.0, max_norm=None)
    c.update(case)
    D, N, B, dyn = c["D"], c["N"], c["B"], c["dyn"]
    ents = {"e": EntitySchema(num_partitions=1)}
    rhs_ent = "e"
    if c["separate"]:
        ents["f"] = EntitySchema(num_partitions=1)
        rhs_ent = "f"
    nrel_schemas = 1 if dyn else c["n_rel_std"]
    rels = [RelationSchema(name=f"r{i}", lhs="e", rhs=rhs_ent, operator=c["op"],
                           weight=(c["rel_weight"] if i == c["rel_idx"] else 1.0)) for i in range(nrel_schemas)]
    # batch_size must be a multiple of num_batch_negs (model.py:879-883); a batch handed to the
    # trainer may still be shorter (the last batch of a bucket), which is what B != multiple tests.
    cfg_batch = max(B, 1) if c["nb"] == 0 else ((B - 1) // c["nb"] + 1) * c["nb"]
    cfg = ConfigSchema(entities=ents, relations=rels, dimension=D, entity_path="x", edge_paths=["y"],
                       checkpoint_path="z", comparator=c["comp"], loss_fn=c["loss"], margin=c["margin"],
                       global_emb=c["global_emb"], regularization_coef=c["reg_coef"], max_norm=c["max_norm"], batch_size=cfg_batch, num_batch_negs=c["nb"], num_uniform_negs=c["nu"],
                       lr=c["lr"], relation_lr=c["relation_lr"], dynamic_relations=dyn,
                       disable_lhs_negs=c["disable_lhs"], disable_rhs_negs=c["disable_rhs"])
    if dyn:
        class RelCount:
            def __init__(self, path): pass
            def load_count(self): return c["R"]
        M.RELATION_TYPE_STORAGES.registry["x"] = RelCount
        M.RELATION_TYPE_STORAGES.registry[""] = RelCount
    model = make_model(cfg)
    seed = sum(ord(ch) for ch in c["name"]) * 7919 % (2 ** 31)
    torch.manual_seed(seed)
    with torch.no_grad():
        for prm in model.parameters():
            prm.add_(torch.randn_like(prm) * 0.3)
    # Trainer and its model optimizer are built BEFORE embeddings are attached (train_cpu.py:463-472).
    trainer = Trainer(make_optimizer(cfg, model.parameters(), False),
                      LOSS_FUNCTIONS.get_class(c["loss"])(margin=c["margin"]),
                      [r.weight for r in cfg.relations])
    emb_l = torch.nn.Parameter(torch.randn(N, D) * c["w_scale"])
    model.set_embeddings("e", Side.LHS, emb_l)
    opt_l = make_optimizer(cfg, [emb_l], True)
    trainer.partitioned_optimizers["e", 0] = opt_l
    opt_l.state[emb_l]["sum"].copy_(torch.rand(N) * 0.5)
    if c["separate"]:
        N2 = c["N2"]
        emb_r = torch.nn.Parameter(torch.randn(N2, D) * c["w_scale"])
        opt_r = make_optimizer(cfg, [emb_r], True)
        trainer.partitioned_optimizers["f", 0] = opt_r
        opt_r.state[emb_r]["sum"].copy_(torch.rand(N2) * 0.5)
    else:
        N2, emb_r, opt_r = N, emb_l, opt_l
    model.set_embeddings(rhs_ent, Side.RHS, emb_r)

    def op_tables():
        """Pack operator parameters as [R, width] tables (complex: [real|imag]; affine: [A|t])."""
        out = {}
        for side, ops in (("rhs", model.rhs_operators), ("lhs", model.lhs_operators)):
            mods = [o for o in ops]
            if all(o is None for o in mods) or c["op"] == "none":
                out[side] = None
                continue
            rows = []
            for o in mods:
                sd = {k: v.detach() for k, v in o.named_parameters()}
                if c["op"] in ("diagonal", "translation"):
                    t = next(iter(sd.values()))
                elif c["op"] == "complex_diagonal":
                    t = torch.cat([sd["real"], sd["imag"]], -1)
                elif c["op"] == "linear":
                    a = next(iter(sd.values()))
                    t = a.reshape(a.shape[:-2] + (D * D,))
                else:
                    a = sd["linear_transformations" if dyn else "linear_transformation"]
                    tr = sd["translations" if dyn else "translation"]
                    t = torch.cat([a.reshape(a.shape[:-2] + (D * D,)), tr], -1)
                rows.append(t if t.dim() == 2 else t.unsqueeze(0))
            out[side] = torch.cat(rows, 0).numpy().copy()
        return out

    def acc_tables():
        out = {}
        opt = trainer.model_optimizer
        for side, ops in (("rhs", model.rhs_operators), ("lhs", model.lhs_operators)):
            if all(o is None for o in ops) or c["op"] == "none":
                out[side] = None
                continue
            rows = []
            for o in ops:
                sd = {k: opt.state[v]["sum"] for k, v in o.named_parameters()}
                if c["op"] in ("diagonal", "translation"):
                    t = next(iter(sd.values()))
                elif c["op"] == "complex_diagonal":
                    t = torch.cat([sd["real"], sd["imag"]], -1)
                elif c["op"] == "linear":
                    a = next(iter(sd.values()))
                    t = a.reshape(a.shape[:-2] + (D * D,))
                else:
                    a = sd["linear_transformations" if dyn else "linear_transformation"]
                    tr = sd["translations" if dyn else "translation"]
                    t = torch.cat([a.reshape(a.shape[:-2] + (D * D,)), tr], -1)
                rows.append(t if t.dim() == 2 else t.unsqueeze(0))
            out[side] = torch.cat(rows, 0).numpy().copy()
        return out

    out = {"config": json.dumps({k: v for k, v in c.items()}),
           "W_lhs0": emb_l.detach().numpy().copy(), "G_lhs0": opt_l.state[emb_l]["sum"].numpy().copy()}
    if c["separate"]:
        out["W_rhs0"] = emb_r.detach().numpy().copy()
        out["G_rhs0"] = opt_r.state[emb_r]["sum"].numpy().copy()
    t0 = op_tables()
    for side in ("rhs", "lhs"):
        if t0[side] is not None:
            out[f"theta_{side}0"] = t0[side]

    def glob_tables():
        """{entity type: (vector, AsyncAdagrad accumulator)} of the model's global embeddings."""
        if model.global_embs is None:
            return {}
        opt = trainer.model_optimizer
        return {k[len(model.EMB_PREFIX):]: (p.detach().numpy().copy(), opt.state[p]["sum"].numpy().copy())
                for k, p in model.global_embs.items()}

    for ent, (g, _) in glob_tables().items():
        out[f"glob_{ent}0"] = g
    hi_l = c["id_range"] or N
    hi_r = c["id_range"] or N2
    for step in range(c["steps"]):
        lhs = torch.randint(hi_l, (B,))
        rhs = torch.randint(hi_r, (B,))
        if dyn:
            rel = torch.randint(c["R"], (B,))
            if "unseen" in c["name"]:
                rel = torch.randint(5, (B,)) * 3  # most rows of the table never touched
        else:
            rel = torch.tensor(c["rel_idx"])
        weight = torch.rand(B) * 2.0 + 0.1 if c["edge_weight"] else None
        draw_seed = seed + 1000 + step
        torch.manual_seed(draw_seed)
        stats = trainer.process_one_batch(model, EdgeList(EntityList.from_tensor(lhs), EntityList.from_tensor(rhs), rel, weight))
        if weight is not None:
            out[f"weight_{step}"] = weight.numpy()
        # replay the uniform-negative draws: lhs side first, then rhs side (model.py:802-821)
        P = min(c["nu"], B) if c["nb"] == 0 else min(c["nb"], B)
        C = (B - 1) // P + 1
        torch.manual_seed(draw_seed)
        ul = ur = None
        if not c["disable_lhs"] and c["nu"] > 0:
            ul = torch.randint(0, N, (C, c["nu"]))
        if not c["disable_rhs"] and c["nu"] > 0:
            ur = torch.randint(0, N2, (C, c["nu"]))
        out[f"lhs_{step}"] = lhs.numpy()
        out[f"rhs_{step}"] = rhs.numpy()
        out[f"rel_{step}"] = rel.numpy()
        out[f"ul_{step}"] = ul.numpy() if ul is not None else np.zeros((C, 0), np.int64)
        out[f"ur_{step}"] = ur.numpy() if ur is not None else np.zeros((C, 0), np.int64)
        out[f"loss_{step}"] = np.float64(stats.metrics["loss"])
        out[f"reg_{step}"] = np.float64(stats.metrics["reg"])
        out[f"violators_lhs_{step}"] = np.int64(stats.metrics["violators_lhs"])
        out[f"violators_rhs_{step}"] = np.int64(stats.metrics["violators_rhs"])
        out[f"W_lhs_after_{step}"] = emb_l.detach().numpy().copy()
        out[f"G_lhs_after_{step}"] = opt_l.state[emb_l]["sum"].numpy().copy()
        if c["separate"]:
            out[f"W_rhs_after_{step}"] = emb_r.detach().numpy().copy()
            out[f"G_rhs_after_{step}"] = opt_r.state[emb_r]["sum"].numpy().copy()
        for ent, (g, a) in glob_tables().items():
            out[f"glob_{ent}_after_{step}"] = g
            out[f"gacc_{ent}_after_{step}"] = a
        t1, a1 = op_tables(), acc_tables()
        for side in ("rhs", "lhs"):
            if t1[side] is not None:
                out[f"theta_{side}_after_{step}"] = t1[side]
                out[f"acc_{side}_after_{step}"] = a1[side]
    # forward scores of one more batch on the final state (no update): model.forward only
    lhs = torch.randint(hi_l, (B,))
    rhs = torch.randint(hi_r, (B,))
    rel = torch.randint(c["R"], (B,)) if dyn else torch.tensor(c["rel_idx"])
    torch.manual_seed(seed + 5000)
    with torch.no_grad():
        scores, _ = model(EdgeList(EntityList.from_tensor(lhs), EntityList.from_tensor(rhs), rel))
    P = min(c["nu"], B) if c["nb"] == 0 else min(c["nb"], B)
    C = (B - 1) // P + 1
    torch.manual_seed(seed + 5000)
    ul = torch.randint(0, N, (C, c["nu"])) if (not c["disable_lhs"] and c["nu"] > 0) else None
    ur = torch.randint(0, N2, (C, c["nu"])) if (not c["disable_rhs"] and c["nu"] > 0) else None
    out.update(fw_lhs=lhs.numpy(), fw_rhs=rhs.numpy(), fw_rel=rel.numpy(),
               fw_ul=ul.numpy() if ul is not None else np.zeros((C, 0), np.int64),
               fw_ur=ur.numpy() if ur is not None else np.zeros((C, 0), np.int64),
               fw_lhs_pos=scores.lhs_pos.numpy(), fw_rhs_pos=scores.rhs_pos.numpy(),
               fw_lhs_neg=scores.lhs_neg.numpy(), fw_rhs_neg=scores.rhs_neg.numpy())
    np.savez_compressed(os.path.join(HERE, f"step_{c['name']}.npz"), **out)
    print(f"step_{c['name']}.npz  loss[0]={float(out['loss_0']):.6g}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a PyTorch-BigGraph checkout")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    _bootstrap(args.reference)
    if args.only in (None, "unit"):
        record_unit_calls()
    if args.only in (None, "steps"):
        for case in CASES:
            run_case(case)
    elif args.only not in ("unit",):          # --only <substring>: the step cases whose name contains it
        for case in CASES:
            if args.only in case["name"]:
                run_case(case)


if __name__ == "__main__":
    main()
