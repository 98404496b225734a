"""The device RankingEvaluator against ranks / MRR / hits computed from the oracle's forward scores
(eval.py:43-81 restated in NumPy here: rank = 1 + #(neg >= pos), both sides averaged)."""
import numpy as np
import pytest

from golden_util import batch_of, load_step, oracle_config, oracle_state
from oracle import pbg_step as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["partial_last_chunk", "c3_none_dot_softmax", "c5_dyn_complex_l2_logistic",
                                  "std_linear_dot_ranking", "disable_lhs_negs", "uniform_only_mode"])
def test_ranking_evaluator_matches_oracle_scores(name):
    import torchbiggraph_b200 as T
    from b200_util import Rig
    c, z = load_step(name)
    ocfg, ost = oracle_config(c), oracle_state(c, z)
    rig = Rig.from_oracle_state(c, ost)
    lhs, rhs, rel, ul, ur = batch_of(c, z, 0)
    sc = O.score_batch(ocfg, ost, lhs, rhs, rel, ul, ur)
    ev = T.B200RankingEvaluator(T.LOSS_FUNCTIONS.get_class(c["loss"])(margin=c["margin"]),
                                [r.weight for r in rig.cfg.relations])
    st = ev.process_one_batch(rig.model, rig.edges(lhs, rhs, rel), ul, ur)
    n = len(lhs)
    ranks, aucs, losses = [], [], 0.0
    for side in ("lhs", "rhs"):
        pos, neg = sc[f"{side}_pos"], sc[f"{side}_neg"]
        val, _, _ = O.loss_forward_backward(c["loss"], c["margin"], pos, neg)
        losses += val
        if neg.size:
            ranks.append((neg >= pos[:, None]).sum(1) + 1)
            aucs.append(float((pos[:, None] > neg).mean()))      # exact value the randomized AUC estimates
    w = 1.0 if c["dyn"] else ([c["rel_weight"] if i == c["rel_idx"] else 1.0 for i in range(c["n_rel_std"])][c["rel_idx"]])
    assert st.count == n
    assert st.metrics["loss"] == pytest.approx(w * losses, rel=1e-4, abs=1e-3)
    mean_of_sums = lambda xs: float(np.mean([x.sum() for x in xs]))
    # a negative that ties with its positive (same entity) may fall either side of `>=` in fp32
    ties = sum(int((np.abs(sc[f"{s}_neg"] - sc[f"{s}_pos"][:, None]) <= 2e-5 * (1 + np.abs(sc[f"{s}_pos"][:, None]))).sum())
               for s in ("lhs", "rhs"))
    assert abs(st.metrics["pos_rank"] - mean_of_sums(ranks)) <= ties / len(ranks) + 1e-6
    assert abs(st.metrics["mrr"] - mean_of_sums([1.0 / r for r in ranks])) <= ties / len(ranks) + 1e-4
    for key, lim in (("r1", 1), ("r10", 10), ("r50", 50)):
        assert abs(st.metrics[key] - mean_of_sums([(r <= lim) for r in ranks])) <= ties / len(ranks) + 1e-6
    # `count` random pairs per side: standard error of the mean AUC is at most 0.5 / sqrt(count)
    assert abs(st.metrics["auc"] / n - float(np.mean(aucs))) <= 4 * 0.5 / np.sqrt(n)


def _allnegs_rig(z, cfg_o, st_o):
    """Model and evaluator for a recorded all_negs case (tests/golden/allnegs_*.npz)."""
    import torch
    import torchbiggraph_b200 as T
    sep, dyn = bool(z["separate"]), bool(z["dyn"])
    ents = {"e": T.EntitySchema()}
    rhs_ent = "e"
    if sep:
        ents["f"] = T.EntitySchema()
        rhs_ent = "f"
    cfg = T.ConfigSchema(entities=ents, relations=[T.RelationSchema("r0", "e", rhs_ent, operator=str(z["op"]), all_negs=True)],
                         dimension=z["W_lhs"].shape[1], comparator=str(z["comp"]), loss_fn=str(z["loss"]), margin=float(z["margin"]),
                         batch_size=1000, num_batch_negs=50, num_uniform_negs=0, dynamic_relations=dyn,
                         num_dynamic_rels=int(z["R"]) if dyn else 0)
    model = T.make_model(cfg, "cuda")
    f32 = lambda a: torch.tensor(np.asarray(a, np.float32), device="cuda").contiguous()
    Wl = f32(z["W_lhs"])
    Wr = f32(z["W_rhs"]) if sep else Wl
    model.set_embeddings("e", T.Side.LHS, Wl)
    model.set_embeddings(rhs_ent, T.Side.RHS, Wr)
    if model.rhs_op_table is not None:
        model.rhs_op_table.copy_(f32(z["theta_rhs"]))
    if model.lhs_op_table is not None:
        model.lhs_op_table.copy_(f32(z["theta_lhs"]))
    ev = T.B200RankingEvaluator(T.LOSS_FUNCTIONS.get_class(str(z["loss"]))(margin=float(z["margin"])), [1.0])
    return T, model, ev


def _allnegs_names():
    from test_oracle_golden import allnegs_cases
    return allnegs_cases()


@pytest.mark.parametrize("name", _allnegs_names())
def test_ranking_against_all_entities_matches_the_reference_evaluator(name):
    """Relations with all_negs=True: rank of the true entity among ALL rows of the side's table, the true entity itself
    ignored (model.py:582-617), against the Stats the reference's RankingEvaluator returned for the same batch."""
    import torch
    from test_oracle_golden import allnegs_stats, load_allnegs
    cfg_o, st_o, z = load_allnegs(name)
    T, model, ev = _allnegs_rig(z, cfg_o, st_o)
    t = lambda a: torch.tensor(np.asarray(a, np.int64))
    edges = T.EdgeList(T.EntityList.from_tensor(t(z["lhs"])), T.EntityList.from_tensor(t(z["rhs"])), t(z["rel"]))
    st = ev.process_one_batch(model, edges)
    n = int(z["stat_count"])
    assert st.count == n
    assert st.metrics["loss"] == pytest.approx(float(z["stat_loss"]), rel=1e-4)
    # candidates whose score ties with the positive up to fp32 rounding may fall either side of `>=`
    sc = O.score_all_negs(cfg_o, st_o, z["lhs"], z["rhs"], z["rel"])
    ties = sum(int((np.abs(sc[f"{s}_neg"] - sc[f"{s}_pos"][:, None]) <= 2e-5 * (1 + np.abs(sc[f"{s}_pos"][:, None]))).sum()) for s in ("lhs", "rhs"))
    assert abs(st.metrics["pos_rank"] - float(z["stat_pos_rank"])) <= ties / 2 + 1e-6
    assert abs(st.metrics["mrr"] - float(z["stat_mrr"])) <= ties / 2 + 1e-4
    for k in ("r1", "r10", "r50"):
        assert abs(st.metrics[k] - float(z["stat_" + k])) <= ties / 2 + 1e-6
    exact_auc = allnegs_stats(cfg_o, sc)["auc"]
    assert abs(st.metrics["auc"] / n - exact_auc) <= 4 * 0.5 / np.sqrt(n)


def test_all_negs_relations_are_not_trained():
    from test_oracle_golden import load_allnegs
    import torch
    cfg_o, st_o, z = load_allnegs("std_translation_dot_softmax")
    T, model, ev = _allnegs_rig(z, cfg_o, st_o)
    tr = T.B200Trainer(T.make_optimizer(model.config, model.parameters(), False), T.LOSS_FUNCTIONS.get_class("softmax")(margin=0.1), [1.0])
    tr.partitioned_optimizers["e", 0] = T.make_optimizer(model.config, [model.lhs_embs["emb_e"]], True)
    t = lambda a: torch.tensor(np.asarray(a, np.int64))
    with pytest.raises(NotImplementedError, match="all_negs"):
        tr.process_one_batch(model, T.EdgeList(T.EntityList.from_tensor(t(z["lhs"])), T.EntityList.from_tensor(t(z["rhs"])), t(0)))
