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
