"""Pins the CPU oracle (oracle/pbg_step.py) to the reference.

(1) every operator / comparator / loss call made by the reference's own known-answer
    tests (recorded in tests/golden/reference_unit_calls.json by make_golden.py);
(2) composed training steps produced by the reference Trainer (tests/golden/step_*.npz).
Runs on CPU only."""
import json
import os

import numpy as np
import pytest

from oracle import pbg_step as O
from golden_util import GOLDEN, batch_of, load_step, oracle_config, oracle_state, step_fixture_names, weight_of


def _arr(d):
    return None if d is None else np.asarray(d["data"], np.float64).reshape(d["shape"])


with open(os.path.join(GOLDEN, "reference_unit_calls.json")) as f:
    UNIT = json.load(f)["records"]


def _op_table(rec):
    p = {k: _arr(v) for k, v in rec["params"].items()}
    name, dyn = rec["name"], rec["kind"] == "dynamic_operator"
    if name == "none":
        return None
    if name in ("diagonal", "translation"):
        t = next(iter(p.values()))
    elif name == "complex_diagonal":
        t = np.concatenate([p["real"], p["imag"]], -1)
    else:
        a = p["linear_transformations" if dyn else "linear_transformation"]
        t = a.reshape(a.shape[:-2] + (-1,))
        if name == "affine":
            t = np.concatenate([t, p["translations" if dyn else "translation"]], -1)
    return t if t.ndim == 2 else t[None]


@pytest.mark.parametrize("i", range(len(UNIT)), ids=[f"{r['kind']}-{r['name']}-{k}" for k, r in enumerate(UNIT)])
def test_reference_unit_vectors(i):
    rec = UNIT[i]
    outs = [_arr(o) for o in rec["outputs"]]
    if rec["kind"] in ("operator", "dynamic_operator"):
        x = _arr(rec["inputs"][0])
        tab = _op_table(rec)
        flat = x.reshape(-1, x.shape[-1])
        if rec["kind"] == "dynamic_operator":
            idx = np.asarray(rec["inputs"][1]["data"], np.int64).reshape(rec["inputs"][1]["shape"]).reshape(-1)
            p = None if tab is None else tab[idx]
        else:
            p = None if tab is None else tab[:1]
        got = O.op_forward(rec["name"], flat, p).reshape(x.shape)
        np.testing.assert_allclose(got, outs[0], rtol=1e-6, atol=1e-6)
        for a in rec["asserted"]:
            np.testing.assert_allclose(got, _arr(a), rtol=5e-5, atol=5e-5)
    elif rec["kind"] == "comparator":
        lp, rp, ln, rn = (_arr(a) for a in rec["inputs"])  # already "prepared" by the reference test
        C = lp.shape[0]
        pos = np.stack([O.compare_pos(rec["name"], lp[c], rp[c]) for c in range(C)])
        lneg = np.stack([O.compare_neg(rec["name"], rp[c], ln[c]) for c in range(C)])
        rneg = np.stack([O.compare_neg(rec["name"], lp[c], rn[c]) for c in range(C)])
        for got, want in zip((pos, lneg, rneg), outs):
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
        for got, a in zip((pos, lneg, rneg), rec["asserted"]):
            np.testing.assert_allclose(got, _arr(a), rtol=5e-5, atol=5e-5)
    else:
        s, S, w = (_arr(a) for a in rec["inputs"])
        val, ds, dS = O.loss_forward_backward(rec["name"], rec.get("margin", 0.0), s, S, w)
        np.testing.assert_allclose(val, outs[0], rtol=2e-6, atol=1e-6)
        for a in rec["asserted"]:
            np.testing.assert_allclose(val, _arr(a), rtol=5e-5, atol=5e-5)


def test_cos_prepare_matches_reference_inputs():
    # the comparator fixtures of the cos tests hold prepared (unit-norm) rows
    recs = [r for r in UNIT if r["kind"] == "comparator" and r["name"] == "cos"]
    assert recs
    for r in recs:
        x = _arr(r["inputs"][0])
        n = np.linalg.norm(x, axis=-1)
        assert np.allclose(n[n > 0], 1.0, atol=1e-5)


@pytest.mark.parametrize("name", step_fixture_names())
def test_composed_step_matches_reference(name):
    c, z = load_step(name)
    cfg = oracle_config(c)
    st = oracle_state(c, z)
    for step in range(c["steps"]):
        stats = O.train_batch(cfg, st, *batch_of(c, z, step), weight_of(c, z, step))
        assert stats["loss"] == pytest.approx(float(z[f"loss_{step}"]), rel=2e-5, abs=1e-4)
        if f"reg_{step}" in z.files:
            assert stats["reg"] == pytest.approx(float(z[f"reg_{step}"]), rel=2e-5, abs=1e-6)
        # `neg > pos` is decided by fp32 rounding where a negative ties with its positive
        assert abs(stats["violators_lhs"] - int(z[f"violators_lhs_{step}"])) <= stats["ties_lhs"]
        assert abs(stats["violators_rhs"] - int(z[f"violators_rhs_{step}"])) <= stats["ties_rhs"]
        np.testing.assert_allclose(st.W_lhs, z[f"W_lhs_after_{step}"], rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(st.G_lhs, z[f"G_lhs_after_{step}"], rtol=2e-5, atol=1e-7)
        if c["separate"]:
            np.testing.assert_allclose(st.W_rhs, z[f"W_rhs_after_{step}"], rtol=2e-5, atol=2e-6)
            np.testing.assert_allclose(st.G_rhs, z[f"G_rhs_after_{step}"], rtol=2e-5, atol=1e-7)
        for side in ("rhs", "lhs"):
            key = f"theta_{side}_after_{step}"
            if key in z and getattr(st, f"theta_{side}") is not None:
                np.testing.assert_allclose(getattr(st, f"theta_{side}"), z[key], rtol=2e-5, atol=2e-6)
                # accumulators are squares of fp32 sums with cancellation in the reference: a little looser
                np.testing.assert_allclose(getattr(st, f"acc_{side}"), z[f"acc_{side}_after_{step}"], rtol=1e-4, atol=1e-7)
        for ent, side in (("e", "lhs"), ("f", "rhs")):
            key = f"glob_{ent}_after_{step}"
            if key in z.files:
                np.testing.assert_allclose(getattr(st, f"glob_{side}"), z[key], rtol=2e-5, atol=2e-6)
                np.testing.assert_allclose(getattr(st, f"gacc_{side}"), z[f"gacc_{ent}_after_{step}"], rtol=1e-4, atol=1e-7)


@pytest.mark.parametrize("name", step_fixture_names())
def test_forward_scores_match_reference(name):
    c, z = load_step(name)
    cfg = oracle_config(c)
    st = oracle_state(c, z)
    for step in range(c["steps"]):
        O.train_batch(cfg, st, *batch_of(c, z, step), weight_of(c, z, step))
    rel = z["fw_rel"] if c["dyn"] else int(z["fw_rel"])
    ul = None if c["disable_lhs"] else z["fw_ul"]
    ur = None if c["disable_rhs"] else z["fw_ur"]
    sc = O.score_batch(cfg, st, z["fw_lhs"], z["fw_rhs"], rel, ul, ur)
    for k in ("lhs_pos", "rhs_pos", "lhs_neg", "rhs_neg"):
        want = z[f"fw_{k}"]
        assert sc[k].shape == want.shape, k
        np.testing.assert_allclose(sc[k], want, rtol=3e-5, atol=3e-5)


def test_wave_of_one_is_a_plain_batch():
    c, z = load_step("sequence_3_batches")
    cfg = oracle_config(c)
    a, b = oracle_state(c, z), oracle_state(c, z)
    for step in range(3):
        s1 = O.train_batch(cfg, a, *batch_of(c, z, step), weight_of(c, z, step))
        s2 = O.train_wave(cfg, b, [batch_of(c, z, step)])[0]
        assert s1 == s2
    assert np.array_equal(a.W_lhs, b.W_lhs) and np.array_equal(a.G_lhs, b.G_lhs)


def test_wave_reads_the_snapshot():
    c, z = load_step("sequence_3_batches")
    cfg = oracle_config(c)
    a, b = oracle_state(c, z), oracle_state(c, z)
    batches = [batch_of(c, z, s) for s in range(3)]
    O.train_wave(cfg, a, batches)
    for bt in batches:
        O.train_batch(cfg, b, *bt)
    # same rows are touched, values differ slightly (stale reads), accumulators too
    assert not np.array_equal(a.W_lhs, b.W_lhs)
    assert np.array_equal(a.W_lhs != z["W_lhs0"], b.W_lhs != z["W_lhs0"])


def _torch_port_cases():
    out = []
    for n in step_fixture_names():
        c, _ = load_step(n)
        if c["op"] in ("linear", "affine") or c["disable_lhs"] or c["disable_rhs"] or c.get("edge_weight") or c.get("global_emb") or c.get("reg_coef") or c.get("max_norm"):
            continue
        out.append(n)
    return out


@pytest.mark.parametrize("name", _torch_port_cases())
def test_torch_port_matches_reference(name):
    """The fp32 PyTorch port that bench.py times as the CPU baseline reproduces the reference."""
    import torch
    from oracle.pbg_step_torch import StepModel
    torch.set_num_threads(1)
    c, z = load_step(name)
    weights = [1.0] if c["dyn"] else [c["rel_weight"] if i == c["rel_idx"] else 1.0 for i in range(c["n_rel_std"])]
    m = StepModel(c["D"], c["op"], c["comp"], c["loss"], c["margin"], c["lr"], c["relation_lr"], c["nb"], c["nu"],
                  c["dyn"], c["R"] if c["dyn"] else c["n_rel_std"], weights)
    W = torch.tensor(z["W_lhs0"]); G = torch.tensor(z["G_lhs0"])
    W2, G2 = (torch.tensor(z["W_rhs0"]), torch.tensor(z["G_rhs0"])) if c["separate"] else (W, G)
    m.attach(W, G, W2, G2)
    with torch.no_grad():
        for side in m.theta:
            m.theta[side].copy_(torch.tensor(z[f"theta_{side}0"]))
    for step in range(c["steps"]):
        lhs, rhs, rel, ul, ur = batch_of(c, z, step)
        rel_t = torch.tensor(rel) if c["dyn"] else rel
        st = m.train_batch(torch.tensor(lhs), torch.tensor(rhs), rel_t, torch.tensor(ul), torch.tensor(ur))
        assert st["loss"] == pytest.approx(float(z[f"loss_{step}"]), rel=1e-5, abs=1e-4)
        np.testing.assert_allclose(W.detach().numpy(), z[f"W_lhs_after_{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(G.numpy(), z[f"G_lhs_after_{step}"], rtol=1e-5, atol=1e-7)
        for side in m.theta:
            np.testing.assert_allclose(m.theta[side].detach().numpy(), z[f"theta_{side}_after_{step}"], rtol=1e-5, atol=1e-6)


# ---------------------------------------------------------------- all_negs relations (model.py:582-617)
def allnegs_cases():
    import glob
    return sorted(os.path.basename(p)[len("allnegs_"):-len(".npz")] for p in glob.glob(os.path.join(GOLDEN, "allnegs_*.npz")))


def load_allnegs(name):
    """(oracle config, oracle state, fixture) of a recorded all_negs case."""
    from oracle.pbg_step import BucketState, StepConfig
    z = np.load(os.path.join(GOLDEN, f"allnegs_{name}.npz"))
    D = z["W_lhs"].shape[1]
    cfg = StepConfig(dim=D, operator=str(z["op"]), comparator=str(z["comp"]), loss=str(z["loss"]), margin=float(z["margin"]),
                     num_batch_negs=50, num_uniform_negs=0, dynamic=bool(z["dyn"]), num_rels=int(z["R"]) if bool(z["dyn"]) else 1)
    Wl = z["W_lhs"].astype(np.float64)
    Wr = z["W_rhs"].astype(np.float64) if bool(z["separate"]) else Wl
    st = BucketState(Wl, np.zeros(len(Wl)), Wr, np.zeros(len(Wr)))
    if z["theta_rhs"].shape[0]:
        st.theta_rhs = z["theta_rhs"].astype(np.float64)
    if z["theta_lhs"].shape[0]:
        st.theta_lhs = z["theta_lhs"].astype(np.float64)
    return cfg, st, z


def allnegs_stats(cfg, sc):
    """RankingEvaluator's Stats (eval.py:43-81) from forward scores: sums over the batch, both sides averaged."""
    from oracle import pbg_step as O
    ranks, loss, aucs = [], 0.0, []
    for side in ("lhs", "rhs"):
        pos, neg = sc[f"{side}_pos"], sc[f"{side}_neg"]
        loss += O.loss_forward_backward(cfg.loss, cfg.margin, pos, neg)[0]
        ranks.append((neg >= pos[:, None]).sum(1) + 1)
        aucs.append(float((pos[:, None] > neg).mean()))
    m = lambda xs: float(np.mean([x.sum() for x in xs]))
    return dict(loss=loss, pos_rank=m(ranks), mrr=m([1.0 / r for r in ranks]), r1=m([r <= 1 for r in ranks]),
                r10=m([r <= 10 for r in ranks]), r50=m([r <= 50 for r in ranks]), auc=float(np.mean(aucs)))


@pytest.mark.parametrize("name", allnegs_cases())
def test_all_negs_scores_and_evaluator_stats_match_the_reference(name):
    from oracle import pbg_step as O
    cfg, st, z = load_allnegs(name)
    sc = O.score_all_negs(cfg, st, z["lhs"], z["rhs"], z["rel"])
    np.testing.assert_allclose(sc["lhs_pos"], z["lhs_pos"], rtol=5e-5, atol=1e-5)
    np.testing.assert_allclose(sc["rhs_pos"], z["rhs_pos"], rtol=5e-5, atol=1e-5)
    # l2: an entity scored against its own row is -sqrt(max(q, 1e-30)) with q = 0 up to fp32 rounding of the expanded
    # form (a few 1e-7, i.e. a score of a few 1e-4) in the reference, and exactly the clamp in float64
    atol = 6e-4 if cfg.comparator == "l2" else 2e-5
    for side in ("lhs", "rhs"):
        want = z[f"{side}_neg"]
        np.testing.assert_allclose(sc[f"{side}_neg"][:, : want.shape[1]], want, rtol=5e-5, atol=atol)
    got = allnegs_stats(cfg, sc)
    assert got["loss"] == pytest.approx(float(z["stat_loss"]), rel=1e-4)
    for k in ("pos_rank", "mrr", "r1", "r10", "r50"):
        assert got[k] == pytest.approx(float(z["stat_" + k]), rel=1e-5, abs=1e-5), k
    n = int(z["stat_count"])
    assert abs(got["auc"] - float(z["stat_auc"]) / n) <= 4 * 0.5 / np.sqrt(n)       # the reference samples n random pairs
