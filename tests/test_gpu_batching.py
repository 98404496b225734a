"""process_in_batches (torchbiggraph/batching.py:91-125 moved onto the device) against the same
batches handed over one at a time through process_one_batch: per-edge weights travel with the
edges, and relations over different entity types are trained by separate library calls in the
reference's batch order.  No uniform negatives, so nothing is drawn at random inside the step."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-4


def _setup(two_types, seed=5, D=32, N=400, M=300):
    import torchbiggraph_b200 as T
    rng = np.random.default_rng(seed)
    ents = {"e": T.EntitySchema()}
    rels = [T.RelationSchema("r0", "e", "e", operator="translation", weight=1.0)]
    if two_types:
        ents["f"] = T.EntitySchema()
        rels += [T.RelationSchema("r1", "e", "f", operator="translation", weight=0.5),
                 T.RelationSchema("r2", "e", "e", operator="translation", weight=2.0)]
    cfg = T.ConfigSchema(entities=ents, relations=rels, dimension=D, comparator="dot", loss_fn="softmax", lr=0.1,
                         batch_size=100, num_batch_negs=50, num_uniform_negs=0)
    We = (rng.standard_normal((N, D)) * 0.1).astype(np.float32)
    Wf = (rng.standard_normal((M, D)) * 0.1).astype(np.float32)
    th = (rng.standard_normal((len(rels), D)) * 0.1).astype(np.float32)

    def build():
        model = T.make_model(cfg, "cuda")
        model.rhs_op_table.copy_(torch.tensor(th).cuda())
        tr = T.B200Trainer(T.make_optimizer(cfg, model.parameters(), False),
                           T.LOSS_FUNCTIONS.get_class("softmax")(margin=0.1), [r.weight for r in rels])
        we, wf = torch.tensor(We).cuda(), torch.tensor(Wf).cuda()
        model.set_embeddings("e", T.Side.LHS, we)
        model.set_embeddings("e", T.Side.RHS, we)
        tr.partitioned_optimizers["e", 0] = T.make_optimizer(cfg, [we], True)
        if two_types:
            model.set_embeddings("f", T.Side.RHS, wf)
            tr.partitioned_optimizers["f", 0] = T.make_optimizer(cfg, [wf], True)
        return model, tr, we, wf

    n = 730
    rel = rng.integers(0, len(rels), n) if two_types else np.zeros(n, np.int64)
    lhs = rng.integers(0, N, n)
    rhs = np.where(rel == 1, rng.integers(0, M, n), rng.integers(0, N, n))
    wgt = (0.5 + rng.random(n) * 3).astype(np.float32)          # mean 2: the weighted total is about twice the plain one
    return T, build, lhs, rhs, rel, wgt


@pytest.mark.parametrize("two_types", [False, True], ids=["one_relation_weighted", "two_entity_types_weighted"])
def test_process_in_batches_equals_batch_by_batch(two_types):
    from torchbiggraph_b200.trainer import _batches_group_by_relation
    T, build, lhs, rhs, rel, wgt = _setup(two_types)
    t = lambda a: torch.tensor(np.asarray(a))
    ent = lambda a: T.EntityList.from_tensor(t(a))
    # (a) the whole edge list in one call of process_in_batches
    model_a, tr_a, we_a, wf_a = build()
    edges = T.EdgeList(ent(lhs), ent(rhs), t(rel) if two_types else t(0), t(wgt))
    torch.manual_seed(123)
    total = T.process_in_batches(100, model_a, tr_a, edges)
    # (b) the same batches in the same order, one process_one_batch each
    model_b, tr_b, we_b, wf_b = build()
    if two_types:
        order = np.argsort(rel, kind="stable")
        torch.manual_seed(123)
        batches = _batches_group_by_relation(t(rel[order]), 100)
    else:
        order = np.arange(len(lhs))
        batches = [(o, min(100, len(lhs) - o), 0) for o in range(0, len(lhs), 100)]
    parts = []
    for off, cnt, r in batches:
        idx = order[off:off + cnt]
        parts.append(tr_b.process_one_batch(model_b, T.EdgeList(ent(lhs[idx]), ent(rhs[idx]), t(r), t(wgt[idx]))))
    want = T.Stats.sum(parts)
    assert total.count == want.count == len(lhs)
    assert total.metrics["loss"] == pytest.approx(want.metrics["loss"], rel=RTOL)
    assert total.metrics["violators_lhs"] == want.metrics["violators_lhs"]
    np.testing.assert_allclose(we_a.cpu().numpy(), we_b.cpu().numpy(), rtol=RTOL, atol=1e-6)
    np.testing.assert_allclose(model_a.rhs_op_table.cpu().numpy(), model_b.rhs_op_table.cpu().numpy(), rtol=RTOL, atol=1e-6)
    if two_types:
        np.testing.assert_allclose(wf_a.cpu().numpy(), wf_b.cpu().numpy(), rtol=RTOL, atol=1e-6)
    # the weights did enter the loss: the unweighted list gives another total
    model_c, tr_c, _, _ = build()
    torch.manual_seed(123)
    plain = T.process_in_batches(100, model_c, tr_c, T.EdgeList(ent(lhs), ent(rhs), t(rel) if two_types else t(0)))
    assert total.metrics["loss"] > 1.5 * plain.metrics["loss"]


def test_relations_with_different_operators_train_like_the_oracle():
    """Standard relations may each have their own operator (torchbiggraph/model.py:368-476 builds one per relation).
    Three relations -- translation, complex_diagonal, none -- over one entity type: process_in_batches cuts the
    batch list where the operator changes and trains every run through the library context of its operator; the
    result is held to the CPU oracle run batch by batch in the same order."""
    import torchbiggraph_b200 as T
    from oracle import pbg_step as O
    from torchbiggraph_b200.trainer import _batches_group_by_relation
    rng = np.random.default_rng(21)
    D, N, n = 16, 300, 640
    ops = ["translation", "complex_diagonal", "none", "translation"]
    weights = [1.0, 0.5, 2.0, 1.5]
    cfg = T.ConfigSchema(entities={"e": T.EntitySchema()},
                         relations=[T.RelationSchema(f"r{i}", "e", "e", operator=o, weight=w) for i, (o, w) in enumerate(zip(ops, weights))],
                         dimension=D, comparator="dot", loss_fn="ranking", margin=0.1, lr=0.1, relation_lr=0.05, batch_size=100,
                         num_batch_negs=50, num_uniform_negs=0)
    model = T.make_model(cfg, "cuda")
    assert model.rhs_op_table is None and set(model.op_groups) == {"translation", "complex_diagonal", "none"}
    W0 = (rng.standard_normal((N, D)) * 0.2).astype(np.float32)
    th = {o: (O.operator_init(o, D, len(m), np.float32) + rng.standard_normal((len(m), D)).astype(np.float32) * 0.2)
          for o, m in model.op_groups.items() if o != "none"}
    for o, t in th.items():
        model.op_tables[o].copy_(torch.tensor(t).cuda())
    tr = T.B200Trainer(T.make_optimizer(cfg, model.parameters(), False), T.LOSS_FUNCTIONS.get_class("ranking")(margin=0.1), weights)
    W = torch.tensor(W0).cuda()
    model.set_embeddings("e", T.Side.LHS, W)
    model.set_embeddings("e", T.Side.RHS, W)
    tr.partitioned_optimizers["e", 0] = T.make_optimizer(cfg, [W], True)
    lhs, rhs, rel = rng.integers(0, N, n), rng.integers(0, N, n), rng.integers(0, len(ops), n)
    t = lambda a: torch.tensor(np.asarray(a))
    torch.manual_seed(77)
    total = T.process_in_batches(100, model, tr, T.EdgeList(T.EntityList.from_tensor(t(lhs)), T.EntityList.from_tensor(t(rhs)), t(rel)))
    # the oracle, relation by relation state, same batches in the same order
    Wo, Go = W0.astype(np.float64), np.zeros(N)
    states = {}
    for o, m in model.op_groups.items():
        st = O.BucketState(Wo, Go, Wo, Go)
        if o != "none":
            st.theta_rhs, st.acc_rhs = th[o].astype(np.float64), np.zeros_like(th[o], np.float64)
        states[o] = st
    order = np.argsort(rel, kind="stable")
    torch.manual_seed(77)
    want = 0.0
    for off, cnt, r in _batches_group_by_relation(t(rel[order]), 100):
        idx = order[off:off + cnt]
        o, local = model.group_of[r]
        ocfg = O.StepConfig(dim=D, operator=o, comparator="dot", loss="ranking", margin=0.1, lr=0.1, relation_lr=0.05,
                            num_batch_negs=50, num_uniform_negs=0, num_rels=len(model.op_groups[o]),
                            relation_weights=[weights[g] for g in model.op_groups[o]])
        chunks = -(-cnt // min(50, cnt))
        want += O.train_batch(ocfg, states[o], lhs[idx], rhs[idx], local, np.zeros((chunks, 0), np.int64), np.zeros((chunks, 0), np.int64))["loss"]
    assert total.count == n
    assert total.metrics["loss"] == pytest.approx(want, rel=RTOL)
    np.testing.assert_allclose(W.cpu().numpy(), Wo, rtol=RTOL, atol=2e-6)
    for o in th:
        np.testing.assert_allclose(model.op_tables[o].cpu().numpy(), states[o].theta_rhs, rtol=RTOL, atol=2e-6, err_msg=o)
