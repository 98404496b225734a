"""The reference-side binding (torchbiggraph_b200/reference_adapter.py) against the reference's OWN classes: its
MultiRelationEmbedder, EdgeList, Trainer and optimizers, imported from a PyTorch-BigGraph checkout (skipped where
there is none; an `h5py` stand-in is put on sys.path for the import only, as tests/golden/make_golden.py does).

Without a GPU this checks everything up to the library call: the adapter is a torchbiggraph AbstractBatchProcessor,
the configuration struct it hands to pbg_create says what the reference config says, the operator tables it packs
ARE the reference's parameters (and AsyncAdagrad state) afterwards -- the reference's own CPU Trainer keeps training
through them with unchanged results -- the bucket struct points at the reference's tensors, and a CPU model is
refused loudly (no fallback)."""
import os
import sys

import numpy as np
import pytest
import torch

REF = os.environ.get("PBG_REFERENCE", "/root/reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "torchbiggraph")), reason="needs a PyTorch-BigGraph checkout")


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from make_golden import _bootstrap
    _bootstrap(REF)
    import torchbiggraph.model as M
    return M


def _build(ref, op, dyn, comp="dot", loss="softmax", R=5, D=16, N=60):
    from torchbiggraph.config import ConfigSchema, EntitySchema, RelationSchema
    from torchbiggraph.model import make_model
    from torchbiggraph.train_cpu import Trainer, make_optimizer
    from torchbiggraph.losses import LOSS_FUNCTIONS
    from torchbiggraph.types import Side
    nrel = 1 if dyn else 2
    cfg = ConfigSchema(entities={"e": EntitySchema(num_partitions=1)},
                       relations=[RelationSchema(name=f"r{i}", lhs="e", rhs="e", operator=op, weight=1.0 + i) for i in range(nrel)],
                       dimension=D, entity_path="x", edge_paths=["y"], checkpoint_path="z", comparator=comp, loss_fn=loss,
                       global_emb=False, batch_size=40, num_batch_negs=20, num_uniform_negs=10, lr=0.1, relation_lr=0.05,
                       dynamic_relations=dyn)
    if dyn:
        class RelCount:
            def __init__(self, path): pass
            def load_count(self): return R
        ref.RELATION_TYPE_STORAGES.registry["x"] = RelCount
        ref.RELATION_TYPE_STORAGES.registry[""] = RelCount
    torch.manual_seed(3)
    model = make_model(cfg)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.2)
    opt = make_optimizer(cfg, model.parameters(), False)
    trainer = Trainer(opt, LOSS_FUNCTIONS.get_class(loss)(margin=cfg.margin), [r.weight for r in cfg.relations])
    emb = torch.nn.Parameter(torch.randn(N, D) * 0.3)
    model.set_embeddings("e", Side.LHS, emb)
    model.set_embeddings("e", Side.RHS, emb)
    trainer.partitioned_optimizers["e", 0] = make_optimizer(cfg, [emb], True)
    return cfg, model, trainer, emb


def _edges(dyn, R, N, n=37, seed=0):
    from torchbiggraph.edgelist import EdgeList
    from torchbiggraph.entitylist import EntityList
    g = torch.Generator().manual_seed(seed)
    rel = torch.randint(0, R, (n,), generator=g) if dyn else torch.tensor(1)
    return EdgeList(EntityList.from_tensor(torch.randint(0, N, (n,), generator=g)),
                    EntityList.from_tensor(torch.randint(0, N, (n,), generator=g)), rel)


@pytest.mark.parametrize("op,dyn", [("translation", False), ("complex_diagonal", True), ("diagonal", True), ("none", False)])
def test_adapter_is_a_reference_batch_processor_over_the_reference_tensors(ref, op, dyn):
    from torchbiggraph.batching import AbstractBatchProcessor
    from torchbiggraph_b200 import _lib
    from torchbiggraph_b200.reference_adapter import OperatorTables, make_reference_trainer
    cfg, model, trainer, emb = _build(ref, op, dyn)
    adapter = make_reference_trainer(cfg, model, model_optimizer=trainer.model_optimizer)
    assert isinstance(adapter, AbstractBatchProcessor)
    nc = adapter.native_config
    assert (nc.dim, nc.op, nc.comparator, nc.loss) == (16, _lib.OPERATOR_CODES[op], _lib.COMPARATOR_CODES["dot"], _lib.LOSS_CODES["softmax"])
    assert nc.dynamic_relations == int(dyn) and nc.num_rels == (5 if dyn else 2)
    assert (nc.num_batch_negs, nc.num_uniform_negs, nc.max_batch_size) == (20, 10, 40)
    assert nc.lr == pytest.approx(0.1) and nc.relation_lr == pytest.approx(0.05)
    # a step of the reference's own trainer, so that its AsyncAdagrad state exists
    trainer.process_one_batch(model, _edges(dyn, 5, 60))
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    tabs = OperatorTables(model, trainer.model_optimizer, op, 16, dyn)
    for n, p in model.named_parameters():                       # packing moved the storage, not the values
        assert torch.equal(p.detach(), before[n]), n
    if op == "none":
        assert tabs.rhs is None
        return
    # the tables ARE the parameters now: a write on one side shows on the other
    ops = [o for o in model.rhs_operators if o is not None]
    first = next(iter(ops[0].parameters()))
    tabs.rhs[0, 0] += 1.0
    assert float(first.detach().reshape(-1)[0]) == pytest.approx(float(before[next(n for n, p in model.named_parameters() if p is first)].reshape(-1)[0]) + 1.0)
    tabs.rhs[0, 0] -= 1.0
    state = trainer.model_optimizer.state[first]["sum"]
    assert state.data_ptr() >= tabs.rhs_acc.data_ptr() and state.data_ptr() < tabs.rhs_acc.data_ptr() + tabs.rhs_acc.numel() * 4
    # the reference's CPU trainer keeps working through the aliased parameters, with the results it had without them
    cfg2, model2, trainer2, emb2 = _build(ref, op, dyn)
    trainer2.process_one_batch(model2, _edges(dyn, 5, 60))
    for seed in (1, 2):
        torch.manual_seed(100 + seed); a = trainer.process_one_batch(model, _edges(dyn, 5, 60, seed=seed))
        torch.manual_seed(100 + seed); b = trainer2.process_one_batch(model2, _edges(dyn, 5, 60, seed=seed))
        assert a.metrics["loss"] == pytest.approx(b.metrics["loss"], rel=1e-6)
    np.testing.assert_allclose(emb.detach().numpy(), emb2.detach().numpy(), rtol=1e-6, atol=1e-7)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), model2.named_parameters()):
        np.testing.assert_allclose(p1.detach().numpy(), p2.detach().numpy(), rtol=1e-6, atol=1e-7, err_msg=n1)


def test_adapter_refuses_a_cpu_model_and_what_it_does_not_bind(ref):
    from torchbiggraph_b200.reference_adapter import make_reference_trainer
    cfg, model, trainer, emb = _build(ref, "translation", False)
    adapter = make_reference_trainer(cfg, model, model_optimizer=trainer.model_optimizer)
    adapter.partitioned_optimizers = trainer.partitioned_optimizers
    with pytest.raises(RuntimeError, match="CUDA device only"):
        adapter.process_one_batch(model, _edges(False, 1, 60))
    cfg_l, model_l, trainer_l, _ = _build(ref, "linear", False)
    ad = make_reference_trainer(cfg_l, model_l, model_optimizer=trainer_l.model_optimizer)
    ad.partitioned_optimizers = trainer_l.partitioned_optimizers
    with pytest.raises((NotImplementedError, RuntimeError)):
        ad.process_one_batch(model_l, _edges(False, 1, 60))


@pytest.mark.gpu
@pytest.mark.parametrize("op,dyn,comp,loss", [("translation", False, "dot", "softmax"), ("complex_diagonal", True, "cos", "ranking"),
                                              ("none", False, "dot", "logistic")])
def test_reference_model_trained_through_the_library_matches_the_reference_trainer(ref, op, dyn, comp, loss):
    """Three batches on the reference's MultiRelationEmbedder (CUDA tensors) through the adapter against the reference's
    own Trainer on a CPU clone; no uniform negatives, so both see the same negatives.  Needs a GPU AND the checkout."""
    from torchbiggraph_b200.reference_adapter import make_reference_trainer
    from torchbiggraph.config import ConfigSchema
    from torchbiggraph.train_cpu import make_optimizer
    from torchbiggraph.types import Side
    import attr
    cfg, model, trainer, emb = _build(ref, op, dyn, comp, loss)
    cfg = attr.evolve(cfg, num_uniform_negs=0)
    cfg_g, model_g, trainer_g, _ = _build(ref, op, dyn, comp, loss)
    model.num_uniform_negs = 0
    model_g.num_uniform_negs = 0
    model_g = model_g.cuda()
    emb_g = torch.nn.Parameter(emb.detach().clone().cuda())
    model_g.set_embeddings("e", Side.LHS, emb_g)
    model_g.set_embeddings("e", Side.RHS, emb_g)
    adapter = make_reference_trainer(cfg, model_g, precision="fp32")
    adapter.partitioned_optimizers["e", 0] = make_optimizer(cfg, [emb_g], True)
    for seed in range(3):
        e = _edges(dyn, 5, 60, seed=seed)
        a = trainer.process_one_batch(model, e)
        b = adapter.process_one_batch(model_g, e)
        assert b.metrics["loss"] == pytest.approx(a.metrics["loss"], rel=1e-4)
    np.testing.assert_allclose(emb_g.detach().cpu().numpy(), emb.detach().numpy(), rtol=1e-4, atol=2e-6)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), model_g.named_parameters()):
        np.testing.assert_allclose(p2.detach().cpu().numpy(), p1.detach().numpy(), rtol=1e-4, atol=2e-6, err_msg=n1)
