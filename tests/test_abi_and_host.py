"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares (no
compute calls), and the host-side mirror of the reference interface behaves like the reference."""
import ctypes
import os
import re

import pytest
import torch

import torchbiggraph_b200 as T
from torchbiggraph_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "pbg_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(pbg_[a-z_0-9]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    names = _declared_functions()
    assert len(names) >= 17
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/pbg_b200.h but not exported"
    bound = {n for n, _, _ in _lib.SYMBOLS}
    assert bound == set(names), f"ctypes binding and header disagree: {bound ^ set(names)}"


def test_version_and_status_strings_need_no_gpu():
    L = _lib.lib()
    assert b"sm_100a" in L.pbg_version()
    assert L.pbg_status_string(0) == b"ok"
    assert b"unsupported" in L.pbg_status_string(_lib.PBG_ERR_UNSUPPORTED)


def test_create_without_a_gpu_fails_loudly_with_a_message():
    if torch.cuda.is_available():
        pytest.skip("this check is for CPU-only hosts")
    L = _lib.lib()
    cfg = _lib.PbgConfig(dim=16, op=0, comparator=0, loss=1, dynamic_relations=0, num_rels=1, num_batch_negs=4,
                         num_uniform_negs=4, disable_lhs_negs=0, disable_rhs_negs=0, precision=0, max_batch_size=8,
                         batches_in_flight=1, margin=0.1, lr=0.1, relation_lr=0.1)
    ctx = ctypes.c_void_p()
    st = L.pbg_create(ctypes.byref(cfg), 0, None, ctypes.byref(ctx))
    assert st in (_lib.PBG_ERR_NO_DEVICE, _lib.PBG_ERR_CUDA)
    assert L.pbg_last_error(ctx)
    L.pbg_destroy(ctx)


def test_config_validation_precedes_device_use():
    L = _lib.lib()
    ctx = ctypes.c_void_p()
    bad = _lib.PbgConfig(dim=18, op=0, comparator=0, loss=1, num_rels=1, num_batch_negs=4, num_uniform_negs=4,
                         max_batch_size=8, batches_in_flight=1)
    assert L.pbg_create(ctypes.byref(bad), 0, None, ctypes.byref(ctx)) == _lib.PBG_ERR_UNSUPPORTED   # dim % 4
    assert b"multiple of 4" in L.pbg_last_error(ctx)
    L.pbg_destroy(ctx)
    lin = _lib.PbgConfig(dim=16, op=4, comparator=0, loss=1, num_rels=1, num_batch_negs=4, num_uniform_negs=4,
                         max_batch_size=8, batches_in_flight=1, dynamic_relations=1)      # one matrix per edge: refused
    assert L.pbg_create(ctypes.byref(lin), 0, None, ctypes.byref(ctx)) == _lib.PBG_ERR_UNSUPPORTED
    L.pbg_destroy(ctx)
    k0 = _lib.PbgConfig(dim=16, op=0, comparator=0, loss=1, num_rels=1, num_batch_negs=4, num_uniform_negs=4,
                        max_batch_size=8, batches_in_flight=0)
    assert L.pbg_create(ctypes.byref(k0), 0, None, ctypes.byref(ctx)) == _lib.PBG_ERR_BAD_ARGUMENT
    L.pbg_destroy(ctx)
    planes = _lib.PbgConfig(dim=16, op=4, comparator=0, loss=1, num_rels=1, num_batch_negs=4, num_uniform_negs=4,
                            max_batch_size=8, batches_in_flight=1, precision=_lib.PRECISION_CODES["bf16x6"])   # matrix operator: outside the bf16-plane tier
    assert L.pbg_create(ctypes.byref(planes), 0, None, ctypes.byref(ctx)) == _lib.PBG_ERR_UNSUPPORTED
    assert b"bf16-plane" in L.pbg_last_error(ctx)
    L.pbg_destroy(ctx)
    assert L.pbg_row_adagrad_static(None, None, 1, 16, None, None, 0, 0.1, None) == 0        # n == 0: nothing to do
    assert L.pbg_row_adagrad_static(None, None, 1, 16, None, None, 5, 0.1, None) == _lib.PBG_ERR_BAD_ARGUMENT


# ---------------------------------------------------------------- registries (plugin.py:16-40)
def test_registries_hold_the_reference_names():
    for name in ("none", "diagonal", "translation", "linear", "affine", "complex_diagonal"):
        assert T.OPERATORS.get_class(name).name == name
        assert T.DYNAMIC_OPERATORS.get_class(name).name == name
    for name in ("dot", "cos", "l2", "squared_l2"):
        assert T.COMPARATORS.get_class(name).native_code is not None
    for name in ("logistic", "ranking", "softmax"):
        assert T.LOSS_FUNCTIONS.get_class(name).native_code is not None
    with pytest.raises(NotImplementedError, match="no_such_operator"):     # plugin.py:35-40; callers catch this type
        T.OPERATORS.get_class("no_such_operator")


def test_reregistering_a_different_class_raises_like_the_reference():
    reg = T.PluginRegistry()

    @reg.register_as("x")
    class A:
        pass

    reg.register_as("x")(A)          # same class again is fine
    reg.register("x", A)
    with pytest.raises(RuntimeError):
        @reg.register_as("x")
        class B:
            pass
    with pytest.raises(RuntimeError):
        reg.register("x", int)
    reg.register("y", int)
    assert reg.get_class("y") is int


def test_custom_loss_without_device_code_is_refused():
    class MyLoss(T.trainer.AbstractLossFunction):
        pass
    with pytest.raises(NotImplementedError):
        T.B200Trainer(None, MyLoss(), [1.0])


# ---------------------------------------------------------------- config
def _cfg(**kw):
    base = dict(entities={"e": T.EntitySchema()}, relations=[T.RelationSchema("r", "e", "e")], dimension=16)
    base.update(kw)
    return T.ConfigSchema(**base)


@pytest.mark.parametrize("kw", [dict(bias=True), dict(regularization_coef=1e-3, regularizer="L2"),
                                dict(half_precision=True), dict(entities={"e": T.EntitySchema(featurized=True)})])
def test_unsupported_config_keys_raise(kw):
    with pytest.raises(NotImplementedError):
        _cfg(**kw).check_supported()


def test_global_embeddings_need_standard_relations():
    _cfg(global_emb=True).check_supported()
    with pytest.raises(RuntimeError, match="global embs"):       # model.py:488-489
        _cfg(global_emb=True, dynamic_relations=True, num_dynamic_rels=3).check_supported()


def test_batch_size_must_be_multiple_of_batch_negs():
    with pytest.raises(RuntimeError, match="multiple of num_batch_negs"):
        _cfg(batch_size=130, num_batch_negs=50).check_supported()


def test_from_reference_copies_the_path_keys():
    class Ref:      # stands for the reference's ConfigSchema (duck-typed)
        entities = {"e": T.EntitySchema(num_partitions=4)}
        relations = [T.RelationSchema("r", "e", "e", weight=2.0, operator="translation")]
        dimension, comparator, loss_fn, margin, lr, relation_lr = 100, "cos", "ranking", 0.1, 0.1, None
        batch_size, num_batch_negs, num_uniform_negs = 1000, 100, 100
        disable_lhs_negs = disable_rhs_negs = dynamic_relations = False
        global_emb, bias, max_norm, regularization_coef, half_precision, init_scale = False, False, None, 0, False, 1e-3
    c = T.ConfigSchema.from_reference(Ref, batches_in_flight=4)
    assert c.dimension == 100 and c.relations[0].weight == 2.0 and c.batches_in_flight == 4
    c.check_supported()


# ---------------------------------------------------------------- edge lists / stats / batching
def test_edgelist_mirrors_reference_behaviour():
    lhs = T.EntityList.from_tensor(torch.tensor([1, 2, 3]))
    rhs = T.EntityList.from_tensor(torch.tensor([4, 5, 6]))
    e = T.EdgeList(lhs, rhs, torch.tensor(1))
    assert e.has_scalar_relation_type() and e.get_relation_type_as_scalar() == 1 and len(e[1:]) == 2
    with pytest.raises(RuntimeError):
        e.get_relation_type_as_vector()
    v = T.EdgeList(lhs, rhs, torch.tensor([0, 1, 0]))
    assert not v.has_scalar_relation_type() and v[torch.tensor([2, 0])].rel.tolist() == [0, 0]
    with pytest.raises(ValueError):
        T.EdgeList(lhs, T.EntityList.from_tensor(torch.tensor([1])), torch.tensor(0))
    with pytest.raises(TypeError):
        T.EntityList.from_tensor(torch.tensor([1.0]))


def test_stats_sum_and_average():
    s = T.Stats.sum([T.Stats(count=2, loss=4.0), T.Stats(count=6, loss=12.0)])
    assert s.count == 8 and s.metrics["loss"] == 16.0 and s.average().metrics["loss"] == 2.0


def test_relation_grouped_batches_cover_every_edge_once():
    from torchbiggraph_b200.trainer import _batches_group_by_relation
    g = torch.Generator().manual_seed(0)
    rel = torch.sort(torch.randint(0, 5, (1234,), generator=g)).values
    batches = _batches_group_by_relation(rel, 100, generator=g)
    seen = torch.zeros(1234, dtype=torch.int)
    for off, n, r in batches:
        assert 0 < n <= 100 and bool((rel[off:off + n] == r).all())
        seen[off:off + n] += 1
    assert bool((seen == 1).all())


def test_batch_list_is_cut_into_runs_that_read_one_pair_of_tables():
    """process_in_batches hands consecutive batches of one (lhs table, rhs table) pair to the library in
    one call and starts a new call where the pair changes; the order of the batches is kept."""
    from torchbiggraph_b200.trainer import _runs_by_table_pair

    class FakeModel:
        num_dynamic_rels = 0
        tabs = {0: (torch.zeros(2, 4), torch.zeros(2, 4))}

        ops = {0: "none", 1: "none", 2: "none"}

        def tables_for(self, r):
            return self.tabs[r]

        def operator_of(self, r):
            return self.ops[r]

    m = FakeModel()
    m.tabs[1] = (m.tabs[0][0], torch.zeros(3, 4))      # relation 1 reads another rhs table
    m.tabs[2] = m.tabs[0]                              # relation 2 shares relation 0's tables
    batches = [(0, 5, 0), (5, 5, 2), (10, 5, 1), (15, 5, 1), (20, 5, 0)]
    runs = _runs_by_table_pair(m, batches)
    assert runs == [[(0, 5, 0), (5, 5, 2)], [(10, 5, 1), (15, 5, 1)], [(20, 5, 0)]]
    assert _runs_by_table_pair(m, []) == []
    m.ops = {0: "none", 1: "none", 2: "translation"}          # a relation with another operator starts a run of its own
    assert _runs_by_table_pair(m, batches) == [[(0, 5, 0)], [(5, 5, 2)], [(10, 5, 1), (15, 5, 1)], [(20, 5, 0)]]
    m.num_dynamic_rels = 3
    assert _runs_by_table_pair(m, batches) == [batches]


def test_optimizer_state_dict_round_trip_keeps_reference_format():
    w = torch.zeros(5, 4)
    opt = T.RowAdagrad([w], lr=0.1)
    opt.sum_for(w).copy_(torch.arange(5.0))
    sd = opt.state_dict()
    assert set(sd) == {"state", "param_groups"} and sd["state"][0]["sum"].tolist() == [0, 1, 2, 3, 4]
    opt2 = T.RowAdagrad([w], lr=0.5)
    opt2.load_state_dict(sd)
    assert opt2.sum_for(w).tolist() == [0, 1, 2, 3, 4] and opt2.lr == 0.1
    with pytest.raises(ValueError):
        T.RowAdagrad([torch.zeros(3)])


def test_model_refuses_cpu_tensors_and_no_fallback():
    with pytest.raises((RuntimeError, AssertionError, ValueError)):
        m = T.make_model(_cfg(), "cpu")
        m.set_embeddings("e", T.Side.LHS, torch.zeros(3, 16))
        tr = T.B200Trainer(None, T.LOSS_FUNCTIONS.get_class("ranking")(margin=0.1), [1.0])
        tr.partitioned_optimizers["e", 0] = T.RowAdagrad([m.lhs_embs["emb_e"]], lr=0.1)
        m.set_embeddings("e", T.Side.RHS, m.lhs_embs["emb_e"])
        tr.process_one_batch(m, T.EdgeList(T.EntityList.from_tensor(torch.tensor([0])),
                                           T.EntityList.from_tensor(torch.tensor([1])), torch.tensor(0)))


def test_bench_names_a_default_tier_per_workload():
    """bench.py's default arithmetic is one of the rtol 1e-4 tensor-core tiers, and every tier has its note."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for name, w in bench.WORKLOADS.items():
        assert w.get("precision", "tf32x3") in ("tf32x3", "bf16x6"), name
    assert set(bench.PRECISION_NOTES) == set(_lib.PRECISION_CODES)
