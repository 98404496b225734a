"""The batch processor that replaces the reference's Trainer (torchbiggraph/train_cpu.py:74-112)
and the batch loop around it (torchbiggraph/batching.py:91-125).

`B200Trainer.process_one_batch(model, batch_edges) -> Stats` is the reference interface
(AbstractBatchProcessor, batching.py:128-165).  `process_in_batches` hands a whole edge list to the
library in one call, which trains `batches_in_flight` batches per wave on the device."""
import ctypes as C
import time
from abc import ABC, abstractmethod
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import _lib
from ._lib import PbgBatch, PbgBatchStats, PbgBucket, PbgConfig, check
from .model import MultiRelationEmbedder, Scores
from .registries import LOSS_FUNCTIONS, AbstractLossFunction
from .row_adagrad import AsyncAdagrad, RowAdagrad
from .types import EdgeList, Stats


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


class _Native:
    """One library context bound to a model's static configuration."""

    def __init__(self, model: MultiRelationEmbedder, max_batch: int, k: int, precision: str, lr: float,
                 relation_lr: Optional[float], margin: float, loss_code: Optional[int] = None,
                 num_batch_negs: Optional[int] = None, num_uniform_negs: Optional[int] = None,
                 op_name: Optional[str] = None):
        cfg = model.config
        self.op_name = model.operator_name if op_name is None else op_name
        if model.device.type != "cuda":
            raise RuntimeError("torchbiggraph_b200 runs on a CUDA device only (no CPU fallback)")
        self.lib = _lib.lib()
        c = PbgConfig()
        c.dim = cfg.dimension
        c.op = _lib.OPERATOR_CODES[self.op_name]
        c.comparator = model.comparator.native_code
        c.loss = _lib.LOSS_CODES[cfg.loss_fn] if loss_code is None else loss_code
        c.dynamic_relations = int(cfg.dynamic_relations)
        c.num_rels = model.num_dynamic_rels if cfg.dynamic_relations else len(model.op_groups[self.op_name])
        c.num_batch_negs = cfg.num_batch_negs if num_batch_negs is None else num_batch_negs
        c.num_uniform_negs = cfg.num_uniform_negs if num_uniform_negs is None else num_uniform_negs
        c.disable_lhs_negs = int(cfg.disable_lhs_negs)
        c.disable_rhs_negs = int(cfg.disable_rhs_negs)
        c.precision = _lib.PRECISION_CODES[precision]
        c.max_batch_size = max_batch
        c.batches_in_flight = k
        c.margin = margin
        c.lr = lr
        c.relation_lr = lr if relation_lr is None else relation_lr
        c.regularization_coef = float(getattr(cfg, "regularization_coef", 0.0))
        c.max_norm = float(getattr(cfg, "max_norm", None) or 0.0)
        self.cfg = c
        self.max_batch = max_batch
        self.device_index = model.device.index if model.device.index is not None else torch.cuda.current_device()
        self.ctx = C.c_void_p()
        stream = torch.cuda.current_stream(self.device_index).cuda_stream
        st = self.lib.pbg_create(C.byref(c), self.device_index, C.c_void_p(stream), C.byref(self.ctx))
        if st != 0:
            msg = self.lib.pbg_last_error(self.ctx).decode() if self.ctx else ""
            self.lib.pbg_destroy(self.ctx)
            self.ctx = None
            if st == _lib.PBG_ERR_UNSUPPORTED:
                raise NotImplementedError(msg)
            raise _lib.PbgError(st, msg)

    def __del__(self):
        if getattr(self, "ctx", None):
            self.lib.pbg_destroy(self.ctx)
            self.ctx = None

    def set_hyper(self, lr, relation_lr, margin):
        check(self.lib.pbg_set_hyperparameters(self.ctx, lr, lr if relation_lr is None else relation_lr, margin), self.ctx)

    def bucket(self, model, relation_idx, states, weights_arr) -> PbgBucket:
        wl, wr = model.tables_for(relation_idx)
        b = PbgBucket()
        b.lhs_emb, b.lhs_rows = wl.data_ptr(), wl.shape[0]
        b.rhs_emb, b.rhs_rows = wr.data_ptr(), wr.shape[0]
        if states is not None:
            gl, gr, al, ar = states[:4]
            b.lhs_state, b.rhs_state = gl.data_ptr(), gr.data_ptr()
            b.rhs_op_state = None if ar is None else ar.data_ptr()
            b.lhs_op_state = None if al is None else al.data_ptr()
        rhs_tab, lhs_tab = model.op_table_for(self.op_name)
        b.rhs_op = None if rhs_tab is None else rhs_tab.data_ptr()
        b.lhs_op = None if lhs_tab is None else lhs_tab.data_ptr()
        b.relation_weights = weights_arr
        gl_, gr_ = model.globals_for(relation_idx)
        if gl_ is not None:
            b.lhs_global, b.rhs_global = gl_.data_ptr(), gr_.data_ptr()
            if states is not None and len(states) > 4:
                b.lhs_global_state, b.rhs_global_state = states[4].data_ptr(), states[5].data_ptr()
        return b

    def score(self, model, edges: EdgeList, ul, ur, seed) -> Scores:
        n = len(edges)
        dev = model.device
        lhs = edges.lhs.to_tensor().to(dev).contiguous()
        rhs = edges.rhs.to_tensor().to(dev).contiguous()
        dyn = model.num_dynamic_rels > 0
        if dyn and edges.has_scalar_relation_type():
            raise TypeError("Need relation for each positive pair")
        if not dyn and not edges.has_scalar_relation_type():
            raise TypeError("All positive pairs must come from the same relation")
        rel = edges.rel.to(dev).contiguous() if dyn else None
        relidx = 0 if dyn else edges.get_relation_type_as_scalar()
        local = 0 if dyn else model.group_of[relidx][1]
        P, Cn, lc, rc = (C.c_int32() for _ in range(4))
        check(self.lib.pbg_neg_columns(self.ctx, n, C.byref(P), C.byref(Cn), C.byref(lc), C.byref(rc)), self.ctx)
        lp = torch.empty(n, device=dev); rp = torch.empty(n, device=dev)
        ln = torch.empty((n, lc.value), device=dev); rn = torch.empty((n, rc.value), device=dev)
        ul = None if ul is None else self._uniform(ul, dev)
        ur = None if ur is None else self._uniform(ur, dev)
        b = self.bucket(model, relidx, None, None)
        check(self.lib.pbg_score_batch(self.ctx, C.byref(b), _ptr(lhs), _ptr(rhs), _ptr(rel), n, local,
                                       _ptr(ul), _ptr(ur), seed, _ptr(lp), _ptr(rp), _ptr(ln), _ptr(rn)), self.ctx)
        return Scores(lp, rp, ln, rn)

    def _uniform(self, u, dev):
        """[chunks, U] ids of ONE batch -> the library's [1, chunks_per_batch, U] layout."""
        u = torch.as_tensor(u, dtype=torch.long)
        lim = self.cfg.num_batch_negs if self.cfg.num_batch_negs > 0 else self.cfg.num_uniform_negs
        P = min(lim, self.max_batch)
        cm = (self.max_batch + P - 1) // P
        out = torch.zeros((cm, self.cfg.num_uniform_negs), dtype=torch.long)
        out[: u.shape[0]] = u.reshape(u.shape[0], -1).cpu()
        return out.to(dev)

    def chunks_per_batch(self) -> int:
        lim = self.cfg.num_batch_negs if self.cfg.num_batch_negs > 0 else self.cfg.num_uniform_negs
        P = min(lim, self.max_batch)
        return (self.max_batch + P - 1) // P


class AbstractBatchProcessor(ABC):
    """torchbiggraph/batching.py:128-165."""

    def __init__(self, loss_fn: AbstractLossFunction, relation_weights: List[float], overrides=None):
        self.loss_fn = loss_fn
        self.relation_weights = relation_weights
        self.overrides = overrides

    @abstractmethod
    def _process_one_batch(self, model, batch_edges: EdgeList) -> Stats:
        pass

    def process_one_batch(self, model, batch_edges: EdgeList) -> Stats:
        if self.overrides is not None:
            raise NotImplementedError("model overrides are not supported by torchbiggraph_b200")
        return self._process_one_batch(model, batch_edges)


class B200Trainer(AbstractBatchProcessor):
    """Trainer(model_optimizer, loss_fn, relation_weights) of train_cpu.py:74-84.  The coordinator
    fills `partitioned_optimizers[(entity, part)]` / `unpartitioned_optimizers[entity]` with
    RowAdagrad objects on partition swap exactly as it does for the reference."""

    def __init__(self, model_optimizer, loss_fn: AbstractLossFunction, relation_weights: List[float]):
        super().__init__(loss_fn, relation_weights)
        if getattr(loss_fn, "native_code", None) is None:
            raise NotImplementedError(f"loss function {type(loss_fn).__name__} has no device code (no CPU fallback)")
        self.model_optimizer = model_optimizer
        self.unpartitioned_optimizers: Dict[str, RowAdagrad] = {}
        self.partitioned_optimizers: Dict[Tuple, RowAdagrad] = {}
        self._native: Optional[_Native] = None          # the context used last
        self._natives: Dict[str, _Native] = {}          # one per operator group
        self._native_key = None
        self.seed = 0
        self._calls = 0
        self._batch_arrays = {}

    # ---- plumbing ------------------------------------------------------------------------------
    def _state_for(self, table: torch.Tensor) -> torch.Tensor:
        for opt in list(self.partitioned_optimizers.values()) + list(self.unpartitioned_optimizers.values()):
            for p in opt.params:
                if p.data_ptr() == table.data_ptr():
                    return opt.sum_for(p)
        raise RuntimeError("no RowAdagrad optimizer registered for an embedding table of this batch")

    def _lr(self) -> float:
        for opt in list(self.partitioned_optimizers.values()) + list(self.unpartitioned_optimizers.values()):
            return opt.lr
        raise RuntimeError("no embedding optimizer registered")

    def _context(self, model: MultiRelationEmbedder, need_batch: int, op_name: Optional[str] = None) -> _Native:
        """The library context of an operator group (one per operator the relations use)."""
        cfg = model.config
        op_name = model.operator_name if op_name is None else op_name
        key = (id(model), cfg.batches_in_flight, cfg.precision)
        if self._native_key != key:
            self._natives = {}
            self._native_key = key
        nat = self._natives.get(op_name)
        if nat is None or nat.max_batch < need_batch:
            margin = getattr(self.loss_fn, "margin", cfg.margin)
            rel_lr = self.model_optimizer.lr if isinstance(self.model_optimizer, AsyncAdagrad) else cfg.relation_lr
            nat = _Native(model, max(cfg.batch_size, need_batch), cfg.batches_in_flight, cfg.precision,
                          self._lr(), rel_lr, margin, loss_code=self.loss_fn.native_code, op_name=op_name)
            self._natives[op_name] = nat
        self._native = nat
        return nat

    def _op_states(self, model, op_name):
        rhs_tab, lhs_tab = model.op_table_for(op_name)
        if rhs_tab is None:
            return None, None
        if not isinstance(self.model_optimizer, AsyncAdagrad):
            raise RuntimeError("the model has operator parameters but model_optimizer is not an AsyncAdagrad over them")
        ar = self.model_optimizer.sum_for(rhs_tab)
        al = None if lhs_tab is None else self.model_optimizer.sum_for(lhs_tab)
        return al, ar

    def train_batches(self, model: MultiRelationEmbedder, lhs: torch.Tensor, rhs: torch.Tensor,
                      rel: Optional[torch.Tensor], batches: List[Tuple[int, int, int]],
                      uniform_lhs: Optional[torch.Tensor] = None, uniform_rhs: Optional[torch.Tensor] = None,
                      want_per_batch: bool = True, weights: Optional[torch.Tensor] = None) -> List[Stats]:
        """Trains the listed (offset, count, relation) batches of the edge arrays.  Edge arrays on
        the CPU are copied by the library (pin them to make the copy asynchronous).  `weights`:
        per-edge weights parallel to the edge arrays (EdgeList.weight), moved to the device here."""
        if not batches:
            return []
        if any(model.relations[0 if model.num_dynamic_rels > 0 else b[2]].all_negs for b in batches):
            raise NotImplementedError("relations with all_negs=True are not trained by torchbiggraph_b200 (the evaluator ranks them)")
        relation_idx = 0 if model.num_dynamic_rels > 0 else batches[0][2]
        op_name = model.operator_of(relation_idx)
        nat = self._context(model, max(b[1] for b in batches), op_name)
        wl, wr = model.tables_for(relation_idx)
        if model.num_dynamic_rels == 0:
            for b in batches:
                if model.tables_for(b[2])[0] is not wl or model.tables_for(b[2])[1] is not wr or model.operator_of(b[2]) != op_name:
                    raise NotImplementedError("batches of one call must read the same pair of tables through the same operator "
                                              "(process_in_batches cuts a list into such runs)")
        al, ar = self._op_states(model, op_name)
        states = (self._state_for(wl), self._state_for(wr), al, ar)
        gl_, gr_ = model.globals_for(relation_idx)
        if gl_ is not None:
            if not isinstance(self.model_optimizer, AsyncAdagrad):
                raise RuntimeError("the model has global embeddings but model_optimizer is not an AsyncAdagrad over them")
            states = states + (self.model_optimizer.sum_for(gl_), self.model_optimizer.sum_for(gr_))
        # the library indexes operator rows and relation weights by the relation's place in its operator group
        dyn = model.num_dynamic_rels > 0
        members = [0] if dyn else model.op_groups[op_name]
        warr = (C.c_float * len(members))(*[self.relation_weights[g] for g in members])
        bucket = nat.bucket(model, relation_idx, states, warr)
        # the descriptor array of a batch list is built once (a trainer is handed the same bucket layout
        # over and over; filling a few hundred ctypes structs costs more host time than launching a wave)
        key = tuple(batches)
        barr = self._batch_arrays.get(key)
        if barr is None:
            barr = (PbgBatch * len(batches))()
            for i, (o, n, r) in enumerate(batches):
                barr[i].offset, barr[i].count, barr[i].rel = o, n, (0 if dyn else model.group_of[r][1])
            if len(self._batch_arrays) > 64:
                self._batch_arrays.clear()
            self._batch_arrays[key] = barr
        sarr = (PbgBatchStats * len(batches))() if want_per_batch else None
        on_host = lhs.device.type == "cpu"
        fn = nat.lib.pbg_train_batches_host if on_host else nat.lib.pbg_train_batches
        for t in (lhs, rhs, rel, uniform_lhs, uniform_rhs):
            if t is not None and (t.dtype != torch.long or not t.is_contiguous() or (t.device.type == "cpu") != on_host):
                raise TypeError("edge and uniform-id arrays must be contiguous int64, all on the host or all on the device")
        self._calls += 1
        if weights is not None:
            if weights.shape[0] != lhs.shape[0]:
                raise ValueError("one weight per edge is needed")
            weights = weights.to(device=model.device, dtype=torch.float32).contiguous()     # kept alive until the call returns
            check(nat.lib.pbg_set_edge_weights(nat.ctx, _ptr(weights)), nat.ctx)
        check(fn(nat.ctx, C.byref(bucket), _ptr(lhs), _ptr(rhs), _ptr(rel), lhs.shape[0], barr, len(batches),
                 _ptr(uniform_lhs), _ptr(uniform_rhs), self.seed + self._calls, sarr), nat.ctx)
        if not want_per_batch:
            return []
        return [Stats(loss=float(s.loss), reg=float(s.reg), violators_lhs=int(s.violators_lhs),
                      violators_rhs=int(s.violators_rhs), count=int(s.count)) for s in sarr]

    def read_stats(self) -> Stats:
        s = PbgBatchStats()
        check(self._native.lib.pbg_read_stats(self._native.ctx, C.byref(s)), self._native.ctx)
        return Stats(loss=float(s.loss), reg=float(s.reg), violators_lhs=int(s.violators_lhs),
                     violators_rhs=int(s.violators_rhs), count=int(s.count))

    # ---- the reference interface ---------------------------------------------------------------
    def _process_one_batch(self, model: MultiRelationEmbedder, batch_edges: EdgeList,
                           uniform_lhs=None, uniform_rhs=None) -> Stats:
        dyn = model.num_dynamic_rels > 0
        if dyn and batch_edges.has_scalar_relation_type():
            raise TypeError("Need relation for each positive pair")
        if not dyn and not batch_edges.has_scalar_relation_type():
            raise TypeError("All positive pairs must come from the same relation")
        n = len(batch_edges)
        if n == 0:
            return Stats(loss=0.0, reg=0.0, violators_lhs=0, violators_rhs=0, count=0)
        dev = model.device
        lhs = batch_edges.lhs.to_tensor().to(dev).contiguous()
        rhs = batch_edges.rhs.to_tensor().to(dev).contiguous()
        rel = batch_edges.rel.to(dev).contiguous() if dyn else None
        r = 0 if dyn else batch_edges.get_relation_type_as_scalar()
        nat = self._context(model, n, model.operator_of(r))
        ul = None if uniform_lhs is None else nat._uniform(uniform_lhs, dev)
        ur = None if uniform_rhs is None else nat._uniform(uniform_rhs, dev)
        wgt = torch.as_tensor(batch_edges.weight) if batch_edges.has_weight() else None
        return self.train_batches(model, lhs, rhs, rel, [(0, n, r)], ul, ur, weights=wgt)[0]

    def process_one_batch(self, model, batch_edges, uniform_lhs=None, uniform_rhs=None) -> Stats:
        if self.overrides is not None:
            raise NotImplementedError("model overrides are not supported by torchbiggraph_b200")
        return self._process_one_batch(model, batch_edges, uniform_lhs, uniform_rhs)


class B200RankingEvaluator(AbstractBatchProcessor):
    """RankingEvaluator (torchbiggraph/eval.py:43-81) on the device: per batch the forward pass, the
    rank of every positive among its negatives on both sides, and Stats(loss, pos_rank, mrr, r1,
    r10, r50, auc, count) as sums the caller averages with Stats.average().  `overrides` takes the
    two keys the reference's evaluator overrides on the model (eval.py:165-172): num_batch_negs and
    num_uniform_negs."""

    def __init__(self, loss_fn: AbstractLossFunction, relation_weights: List[float], overrides=None):
        super().__init__(loss_fn, relation_weights, None)
        if getattr(loss_fn, "native_code", None) is None:
            raise NotImplementedError(f"loss function {type(loss_fn).__name__} has no device code (no CPU fallback)")
        unknown = set(overrides or {}) - {"num_batch_negs", "num_uniform_negs"}
        if unknown:
            raise NotImplementedError(f"model overrides {sorted(unknown)} are not supported by torchbiggraph_b200")
        self.neg_overrides = dict(overrides or {})
        self._native: Optional[_Native] = None
        self._natives: Dict[str, _Native] = {}
        self._key = None
        self.seed = 0
        self._calls = 0

    def _context(self, model, need_batch, op_name=None):
        op_name = model.operator_name if op_name is None else op_name
        key = (id(model),)
        if self._key != key:
            self._natives = {}
            self._key = key
        nat = self._natives.get(op_name)
        if nat is None or nat.max_batch < need_batch:
            cfg = model.config
            nat = _Native(model, max(cfg.batch_size, need_batch), 1, cfg.precision, cfg.lr, cfg.relation_lr,
                          getattr(self.loss_fn, "margin", cfg.margin), loss_code=self.loss_fn.native_code,
                          num_batch_negs=self.neg_overrides.get("num_batch_negs"),
                          num_uniform_negs=self.neg_overrides.get("num_uniform_negs"), op_name=op_name)
            self._natives[op_name] = nat
        self._native = nat
        return nat

    def _process_one_batch(self, model: MultiRelationEmbedder, batch_edges: EdgeList, uniform_lhs=None, uniform_rhs=None) -> Stats:
        dyn = model.num_dynamic_rels > 0
        if dyn and batch_edges.has_scalar_relation_type():
            raise TypeError("Need relation for each positive pair")
        if not dyn and not batch_edges.has_scalar_relation_type():
            raise TypeError("All positive pairs must come from the same relation")
        n = len(batch_edges)
        if n == 0:
            return Stats(loss=0.0, pos_rank=0.0, mrr=0.0, r1=0.0, r10=0.0, r50=0.0, auc=0.0, count=0)
        dev = model.device
        r = 0 if dyn else batch_edges.get_relation_type_as_scalar()
        op_name = model.operator_of(r)
        nat = self._context(model, n, op_name)
        lhs = batch_edges.lhs.to_tensor().to(dev).contiguous()
        rhs = batch_edges.rhs.to_tensor().to(dev).contiguous()
        rel = batch_edges.rel.to(dev).contiguous() if dyn else None
        ul = None if uniform_lhs is None else nat._uniform(uniform_lhs, dev)
        ur = None if uniform_rhs is None else nat._uniform(uniform_rhs, dev)
        members = [0] if dyn else model.op_groups[op_name]
        warr = (C.c_float * len(members))(*[self.relation_weights[g] for g in members])
        bucket = nat.bucket(model, r, None, warr)
        full_r, r = r, (0 if dyn else model.group_of[r][1])     # the library's relation index is local to the operator group
        out = _lib.PbgEvalStats()
        self._calls += 1
        if batch_edges.has_weight():                 # the evaluator's loss is weighted like the trainer's (eval.py:55-56)
            wgt = torch.as_tensor(batch_edges.weight).to(device=dev, dtype=torch.float32).contiguous()
            check(nat.lib.pbg_set_edge_weights(nat.ctx, _ptr(wgt)), nat.ctx)
        if model.relations[0 if dyn else full_r].all_negs:
            # every entity of a side's table is a negative (model.py:582-617): ranks among the whole partition
            st = nat.lib.pbg_eval_batch_all_negs(nat.ctx, C.byref(bucket), _ptr(lhs), _ptr(rhs), _ptr(rel), n, r,
                                                 self.seed + self._calls, C.byref(out))
            if st == _lib.PBG_ERR_UNSUPPORTED:
                raise NotImplementedError(nat.lib.pbg_last_error(nat.ctx).decode())
            check(st, nat.ctx)
        else:
            check(nat.lib.pbg_eval_batch(nat.ctx, C.byref(bucket), _ptr(lhs), _ptr(rhs), _ptr(rel), n, r, _ptr(ul), _ptr(ur),
                                         self.seed + self._calls, C.byref(out)), nat.ctx)
        return Stats(loss=float(out.loss), pos_rank=out.pos_rank, mrr=out.mrr, r1=out.r1, r10=out.r10, r50=out.r50,
                     auc=out.auc, count=int(out.count))

    def process_one_batch(self, model, batch_edges, uniform_lhs=None, uniform_rhs=None) -> Stats:
        return self._process_one_batch(model, batch_edges, uniform_lhs, uniform_rhs)


def _batches_group_by_relation(rel_sorted: torch.Tensor, batch_size: int, generator=None):
    """Batch descriptors over edges sorted by relation: repeatedly pick a relation with
    probability proportional to its remaining edges and emit its next <= batch_size edges
    (batching.py:58-79)."""
    rels, counts = torch.unique_consecutive(rel_sorted, return_counts=True)
    starts = torch.cumsum(counts, 0) - counts
    left = counts.clone()
    out = []
    while int(left.sum()) > 0:
        idx = int(torch.multinomial(left.float(), 1, generator=generator))
        off = int(starts[idx] + counts[idx] - left[idx])
        n = min(batch_size, int(left[idx]))
        out.append((off, n, int(rels[idx])))
        left[idx] -= n
    return out


def process_in_batches(batch_size: int, model: MultiRelationEmbedder, batch_processor: B200Trainer,
                       edges: EdgeList, indices: Optional[torch.Tensor] = None, delay: float = 0.0) -> Stats:
    """torchbiggraph/batching.py:91-125 with the batch loop moved onto the device.  Per-edge weights
    (EdgeList.weight) travel with the edges.  With standard relations the batches come in the
    reference's order (batching.py:58-79); consecutive batches that read the same pair of embedding
    tables go to the library in one call, so relations over different entity types simply cut the
    list into more calls."""
    if indices is not None:
        edges = edges[indices]
    if delay > 0:
        time.sleep(delay)
    n = len(edges)
    if n == 0:
        return Stats(count=0)
    lhs, rhs = edges.lhs.to_tensor().contiguous(), edges.rhs.to_tensor().contiguous()
    weights = torch.as_tensor(edges.weight) if edges.has_weight() else None
    if model.num_dynamic_rels > 0:
        rel = edges.get_relation_type_as_vector().contiguous()
        batches = [(o, min(batch_size, n - o), 0) for o in range(0, n, batch_size)]
    elif edges.has_scalar_relation_type():
        rel = None
        r = edges.get_relation_type_as_scalar()
        batches = [(o, min(batch_size, n - o), r) for o in range(0, n, batch_size)]
    else:
        order = torch.argsort(edges.rel, stable=True)
        lhs, rhs, rel_sorted = lhs[order].contiguous(), rhs[order].contiguous(), edges.rel[order]
        if weights is not None:
            weights = weights[order.to(weights.device)]
        rel = None
        batches = _batches_group_by_relation(rel_sorted.cpu(), batch_size)
    stats: List[Stats] = []
    for run in _runs_by_table_pair(model, batches):
        stats.extend(batch_processor.train_batches(model, lhs, rhs, rel, run, weights=weights))
    return Stats.sum(stats)


def _runs_by_table_pair(model: MultiRelationEmbedder, batches):
    """Cuts a batch list into maximal runs of consecutive batches whose relations read the same
    (lhs table, rhs table) pair through the same operator; one library call trains one run."""
    if model.num_dynamic_rels > 0 or not batches:
        return [batches] if batches else []
    runs, cur, cur_key = [], [], None
    for b in batches:
        wl, wr = model.tables_for(b[2])
        key = (wl.data_ptr(), wr.data_ptr(), model.operator_of(b[2]))
        if cur and key != cur_key:
            runs.append(cur)
            cur = []
        cur_key = key
        cur.append(b)
    runs.append(cur)
    return runs
