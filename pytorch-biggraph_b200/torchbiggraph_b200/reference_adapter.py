"""The reference-side binding: a batch processor that PyTorch-BigGraph's own `train()` accepts as
`trainer=` (torchbiggraph/train.py:30-43) and that trains the REFERENCE's `MultiRelationEmbedder` through
libpbg_b200.so.

    from torchbiggraph_b200.reference_adapter import make_reference_trainer
    trainer = make_reference_trainer(config, model)      # a torchbiggraph AbstractBatchProcessor
    train(config, model=model, trainer=trainer)

It needs the `torchbiggraph` package importable (it subclasses the reference's AbstractBatchProcessor,
torchbiggraph/batching.py:128-165) and nothing else of this package's model classes: the tensors handed to
the library are the reference's own parameters --

  * embedding tables: `model.lhs_embs["emb_<entity>"].weight` (SimpleEmbedding, torchbiggraph/model.py:51-61),
    trained in place;
  * RowAdagrad state: the `sum` vector of the reference optimizer the coordinator registered in
    `trainer.partitioned_optimizers / unpartitioned_optimizers` (torchbiggraph/row_adagrad.py:34-40,
    train_cpu.py:816-842), so `optimizer.state_dict()` and the checkpoint files are what they always were;
  * operator parameters: the library wants one [num_rels, dim] table per side, the reference keeps one
    nn.Parameter per operator (and `real` / `imag` halves for complex_diagonal, torchbiggraph/operators.py:129-157).
    `OperatorTables` allocates the packed tables once and re-points the reference's parameters (and their
    AsyncAdagrad `sum` tensors) at views of them: both sides then read and write the same memory.
"""
import ctypes as C
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib
from ._lib import PbgBatch, PbgBatchStats, PbgBucket, PbgConfig, check

_PARAM_NAMES = {
    "diagonal": (("diagonal",), ("diagonals",)),
    "translation": (("translation",), ("translations",)),
    "complex_diagonal": (("real", "imag"), ("real", "imag")),
}


class OperatorTables:
    """Packed [num_rels, dim] operator tables (and AsyncAdagrad accumulators) aliased by the reference's parameters."""

    def __init__(self, model, model_optimizer, op_name: str, dim: int, dynamic: bool):
        self.rhs = self.lhs = self.rhs_acc = self.lhs_acc = None
        if op_name == "none":
            return
        if op_name not in _PARAM_NAMES:
            raise NotImplementedError(f"operator '{op_name}' is not bound by the reference adapter (use torchbiggraph_b200's own model for linear / affine)")
        names = _PARAM_NAMES[op_name][1 if dynamic else 0]
        self.rhs, self.rhs_acc = self._pack(model.rhs_operators, model_optimizer, names, dim, dynamic)
        if dynamic:
            self.lhs, self.lhs_acc = self._pack(model.lhs_operators, model_optimizer, names, dim, dynamic)

    @staticmethod
    def _pack(ops, optimizer, names, dim, dynamic):
        ops = [o for o in ops if o is not None]
        first = getattr(ops[0], names[0])
        rows = first.shape[0] if dynamic else len(ops)
        table = torch.empty(rows, dim, device=first.device, dtype=torch.float32)
        acc = torch.zeros_like(table)
        width = dim // len(names)
        for i, o in enumerate(ops):
            for j, n in enumerate(names):
                p = getattr(o, n)
                cols = slice(j * width, (j + 1) * width)
                view = table[:, cols] if dynamic else table[i, cols]
                view.copy_(p.data)
                p.data = view                                   # the reference's parameter now lives inside the table
                state = optimizer.state[p] if optimizer is not None and p in optimizer.state else None
                if state is not None and "sum" in state:
                    aview = acc[:, cols] if dynamic else acc[i, cols]
                    aview.copy_(state["sum"])
                    state["sum"] = aview
        return table, acc


def _native_config(config, model, loss_code: int, margin: float, precision: str, batches_in_flight: int) -> PbgConfig:
    dyn = bool(config.dynamic_relations)
    ops = {r.operator for r in config.relations}
    if len(ops) != 1:
        raise NotImplementedError("different operators on different relations are not bound by the reference adapter")
    c = PbgConfig()
    c.dim = config.dimension
    c.op = _lib.OPERATOR_CODES[next(iter(ops))]
    c.comparator = _lib.COMPARATOR_CODES[config.comparator]
    c.loss = loss_code
    c.dynamic_relations = int(dyn)
    c.num_rels = model.num_dynamic_rels if dyn else len(config.relations)
    c.num_batch_negs = config.num_batch_negs
    c.num_uniform_negs = config.num_uniform_negs
    c.disable_lhs_negs = int(config.disable_lhs_negs)
    c.disable_rhs_negs = int(config.disable_rhs_negs)
    c.precision = _lib.PRECISION_CODES[precision]
    c.max_batch_size = config.batch_size
    c.batches_in_flight = batches_in_flight
    c.margin = margin
    c.lr = config.lr
    c.relation_lr = config.lr if config.relation_lr is None else config.relation_lr
    c.regularization_coef = float(config.regularization_coef)
    c.max_norm = float(config.max_norm or 0.0)
    for key in ("bias", "half_precision", "global_emb"):
        if getattr(config, key, False):
            raise NotImplementedError(f"config.{key} is not bound by the reference adapter")
    return c


def make_reference_trainer(config, model, model_optimizer=None, loss_fn=None, relation_weights=None,
                           precision: str = "bf16x6", batches_in_flight: int = 1):
    """Builds the batch processor for the reference's `train(config, model=model, trainer=...)`.  Call it where the
    reference builds its own Trainer: after the model exists and BEFORE embeddings are attached
    (torchbiggraph/train_cpu.py:463-472), so that `model.parameters()` holds the operator parameters only."""
    from torchbiggraph.batching import AbstractBatchProcessor
    from torchbiggraph.losses import LOSS_FUNCTIONS
    from torchbiggraph.stats import Stats
    from torchbiggraph.train_cpu import make_optimizer

    if model_optimizer is None:
        model_optimizer = make_optimizer(config, model.parameters(), False)
    if loss_fn is None:
        loss_fn = LOSS_FUNCTIONS.get_class(config.loss_fn)(margin=config.margin)
    if relation_weights is None:
        relation_weights = [r.weight for r in config.relations]
    loss_code = _lib.LOSS_CODES.get(config.loss_fn)
    if loss_code is None:
        raise NotImplementedError(f"loss function '{config.loss_fn}' has no device code")

    class ReferenceB200Trainer(AbstractBatchProcessor):
        """Trainer (torchbiggraph/train_cpu.py:74-112) whose step runs in libpbg_b200.so."""

        def __init__(self):
            super().__init__(loss_fn, relation_weights)
            self.model_optimizer = model_optimizer
            self.unpartitioned_optimizers: Dict = {}
            self.partitioned_optimizers: Dict = {}
            self.lib = _lib.lib()
            self.ctx = None
            self.tables: Optional[OperatorTables] = None
            self.seed = 0
            self.calls = 0
            self.native_config = _native_config(config, model, loss_code, getattr(loss_fn, "margin", config.margin),
                                                precision, batches_in_flight)

        def _ensure(self, device: torch.device):
            if self.tables is None:
                self.tables = OperatorTables(model, self.model_optimizer, config.relations[0].operator, config.dimension,
                                             bool(config.dynamic_relations))
            if self.ctx is None:
                ctx = C.c_void_p()
                idx = device.index if device.index is not None else torch.cuda.current_device()
                st = self.lib.pbg_create(C.byref(self.native_config), idx,
                                         C.c_void_p(torch.cuda.current_stream(idx).cuda_stream), C.byref(ctx))
                if st != 0:
                    msg = self.lib.pbg_last_error(ctx).decode() if ctx else ""
                    self.lib.pbg_destroy(ctx)
                    if st == _lib.PBG_ERR_UNSUPPORTED:
                        raise NotImplementedError(msg)
                    raise _lib.PbgError(st, msg)
                self.ctx = ctx

        def _sum_of(self, weight: torch.Tensor) -> torch.Tensor:
            for opt in list(self.partitioned_optimizers.values()) + list(self.unpartitioned_optimizers.values()):
                for group in opt.param_groups:
                    for p in group["params"]:
                        if p.data_ptr() == weight.data_ptr():
                            return opt.state[p]["sum"]
            raise RuntimeError("no RowAdagrad optimizer registered for an embedding table of this batch")

        def bucket_for(self, rel_idx: int) -> Tuple[PbgBucket, object]:
            rel = config.relations[rel_idx]
            lhs_w = model.lhs_embs[model.EMB_PREFIX + rel.lhs].weight
            rhs_w = model.rhs_embs[model.EMB_PREFIX + rel.rhs].weight
            if lhs_w.device.type != "cuda":
                raise RuntimeError("torchbiggraph_b200 runs on a CUDA device only (no CPU fallback)")
            self._ensure(lhs_w.device)
            b = PbgBucket()
            b.lhs_emb, b.lhs_rows, b.lhs_state = lhs_w.data_ptr(), lhs_w.shape[0], self._sum_of(lhs_w).data_ptr()
            b.rhs_emb, b.rhs_rows, b.rhs_state = rhs_w.data_ptr(), rhs_w.shape[0], self._sum_of(rhs_w).data_ptr()
            t = self.tables
            if t.rhs is not None:
                b.rhs_op, b.rhs_op_state = t.rhs.data_ptr(), t.rhs_acc.data_ptr()
            if t.lhs is not None:
                b.lhs_op, b.lhs_op_state = t.lhs.data_ptr(), t.lhs_acc.data_ptr()
            weights = (C.c_float * len(self.relation_weights))(*self.relation_weights)
            b.relation_weights = weights
            return b, weights

        def _process_one_batch(self, model_, batch_edges):
            n = len(batch_edges)
            if n == 0:
                return Stats(loss=0.0, reg=0.0, violators_lhs=0, violators_rhs=0, count=0)
            dyn = bool(config.dynamic_relations)
            r = 0 if dyn else batch_edges.get_relation_type_as_scalar()
            bucket, keep = self.bucket_for(r)
            dev = model_.lhs_embs[model_.EMB_PREFIX + config.relations[r].lhs].weight.device
            lhs = batch_edges.lhs.to_tensor().to(dev).contiguous()
            rhs = batch_edges.rhs.to_tensor().to(dev).contiguous()
            rel = batch_edges.rel.to(dev).contiguous() if dyn else None
            if batch_edges.has_weight():
                wgt = batch_edges.weight.to(device=dev, dtype=torch.float32).contiguous()
                check(self.lib.pbg_set_edge_weights(self.ctx, C.c_void_p(wgt.data_ptr())), self.ctx)
            batch = PbgBatch(offset=0, count=n, rel=r)
            out = PbgBatchStats()
            self.calls += 1
            torch.cuda.current_stream(dev).synchronize()
            check(self.lib.pbg_train_batches(self.ctx, C.byref(bucket), C.c_void_p(lhs.data_ptr()), C.c_void_p(rhs.data_ptr()),
                                             None if rel is None else C.c_void_p(rel.data_ptr()), n, C.byref(batch), 1,
                                             None, None, self.seed + self.calls, C.byref(out)), self.ctx)
            return Stats(loss=float(out.loss), reg=float(out.reg), violators_lhs=int(out.violators_lhs),
                         violators_rhs=int(out.violators_rhs), count=int(out.count))

        def __del__(self):
            if getattr(self, "ctx", None):
                self.lib.pbg_destroy(self.ctx)
                self.ctx = None

    return ReferenceB200Trainer()
