"""Device-resident model state for the training step, with MultiRelationEmbedder's surface
(torchbiggraph/model.py:366-476): set_embeddings / clear_all_embeddings, lhs_operators /
rhs_operators, num_dynamic_rels, and forward(edges) -> Scores.

Nothing here computes: the tensors are handed to the native library by pointer."""
from typing import Dict, List, NamedTuple, Optional

import torch

from .config import ConfigSchema
from .registries import COMPARATORS, DYNAMIC_OPERATORS, OPERATORS
from .types import EdgeList, Side


class Scores(NamedTuple):          # torchbiggraph/model.py:359-363
    lhs_pos: torch.Tensor
    rhs_pos: torch.Tensor
    lhs_neg: torch.Tensor
    rhs_neg: torch.Tensor


class MultiRelationEmbedder:
    EMB_PREFIX = "emb_"

    def __init__(self, config: ConfigSchema, device: torch.device):
        config.check_supported()
        self.config = config
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.relations = config.relations
        self.entities = config.entities
        self.num_dynamic_rels = config.num_dynamic_rels if config.dynamic_relations else 0
        if config.dynamic_relations and self.num_dynamic_rels <= 0:
            raise RuntimeError("Dynamic relations are enabled, so the count of relation types is needed "
                               "(config.num_dynamic_rels)")
        self.num_batch_negs = config.num_batch_negs
        self.num_uniform_negs = config.num_uniform_negs
        self.disable_lhs_negs = config.disable_lhs_negs
        self.disable_rhs_negs = config.disable_rhs_negs
        self.comparator = COMPARATORS.get_class(config.comparator)()
        if self.comparator.native_code is None:
            raise NotImplementedError(f"comparator '{config.comparator}' has no device code")
        D = config.dimension
        dyn = config.dynamic_relations
        registry = DYNAMIC_OPERATORS if dyn else OPERATORS
        # Relations are grouped by operator (standard relations may mix them, model.py:368-476 builds one operator
        # per relation): each group has its own [relations of the group, width] parameter table (width = dim;
        # dim * dim (+ dim) for linear (affine)), and a batch is trained by the library context of its group.
        # With dynamic relations there is one group and a second table for the lhs-side operators.
        self.op_groups: Dict[str, List[int]] = {}
        for i, r in enumerate(config.relations):
            self.op_groups.setdefault(r.operator, []).append(i)
        self.group_of: List[tuple] = [(r.operator, self.op_groups[r.operator].index(i)) for i, r in enumerate(config.relations)]
        self.op_tables: Dict[str, Optional[torch.Tensor]] = {}
        self.lhs_op_tables: Dict[str, Optional[torch.Tensor]] = {}
        protos = {}
        for op_name, members in self.op_groups.items():
            if dyn and op_name in ("linear", "affine"):
                raise NotImplementedError(f"operator '{op_name}' with dynamic relations has no device code (and no CPU fallback)")
            op_cls = registry.get_class(op_name)
            if op_cls.native_code is None:
                raise NotImplementedError(f"operator '{op_name}' has no device code")
            rows = self.num_dynamic_rels if dyn else len(members)
            proto = op_cls(D, rows) if dyn else op_cls(D)
            init = proto.init_table(rows)
            protos[op_name] = (op_cls, rows, init)
            self.op_tables[op_name] = None if init is None else init.to(self.device)
            self.lhs_op_tables[op_name] = None if init is None or not dyn else init.clone().to(self.device)
        # the single-operator case keeps its plain attributes
        self.operator_name = config.relations[0].operator
        self.num_rels = self.num_dynamic_rels if dyn else len(self.op_groups[self.operator_name])
        self.rhs_op_table: Optional[torch.Tensor] = self.op_tables[self.operator_name] if len(self.op_groups) == 1 else None
        self.lhs_op_table: Optional[torch.Tensor] = self.lhs_op_tables[self.operator_name] if len(self.op_groups) == 1 else None
        self.lhs_operators: List[Optional[object]] = []
        self.rhs_operators: List[Optional[object]] = []
        for i, rel in enumerate(config.relations):
            op_cls, rows, init = protos[rel.operator]
            if init is None:
                self.lhs_operators.append(None)
                self.rhs_operators.append(None)
                continue
            local = self.group_of[i][1]
            r = op_cls(D, rows) if dyn else op_cls(D)
            r.table = self.op_tables[rel.operator] if dyn else self.op_tables[rel.operator][local:local + 1]
            self.rhs_operators.append(r)
            if dyn:
                l = op_cls(D, rows)
                l.table = self.lhs_op_tables[rel.operator]
                self.lhs_operators.append(l)
            else:
                self.lhs_operators.append(None)
        self.lhs_embs: Dict[str, torch.Tensor] = {}
        self.rhs_embs: Dict[str, torch.Tensor] = {}
        # config.global_emb: one [dimension] vector per entity type, initialised to zero and trained
        # by the model optimizer (model.py:433-441)
        self.global_embs: Optional[Dict[str, torch.Tensor]] = None
        if config.global_emb:
            self.global_embs = {self.EMB_PREFIX + e: torch.zeros(D, device=self.device) for e in config.entities}
        self._scorer = None

    # ---- parameters other than embeddings: what model_optimizer steps (train_cpu.py:468) ----
    def parameters(self):
        glob = [] if self.global_embs is None else list(self.global_embs.values())
        tabs = [t for t in self.op_tables.values() if t is not None] + [t for t in self.lhs_op_tables.values() if t is not None]
        return tabs + glob

    def operator_of(self, relation_idx: int) -> str:
        return self.relations[relation_idx].operator

    def op_table_for(self, op_name: str):
        """(rhs-side table, lhs-side table) of an operator group."""
        return self.op_tables[op_name], self.lhs_op_tables[op_name]

    def globals_for(self, relation_idx: int):
        """(lhs, rhs) global embedding of the relation's entity types, or (None, None)."""
        if self.global_embs is None:
            return None, None
        rel = self.relations[relation_idx]
        return self.global_embs[self.EMB_PREFIX + rel.lhs], self.global_embs[self.EMB_PREFIX + rel.rhs]

    def set_embeddings(self, entity: str, side: Side, weights: torch.Tensor) -> None:
        if weights.dim() != 2 or weights.shape[1] != self.config.dimension or weights.dtype != torch.float32:
            raise TypeError("embeddings must be float32 [rows, dimension]")
        if weights.device != self.device or not weights.is_contiguous():
            raise ValueError(f"embeddings must be contiguous tensors on {self.device} (they are trained in place)")
        side.pick(self.lhs_embs, self.rhs_embs)[self.EMB_PREFIX + entity] = weights

    def clear_all_embeddings(self) -> None:
        self.lhs_embs.clear()
        self.rhs_embs.clear()

    def tables_for(self, relation_idx: int):
        rel = self.relations[relation_idx]
        return self.lhs_embs[self.EMB_PREFIX + rel.lhs], self.rhs_embs[self.EMB_PREFIX + rel.rhs]

    def forward(self, edges: EdgeList, uniform_lhs=None, uniform_rhs=None, seed: int = 0) -> Scores:
        """Scores of one batch (model.py:624-762) computed by the library's forward kernels.
        uniform_lhs / uniform_rhs: optional int64 [chunks, num_uniform_negs] row ids."""
        from .trainer import _Native
        op_name = self.operator_name if self.num_dynamic_rels > 0 or not edges.has_scalar_relation_type() \
            else self.operator_of(edges.get_relation_type_as_scalar())
        if self._scorer is None:
            self._scorer = {}
        if op_name not in self._scorer or self._scorer[op_name].max_batch < len(edges):
            self._scorer[op_name] = _Native(self, max_batch=max(self.config.batch_size, len(edges)), k=1,
                                            precision=self.config.precision, lr=self.config.lr,
                                            relation_lr=self.config.relation_lr, margin=self.config.margin, op_name=op_name)
        return self._scorer[op_name].score(self, edges, uniform_lhs, uniform_rhs, seed)

    __call__ = forward


def make_model(config: ConfigSchema, device="cuda") -> MultiRelationEmbedder:
    """torchbiggraph/model.py:859-924."""
    return MultiRelationEmbedder(config, torch.device(device))
