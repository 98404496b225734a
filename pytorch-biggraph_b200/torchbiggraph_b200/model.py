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
        op_name = config.relations[0].operator
        if config.dynamic_relations and op_name in ("linear", "affine"):
            raise NotImplementedError(f"operator '{op_name}' with dynamic relations has no device code (and no CPU fallback)")
        self.operator_name = op_name
        D = config.dimension
        rows = self.num_dynamic_rels if config.dynamic_relations else len(config.relations)
        self.num_rels = rows
        registry = DYNAMIC_OPERATORS if config.dynamic_relations else OPERATORS
        op_cls = registry.get_class(op_name)
        if op_cls.native_code is None:
            raise NotImplementedError(f"operator '{op_name}' has no device code")
        proto = op_cls(D, rows) if config.dynamic_relations else op_cls(D)
        init = proto.init_table(rows)
        # one [num_rels, width] table per side (width = dim; dim*dim (+dim) for linear (affine));
        # standard relations only have the rhs one
        self.rhs_op_table: Optional[torch.Tensor] = None if init is None else init.to(self.device)
        self.lhs_op_table: Optional[torch.Tensor] = (
            None if init is None or not config.dynamic_relations else init.clone().to(self.device))
        self.lhs_operators: List[Optional[object]] = []
        self.rhs_operators: List[Optional[object]] = []
        for i, _ in enumerate(config.relations):
            if init is None:
                self.lhs_operators.append(None)
                self.rhs_operators.append(None)
                continue
            r = op_cls(D, rows) if config.dynamic_relations else op_cls(D)
            r.table = self.rhs_op_table if config.dynamic_relations else self.rhs_op_table[i:i + 1]
            self.rhs_operators.append(r)
            if config.dynamic_relations:
                l = op_cls(D, rows)
                l.table = self.lhs_op_table
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
        return [t for t in (self.rhs_op_table, self.lhs_op_table) if t is not None] + glob

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
        if self._scorer is None:
            self._scorer = _Native(self, max_batch=max(self.config.batch_size, len(edges)), k=1,
                                   precision=self.config.precision, lr=self.config.lr,
                                   relation_lr=self.config.relation_lr, margin=self.config.margin)
        return self._scorer.score(self, edges, uniform_lhs, uniform_rhs, seed)

    __call__ = forward


def make_model(config: ConfigSchema, device="cuda") -> MultiRelationEmbedder:
    """torchbiggraph/model.py:859-924."""
    return MultiRelationEmbedder(config, torch.device(device))
