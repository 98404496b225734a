"""The subset of the reference's ConfigSchema (torchbiggraph/config.py:40-536) that the training
step reads, with the same key names and meanings.  `from_reference` accepts the reference's own
ConfigSchema object (duck-typed) so that a stock config file drives this path unchanged.

Keys with no device code are refused where the trainer is built (NotImplementedError), never
silently ignored: bias, half_precision, featurized entities, per-entity dimensions.  Relations with
all_negs=True are ranked by the evaluator against every entity of a side (B200RankingEvaluator); the
trainer refuses them, as the reference's GPU trainer has no use for them either."""
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class EntitySchema:
    num_partitions: int = 1
    featurized: bool = False
    dimension: Optional[int] = None


@dataclass
class RelationSchema:
    name: str
    lhs: str
    rhs: str
    weight: float = 1.0
    operator: str = "none"
    all_negs: bool = False


@dataclass
class ConfigSchema:
    entities: Dict[str, EntitySchema]
    relations: List[RelationSchema]
    dimension: int
    comparator: str = "cos"
    loss_fn: str = "ranking"
    margin: float = 0.1
    lr: float = 1e-2
    relation_lr: Optional[float] = None
    batch_size: int = 1000
    num_batch_negs: int = 50
    num_uniform_negs: int = 50
    disable_lhs_negs: bool = False
    disable_rhs_negs: bool = False
    dynamic_relations: bool = False
    init_scale: float = 1e-3
    # one trained vector per entity type added to every embedding of the type (model.py:433-441,
    # 486-492).  The reference's default is True; here a config built by hand starts without,
    # from_reference() copies whatever the reference config says.
    global_emb: bool = False
    # keys the reference has and this path refuses when set
    bias: bool = False
    max_norm: Optional[float] = None
    regularization_coef: float = 0.0    # N3 regularizer weight (regularizers.py:51-97)
    regularizer: str = "N3"
    half_precision: bool = False
    # keys of this implementation
    precision: str = "fp32"        # "fp32" | "tf32x3" | "tf32" | "bf16x6" | "bf16x3": arithmetic of the contractions
    batches_in_flight: int = 1     # 1 = the reference's sequential batches
    num_dynamic_rels: int = 0      # count of relation types when dynamic_relations (the reference
                                   # reads it from dynamic_rel_count.txt, model.py:866-870)

    @classmethod
    def from_reference(cls, cfg, num_dynamic_rels: int = 0, **overrides) -> "ConfigSchema":
        ents = {k: EntitySchema(v.num_partitions, v.featurized, getattr(v, "dimension", None))
                for k, v in cfg.entities.items()}
        rels = [RelationSchema(r.name, r.lhs, r.rhs, r.weight, r.operator, r.all_negs) for r in cfg.relations]
        kw = dict(entities=ents, relations=rels, dimension=cfg.dimension, num_dynamic_rels=num_dynamic_rels)
        for k in ("comparator", "loss_fn", "margin", "lr", "relation_lr", "batch_size", "num_batch_negs",
                  "num_uniform_negs", "disable_lhs_negs", "disable_rhs_negs", "dynamic_relations", "init_scale",
                  "global_emb", "bias", "max_norm", "regularization_coef", "regularizer", "half_precision"):
            if hasattr(cfg, k):
                kw[k] = getattr(cfg, k)
        kw.update(overrides)
        return cls(**kw)

    def check_supported(self) -> None:
        bad = []
        if self.global_emb and self.dynamic_relations:
            raise RuntimeError("Cannot have global embs with dynamic rels")          # model.py:488-489
        if self.bias:
            bad.append("bias=True")
        if self.max_norm is not None and self.max_norm <= 0:
            raise ValueError("max_norm must be positive")
        if self.regularization_coef != 0 and self.regularizer != "N3":
            bad.append(f"regularizer '{self.regularizer}'")
        if self.regularization_coef != 0 and any(r.operator in ("linear", "affine") for r in self.relations):
            bad.append("regularization with linear / affine operators (the reference has none either, operators.py:39-40)")
        if self.half_precision:
            bad.append("half_precision=True")
        if any(e.featurized for e in self.entities.values()):
            bad.append("featurized entities")
        if any(e.dimension not in (None, self.dimension) for e in self.entities.values()):
            bad.append("per-entity dimensions")
        if bad:
            raise NotImplementedError(
                "torchbiggraph_b200 has no device code for: " + ", ".join(bad) + " (and no CPU fallback)")
        if self.num_batch_negs > 0 and self.batch_size % self.num_batch_negs != 0:
            raise RuntimeError("Batch size (%d) must be a multiple of num_batch_negs (%d)"
                               % (self.batch_size, self.num_batch_negs))   # model.py:879-883
        if self.dynamic_relations and len(self.relations) != 1:
            raise RuntimeError("Dynamic relations are enabled, so there should only be one entry in "
                               "config.relations with config for all relations.")   # model.py:861-865
