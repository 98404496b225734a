"""torchbiggraph_b200: PyTorch-BigGraph's per-bucket training step on B200 (sm_100a).

Host-side mirror of the reference interface for this path (registries, config keys, EdgeList,
Stats, Trainer, process_in_batches) over the C-ABI library libpbg_b200.so."""
from .config import ConfigSchema, EntitySchema, RelationSchema
from .model import MultiRelationEmbedder, Scores, make_model
from .plugin import PluginRegistry
from .registries import COMPARATORS, DYNAMIC_OPERATORS, LOSS_FUNCTIONS, OPERATORS
from .row_adagrad import AsyncAdagrad, RowAdagrad, make_optimizer
from .trainer import AbstractBatchProcessor, B200RankingEvaluator, B200Trainer, process_in_batches
from .types import EdgeList, EntityList, Side, Stats

__all__ = [
    "ConfigSchema", "EntitySchema", "RelationSchema", "MultiRelationEmbedder", "Scores", "make_model",
    "PluginRegistry", "COMPARATORS", "DYNAMIC_OPERATORS", "LOSS_FUNCTIONS", "OPERATORS", "AsyncAdagrad",
    "RowAdagrad", "make_optimizer", "AbstractBatchProcessor", "B200RankingEvaluator", "B200Trainer", "process_in_batches",
    "EdgeList", "EntityList", "Side", "Stats",
]
