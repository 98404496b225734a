"""Input / output types at the boundary of the training step, with the reference's names.

EdgeList / EntityList follow torchbiggraph/edgelist.py:16-179 and entitylist.py:16-135 for the
non-featurized case (featurized entities are refused: there is no device code for them);
Stats follows torchbiggraph/stats.py:23-92; Side follows torchbiggraph/types.py."""
from collections import defaultdict
from enum import Enum
from typing import Any, Iterable, Sequence, Union

import torch


class Side(Enum):
    LHS = 0
    RHS = 1

    def pick(self, lhs, rhs):
        return lhs if self is Side.LHS else rhs


class EntityList:
    @classmethod
    def empty(cls) -> "EntityList":
        return cls(torch.empty((0,), dtype=torch.long))

    @classmethod
    def from_tensor(cls, tensor: torch.Tensor) -> "EntityList":
        return cls(tensor)

    @classmethod
    def cat(cls, entity_lists: Sequence["EntityList"]) -> "EntityList":
        return cls(torch.cat([e.tensor for e in entity_lists]))

    def __init__(self, tensor: torch.Tensor, tensor_list: Any = None) -> None:
        if tensor_list is not None:
            raise NotImplementedError("featurized entities have no device code in torchbiggraph_b200")
        if tensor.dim() != 1 or tensor.dtype != torch.long:
            raise TypeError(f"Expected long tensor with 1 dimension, got {tensor.dtype} with {tensor.dim()}")
        self.tensor = tensor

    def to_tensor(self) -> torch.Tensor:
        return self.tensor

    def __getitem__(self, index) -> "EntityList":
        if isinstance(index, int):
            return EntityList(self.tensor[index:index + 1])
        return EntityList(self.tensor[index])

    def __len__(self) -> int:
        return self.tensor.shape[0]

    def to(self, *args, **kwargs) -> "EntityList":
        return EntityList(self.tensor.to(*args, **kwargs))


class EdgeList:
    @classmethod
    def empty(cls) -> "EdgeList":
        return cls(EntityList.empty(), EntityList.empty(), torch.empty((0,), dtype=torch.long))

    def __init__(self, lhs: EntityList, rhs: EntityList, rel: torch.Tensor, weight: Any = None) -> None:
        if not isinstance(lhs, EntityList) or not isinstance(rhs, EntityList):
            raise TypeError("lhs and rhs must be EntityList")
        if len(lhs) != len(rhs):
            raise ValueError(f"The lhs and rhs entity lists have different lengths ({len(lhs)} != {len(rhs)})")
        if not torch.is_tensor(rel) or rel.dtype != torch.long or rel.dim() > 1:
            raise TypeError("rel must be a long tensor with 0 or 1 dimensions")
        if rel.dim() == 1 and rel.shape[0] != len(lhs):
            raise ValueError("The relation type has a different length than the entity lists")
        self.lhs, self.rhs, self.rel, self.weight = lhs, rhs, rel, weight

    def has_scalar_relation_type(self) -> bool:
        return self.rel.dim() == 0

    def get_relation_type_as_scalar(self) -> int:
        if self.rel.dim() != 0:
            raise RuntimeError("The relation type isn't a scalar")
        return int(self.rel)

    def get_relation_type_as_vector(self) -> torch.Tensor:
        if self.rel.dim() == 0:
            raise RuntimeError("The relation type is a scalar")
        return self.rel

    def get_relation_type(self) -> Union[int, torch.Tensor]:
        return self.get_relation_type_as_scalar() if self.has_scalar_relation_type() else self.rel

    def has_weight(self) -> bool:
        return self.weight is not None

    def __getitem__(self, index) -> "EdgeList":
        if isinstance(index, int):
            index = slice(index, index + 1)
        sub_rel = self.rel if self.has_scalar_relation_type() else self.rel[index]
        sub_w = self.weight[index] if self.has_weight() else None
        return EdgeList(self.lhs[index], self.rhs[index], sub_rel, sub_w)

    def __len__(self) -> int:
        return len(self.lhs)

    def to(self, *args, **kwargs) -> "EdgeList":
        return EdgeList(self.lhs.to(*args, **kwargs), self.rhs.to(*args, **kwargs), self.rel.to(*args, **kwargs),
                        self.weight.to(*args, **kwargs) if self.has_weight() else None)


class Stats:
    def __init__(self, *, count: int, **metrics: float) -> None:
        self.count = count
        self.metrics = metrics

    @classmethod
    def sum(cls, stats: Iterable["Stats"]) -> "Stats":
        total = defaultdict(lambda: 0)
        n = 0
        for s in stats:
            n += s.count
            for k, v in s.metrics.items():
                total[k] += v
        return cls(count=n, **total)

    def average(self) -> "Stats":
        if self.count == 0:
            return self
        return type(self)(count=self.count, **{k: v / self.count for k, v in self.metrics.items()})

    def __str__(self) -> str:
        return "%s , count:  %d" % (" , ".join("%s:  %.6g" % (k, v) for k, v in self.metrics.items()), self.count)

    def __eq__(self, other) -> bool:
        return isinstance(other, Stats) and self.count == other.count and self.metrics == other.metrics
