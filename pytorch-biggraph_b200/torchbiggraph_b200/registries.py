"""The plugin registries of the training step, with the reference's names and lookup API:
OPERATORS / DYNAMIC_OPERATORS (torchbiggraph/operators.py:46, 194), COMPARATORS
(torchbiggraph/model.py:156), LOSS_FUNCTIONS (torchbiggraph/losses.py:50).

A registered class here does not compute anything in Python: it names the device code that
implements it (`native_code`) and, for operators, owns the parameter table the kernels read and
update in place.  Registering a class without device code is allowed (the registry is the
reference's), but building a trainer with it raises NotImplementedError: there is no CPU or
PyTorch fallback."""
from typing import Optional

import torch

from ._lib import COMPARATOR_CODES, LOSS_CODES, OPERATOR_CODES
from .plugin import PluginRegistry


# ----------------------------------------------------------------------------- operators
class AbstractOperator:
    """One relation's operator (operators.py:21-43).  `table` is the [1, width] float32 parameter
    row the device code uses; `state` its AsyncAdagrad accumulator."""
    native_code: Optional[int] = None
    name = "?"

    def __init__(self, dim: int):
        self.dim = dim
        self.table: Optional[torch.Tensor] = None

    def init_table(self, rows: int) -> Optional[torch.Tensor]:
        return None


class AbstractDynamicOperator(AbstractOperator):
    """All relations' operators as one [num_operations, width] table (operators.py:160-191)."""

    def __init__(self, dim: int, num_operations: int):
        super().__init__(dim)
        self.num_operations = num_operations


OPERATORS = PluginRegistry[AbstractOperator]()
DYNAMIC_OPERATORS = PluginRegistry[AbstractDynamicOperator]()


def _ones(rows, dim):
    return torch.ones((rows, dim), dtype=torch.float32)


def _zeros(rows, dim):
    return torch.zeros((rows, dim), dtype=torch.float32)


def _complex_init(rows, dim):
    if dim % 2 != 0:
        raise ValueError("Need even dimension as 1st half is real and 2nd half is imaginary coordinates")
    t = torch.zeros((rows, dim), dtype=torch.float32)
    t[:, : dim // 2] = 1.0          # real = 1, imag = 0 (operators.py:139-140)
    return t


def _linear_init(rows, dim):
    # one row-major D x D matrix per relation, identity at the start (operators.py:91-92)
    return torch.eye(dim, dtype=torch.float32).reshape(1, -1).repeat(rows, 1)


def _affine_init(rows, dim):
    # [matrix | translation], identity and zero at the start (operators.py:105-107)
    return torch.cat([_linear_init(rows, dim), torch.zeros((rows, dim), dtype=torch.float32)], dim=1)


_INIT = {"none": lambda r, d: None, "diagonal": _ones, "translation": _zeros, "complex_diagonal": _complex_init,
         "linear": _linear_init, "affine": _affine_init}


def _make(name, base, registry):
    code = OPERATOR_CODES[name]

    class _Op(base):
        native_code = code

        def init_table(self, rows: int):
            if name in _INIT:
                return _INIT[name](rows, self.dim)
            raise NotImplementedError(f"operator '{name}' has no device code in torchbiggraph_b200")

    _Op.name = name
    _Op.__name__ = "".join(p.capitalize() for p in name.split("_")) + ("DynamicOperator" if base is AbstractDynamicOperator else "Operator")
    registry.register_as(name)(_Op)
    return _Op


for _n in ("none", "diagonal", "translation", "linear", "affine", "complex_diagonal"):
    _make(_n, AbstractOperator, OPERATORS)
    _make(_n, AbstractDynamicOperator, DYNAMIC_OPERATORS)


# --------------------------------------------------------------------------- comparators
class AbstractComparator:
    native_code: Optional[int] = None


COMPARATORS = PluginRegistry[AbstractComparator]()
for _n, _c in COMPARATOR_CODES.items():
    COMPARATORS.register_as(_n)(type(_n.capitalize() + "Comparator", (AbstractComparator,), {"native_code": _c, "name": _n}))


# -------------------------------------------------------------------------------- losses
class AbstractLossFunction:
    native_code: Optional[int] = None

    def __init__(self, **kwargs):
        pass


LOSS_FUNCTIONS = PluginRegistry[AbstractLossFunction]()


@LOSS_FUNCTIONS.register_as("logistic")
class LogisticLossFunction(AbstractLossFunction):
    native_code = LOSS_CODES["logistic"]
    name = "logistic"


@LOSS_FUNCTIONS.register_as("ranking")
class RankingLossFunction(AbstractLossFunction):
    native_code = LOSS_CODES["ranking"]
    name = "ranking"

    def __init__(self, *, margin, **kwargs):
        super().__init__()
        self.margin = margin


@LOSS_FUNCTIONS.register_as("softmax")
class SoftmaxLossFunction(AbstractLossFunction):
    native_code = LOSS_CODES["softmax"]
    name = "softmax"
