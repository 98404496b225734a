"""Optimizer objects the coordinator sees (swap on partition change, checkpoint via state_dict).

The arithmetic runs inside the library's update kernels; these objects own the state tensors and
keep the reference's checkpoint format:
  RowAdagrad   one float32 `sum` per embedding row   (torchbiggraph/row_adagrad.py:20-46)
  AsyncAdagrad one float32 `sum` per parameter       (torchbiggraph/async_adagrad.py:19-87)
`state_dict()` / `load_state_dict()` use torch.optim.Optimizer's layout
({"state": {0: {"sum": tensor}}, "param_groups": [...]}), which is what the reference pickles into
checkpoints (torchbiggraph/checkpoint_storage.py:156-184)."""
from typing import Iterable, List

import torch


class _SumOptimizer:
    def __init__(self, params: Iterable[torch.Tensor], lr: float, per_row: bool):
        self.params: List[torch.Tensor] = list(params)
        self.lr = lr
        self.state = {}
        for p in self.params:
            if per_row and p.dim() != 2:
                raise ValueError("RowAdagrad only works on 2D tensors")
            shape = (p.shape[0],) if per_row else tuple(p.shape)
            self.state[id(p)] = {"sum": torch.zeros(shape, dtype=torch.float32, device=p.device)}

    def sum_for(self, p: torch.Tensor) -> torch.Tensor:
        return self.state[id(p)]["sum"]

    def step(self, closure=None):
        """No-op: the optimizer step of a batch is fused into the training-step kernels."""
        return None

    def share_memory(self):
        return None

    def state_dict(self):
        return {"state": {i: {"sum": self.state[id(p)]["sum"].detach().cpu().clone()} for i, p in enumerate(self.params)},
                "param_groups": [{"lr": self.lr, "lr_decay": 0, "weight_decay": 0, "params": list(range(len(self.params)))}]}

    def load_state_dict(self, sd):
        for i, p in enumerate(self.params):
            src = sd["state"][i]["sum"]
            dst = self.state[id(p)]["sum"]
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"optimizer state shape {tuple(src.shape)} does not match {tuple(dst.shape)}")
            dst.copy_(src.to(dst.device, torch.float32))
        groups = sd.get("param_groups")
        if groups:
            self.lr = groups[0].get("lr", self.lr)


class RowAdagrad(_SumOptimizer):
    def __init__(self, params, lr=1e-2, lr_decay=0, weight_decay=0):
        assert lr_decay == 0, "lr_decay not currently supported."
        if weight_decay != 0:
            raise RuntimeError("weight_decay option is not compatible with sparse gradients")
        super().__init__(params, lr, per_row=True)


class AsyncAdagrad(_SumOptimizer):
    def __init__(self, params, lr=1e-2):
        super().__init__(params, lr, per_row=False)


class DummyOptimizer(_SumOptimizer):
    def __init__(self):
        super().__init__([], 0.0, per_row=False)


def make_optimizer(config, params: Iterable[torch.Tensor], is_emb: bool):
    """torchbiggraph/train_cpu.py:215-230."""
    params = list(params)
    if len(params) == 0:
        return DummyOptimizer()
    if is_emb:
        return RowAdagrad(params, lr=config.lr)
    lr = config.relation_lr if config.relation_lr is not None else config.lr
    return AsyncAdagrad(params, lr=lr)
