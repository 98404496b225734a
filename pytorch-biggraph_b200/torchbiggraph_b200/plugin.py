"""Name -> class registries with the reference's interface (torchbiggraph/plugin.py:16-40):
`register_as(name)` decorator, `get_class(name)`, and a RuntimeError when a different class is
registered twice under one name."""
from typing import Callable, Dict, Generic, Type, TypeVar

T = TypeVar("T")


class PluginRegistry(Generic[T]):
    def __init__(self) -> None:
        self.registry: Dict[str, Type[T]] = {}

    def register_as(self, name: str) -> Callable[[Type[T]], Type[T]]:
        def decorator(class_: Type[T]) -> Type[T]:
            reg_class = self.registry.setdefault(name, class_)
            if reg_class is not class_:
                raise RuntimeError(f"Attempting to re-register {name} which was already set to {reg_class!r} with {class_!r}")
            return class_
        return decorator

    def get_class(self, name: str) -> Type[T]:
        try:
            return self.registry[name]
        except KeyError:
            raise RuntimeError(f"Cannot find plugin '{name}'. Available: {sorted(self.registry)}") from None
