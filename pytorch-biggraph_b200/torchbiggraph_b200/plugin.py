"""Name -> class registries with the reference's interface (torchbiggraph/plugin.py:16-40):
`register(name, class_)`, the `register_as(name)` decorator, `get_class(name)` raising
NotImplementedError for an unknown name (callers catch that type, plugin.py:46-49), and a
RuntimeError when a different class is registered twice under one name."""
from typing import Callable, Dict, Generic, Type, TypeVar

T = TypeVar("T")


class PluginRegistry(Generic[T]):
    def __init__(self) -> None:
        self.registry: Dict[str, Type[T]] = {}

    def register(self, name: str, class_: Type[T]) -> None:
        known = self.registry.setdefault(name, class_)
        if known is not class_:
            raise RuntimeError(f"Attempting to re-register {name} which was already set to {known!r}")

    def register_as(self, name: str) -> Callable[[Type[T]], Type[T]]:
        def decorator(class_: Type[T]) -> Type[T]:
            self.register(name, class_)
            return class_
        return decorator

    def get_class(self, name: str) -> Type[T]:
        if name not in self.registry:
            raise NotImplementedError(f"Unknown name {name} (known names: {', '.join(sorted(self.registry))})")
        return self.registry[name]
