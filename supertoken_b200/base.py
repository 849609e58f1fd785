"""Trainer base class of the drop-in.

When the reference package is importable (the drop-in deployment), its own
``BaseTrainer`` is used so that ``isinstance`` checks in the reference's launcher hold
(``gpu_tokenizer/dist/launcher.py:134-138``).  Otherwise a local ABC with the same abstract
surface (``gpu_tokenizer/trainers/base.py:128-192``) stands in.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from types import MappingProxyType
from typing import Any, Mapping

try:  # pragma: no cover - only when the reference is on sys.path
    from gpu_tokenizer.trainers.base import BaseTrainer as _RefBase  # type: ignore
except Exception:  # reference not installed: local mirror
    _RefBase = None


class _LocalBaseTrainer(ABC):
    def __init__(self) -> None:
        self._metrics_registry: dict[str, Any] = {}
        self._metrics_view: Mapping[str, Any] = MappingProxyType(self._metrics_registry)

    def register_metrics_tracker(self, name: str, tracker: Any | None) -> None:
        if tracker is None:
            self._metrics_registry.pop(str(name), None)
        else:
            self._metrics_registry[str(name)] = tracker

    def _metrics_mapping(self) -> Mapping[str, Any]:
        return self._metrics_view

    @abstractmethod
    def fit(self, *args: Any, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def state_dict(self, *args: Any, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def load_state_dict(self, state_dict: Mapping[str, Any], *args: Any, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def save_checkpoint(self, path, *args: Any, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def load_checkpoint(self, path, *args: Any, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def save_artifacts(self, output_dir, *args: Any, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def metrics(self) -> Mapping[str, Any]: ...


BaseTrainer = _RefBase if _RefBase is not None else _LocalBaseTrainer
