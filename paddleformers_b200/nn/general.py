"""Registry pattern shared by the layer factories: a class-level table of named implementations and a ``create``
class method that picks one, so that a model file never hard-codes which linear / norm / attention variant it gets
(paddleformers/nn/general.py:19-57 ``GeneralInterface``)."""
from __future__ import annotations

from typing import Callable, Dict


class GeneralInterface:
    _global_mapping: Dict[str, Callable] = {}

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        cls._global_mapping = dict(cls._global_mapping)      # every factory owns its table

    @classmethod
    def register(cls, key: str, value: Callable):
        cls._global_mapping[key] = value

    @classmethod
    def get(cls, key: str) -> Callable:
        if key not in cls._global_mapping:
            raise KeyError(f"{cls.__name__}: unknown implementation {key!r}; registered: {sorted(cls._global_mapping)}")
        return cls._global_mapping[key]

    @classmethod
    def valid_keys(cls):
        return sorted(cls._global_mapping)
