"""Singleton that assembles an `AlgorithmCollection` from user builders, selectors and the default
algorithms (reference: python/mscclpp/ext/algorithm_collection_builder.py:14-68)."""
from __future__ import annotations

import atexit
from typing import Union

from .._core import native as _loader
from .._core.algorithm import Algorithm, AlgorithmBuilder, AlgorithmCollection

__all__ = ["AlgorithmCollectionBuilder"]


class AlgorithmCollectionBuilder:
    _instance = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
        return cls._instance

    @classmethod
    def reset(cls):
        if cls._instance is not None:
            _loader.load().AlgorithmCollectionBuilder.reset()
            cls._instance = None

    def __init__(self):
        if not hasattr(self, "_initialized"):
            self._builder = _loader.load().AlgorithmCollectionBuilder.get_instance()
            self._initialized = True

    def add_algorithm_builder(self, algorithm_builder: Union[AlgorithmBuilder, Algorithm]):
        if isinstance(algorithm_builder, AlgorithmBuilder):
            self._builder.add_algorithm_builder(algorithm_builder._algorithm_builder)
            return
        if isinstance(algorithm_builder, Algorithm):
            # a ready algorithm (a compiled DSL plan, or a native one made in Python) is its own builder
            self._builder.add_dsl_algorithm_builder(algorithm_builder._algorithm)
            return
        raise ValueError("the argument must be an AlgorithmBuilder or an Algorithm")

    def set_algorithm_selector(self, selector):
        self._builder.set_algorithm_selector(selector)

    def set_fallback_algorithm_selector(self, selector):
        self._builder.set_fallback_algorithm_selector(selector)

    def build(self) -> AlgorithmCollection:
        return AlgorithmCollection(self._builder.build())

    def build_default_algorithms(self, heap) -> AlgorithmCollection:
        """Default native algorithms on a symmetric heap (`SymmetricMemory` or the native `SymmetricHeap`).

        The reference takes a scratch buffer and a flag buffer here; in this library both live inside the
        symmetric heap, so the heap is the only argument."""
        native_heap = getattr(heap, "heap", heap)
        return AlgorithmCollection(self._builder.build_default_algorithms(native_heap))


atexit.register(AlgorithmCollectionBuilder.reset)
