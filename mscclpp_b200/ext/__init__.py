"""Extensions on top of the core: the default algorithm collection."""
from .algorithm_collection_builder import AlgorithmCollectionBuilder  # noqa: F401

__all__ = ["AlgorithmCollectionBuilder"]
