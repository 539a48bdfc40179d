"""The algorithm DSL: describe a collective as per-rank, per-thread-block operations over chunks and
channels, and compile it to the JSON execution plan the executor runs. Pure Python, no GPU needed."""
from .utils import AlgoSpec, ReplicationPolicy  # noqa: F401
