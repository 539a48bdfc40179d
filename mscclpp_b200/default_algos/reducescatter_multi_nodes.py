"""`reducescatter_multi_nodes` under the module name the reference uses (python/mscclpp/default_algos/reducescatter_multi_nodes.py);
the program itself lives in `multi_node.py` with the other hierarchical algorithms."""
from .multi_node import reducescatter_multi_nodes

__all__ = ["reducescatter_multi_nodes"]
