from .collectives import (all_gather, all_reduce, all_reduce_rmsnorm, all_to_all, broadcast, reduce_scatter,  # noqa: F401
                          select_allreduce)
from .gemm import gemm_bf16  # noqa: F401
