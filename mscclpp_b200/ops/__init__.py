from .collectives import all_gather, all_reduce, all_reduce_rmsnorm, reduce_scatter, select_allreduce  # noqa: F401
from .gemm import gemm_bf16  # noqa: F401
