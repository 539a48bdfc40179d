"""Benchmarks and the offline tuner (device-timed, max over ranks):

    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.bench_collective --collective allreduce
    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.sp_mlp
    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.moe
    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.tuner --out tuned.json
"""
