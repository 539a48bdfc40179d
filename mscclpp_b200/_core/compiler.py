"""`compile` (DSL function -> cached plan -> `Algorithm`) and `compile_native` (a .cu file with pybind11
bindings -> cached extension module), reference: python/mscclpp/_core/compiler.py:45-355.

Differences that matter to a user: the cache key is a BLAKE2b digest (the blake3 package is not a
dependency here) and native code is compiled for sm_100a only.
"""
from __future__ import annotations

import fcntl
import hashlib
import importlib.util
import inspect
import json
import os
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import Any, Callable

from . import native as _loader
from .algorithm import Algorithm

__all__ = ["DslCompiler", "NativeCodeCompiler"]

ARCH = "sm_100a"


def _stable_json_bytes(obj: Any) -> bytes:
    return json.dumps(obj, sort_keys=True, ensure_ascii=False, separators=(",", ":")).encode("utf-8")


def _digest(data: bytes) -> str:
    return hashlib.blake2b(data, digest_size=32).hexdigest()


def _cache_dir() -> Path:
    if _loader.available():
        return Path(_loader.load().env().cache_dir)
    return Path(os.environ.get("MSCCLPP_CACHE_DIR", Path.home() / ".cache" / "mscclpp"))


class DslCompiler:
    """Callable singleton behind `mscclpp_b200.compile`."""

    def __call__(self, algo: Callable, algo_spec, rank: int, **kwds) -> Algorithm:
        return self.compile(algo, algo_spec, rank, **kwds)

    def plan_path(self, algo: Callable, algo_spec, **kwargs) -> Path:
        """Compile (or find in the cache) and return the path of the plan JSON; needs no GPU and no native library."""
        if not callable(algo):
            raise ValueError("The 'algo' argument must be a callable (e.g., a function or class).")
        from .. import __version__

        try:
            source = inspect.getsource(algo)
        except (OSError, TypeError):
            source = repr(algo)
        plan_id = _digest(_stable_json_bytes({
            "version": __version__,
            "algo_name": algo_spec.name,
            "collective": getattr(algo_spec.collective, "name", str(algo_spec.collective)),
            "tags": sorted(algo_spec.tags.items()),
            "source_hash": _digest(source.encode("utf-8")),
            "kwargs": sorted((k, repr(v)) for k, v in kwargs.items()),
            "envs": {
                "nranks_per_node": algo_spec.nranks_per_node,
                "world_size": algo_spec.world_size,
                "instances": algo_spec.instances,
                "protocol": algo_spec.protocol,
            },
        }))
        plan_dir = _cache_dir()
        plan_dir.mkdir(parents=True, exist_ok=True)
        path = plan_dir / f"{plan_id}.json"
        if not path.exists():
            prog = algo(algo_spec, **kwargs)
            tmp = path.with_suffix(f".json.tmp.{os.getpid()}")
            with open(tmp, "w") as f:
                f.write(prog.to_json(indent=None, separators=(",", ":"), ensure_ascii=False))
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, path)  # atomic: concurrent ranks write identical content
        return path

    def compile(self, algo: Callable, algo_spec, rank: int, **kwargs) -> Algorithm:
        path = self.plan_path(algo, algo_spec, **kwargs)
        plan = _loader.load().ExecutionPlan(str(path), rank)
        return Algorithm(id=path.stem, execution_plan=plan,
                         constraint=Algorithm.Constraint(world_size=algo_spec.world_size, n_ranks_per_node=algo_spec.nranks_per_node),
                         tags=algo_spec.tags)


class NativeCodeCompiler:
    """Callable singleton behind `mscclpp_b200.compile_native`: nvcc-compiles a user's .cu file (which carries its
    own pybind11 module definition) against this library's headers and loads it."""

    def __init__(self):
        self._initialized = False

    def _do_init(self):
        import pybind11

        from .. import get_include, get_lib

        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        nvcc = os.path.join(cuda_home, "bin", "nvcc")
        self._compiler = nvcc if os.path.exists(nvcc) else "nvcc"
        self._device_arch = ARCH
        lib = get_lib()
        self._default_options = [
            "-std=c++17", "-O3", "--shared", "-lineinfo",
            f"-I{sysconfig.get_path('include')}", f"-I{pybind11.get_include()}",
            "-gencode=arch=compute_100a,code=sm_100a",
            "--compiler-options", "-fPIC",
            "--linker-options", f"-rpath,{lib}",
            f"-I{get_include()}", f"-L{lib}", "-lmscclpp_b200",
        ]
        self._cache_dir = _cache_dir() / "native"
        self._cache_dir.mkdir(parents=True, exist_ok=True)
        self._initialized = True

    def get_arch(self) -> str:
        if not self._initialized:
            self._do_init()
        return self._device_arch

    def __call__(self, name: str, file: str, **kwds):
        return self.compile(name, file, **kwds)

    def compile(self, name: str, file: str):
        if not self._initialized:
            self._do_init()
        if not os.path.isfile(file):
            raise FileNotFoundError(f"The specified source file does not exist: {file}")
        from .. import __version__

        with open(file, "rb") as f:
            source_hash = _digest(f.read())
        cache_key = _digest(_stable_json_bytes({
            "version": __version__, "source_hash": source_hash, "compiler": self._compiler,
            "options": self._default_options, "arch": self._device_arch,
        }))
        output_file = self._cache_dir / f"{name}-{cache_key}.so"
        with open(str(output_file) + ".lock", "w") as lock:
            fcntl.flock(lock, fcntl.LOCK_EX)
            if not output_file.exists():
                tmp = Path(str(output_file) + f".tmp.{os.getpid()}")
                cmd = [self._compiler] + self._default_options + ["-o", str(tmp), file]
                try:
                    subprocess.run(cmd, check=True, capture_output=True, text=True)
                    os.replace(tmp, output_file)
                except FileNotFoundError as e:
                    tmp.unlink(missing_ok=True)
                    raise RuntimeError(f"Compiler '{self._compiler}' not found. Make sure it's installed and in PATH.") from e
                except subprocess.CalledProcessError as e:
                    tmp.unlink(missing_ok=True)
                    raise RuntimeError(f"Compilation failed with return code {e.returncode}.\nCommand: {' '.join(cmd)}\n"
                                       f"Stdout: {e.stdout}\nStderr: {e.stderr}") from e
        existing = sys.modules.get(name)
        if existing is not None and getattr(existing, "__mscclpp_cache_key__", None) == cache_key:
            return existing
        _loader.load()  # the user's module resolves the pybind11 types registered by the runtime module
        spec = importlib.util.spec_from_file_location(name, output_file)
        if spec is None or spec.loader is None:
            raise ImportError(f"Could not load module '{name}' from '{output_file}'")
        module = importlib.util.module_from_spec(spec)
        module.__mscclpp_cache_key__ = cache_key
        sys.modules[name] = module
        spec.loader.exec_module(module)
        return module
