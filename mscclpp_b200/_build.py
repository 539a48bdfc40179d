"""In-tree build of the native libraries with nvcc (sm_100a only).

Produces, next to this file under ``lib/``:
  libmscclpp_b200.so        core runtime + every CUDA kernel (C++ API, namespace mscclpp)
  libmscclpp_b200_nccl.so   NCCL-API shim (C ABI) on top of the core
  _native.<abi>.so          pybind11 bindings used by the Python package
Objects are cached under ``build/`` and rebuilt when their source, any header or the flags change.
Run ``python -m mscclpp_b200._build`` to build from the command line.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
BUILD = ROOT / "build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=default",
              "-Xcudafe", "--diag_suppress=177"]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _cuda_home() -> Path:
    return Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".hpp", ".cuh", ".h"):
            h.update(p.read_bytes())
    return h.hexdigest()


def _sources(sub: str, exts=(".cc", ".cu", ".cpp")) -> list[Path]:
    d = CSRC / sub
    return sorted(p for p in d.iterdir() if p.suffix in exts) if d.exists() else []


def _compile_one(src: Path, extra_inc: list[str], hdr_digest: str, verbose: bool) -> Path:
    is_cu = src.suffix == ".cu"
    inc = ["-I", str(CSRC / "include"), "-I", str(CSRC), "-I", str(_cuda_home() / "include")] + extra_inc
    if is_cu:
        cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + inc + ["-c", str(src)]
    else:
        cmd = ["g++"] + CXX_FLAGS + inc + ["-c", str(src)]
    key = hashlib.sha256((" ".join(cmd) + hdr_digest).encode() + src.read_bytes()).hexdigest()[:16]
    obj = BUILD / f"{src.parent.name}_{src.stem}.o"
    stamp = BUILD / f"{src.parent.name}_{src.stem}.stamp"
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj
    if verbose:
        print(f"[build] {src.relative_to(ROOT)}", flush=True)
    res = subprocess.run(cmd + ["-o", str(obj)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp.write_text(key)
    return obj


def _link(objs: list[Path], out: Path, extra: list[str], verbose: bool) -> None:
    newest = max(o.stat().st_mtime for o in objs)
    if out.exists() and out.stat().st_mtime >= newest:
        return
    # link into a temporary name and rename: a reader (an importing process, a snapshot) never sees a partial library
    tmp = out.with_name(out.name + f".tmp.{os.getpid()}")
    cmd = [_nvcc(), "-shared", "-o", str(tmp)] + [str(o) for o in objs] + ARCH_FLAGS + [
        "-cudart", "static", "-Xlinker", "-rpath,$ORIGIN", "-lpthread", "-ldl", "-lrt"] + extra
    if verbose:
        print(f"[link] {out.relative_to(ROOT)}", flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, out)


def native_module_path() -> Path:
    return LIB / ("_native" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(verbose: bool = True, jobs: int | None = None) -> dict[str, Path]:
    """Compile and link everything that is out of date. Returns the produced libraries."""
    import pybind11

    LIB.mkdir(exist_ok=True)
    BUILD.mkdir(exist_ok=True)
    hdr = _headers_digest()
    core_srcs = _sources("core") + _sources("kernels") + _sources("executor") + _sources("ext")
    nccl_srcs = _sources("nccl")
    bind_srcs = _sources("bindings")
    py_inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    jobs = jobs or max(1, (os.cpu_count() or 4))
    with ThreadPoolExecutor(jobs) as pool:
        core_f = [pool.submit(_compile_one, s, [], hdr, verbose) for s in core_srcs]
        nccl_f = [pool.submit(_compile_one, s, [], hdr, verbose) for s in nccl_srcs]
        bind_f = [pool.submit(_compile_one, s, py_inc, hdr, verbose) for s in bind_srcs]
        core_o = [f.result() for f in core_f]
        nccl_o = [f.result() for f in nccl_f]
        bind_o = [f.result() for f in bind_f]
    out = {}
    core_lib = LIB / "libmscclpp_b200.so"
    _link(core_o, core_lib, [], verbose)
    out["core"] = core_lib
    if nccl_o:
        nccl_lib = LIB / "libmscclpp_b200_nccl.so"
        _link(nccl_o, nccl_lib, ["-L", str(LIB), "-lmscclpp_b200"], verbose)
        out["nccl"] = nccl_lib
    audit_src = CSRC / "nccl_audit" / "audit_nccl.cc"
    if audit_src.exists():
        # tiny stand-alone library (no CUDA, no dependency on the core): plain g++
        audit_lib = LIB / "libmscclpp_b200_audit_nccl.so"
        if not audit_lib.exists() or audit_lib.stat().st_mtime < audit_src.stat().st_mtime:
            tmp = audit_lib.with_name(audit_lib.name + f".tmp.{os.getpid()}")
            res = subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", str(audit_src), "-o", str(tmp), "-ldl"],
                                 capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"audit shim build failed:\n{res.stderr}")
            os.replace(tmp, audit_lib)
            if verbose:
                print(f"[link] {audit_lib.relative_to(ROOT)}", flush=True)
        out["audit"] = audit_lib
    if bind_o:
        mod = native_module_path()
        _link(bind_o, mod, ["-L", str(LIB), "-lmscclpp_b200"], verbose)
        out["native"] = mod
    return out


if __name__ == "__main__":
    for name, path in build(verbose=True).items():
        print(f"{name}: {path}")
