"""Writes the API reference (docs/api-reference.md) from the package itself: every public Python name with its signature
and the first paragraph of its docstring, every class and function of the native module with the signatures pybind11
records, and every public C++ header with the comment that opens it.

    python -m mscclpp_b200.utils.apidoc > docs/api-reference.md

Runs without a GPU. The reference project publishes a Sphinx + Doxygen site for the same purpose (docs/cpp_api.rst,
docs/py_api.rst); here the reference is one Markdown file that is regenerated when the API changes and checked by
tests/test_docs.py against the live package."""
from __future__ import annotations

import importlib
import inspect
import os
import re
import sys
from typing import Iterable, List

PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PYTHON_MODULES = [
    ("mscclpp_b200", "Top-level package (the names of the reference's `mscclpp` package plus the symmetric-heap API)"),
    ("mscclpp_b200.ops", "Collectives and GEMM on symmetric tensors"),
    ("mscclpp_b200.ops.collectives", "Allreduce / allgather / reduce-scatter / broadcast / all-to-all entry points and the selector"),
    ("mscclpp_b200.ops.gemm", "tcgen05 GEMM entry points"),
    ("mscclpp_b200.parallel.tp_layer", "Tensor-parallel fused layer"),
    ("mscclpp_b200.parallel.sp_layer", "Sequence-parallel fused layers"),
    ("mscclpp_b200.parallel.moe", "Expert-parallel dispatch / combine"),
    ("mscclpp_b200.ext", "Algorithm collection builder"),
    ("mscclpp_b200.language", "DSL for execution plans"),
    ("mscclpp_b200.language.interpreter", "numpy plan interpreter and plan validator"),
    ("mscclpp_b200.default_algos", "Plans shipped with the package"),
    ("mscclpp_b200.utils", "Kernel builder, packing helpers, dtype maps"),
    ("mscclpp_b200.utils.npkit_trace", "Trace conversion"),
    ("mscclpp_b200.benchmark.bench_collective", "Collective benchmark"),
    ("mscclpp_b200.benchmark.check_perf", "Performance-regression gate"),
    ("mscclpp_b200.benchmark.tuner", "Offline tuner"),
    ("mscclpp_b200.compat", "`import mscclpp` compatibility"),
]


def first_paragraph(doc: str | None) -> str:
    if not doc:
        return ""
    text = inspect.cleandoc(doc)
    para = text.split("\n\n", 1)[0]
    return " ".join(line.strip() for line in para.splitlines())


def signature_of(obj) -> str:
    try:
        return str(inspect.signature(obj))
    except (TypeError, ValueError):
        doc = getattr(obj, "__doc__", "") or ""
        first = doc.strip().splitlines()[0] if doc.strip() else ""
        m = re.match(r"^\w+(\(.*\))(\s*->\s*.+)?$", first)  # pybind11 puts the signature on the first docstring line
        return tidy(m.group(1) + (m.group(2) or "")) if m else "(...)"


def tidy(sig: str) -> str:
    """pybind11 signatures without the module path, the self parameter and the long spellings of int and float."""
    sig = sig.replace("mscclpp_b200.lib._native.", "")
    sig = sig.replace("typing.SupportsInt | typing.SupportsIndex", "int").replace("typing.SupportsFloat | typing.SupportsIndex", "float")
    sig = sig.replace("collections.abc.", "").replace("typing.", "")
    sig = re.sub(r"^\(self: [\w.]+(, )?", "(", sig)
    return sig


def pybind_doc(obj) -> str:
    """Docstring of a pybind11 callable without its leading signature line."""
    doc = (getattr(obj, "__doc__", "") or "").strip()
    lines = doc.splitlines()
    if lines and re.match(r"^\w+\(.*\)", lines[0]):
        lines = lines[1:]
    return first_paragraph("\n".join(lines))


def public_names(mod) -> List[str]:
    names = getattr(mod, "__all__", None)
    if names is None:
        names = [n for n in vars(mod) if not n.startswith("_")]
        names = [n for n in names if getattr(getattr(mod, n), "__module__", mod.__name__) == mod.__name__]
    return sorted(set(names))


def describe_class(cls, out: List[str], native: bool) -> None:
    members = getattr(cls, "__members__", None)
    if native and isinstance(members, dict) and members:  # a pybind11 enum
        out.append("  * values: " + ", ".join(f"`{k}`" for k in members))
        return
    for name, member in sorted(vars(cls).items()):
        if name.startswith("_") and name != "__init__":
            continue
        if isinstance(member, property) or type(member).__name__ in ("getset_descriptor", "instancemethod") and False:
            pdoc = first_paragraph(getattr(member, "__doc__", ""))
            if re.match(r"^\w+\(", pdoc):  # pybind11's generated "name(self: object, /) -> str"
                pdoc = ""
            out.append(f"  * `{name}` (property) {pdoc}".rstrip())
        elif isinstance(member, (staticmethod, classmethod)):
            fn = member.__func__
            out.append(f"  * `{name}{signature_of(fn)}` {first_paragraph(fn.__doc__)}".rstrip())
        elif callable(member):
            doc = pybind_doc(member) if native else first_paragraph(getattr(member, "__doc__", ""))
            if name == "__init__" and (member is object.__init__ or "See help(type(self))" in (doc or "")):
                continue
            if doc.startswith("Overloaded function."):
                overloads = re.findall(r"^\d+\. \w+(\(.*)$", getattr(member, "__doc__", "") or "", re.M)
                for o in overloads:
                    out.append(f"  * `{name}{tidy(o)}`")
                continue
            out.append(f"  * `{name}{signature_of(member)}` {doc}".rstrip())
        elif isinstance(member, property):
            out.append(f"  * `{name}` (property)")


def describe_module(modname: str, title: str, out: List[str], native: bool = False) -> None:
    try:
        mod = importlib.import_module(modname)
    except Exception as e:  # noqa: BLE001
        out.append(f"### `{modname}`\n\n(not importable here: {e})\n")
        return
    out.append(f"### `{modname}` - {title}\n")
    doc = first_paragraph(mod.__doc__)
    if doc:
        out.append(doc + "\n")
    for name in public_names(mod):
        obj = getattr(mod, name, None)
        if obj is None or inspect.ismodule(obj):
            continue
        if inspect.isclass(obj):
            is_native = native or obj.__module__.endswith("_native")
            base = first_paragraph(obj.__doc__) if not is_native else pybind_doc(obj)
            out.append(f"* **class `{name}`** {base}".rstrip())
            describe_class(obj, out, is_native)
        elif callable(obj):
            is_native = native or type(obj).__name__ == "builtin_function_or_method"
            doc = pybind_doc(obj) if is_native else first_paragraph(obj.__doc__)
            out.append(f"* `{name}{signature_of(obj)}` {doc}".rstrip())
        else:
            out.append(f"* `{name}` = `{obj!r}`"[:200])
    out.append("")


def header_summaries() -> Iterable[str]:
    inc = os.path.join(PKG_ROOT, "csrc", "include", "mscclpp")
    for root, _dirs, files in sorted(os.walk(inc)):
        for f in sorted(files):
            if not f.endswith((".hpp", ".h", ".cuh")):
                continue
            path = os.path.join(root, f)
            rel = os.path.relpath(path, os.path.join(PKG_ROOT, "csrc", "include"))
            comment: List[str] = []
            with open(path) as fh:
                for line in fh:
                    s = line.strip()
                    if s.startswith("//"):
                        comment.append(s.lstrip("/").strip())
                    elif s == "" and not comment:
                        continue
                    else:
                        break
            names = []
            with open(path) as fh:
                text = fh.read()
            for m in re.finditer(r"^(?:class|struct|union|enum class)\s+(?:alignas\(\d+\)\s+)?([A-Z]\w+)\b(?!\s*;)", text, re.M):
                if m.group(1) not in names:
                    names.append(m.group(1))
            summary = " ".join(comment)
            yield f"* `<{rel}>` {summary}" + (f" Declares: {', '.join('`' + n + '`' for n in names[:24])}." if names else "")


def generate() -> str:
    out: List[str] = []
    out.append("# API reference\n")
    out.append("Generated by `python -m mscclpp_b200.utils.apidoc` from the package itself; do not edit by hand. Guides: "
               "`quickstart.md`, `tutorials.md`, `torch-integration.md`, `fused-layers.md`, `dsl.md`, `nccl-shim.md`, `tracing.md`, `api-parity.md`.\n")
    out.append("## Python\n")
    for modname, title in PYTHON_MODULES:
        describe_module(modname, title, out)
    out.append("## Native module (`mscclpp_b200.native()`)\n")
    out.append("The pybind11 module behind the package: host classes of the C++ API plus the kernel launchers. Pointers are "
               "passed as integers (`tensor.data_ptr()`), streams as `torch.cuda.Stream.cuda_stream`.\n")
    try:
        import mscclpp_b200 as mp

        native = mp.native()
        names = sorted(n for n in dir(native) if not n.startswith("_"))
        for name in names:
            obj = getattr(native, name)
            if inspect.ismodule(obj):
                out.append(f"* **submodule `{name}`**: " + ", ".join(f"`{m}`" for m in sorted(dir(obj)) if not m.startswith("_")))
            elif inspect.isclass(obj):
                out.append(f"* **class `{name}`** {pybind_doc(obj)}".rstrip())
                describe_class(obj, out, True)
            elif callable(obj):
                out.append(f"* `{name}{signature_of(obj)}` {pybind_doc(obj)}".rstrip())
        out.append("")
    except Exception as e:  # noqa: BLE001
        out.append(f"(native module not loadable here: {e})\n")
    out.append("## C++ headers (`mscclpp_b200/csrc/include`)\n")
    out.extend(header_summaries())
    out.append("")
    out.append("## C ABI\n")
    out.append("* `<mscclpp/ext/nccl/nccl.h>`: the NCCL 2.x C ABI implemented by `libmscclpp_b200_nccl.so` (see `nccl-shim.md`).")
    out.append("* `<mscclpp/ext/tp_layer_noalloc.h>`: `mscclpp_b200_tp_layer_noalloc`, `mscclpp_b200_tp_layer_noalloc_status` - the "
               "fused GEMM + residual + RMSNorm layer on one GPU with no device allocation at run time.")
    out.append("")
    # defaults that hold a path of this installation are shown relative to the package
    return "\n".join(out).replace(PKG_ROOT, "<package>").replace(os.path.dirname(PKG_ROOT), "<site>")


def main(argv=None) -> int:
    sys.stdout.write(generate())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
