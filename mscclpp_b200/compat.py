"""Import-name compatibility: let code written as `import mscclpp` / `from mscclpp.language.x import y`
run on this package unchanged.

`install()` registers a meta-path finder that resolves `mscclpp` and every `mscclpp.<sub>` to the
corresponding `mscclpp_b200` module object (the same object, not a copy, so module-level state such as
the DSL's current program is shared). It refuses to shadow a real `mscclpp` that is already imported.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import sys

_ALIAS = "mscclpp"
_TARGET = "mscclpp_b200"


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target_name: str):
        self._target_name = target_name

    def create_module(self, spec):
        return importlib.import_module(self._target_name)

    def exec_module(self, module):  # already executed under its real name
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != _ALIAS and not fullname.startswith(_ALIAS + "."):
            return None
        real = _TARGET + fullname[len(_ALIAS):]
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        spec = importlib.machinery.ModuleSpec(fullname, _AliasLoader(real), is_package=real_spec.submodule_search_locations is not None)
        return spec


_finder = None


def install() -> None:
    global _finder
    if _finder is not None:
        return
    if _ALIAS in sys.modules and getattr(sys.modules[_ALIAS], "__name__", "") != _TARGET:
        raise ImportError("a different `mscclpp` package is already imported in this process")
    import importlib.util  # noqa: F401  (used by the finder)

    _finder = _AliasFinder()
    sys.meta_path.insert(0, _finder)


def uninstall() -> None:
    global _finder
    if _finder is not None:
        sys.meta_path.remove(_finder)
        _finder = None
    for name in [n for n in sys.modules if n == _ALIAS or n.startswith(_ALIAS + ".")]:
        del sys.modules[name]
