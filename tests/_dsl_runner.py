"""Runs one DSL example script and prints the plan it prints.

usage: _dsl_runner.py {reference|ours} <reference python dir or ''> script.py [script args...]
`reference` imports the reference DSL as a bare package (its top-level __init__ needs native
bindings and cupy, the DSL subpackage does not); `ours` maps the `mscclpp` import name onto this
package."""
import os
import runpy
import sys
import types

mode, ref_dir, script = sys.argv[1], sys.argv[2], sys.argv[3]
sys.argv = [script] + sys.argv[4:]
if mode == "reference":
    stub = types.ModuleType("mscclpp")
    stub.__path__ = [os.path.join(ref_dir, "mscclpp")]
    sys.modules["mscclpp"] = stub
else:
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from mscclpp_b200 import compat

    compat.install()
runpy.run_path(script, run_name="__main__")
