"""`python -m mscclpp_b200 --install` writes the default DSL plans into `<cache>/default/`, where the
algorithm collection builder (and with it the NCCL shim) picks them up
(reference: python/mscclpp/__main__.py:101-140)."""
from __future__ import annotations

import argparse
import os
import shutil
from pathlib import Path

from .default_algos import default_algo_configs


def default_plan_dir() -> Path:
    return Path(os.environ.get("MSCCLPP_CACHE_DIR", Path.home() / ".cache" / "mscclpp")) / "default"


def create_default_plans(plan_dir: Path | None = None, verbose: bool = True) -> list:
    plan_dir = Path(plan_dir) if plan_dir is not None else default_plan_dir()
    if plan_dir.exists():
        shutil.rmtree(plan_dir)
    plan_dir.mkdir(parents=True)
    written = []
    for config in default_algo_configs():
        path = plan_dir / config["filename"]
        try:
            prog = config["function"](config["spec"], **config.get("additional_kwargs", {}))
            with open(path, "w", encoding="utf-8") as f:
                f.write(prog.to_json())
            written.append(path)
        except Exception as e:  # one bad plan must not stop the installation of the others
            print(f"Error creating plan for {config['spec'].name}: {e}")
    if verbose:
        print(f"wrote {len(written)} plans to {plan_dir}")
    return written


def main(argv=None):
    parser = argparse.ArgumentParser(prog="python -m mscclpp_b200")
    parser.add_argument("--install", action="store_true", help="install the default execution plans into the cache directory")
    args = parser.parse_args(argv)
    if args.install:
        create_default_plans()
    else:
        parser.print_help()


if __name__ == "__main__":
    main()
