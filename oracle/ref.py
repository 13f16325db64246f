"""Test infrastructure: the reference itself, installed beside the CPU oracle.

The reference compiler is pure Python (package ``mlc`` plus its ``tests/``).
:func:`install` copies those files from a checkout of the reference into
``oracle/_ref/`` -- a directory that is never committed -- so that machines
without the checkout can still run the reference's own code:

* as the checker of the drop-in boundary (``tests/test_gpu_reference.py`` drives
  ``mlc.compile`` with this backend installed against the reference's torch
  backend, ``mlc/codegen/torch_backend.py:100-248``;
  ``tests/test_gpu_reference_suite.py`` runs the reference's own test files on
  the GPU with this backend installed),
* as the timed CPU baseline (``bench.py --impl reference`` and the
  ``cpu_baseline`` leg), and
* as the comparison arm that runs the reference's stock Triton build
  (``mlc/runtime/triton_runtime.py:60-97``) on the same GPU.

Only tests, the smoke check and ``bench.py`` may import this module; nothing in
the product package does.  Nothing is copied into tracked files.

    python oracle/ref.py [--from /path/to/mlc-compiler]
"""

from __future__ import annotations

import argparse
import os
import pathlib
import shutil
import sys

HERE = pathlib.Path(__file__).resolve().parent
DEST = HERE / "_ref"
#: what the checker needs of a checkout: the package and its test suite (model zoo
#: included), which ``tests/test_gpu_reference_suite.py`` runs on the GPU unmodified
PIECES = ("mlc", "tests")


def default_source() -> pathlib.Path:
    env = os.environ.get("MLC_REFERENCE")
    return pathlib.Path(env) if env else HERE.parent.parent / "reference"


def install(source: str | os.PathLike | None = None, quiet: bool = False) -> pathlib.Path | None:
    """Copy the reference's Python files into ``oracle/_ref``; returns the
    directory, or None (with a message) when no checkout is found.  An existing
    copy is refreshed."""
    src = pathlib.Path(source) if source else default_source()
    if not (src / "mlc" / "api.py").exists():
        if not quiet:
            print(f"oracle/ref: no reference checkout at {src}; keeping "
                  f"{'the existing' if present() else 'no'} copy")
        return DEST if present() else None
    if DEST.exists():
        shutil.rmtree(DEST)
    DEST.mkdir(parents=True)
    ignore = shutil.ignore_patterns("__pycache__", "*.pyc")
    for piece in PIECES:
        s, d = src / piece, DEST / piece
        d.parent.mkdir(parents=True, exist_ok=True)
        if s.is_dir():
            shutil.copytree(s, d, ignore=ignore)
        else:
            shutil.copy2(s, d)
    if not quiet:
        n = sum(1 for _ in DEST.rglob("*.py"))
        print(f"oracle/ref: installed {n} files of the reference into {DEST}")
    return DEST


def present() -> bool:
    return (DEST / "mlc" / "api.py").exists()


def path() -> pathlib.Path | None:
    """Where the reference can be imported from: the installed copy first, a
    checkout named by ``$MLC_REFERENCE`` (or lying beside this repository) second."""
    if present():
        return DEST
    src = default_source()
    return src if (src / "mlc" / "api.py").exists() else None


def activate() -> pathlib.Path:
    """Put the reference on ``sys.path`` (without letting it write bytecode into a
    read-only checkout) and return its directory; raises when it is absent."""
    p = path()
    if p is None:
        raise ImportError("the reference is not installed: run `python oracle/ref.py --from "
                          "<checkout>` (or __graft_entry__.build()) where a checkout exists")
    sys.dont_write_bytecode = True
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))
    return p


def test_models():
    """The reference's ten test modules (``tests/models.py:112-126``) as
    ``[(name, module, inputs)]``."""
    p = activate()
    import importlib.util

    spec = importlib.util.spec_from_file_location("_mlc_ref_test_models", p / "tests" / "models.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.all_models()


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--from", dest="source", default=None)
    a = ap.parse_args()
    raise SystemExit(0 if install(a.source) is not None else 1)
