"""Loader of the native extension ``scalingcontrasts_b200._C`` (built in-tree by ``setup.py build_ext --inplace``).

On a machine with a GPU a missing extension is an error, never a silent fallback: ``native()`` raises with the build
command. Code that can run without it (the CPU oracle, the CPU streamed loss) asks ``available()`` first.
"""
from __future__ import annotations

import importlib
import os
import subprocess
import sys
from typing import Optional

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_module = None
_error: Optional[BaseException] = None


def _try_import():
    global _module, _error
    if _module is not None or _error is not None:
        return
    try:
        import torch  # noqa: F401  (the extension links against torch's libraries)

        # SC_NATIVE_VARIANT=bounds loads the bounds-checked debug build of the same sources instead
        variant = os.environ.get("SC_NATIVE_VARIANT", "")
        _module = importlib.import_module("scalingcontrasts_b200._C" + ("_" + variant if variant else ""))
    except BaseException as error:  # ImportError, or OSError from the dynamic loader
        _error = error


def available() -> bool:
    _try_import()
    return _module is not None


def native():
    """The extension module; raises when it has not been built."""
    _try_import()
    if _module is None:
        raise RuntimeError(
            "scalingcontrasts_b200._C is not built or failed to load "
            f"({_error!r}); build it with: python setup.py build_ext --inplace  (from {_ROOT})")
    return _module


def build(verbose: bool = False) -> None:
    """Compiles every CUDA source for sm_100a in-tree and imports the result."""
    global _module, _error
    environment = dict(os.environ)
    environment.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    command = [sys.executable, "setup.py", "build_ext", "--inplace"]
    result = subprocess.run(command, cwd=_ROOT, env=environment, stdout=None if verbose else subprocess.PIPE,
                            stderr=None if verbose else subprocess.STDOUT, text=True)
    if result.returncode != 0:
        raise RuntimeError("native build failed:\n" + (result.stdout or "")[-8000:])
    _module, _error = None, None
    importlib.invalidate_caches()
    native()
