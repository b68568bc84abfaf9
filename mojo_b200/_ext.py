"""Loader of the native extension (`mojo_b200/_C*.so` + `mojo_b200/lib/libb2kernels.so`).

The extension is built in-tree by `python -m mojo_b200.build`. There is no silent fallback: code that needs a
kernel calls `require()` and gets an ImportError naming the build command when the shared objects are missing.
CPU-only hosts still get the engine runtime (KV manager, scheduler) from the same module.
"""
from __future__ import annotations

import ctypes
import importlib
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_C = None
_err: Exception | None = None
_lib = None


def _load():
    global _C, _err
    if _C is not None or _err is not None:
        return
    try:
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        _C = importlib.import_module("mojo_b200._C")
    except Exception as e:  # noqa: BLE001
        _err = e


def available() -> bool:
    _load()
    return _C is not None


def require():
    """Return the extension module or raise with the build instruction."""
    _load()
    if _C is None:
        raise ImportError(
            "mojo_b200 native extension is not built or failed to load "
            f"({_err!r}); run `python -m mojo_b200.build` in the source tree"
        )
    return _C


def kernels_lib() -> ctypes.CDLL:
    """The plain-C kernel library, for callers that bypass PyTorch (ctypes)."""
    global _lib
    if _lib is None:
        path = _ROOT / "lib" / "libb2kernels.so"
        if not path.exists():
            raise ImportError(f"{path} missing; run `python -m mojo_b200.build`")
        _lib = ctypes.CDLL(str(path))
    return _lib
