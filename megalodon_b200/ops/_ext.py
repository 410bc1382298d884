"""Loader for the in-tree CUDA extension `megalodon_b200/_C*.so`.

The extension is built in-tree by `python setup.py build_ext --inplace` (or
`__graft_entry__.build()`).  On a machine with a GPU a missing extension is an
error: operators never fall back silently to library kernels unless
`MEGALODON_B200_ALLOW_FALLBACK=1` is set explicitly.
"""
from __future__ import annotations

import importlib
import os

_EXT = None
_ERR = None


def load():
    global _EXT, _ERR
    if _EXT is not None or _ERR is not None:
        return _EXT
    try:
        import torch  # noqa: F401  (the extension links against libtorch)
        _EXT = importlib.import_module("megalodon_b200._C")
    except Exception as e:  # noqa: BLE001
        _ERR = e
    return _EXT


def have_ext() -> bool:
    return load() is not None


def allow_fallback() -> bool:
    return os.environ.get("MEGALODON_B200_ALLOW_FALLBACK", "0") == "1"


def require():
    ext = load()
    if ext is None:
        raise RuntimeError(
            "megalodon_b200._C (the sm_100a CUDA extension) is not built or failed to load: "
            f"{_ERR!r}.  Build it with `python setup.py build_ext --inplace`, or set "
            "MEGALODON_B200_ALLOW_FALLBACK=1 to run the PyTorch reference operators.")
    return ext


def native_for(t) -> bool:
    """True when operator calls on tensor `t` must take the CUDA-kernel path."""
    if not t.is_cuda:
        return False
    if have_ext():
        return True
    if allow_fallback():
        return False
    require()
    return False
