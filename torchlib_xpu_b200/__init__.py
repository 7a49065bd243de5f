"""B200-native table-batched-embedding (TBE) and jagged-tensor kernels behind torch.ops.fbgemm.*.

Importing the package loads the C-ABI library (libb200tbe.so) and, when it has been built, the
torch operator library that registers torch.ops.fbgemm.*. There is no CPU or eager fallback: a
missing library is an error.
"""
from __future__ import annotations

from . import cabi  # noqa: F401

__all__ = ["cabi", "load_torch_ops"]

_ops_loaded = False


def load_torch_ops() -> None:
    """Registers torch.ops.fbgemm.* (idempotent). Raises a descriptive error when the operator
    library is missing or cannot be loaded."""
    global _ops_loaded
    if _ops_loaded:
        return
    import os

    import torch

    from . import _build

    cabi.lib()
    path = _build.TORCH_OPS_LIB
    if not os.path.exists(path):
        raise RuntimeError(
            "libb200tbe_torch_ops.so is not built (%s). Run `python -m torchlib_xpu_b200._build`." % path)
    try:
        torch.ops.load_library(path)
    except Exception as exc:  # the loader error alone rarely names the cause
        raise RuntimeError(
            "could not load %s: %s\nLikely causes: built against another torch version; an "
            "fbgemm_gpu install that already defines torch.ops.fbgemm.*; libb200tbe.so missing "
            "next to it." % (path, exc)) from exc
    _ops_loaded = True
