"""B200-native table-batched-embedding (TBE) and jagged-tensor kernels behind torch.ops.fbgemm.*.

Importing the package loads the C-ABI library (libb200tbe.so) and the torch operator library on top
of it, which registers torch.ops.fbgemm.* as a side effect of being loaded -- the same contract as
the reference plugin, whose import registers it with its host framework
(packages/torchcodec-xpu/src/torchcodec_xpu/__init__.py:25-32 and :56). There is no CPU or eager
fallback: a missing library is an error.
"""
from __future__ import annotations

import os

from . import cabi  # noqa: F401

__all__ = ["cabi", "load_torch_ops"]

_ops_loaded = False


def load_torch_ops() -> None:
    """Registers torch.ops.fbgemm.* (idempotent; runs at import). Raises a descriptive error when
    the operator library is missing or cannot be loaded."""
    global _ops_loaded
    if _ops_loaded:
        return
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


def _build_in_progress() -> bool:
    """True while the libraries are being (re)built: `python -m torchlib_xpu_b200._build`, or a
    caller that sets B200TBE_BUILDING=1 around its call of _build.build_all()."""
    import sys

    if os.environ.get("B200TBE_BUILDING") == "1":
        return True
    return any(a.endswith("torchlib_xpu_b200._build") for a in getattr(sys, "orig_argv", []))


# Registration is the import's side effect, as in the reference plugin. Only the build, which has
# to import the package's _build module before the libraries exist (or while they are stale),
# goes without.
if not _build_in_progress():
    load_torch_ops()
