"""Loader of the PyTorch extension module `_C` (built in-tree by ultra_ep_b200.build)."""

from __future__ import annotations

import importlib

_C = None


def load():
    """Import ultra_ep_b200._C; a missing extension is an error, there is no fallback."""
    global _C
    if _C is None:
        try:
            import torch  # noqa: F401  (libtorch must be loaded before the extension)

            _C = importlib.import_module("ultra_ep_b200._C")
        except ImportError as e:
            raise ImportError(
                "ultra_ep_b200._C is not built or cannot be loaded; run `python -m ultra_ep_b200.build` "
                f"(there is no non-CUDA fallback): {e}") from e
    return _C
