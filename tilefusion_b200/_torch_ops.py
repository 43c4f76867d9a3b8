"""Loads the operator layer (``libtilefusion_b200_torch.so``).

Loading the shared object runs its static registrars, after which
``torch.ops.tilefusion.flash_attention`` and the decode operators exist --
the same mechanism as TileFusion's ``python/__init__.py:19-40``.
"""

from __future__ import annotations

from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_BIND_PATH = _PKG / "libtilefusion_b200_torch.so"
_loaded = False


def ensure_loaded() -> None:
    global _loaded
    if _loaded:
        return
    from . import _cabi

    _cabi.lib()
    from .build import build_torch_binding

    build_torch_binding()     # no-op when the library matches the sources
    try:
        torch.ops.load_library(str(_BIND_PATH))
    except OSError as e:  # pragma: no cover - depends on the machine
        raise RuntimeError(f"Failed to load library from {_BIND_PATH}") from e
    _loaded = True
