"""The llama graph over GGUF files as a registered model family (see models.py)."""
from __future__ import annotations

from .models import Family, register


def _open(src, **kw):
    from .engine import Engine
    return Engine(src.gguf, **kw)


LLAMA = register(Family(name="llama", source="gguf", open_engine=_open))
