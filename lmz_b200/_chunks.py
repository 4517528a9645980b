"""ctypes signatures of the additive whole-chunk entry points."""
from __future__ import annotations

import ctypes


def bind(lib) -> None:
    pass
