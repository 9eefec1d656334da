"""Process-grid factorisation (reference: include/utils/decomp.hpp:23-56)."""
from __future__ import annotations

import math
from typing import Tuple


def npfactx(np_: int) -> Tuple[int, int]:
    return np_, 1


def npfacty(np_: int) -> Tuple[int, int]:
    return 1, np_


def npfact2d(np_: int, row_master: bool = True) -> Tuple[int, int]:
    """Split ``np_`` into nx*ny with the smaller factor the largest divisor <= sqrt(np_);
    a prime count degenerates to np_ x 1 (or 1 x np_ when ``row_master`` is false)."""
    up = int(math.isqrt(np_))
    while up > 1:
        if np_ % up == 0:
            return (up, np_ // up) if row_master else (np_ // up, up)
        up -= 1
    return (np_, 1) if row_master else (1, np_)
