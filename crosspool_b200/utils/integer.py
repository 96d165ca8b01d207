"""Range checks for integers that cross into native code (ctypes silently wraps out-of-range values).
Reference: src/xpool/utils/integer.py."""

from __future__ import annotations

UINT64_MAX = (1 << 64) - 1
SINT64_MAX = (1 << 63) - 1
UINT32_MAX = (1 << 32) - 1


def _ints(values) -> None:
    for v in values:
        if isinstance(v, bool) or not hasattr(v, "__index__"):      # NumPy and torch integer scalars pass
            raise TypeError(f"expected an integer, got {type(v).__name__} ({v!r})")


def ensure_uint64(*values: int) -> None:
    _ints(values)
    for v in values:
        if not 0 <= v <= UINT64_MAX:
            raise OverflowError(f"{v} does not fit an unsigned 64-bit integer")


def ensure_uint32(*values: int) -> None:
    _ints(values)
    for v in values:
        if not 0 <= v <= UINT32_MAX:
            raise OverflowError(f"{v} does not fit an unsigned 32-bit integer")


def ensure_sint64_nonnegative(*values: int) -> None:
    _ints(values)
    for v in values:
        if not 0 <= v <= SINT64_MAX:
            raise OverflowError(f"{v} is negative or does not fit a signed 64-bit integer")
