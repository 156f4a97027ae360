"""Poison-and-verify mode for the kernel wrappers (race / coverage detection without a sanitizer).

With ``TORCHURE_B200_POISON=1`` (or ``enable()``), every output buffer that ``ops/kernels.py`` allocates for a kernel
that must overwrite it completely is first filled with NaN and remembered; ``verify()`` synchronises and raises if
any remembered buffer still holds a NaN, naming the wrapper that allocated it.  A kernel that skips a tile, a row or
a tail element, or a consumer that runs before its producer, shows up as a surviving sentinel.  Inputs containing NaN
are the caller's business: use finite test data.  Costs one fill per output, so it is a debugging mode only.
"""

from __future__ import annotations

import os

import torch

_enabled = os.environ.get("TORCHURE_B200_POISON", "0") == "1"
_pending: list[tuple[str, torch.Tensor]] = []


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = on
    if not on:
        _pending.clear()


def enabled() -> bool:
    return _enabled


def new_output(name: str, *shape, dtype, device) -> torch.Tensor:
    """``torch.empty`` for a kernel output; poisoned and tracked when the mode is on."""
    t = torch.empty(*shape, dtype=dtype, device=device)
    if _enabled and t.is_floating_point():
        t.fill_(float("nan"))
        _pending.append((name, t))
    return t


def verify() -> int:
    """Check every tracked output; returns how many were checked.  Raises on a surviving sentinel."""
    if not _pending:
        return 0
    torch.cuda.synchronize()
    bad = []
    for name, t in _pending:
        n = int(torch.isnan(t).sum().item())
        if n:
            bad.append(f"{name}: {n} of {t.numel()} elements of shape {tuple(t.shape)} were never written")
    checked = len(_pending)
    _pending.clear()
    if bad:
        raise RuntimeError("poison check failed:\n  " + "\n  ".join(bad))
    return checked
