"""Hand-written sm_100a kernels and their plain PyTorch oracles.

``available()`` is true when the CUDA extension (``torchure_b200/_C*.so``, built in-tree
by ``python -m torchure_b200.build``) is loaded and a Blackwell GPU is present.  On a
machine with a GPU, a missing extension is an error, not a silent fallback: set
``TORCHURE_B200_ALLOW_FALLBACK=1`` to run the PyTorch oracle path on purpose.
"""

from __future__ import annotations

import os

import torch

_EXT = None
_TRIED = False


def ext():
    """The loaded extension module, or None."""
    global _EXT, _TRIED
    if not _TRIED:
        _TRIED = True
        try:
            from torchure_b200 import _C  # type: ignore

            _EXT = _C
        except ImportError as e:  # not built
            _EXT = None
            if torch.cuda.is_available() and os.environ.get("TORCHURE_B200_ALLOW_FALLBACK") != "1":
                raise RuntimeError(
                    "a GPU is present but the torchure_b200 CUDA extension is not built "
                    "(run `python -m torchure_b200.build`); set TORCHURE_B200_ALLOW_FALLBACK=1 "
                    "to use the PyTorch oracle path deliberately") from e
    return _EXT


_FORCED_OFF = False


def force_fallback(flag: bool = True) -> None:
    """Route every op to its PyTorch oracle (used by A/B tests)."""
    global _FORCED_OFF
    _FORCED_OFF = flag


def available() -> bool:
    if _FORCED_OFF or not torch.cuda.is_available():
        return False
    if ext() is None:
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


# launch counter: every Python wrapper that launches one of OUR kernels adds to it
_LAUNCHES = 0


def count_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launches() -> int:
    return _LAUNCHES


def reset_launches() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def set_compute_sm_reserve(n: int) -> None:
    """Persistent compute kernels (GEMM) launch on `SM count - n` CTAs, leaving room for communication kernels
    that must be resident at the same time as the backward pass they overlap."""
    e = ext()
    if e is not None:
        e.set_sm_reserve(int(n))
