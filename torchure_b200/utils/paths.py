"""Project directory resolution (reference ``torchure/utils.py:40-43``): checkpoints live under
``$TORCHURE_B200_HOME`` when set, else under the directory that holds the package."""

from __future__ import annotations

import os
from pathlib import Path


def get_project_dir() -> str:
    env = os.environ.get("TORCHURE_B200_HOME")
    if env:
        return env
    return str(Path(__file__).resolve().parents[2])
