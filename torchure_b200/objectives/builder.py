"""Objective registry (reference ``torchure/objectives/builder.py:9-16``)."""

from torchure_b200.objectives.autoregressive import ARObjective

OBJECTIVES = {"AR": ARObjective}


def build_objective(name: str, cfg: dict):
    if name not in OBJECTIVES:
        raise KeyError(f"unknown objective {name!r}; known: {sorted(OBJECTIVES)}")
    return OBJECTIVES[name](**cfg)
