from torchure_b200.objectives.autoregressive import ARObjective  # noqa: F401
from torchure_b200.objectives.builder import OBJECTIVES, build_objective  # noqa: F401
