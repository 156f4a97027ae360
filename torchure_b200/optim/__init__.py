from torchure_b200.optim.adamw import AdamW  # noqa: F401
from torchure_b200.optim.builder import build_optimizer, build_scheduler  # noqa: F401
from torchure_b200.optim.scheduler import CosineWithWarmup, WarmupStableDecay, wsd_scale  # noqa: F401
