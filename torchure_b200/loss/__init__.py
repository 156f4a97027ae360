from torchure_b200.loss.cross_entropy import cross_entropy_loss, shift_labels  # noqa: F401
from torchure_b200.loss.fused_linear_ce import fused_linear_cross_entropy  # noqa: F401
