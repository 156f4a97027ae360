from torchure_b200.core.collective import (all_gather, all_reduce, all_to_all, barrier, broadcast,  # noqa: F401
                                           reduce_scatter, ring_send_recv, send_recv)
from torchure_b200.core.grad_helper import clip_grad_norm, grad_norm_and_coef  # noqa: F401
from torchure_b200.core.mesh import Mesh  # noqa: F401
