from torchure_b200.models.builder import MODELS, build_model  # noqa: F401
from torchure_b200.models.llama3 import Llama3  # noqa: F401
from torchure_b200.models.qwen3 import Qwen3, flops_per_token  # noqa: F401
from torchure_b200.models.qwen3_moe import Qwen3MoE  # noqa: F401
