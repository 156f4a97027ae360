from torchure_b200.ckpt.checkpointer import Checkpointer  # noqa: F401
