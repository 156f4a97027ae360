from torchure_b200.parallel.ddp import DDP, plan_buckets  # noqa: F401
