"""Parallelism strategies: DDP (fused NVLink reducer), FSDP/HSDP, tensor/sequence, context (ring attention),
Ulysses, expert and pipeline parallelism, plus placement bookkeeping."""

from torchure_b200.parallel.ddp import DDP, plan_buckets  # noqa: F401
