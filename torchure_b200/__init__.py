"""torchure_b200: a Blackwell (sm_100a) native LLM pretraining stack.

Layers, bottom to top:

* ``core``       named device mesh, mesh-aware collectives, symmetric memory, grad clipping
* ``ops``        hand-written sm_100a kernels (tcgen05 GEMM, attention, norms, RoPE, CE,
                 AdamW, NVLink collectives) with plain PyTorch oracles of the same ops
* ``parallel``   DDP (fused bucket all-reduce), FSDP/HSDP, tensor/sequence, context,
                 expert and pipeline parallel building blocks
* ``models``     Qwen3 dense (and the llama3 variant of the same block)
* ``loss`` / ``objectives`` / ``optim`` / ``data`` / ``ckpt``  workload plug-ins
* ``train``      trainer, CLI entry point and the overlap profiler
"""

__version__ = "0.1.0"
