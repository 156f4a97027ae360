"""Tiny model / config factories shared by the CPU tests."""

from __future__ import annotations

TINY = dict(num_layers=2, num_heads=2, num_kv_heads=1, emb_dim=32, head_dim=16, vocab_size=64, ffn_dim=64)

# the "plumbing and parity" configuration: hidden 256, 4 layers, 4/2 heads, head_dim 64, ffn 768, vocab 4096
PARITY = dict(num_layers=4, num_heads=4, num_kv_heads=2, emb_dim=256, head_dim=64, vocab_size=4096, ffn_dim=768,
              norm_eps=1e-6, rope_theta=1e6)


def parity_config(world: int, steps: int = 5, run_name: str = "parity", accumulation: int = 2, resume=None,
                  save_steps: int = 1000, mesh: dict | None = None) -> dict:
    return {
        "model": {"name": "qwen3_dense", "config": dict(PARITY)},
        "mesh": dict(mesh) if mesh is not None else {"dp": world},
        "seed": 1234,
        "optimizer": {"name": "adamw", "config": {"lr": 3e-4, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                  "fused": False},
                      "max_norm": 1.0,
                      "scheduler": {"type": "wsd", "warmup_ratio": 0.2, "decay_ratio": 0.2, "total_steps": steps}},
        "objective": {"name": "AR", "config": {"ignore_index": -100, "fused_linear_ce": True, "ce_chunk_size": 128}},
        "data": {"name": "synthetic", "synthetic": True, "seed": 7, "mean_doc_len": 128, "eos_id": 0,
                 "num_workers": 0, "global_batch_size": 2 * world * accumulation, "micro_batch_size": 2,
                 "seq_len": 256},
        "ddp": {"bucket_mb": 0.25},
        "checkpointing": {"save_steps": save_steps, "resume": resume},
        "run_name": run_name,
    }
