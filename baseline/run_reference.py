"""Reference arm of the benchmark: the unmodified reference, through its own Trainer.

The reference package is installed offline into ``baseline/_ref`` (``pip install --no-index
--no-deps --ignore-requires-python --target baseline/_ref``; its metadata pins python 3.14 and
torch 2.10, neither of which exists in this image, so dependency resolution is skipped).  Its
model, DDP, objective, fused linear+CE, optimizer, scheduler, prefetcher and ``train_step`` run
as shipped, including per-block ``torch.compile``.  Only three names of its trainer module are
replaced before the Trainer is built, because the stock ones need the network or a writable
source tree: the tokenizer constructor, the dataset builder (replaced by the same synthetic packed
source our arm uses, with pinned batches) and the checkpoint root.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


class _FakeTokenizer:
    @classmethod
    def from_pretrained(cls, name):
        return cls()


def run_reference(args, cfg: dict, timed_steps, max_over_ranks, ClockSampler) -> None:
    if not os.path.isdir(os.path.join(REF_DIR, "torchure")):
        return _unavailable("baseline/_ref is missing: the reference package was not installed on this box")
    try:
        import torch
        import torch.distributed as dist

        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
        sys.path.insert(0, REF_DIR)
        import torchure.train.trainer as ref_trainer  # noqa: E402
    except Exception as e:  # pragma: no cover - depends on the box
        return _unavailable(f"reference import failed: {type(e).__name__}: {e}"[:200])

    from torchure_b200.data.synthetic import SyntheticLoader
    from torchure_b200.train.train import init_distributed

    rank, local_rank, world = init_distributed()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    vocab = cfg["model"]["config"]["vocab_size"]

    def synthetic_builder(data_cfg, tokenizer, ignore_id, dp_rank, dp_size):
        return SyntheticLoader(seq_len=data_cfg["seq_len"], micro_batch_size=data_cfg["micro_batch_size"],
                               vocab_size=vocab, eos_id=data_cfg.get("eos_id", 0), seed=data_cfg.get("seed", 0),
                               mean_doc_len=data_cfg.get("mean_doc_len", 1024), dp_rank=dp_rank, dp_size=dp_size)

    work = tempfile.mkdtemp(prefix="ref_bench_")
    ref_trainer.Tokenizer = _FakeTokenizer
    ref_trainer.build_dataloader = synthetic_builder
    ref_trainer.PROJECT_DIR = work
    cfg = json.loads(json.dumps(cfg))
    cfg["compile"] = True
    cfg_path = os.path.join(work, f"cfg_rank{rank}.json")
    with open(cfg_path, "w") as f:
        json.dump(cfg, f)

    trainer = ref_trainer.Trainer(cfg_path, rank, local_rank, world, benchmark=True)

    def step():
        metrics, _seconds = trainer.train_step()  # the reference's own sync-bracketed step
        return metrics

    for _ in range(max(5, args.warmup)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    dev_ms, _, _ = timed_steps(step, args.steps, read_loss=False)
    e2e_ms, _, last_loss = timed_steps(step, args.steps, read_loss=True)
    clocks = sampler.stop() if rank == 0 else None
    dev_ms, e2e_ms = max_over_ranks(dev_ms), max_over_ranks(e2e_ms)
    seq = cfg["data"]["seq_len"]
    tokens = seq * cfg["data"]["global_batch_size"] * args.steps
    if rank == 0:
        mbs = cfg["data"]["micro_batch_size"]
        print(json.dumps({
            "metric": "Qwen3-0.6B bf16 global tokens/sec @seq4096 bs2/GPU" if args.model == "0.6b"
                      else "Qwen3-4B bf16 global tokens/sec @seq4096 bs1/GPU",
            "impl": "reference", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(5, args.warmup), "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic packed uniform tokens, random-init weights",
            "config": {"model": f"qwen3-{args.model}", "ffn_dim": cfg["model"]["config"]["ffn_dim"],
                       "global_batch": mbs * world, "micro_batch": mbs, "seq_len": seq, "parallelism": f"dp{world}",
                       "ce_chunk": cfg["objective"]["config"]["ce_chunk_size"], "grad_clip": 1.0,
                       "l2": "per-step working set (>10 GB) exceeds the 126 MB L2; no explicit flush",
                       "torch": torch.__version__, "arch_list": torch.cuda.get_arch_list()},
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 2 * mbs * seq * 8, "d2h_bytes_per_step": 4, "last_loss": last_loss},
            "clocks": clocks, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }), flush=True)
    dist.destroy_process_group()
