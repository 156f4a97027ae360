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


def run_reference(args, cfg: dict, timed_steps, max_over_ranks, ClockSampler, shared_config, kernel_census) -> None:
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

    def synced_step():
        metrics, _seconds = trainer.train_step()  # the reference's own sync-bracketed step
        return metrics

    # `train_step` is the step body wrapped by the reference's `record_time` closure (two device synchronisations
    # per step).  The body itself, unwrapped, is timed as the headline so that neither arm drains the queue inside
    # the timed region; the wrapped call is timed as `synced`.
    wrapped = type(trainer).train_step
    body = None
    for cell in getattr(wrapped, "__closure__", None) or ():
        if callable(cell.cell_contents):
            body = cell.cell_contents
    step = (lambda: body(trainer)) if body is not None else synced_step

    for _ in range(max(5, args.warmup)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    dev_ms, _, _ = timed_steps(step, args.steps, read_loss=False)
    e2e_ms, _, last_loss = timed_steps(step, args.steps, read_loss=True)
    sync_ms, _, _ = timed_steps(synced_step, args.steps, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    dev_ms, e2e_ms, sync_ms = max_over_ranks(dev_ms), max_over_ranks(e2e_ms), max_over_ranks(sync_ms)
    census = None
    if getattr(args, "census", 0):
        census = kernel_census(step) if rank == 0 else step()
    seq = cfg["data"]["seq_len"]
    tokens = seq * cfg["data"]["global_batch_size"] * args.steps
    if rank == 0:
        mbs = cfg["data"]["micro_batch_size"]
        shared = shared_config(args.model, cfg, world, cfg["objective"]["config"]["ce_chunk_size"])
        shared["sync_per_step"] = body is None
        print(json.dumps({
            "metric": "Qwen3-0.6B bf16 global tokens/sec @seq4096 bs2/GPU" if args.model == "0.6b"
                      else "Qwen3-4B bf16 global tokens/sec @seq4096 bs1/GPU",
            "impl": "reference", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(5, args.warmup), "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic packed uniform tokens, random-init weights",
            "config": shared,
            "torch": torch.__version__, "arch_list": torch.cuda.get_arch_list(),
            "synced": {"value": tokens / (sync_ms / 1e3), "unit": "tokens/s", "ms_per_step": sync_ms / args.steps,
                       "note": "device synchronize before and after every step (the reference's record_time)"},
            "kernel_census": census,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 2 * mbs * seq * 8, "d2h_bytes_per_step": 4, "last_loss": last_loss},
            "clocks": clocks, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }), flush=True)
    dist.destroy_process_group()
