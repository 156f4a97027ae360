"""Dataloader construction (reference ``torchure/dataloader/builder.py:50-113``).

Two sources behind one call:

* ``data.synthetic: true`` (or ``data.name == "synthetic"``): the seeded synthetic packed
  source of ``data/synthetic.py``; needs no tokenizer and no network.
* otherwise a HuggingFace streaming dataset: shuffle buffer -> per-dp-coordinate shard ->
  tokenizer + stream packer as a batched ``map`` -> torchdata ``StatefulDataLoader`` with
  pinned batches, whose ``state_dict`` is what ``dataloader_dp{r}.pt`` stores.
"""

from __future__ import annotations

import torch

from torchure_b200.data.packers import BESTFIT_PACKERS, PACKERS
from torchure_b200.data.synthetic import SyntheticLoader


class Collator:
    """Stack packed rows; labels are a clone (shifting is the objective's job)."""

    def __init__(self, tokenizer=None, ignore_index: int = -100):
        self.tokenizer = tokenizer
        self.ignore_index = ignore_index

    def __call__(self, examples):
        ids = torch.tensor([ex["input_ids"] for ex in examples], dtype=torch.long)
        return {"input_ids": ids, "labels": ids.clone()}


def is_synthetic(data_cfg: dict) -> bool:
    return bool(data_cfg.get("synthetic", False)) or data_cfg.get("name") == "synthetic"


def build_dataloader(data_cfg: dict, tokenizer, ignore_id: int, dp_rank: int, dp_size: int):
    if is_synthetic(data_cfg):
        return SyntheticLoader(
            seq_len=data_cfg["seq_len"], micro_batch_size=data_cfg["micro_batch_size"],
            vocab_size=data_cfg["vocab_size"], eos_id=data_cfg.get("eos_id", 0), seed=data_cfg.get("seed", 0),
            mean_doc_len=data_cfg.get("mean_doc_len", 1024), dp_rank=dp_rank, dp_size=dp_size,
        )
    import datasets
    from datasets.distributed import split_dataset_by_node
    from torchdata.stateful_dataloader import StatefulDataLoader

    ds = datasets.load_dataset(data_cfg["name"], data_cfg.get("config"), split=data_cfg.get("split", "train"),
                               streaming=True)
    if dp_rank == 0:
        print(f"num shards: {ds.num_shards}")
    if data_cfg["text_field"] != "text":
        ds = ds.rename_column(data_cfg["text_field"], "text")
    ds = ds.shuffle(buffer_size=data_cfg["shuffle_buffer"], seed=data_cfg["seed"])
    ds = split_dataset_by_node(ds, rank=dp_rank, world_size=dp_size)
    eos_id = tokenizer.token_to_id(data_cfg["eos_token"])
    pad_id = tokenizer.token_to_id(data_cfg["pad_token"])
    assert eos_id is not None, f"eos_token {data_cfg['eos_token']!r} is not in the tokenizer vocabulary"
    assert pad_id is not None, f"pad_token {data_cfg['pad_token']!r} is not in the tokenizer vocabulary"
    kind = data_cfg.get("packer", "list")
    packer_cls = {**PACKERS, **BESTFIT_PACKERS}[kind]
    packer = packer_cls(tokenizer, data_cfg["seq_len"], eos_id, pad_id)
    ds = ds.map(packer, batched=True, batch_size=data_cfg.get("pack_batch", 1000), remove_columns=ds.column_names)
    workers = data_cfg["num_workers"]
    return StatefulDataLoader(ds, batch_size=data_cfg["micro_batch_size"], num_workers=workers,
                              collate_fn=Collator(tokenizer, ignore_id), persistent_workers=workers > 0,
                              pin_memory=torch.cuda.is_available())
