"""Merge the per-coordinate model files of a checkpoint into the unsharded layout.

Strategies that split tensors write one ``model_shard{k}.pt`` per coordinate of their axis (tensor parallel: rows or
columns of every block matrix; pipeline: the blocks of a stage under the keys of the whole model; expert parallel: a
slice of every layer's stacked experts).  ``merge_model_shards`` rebuilds the ``model.pt`` a run without that axis
writes (the reference's layout, ``torchure/checkpoint/checkpointer.py:18-102``), so a sharded run's weights can be
loaded by the dense model, by another mesh, or by external tooling::

    python -m torchure_b200.ckpt.merge checkpoints/<run_name> <step> [--out model.pt]

FSDP / HSDP checkpoints already hold an unsharded ``model.pt``.
"""

from __future__ import annotations

import argparse
import os

import torch

from torchure_b200.ckpt.checkpointer import Checkpointer

# module-path suffixes of the matrices tensor parallelism splits, and the dimension it splits them along
_TP_ROWS = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")
_TP_COLS = ("o_proj.weight", "down_proj.weight")
_EP_STACKED = ("ffn.w_gate", "ffn.w_up", "ffn.w_down")


def split_axis(mesh: dict) -> str | None:
    for axis in ("tp", "pp", "ep"):
        if mesh.get(axis, 1) > 1:
            return axis
    return None


def merge_state_dicts(shards: list[dict], axis: str) -> dict:
    """`shards` in coordinate order along `axis` ("tp", "pp" or "ep")."""
    if axis == "pp":
        out: dict = {}
        for sd in shards:
            out.update(sd)      # disjoint blocks; a tied embedding appears as token_emb on the first stage and as
        return out              # lm_head on the last, which is how the whole model's state dict lists it too
    out = {}
    for key, first in shards[0].items():
        if axis == "tp" and key.endswith(_TP_ROWS):
            out[key] = torch.cat([sd[key] for sd in shards], dim=0)
        elif axis == "tp" and key.endswith(_TP_COLS):
            out[key] = torch.cat([sd[key] for sd in shards], dim=1)
        elif axis == "ep" and key.endswith(_EP_STACKED):
            out[key] = torch.cat([sd[key] for sd in shards], dim=0)
        else:
            out[key] = first    # replicated
    return out


def merge_model_shards(root: str, step: int) -> dict:
    """The unsharded model state dict of checkpoint `step` under `root` (``checkpoints/<run_name>``)."""
    ck = Checkpointer(root)
    assert ck.valid_step(step) is not None, f"checkpoint step {step} under {root} does not exist or is incomplete"
    mesh = ck.load_trainer(step)["config"]["mesh"]
    axis = split_axis(mesh)
    if axis is None:
        return ck._read(step, "model.pt")
    return merge_state_dicts([ck._read(step, f"model_shard{k}.pt") for k in range(mesh[axis])], axis)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("root", help="checkpoint directory of the run (checkpoints/<run_name>)")
    ap.add_argument("step", type=int)
    ap.add_argument("--out", default=None, help="where to write the merged state dict (default: <root>/<step>/model.pt)")
    args = ap.parse_args()
    merged = merge_model_shards(args.root, args.step)
    out = args.out or os.path.join(args.root, str(args.step), "model.pt")
    tmp = out + ".tmp"
    torch.save(merged, tmp)
    os.replace(tmp, out)
    print(f"wrote {out}: {len(merged)} tensors, {sum(v.numel() for v in merged.values()):,} elements")


if __name__ == "__main__":
    main()
