"""JSON run configuration: loading, defaults and validation.

Schema (superset of the reference's seven ``configs/*.json``; reference readers:
``torchure/train/trainer.py:73-133``)::

    model         {name, config{num_layers, num_heads, num_kv_heads, emb_dim, head_dim, vocab_size,
                   [ffn_dim], [norm_eps], [rope_theta], [impl]}}
    mesh          {axis: size, ...}   product == WORLD_SIZE.  Data axes: "dp" (DDP), or "dp_shard" (FSDP2) with an
                  optional "dp_replicate" in front of it (HSDP); at least one is required.  After "dp", one of:
                  "tp" shards every block (Megatron column / row split); "cp" splits every sequence into zigzag
                  chunks and runs attention as a ring; "pp" cuts the blocks into pipeline stages; "ep" (model
                  "qwen3_moe") spreads the experts of every layer and is a data axis as well.
    optimizer     {name, config{lr, weight_decay, betas, fused}, [max_norm],
                   scheduler{type, warmup_ratio, decay_ratio, total_steps}}
    objective     {name, config{ignore_index, fused_linear_ce, ce_chunk_size}}
    data          {name | synthetic, tokenizer, eos_token, pad_token, text_field, shuffle_buffer, seed,
                   num_workers, global_batch_size, micro_batch_size, seq_len, [pack_batch], [packer],
                   synthetic extras: vocab_size, eos_id, mean_doc_len}
    [ddp]         {bucket_mb, [fused], [merge_small], [comm_sms], [early_embedding]}
    [fsdp]        {[comm_sms]}
    [tp]          {[sequence_parallel], [loss_parallel]: the fused CE computes V / tp rows of the head per rank}
    [cp]          {[kind]: "ring" | "ulysses"}     with mesh {"dp": D, "cp": C}: zigzag ring attention, or heads <->
                  sequence all-to-alls around whole-sequence attention
    [pp]          {[schedule]: "1f1b" | "gpipe"}   with mesh {"dp": D, "pp": P}: contiguous stages of blocks
    [comm]        {backend: "sm100" | "torch", [max_bytes]}
    checkpointing {save_steps, resume: null|"auto"|int, [resume_scheduler], [keep_last]: complete steps kept on disk,
                   [async]: files written by a background thread from host snapshots,
                   [on_signal]: checkpoint and leave at the next log cadence after SIGTERM / SIGUSR1}
    run_name      str
    [eval]        {every: steps between held-out evaluations (0 = never), [batches]: micro-batches per rank,
                   [data]: overrides of the data section for the held-out stream}
    [init_from]   str    path of an unsharded model state dict to start from (any mesh; optimizer state starts fresh)
    [wandb]       {enabled, project, entity}
    [compile]     bool   per-block fused execution (hand-written kernels) on/off
    [torch_compile] bool, [compile_mode] str, [compile_backend] str
                  with compile=false: torch.compile every block of the PyTorch path
    [log_every]   int
"""

from __future__ import annotations

import json
import math

DATA_AXES = ("dp", "dp_replicate", "dp_shard")
MESH_AXES = DATA_AXES + ("tp", "cp", "pp", "ep")
REQUIRED = ("model", "mesh", "optimizer", "objective", "data", "checkpointing", "run_name")


class ConfigError(ValueError):
    pass


def load_config(path: str) -> dict:
    with open(path) as f:
        cfg = json.load(f)
    return validate_config(cfg)


def validate_config(cfg: dict, world_size: int | None = None) -> dict:
    for key in REQUIRED:
        if key not in cfg:
            raise ConfigError(f"config is missing the {key!r} section")
    mesh = cfg["mesh"]
    unknown = [a for a in mesh if a not in MESH_AXES]
    if unknown:
        raise ConfigError(f"unknown mesh axes {unknown}; known: {list(MESH_AXES)}")
    if mesh.get("ep", 1) > 1:
        if list(mesh)[: 2] != ["dp", "ep"] or len(mesh) != 2:
            raise ConfigError('expert parallelism is selected by mesh {"dp": D, "ep": E} (in this order, no other axis)')
        experts = cfg["model"]["config"].get("num_experts", 0) if cfg["model"].get("name") == "qwen3_moe" else 0
        if experts == 0 or experts % mesh["ep"] != 0:
            raise ConfigError('"ep" needs the mixture-of-experts model ("qwen3_moe") with num_experts divisible by ep')
    if mesh.get("tp", 1) > 1 and ("dp_shard" in mesh or "dp_replicate" in mesh):
        raise ConfigError('"tp" combines with "dp" only (not with "dp_shard" / "dp_replicate")')
    data_axes = [a for a in mesh if a in DATA_AXES]
    if not data_axes:
        raise ConfigError('mesh must define a data axis: "dp", or "dp_shard" (optionally after "dp_replicate")')
    if "dp" in mesh and ("dp_shard" in mesh or "dp_replicate" in mesh):
        raise ConfigError('"dp" (DDP) cannot be combined with "dp_shard" / "dp_replicate" (FSDP / HSDP)')
    if "dp_replicate" in mesh and "dp_shard" not in mesh:
        raise ConfigError('"dp_replicate" needs a "dp_shard" axis (HSDP); use "dp" for plain replication')
    if "dp_replicate" in mesh and list(mesh).index("dp_replicate") > list(mesh).index("dp_shard"):
        raise ConfigError('"dp_replicate" must come before "dp_shard" in the mesh')
    if mesh.get("cp", 1) > 1:
        if list(mesh)[: 2] != ["dp", "cp"] or len(mesh) != 2:
            raise ConfigError('context parallelism is selected by mesh {"dp": D, "cp": C} (in this order, no other axis)')
        if cfg.get("data", {}).get("seq_len", 0) % (2 * mesh["cp"]) != 0:
            raise ConfigError(f"seq_len must be a multiple of 2 x cp = {2 * mesh['cp']} (zigzag chunks)")
        kind = cfg.get("cp", {}).get("kind", "ring")
        if kind not in ("ring", "ulysses"):
            raise ConfigError('cp.kind must be "ring" or "ulysses"')
        if kind == "ulysses" and cfg["model"]["config"].get("num_kv_heads", mesh["cp"]) % mesh["cp"] != 0:
            raise ConfigError("Ulysses needs the number of KV heads to be a multiple of cp")
    if mesh.get("pp", 1) > 1:
        if list(mesh)[: 2] != ["dp", "pp"] or len(mesh) != 2:
            raise ConfigError('pipeline parallelism is selected by mesh {"dp": D, "pp": P} (in this order, no other axis)')
        if cfg["model"]["config"].get("num_layers", mesh["pp"]) < mesh["pp"]:
            raise ConfigError("more pipeline stages than transformer blocks")
        if cfg.get("pp", {}).get("schedule", "1f1b") not in ("1f1b", "gpipe"):
            raise ConfigError('pp.schedule must be "1f1b" or "gpipe"')
    if world_size is not None and math.prod(mesh.values()) != world_size:
        raise ConfigError(f"mesh {mesh} does not cover world size {world_size}")
    opt = cfg["optimizer"]
    for key in ("name", "config", "scheduler"):
        if key not in opt:
            raise ConfigError(f"optimizer.{key} is required")
    sched = opt["scheduler"]
    for key in ("type", "total_steps"):
        if key not in sched:
            raise ConfigError(f"optimizer.scheduler.{key} is required")
    data = cfg["data"]
    for key in ("global_batch_size", "micro_batch_size", "seq_len"):
        if key not in data:
            raise ConfigError(f"data.{key} is required")
    dp = math.prod(mesh[a] for a in data_axes) * mesh.get("ep", 1)      # the ranks of an ep group read different rows
    per_backward = data["micro_batch_size"] * dp
    if data["global_batch_size"] % per_backward != 0:
        raise ConfigError(
            f"global_batch_size {data['global_batch_size']} must be divisible by micro_batch_size "
            f"{data['micro_batch_size']} x dp {dp} = {per_backward}")
    ck = cfg["checkpointing"]
    if "save_steps" not in ck or "resume" not in ck:
        raise ConfigError("checkpointing needs save_steps and resume")
    if not (ck["resume"] is None or ck["resume"] == "auto" or isinstance(ck["resume"], int)):
        raise ConfigError('checkpointing.resume must be null, "auto" or a step number')
    return cfg
