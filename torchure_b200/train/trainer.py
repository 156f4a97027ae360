"""Training orchestration.

Lifecycle (reference ``torchure/train/trainer.py:61-146``): mesh -> model -> init ->
parallelize -> objective -> optimizer -> scheduler -> data -> resume -> prefetcher.
The mesh of the config selects the strategy: ``dp`` builds DDP; ``dp_shard`` (optionally after
``dp_replicate``) builds FSDP2 / HSDP (``parallel/fsdp_engine.py`` on the sm_100a engine,
``parallel/fsdp.py`` hooks on the PyTorch path); after ``dp``, one more axis selects a model-parallel
family: ``tp`` shards every block (``parallel/tensor_parallel.py``; ``tp.sequence_parallel``,
``tp.loss_parallel``), ``cp`` splits every sequence (ring attention inside the engine, or Ulysses with
``cp.kind``), ``pp`` cuts the blocks into pipeline stages (``_pipeline_step``), ``ep`` spreads the experts of the
mixture-of-experts model (``_expert_step``).
One optimizer step (reference ``trainer.py:371-402``): K micro-batches of forward+backward
with ``requires_sync`` only on the last, ``ddp.sync()``, global grad-norm clip, optimizer,
``zero_grad``, scheduler, loss averaged over dp.

GPU specifics: gradient buckets are reduced by the fused NVLink kernel, the clip
coefficient stays on the device and is applied inside the AdamW kernel, and nothing in a
step reads a device value on the host; only the logging cadence synchronises.
"""

from __future__ import annotations

import os
from datetime import datetime

import torch

from torchure_b200.ckpt import Checkpointer
from torchure_b200.config import DATA_AXES, load_config, validate_config
from torchure_b200.core.collective import all_reduce, barrier, enable_sm100
from torchure_b200.core.grad_helper import clip_grad_norm, grad_norm_and_coef
from torchure_b200.core.mesh import Mesh
from torchure_b200.data import CUDAPrefetcher, build_dataloader, is_synthetic
from torchure_b200.models import build_model
from torchure_b200.objectives import build_objective
from torchure_b200.optim import build_optimizer, build_scheduler
from torchure_b200.parallel.ddp import DDP
from torchure_b200.utils import debug_time, get_project_dir, record_time

try:
    import wandb  # type: ignore

    HAS_WANDB = True
except Exception:  # pragma: no cover - optional dependency
    wandb = None
    HAS_WANDB = False

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


class Trainer:
    def __init__(self, config: str | dict, rank: int, local_rank: int, world_size: int, benchmark: bool = False,
                 device: str | None = None):
        self.config = load_config(config) if isinstance(config, str) else validate_config(config)
        validate_config(self.config, world_size)
        self.rank, self.world_size, self.benchmark = rank, world_size, benchmark
        if device is None:
            device = f"cuda:{local_rank}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        if self.on_gpu:
            torch.cuda.set_device(self.device)
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
        self.mesh = Mesh(self.config["mesh"])
        # the data axis: "dp", "dp_shard", or the row-major product of ("dp_replicate", "dp_shard")
        data_axes = tuple(a for a in self.mesh.axes() if a in DATA_AXES)
        if len(data_axes) > 1:
            self.mesh.flatten(data_axes, "data")
            self.data_axis = "data"
        else:
            self.data_axis = data_axes[0]
        self.dp_size = self.mesh.size(self.data_axis)
        # gradients (and the reported loss) are averaged over every replica of the parameters: the data axis and,
        # under context parallelism, the ranks that hold the other chunks of the same sequences
        self.cp_size = self.mesh.size("cp") if "cp" in self.mesh.axes() else 1
        self.pp_size = self.mesh.size("pp") if "pp" in self.mesh.axes() else 1
        self.ep_size = self.mesh.size("ep") if "ep" in self.mesh.axes() else 1
        if self.ep_size > 1:
            # the ranks of an expert-parallel group read different rows: the axis is a data axis as well, and the
            # shared (non-expert) parameters are averaged over dp x ep
            assert data_axes == ("dp",) and len(self.mesh.axes()) == 2, "ep combines with plain dp only"
            self.mesh.flatten(("dp", "ep"), "dp_ep")
            self.data_axis = self.grad_axis = "dp_ep"
            self.dp_size = self.mesh.size("dp_ep")
        self.grad_axis = self.data_axis
        if self.cp_size > 1:
            assert data_axes == ("dp",) and "tp" not in self.mesh.axes(), "cp combines with plain dp only"
            self.mesh.flatten(("dp", "cp"), "dp_cp")
            self.grad_axis = "dp_cp"
        comm_cfg = self.config.get("comm", {})
        if self.on_gpu and comm_cfg.get("backend", "sm100") == "sm100":
            from torchure_b200 import ops

            if ops.available():
                axes = [self.grad_axis] + [a for a in ("tp",) if a in self.mesh.axes()]
                if self.cp_size > 1 and self.config.get("cp", {}).get("kind", "ring") == "ulysses":
                    axes.append("cp")       # the two all-to-alls around attention run on the NVLink kernel
                for axis in axes:
                    persistent = 0
                    if axis == "tp" and self.config.get("tp", {}).get("sequence_parallel", False):
                        # operands of the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels live in the axis'
                        # symmetric region: the shard and the gathered copy of the widest activation (bf16) and one
                        # fp32 reduce-scatter target, each kept per shape
                        d = self.config["data"]
                        mc = self.config["model"]["config"]
                        tokens = d["micro_batch_size"] * d["seq_len"]
                        widest = max(mc["emb_dim"], mc.get("ffn_dim") or 0, mc["num_heads"] * (mc.get("head_dim") or 128))
                        persistent = tokens * widest * 24 + (8 << 20)
                    enable_sm100(self.mesh, axis, comm_cfg.get("max_bytes", 64 << 20), persistent)

        self.ignore_index = self.config["objective"]["config"]["ignore_index"]
        self.tokenizer = None
        if not is_synthetic(self.config["data"]):
            from tokenizers import Tokenizer

            name = self.config["data"]["tokenizer"]
            # a hub id as in the reference's configs, or the path of a local tokenizer.json (no network needed)
            self.tokenizer = Tokenizer.from_file(name) if os.path.isfile(name) else Tokenizer.from_pretrained(name)

        self.model = self._build_model()
        self._init_weights(self.model)
        if self.config.get("init_from"):
            # warm start: an unsharded model state dict (a `model.pt` of any run, or the output of `ckpt.merge` for
            # runs that wrote shard files) replaces the initialisation BEFORE the strategy slices, stages or shards
            # the model, so the weights of a run on one mesh can start a run on another.  Optimizer state starts fresh
            state = torch.load(self.config["init_from"], map_location="cpu", weights_only=True)
            self.model.load_state_dict(state)
        self.model = self._parallelize(self.model)
        self.objective = build_objective(self.config["objective"]["name"], self.config["objective"]["config"])
        opt_cfg = self.config["optimizer"]
        self.optimizer = build_optimizer(self.model, opt_cfg["name"], opt_cfg["config"], params=self._opt_params)
        self.scheduler = build_scheduler(self.optimizer, opt_cfg["scheduler"])
        self.num_train_steps = opt_cfg["scheduler"]["total_steps"]
        self.max_norm = opt_cfg.get("max_norm")
        self._wire_engine()
        # the ring exchange of context parallelism goes through library p2p calls on a side stream: not captured
        self.use_cuda_graph = (bool(self.config.get("cuda_graph", False)) and self.on_gpu and self.cp_size == 1
                               and self.pp_size == 1 and not hasattr(self.model, "expert_params"))
        self._graph = None
        self._graph_eager_left = int(self.config.get("cuda_graph_warmup", 3))

        self.dataloader = self._build_dataloader()
        data_cfg = self.config["data"]
        self.global_batch_size = data_cfg["global_batch_size"]
        self.micro_batch_size = data_cfg["micro_batch_size"]
        self.microbatches_per_step = self.global_batch_size // (self.micro_batch_size * self.dp_size)
        self.log_every = int(self.config.get("log_every", 1))

        stamp = datetime.now().strftime("%Y-%m-%d_%H-%M-%S")
        self.run_name = f"{self.config['run_name']}_{stamp}"
        # keyed on the config's run_name alone so a relaunch finds its own checkpoints
        self.checkpointer_path = os.path.join(get_project_dir(), "checkpoints", self.config["run_name"])
        self.checkpointer = Checkpointer(self.checkpointer_path,
                                         background=bool(self.config["checkpointing"].get("async", False)))
        self._unmarked_step: int | None = None
        ck = self.config["checkpointing"]
        self.resume, self.save_steps = ck["resume"], ck["save_steps"]
        self.resume_scheduler = ck.get("resume_scheduler", True)
        self.resume_wandb_id: str | None = None
        self.start_step = self._resume()
        self._setup_wandb()
        self.prefetcher = CUDAPrefetcher(self.dataloader, self.device)

    # -- construction --------------------------------------------------------------------------
    def _build_model(self):
        """``compile: false`` selects the PyTorch path (the oracle) instead of the sm_100a engine.  On that path
        ``torch_compile: true`` compiles every transformer block and the final norm in place, one region per block as
        the reference does (``torchure/train/trainer.py:223-244``), with the reference's ``compile_mode`` key (and
        ``compile_backend`` for a Dynamo backend other than Inductor)."""
        mc = dict(self.config["model"]["config"])
        if not self.config.get("compile", True):
            mc["impl"] = "torch"
        model = build_model(self.config["model"]["name"], mc)
        if self.config.get("torch_compile", False) and mc.get("impl") == "torch":
            # `compile_mode` is the reference's key (an Inductor mode); `compile_backend` selects another Dynamo backend
            # (e.g. "aot_eager", which needs no host compiler)
            backend = self.config.get("compile_backend", "inductor")
            kw = {"mode": self.config.get("compile_mode", "default")} if backend == "inductor" else {"backend": backend}
            for block in model.blocks:
                block.compile(**kw)
            model.norm.compile(**kw)
        return model

    def _init_weights(self, model) -> None:
        model.to(self.device)
        seed = self.config.get("seed")
        if seed is not None:
            torch.manual_seed(int(seed))
        model.init_weights()

    def _parallelize(self, model):
        """Build the strategy the mesh asks for.  ``self.ddp`` is the data-parallel strategy object whatever its kind
        (``requires_sync``, ``sync()``, ``sq_norm()``); ``self._opt_params`` is what the optimizer must hold when
        that is not ``model.parameters()`` (flat or row shards)."""
        axes = self.mesh.axes()
        self._opt_params = None
        self.sharded = "dp_shard" in axes
        self.tp_size = self.mesh.size("tp") if "tp" in axes else 1
        self.ddp_experts = None
        if hasattr(model, "expert_params"):
            # mixture-of-experts model: PyTorch blocks.  With an "ep" axis every rank keeps its slice of each layer's
            # experts; expert gradients are reduced over "dp" only (the other ranks of the ep group hold other
            # experts), everything else over dp x ep
            assert not self.sharded and self.tp_size == 1 and self.cp_size == 1 and self.pp_size == 1, \
                "the mixture-of-experts model combines with dp and ep only"
            ddp_cfg = self.config.get("ddp", {})
            kw = dict(bucket_mb=ddp_cfg.get("bucket_mb", 25), fused=False, merge_small=ddp_cfg.get("merge_small", True))
            if self.ep_size > 1:
                model.shard_experts(self.mesh, "ep")
                experts = model.expert_params()
                mine = {id(p) for p in experts}
                shared = [p for p in model.parameters() if id(p) not in mine]
                self.ddp = DDP(model, self.mesh, dim=self.grad_axis, params=shared, **kw)
                self.ddp_experts = DDP(model, self.mesh, dim="dp", params=experts, **kw)
            else:
                self.ddp = DDP(model, self.mesh, dim=self.grad_axis, **kw)
            return model
        if self.pp_size > 1:
            # every rank built the whole model from the same seed and keeps its stage: contiguous blocks, the first
            # stage also the embedding, the last the final norm and the head.  Stages run the PyTorch blocks; their
            # replicas along "dp" are averaged by the bucketed reducer
            from torchure_b200.parallel.pipeline import PipelineStage

            assert not self.sharded and self.tp_size == 1 and self.cp_size == 1, "pp combines with plain dp only"
            model.impl = "torch"
            stage = PipelineStage(model, self.mesh, "pp")
            stage.sync_tied_weight()
            ddp_cfg = self.config.get("ddp", {})
            self.ddp = DDP(stage, self.mesh, dim=self.data_axis, bucket_mb=ddp_cfg.get("bucket_mb", 25), fused=False,
                           merge_small=ddp_cfg.get("merge_small", True))
            return stage
        assert not (self.sharded and self.tp_size > 1), "dp_shard and tp cannot be combined yet"
        if "tp" in axes and self.mesh.size("tp") > 1:
            from torchure_b200.parallel.tensor_parallel import parallelize_model

            parallelize_model(model, self.mesh, "tp",
                              sequence_parallel=self.config.get("tp", {}).get("sequence_parallel", False))
            if self.config.get("tp", {}).get("loss_parallel", False):
                # the fused linear + CE computes only this rank's V / tp rows of the head (`vocab_parallel`); the
                # head's weight gradient is then complete in those rows only, and `_gather_head_rows` completes it
                assert self.config["objective"]["config"].get("fused_linear_ce", True), "loss_parallel needs the fused CE"
                assert model.cfg["vocab_size"] % self.tp_size == 0, "loss_parallel: vocabulary not divisible by tp"
                model.vocab_parallel = (self.mesh, "tp")
        if self.sharded:
            replicate = "dp_replicate" if "dp_replicate" in axes else None
            engine_path = self.on_gpu and getattr(model, "impl", "torch") != "torch"
            if engine_path:
                from torchure_b200 import ops

                engine_path = ops.available() and self.mesh.size("dp_shard") > 1
            if engine_path:
                from torchure_b200.parallel.fsdp_engine import EngineFSDP

                self.ddp = EngineFSDP(model, self.mesh, "dp_shard", replicate,
                                      comm_sms=self.config.get("fsdp", {}).get("comm_sms", 16))
            else:
                from torchure_b200.parallel.fsdp import FSDP

                model.impl = "torch"    # the hook-driven units swap parameter storage under plain modules
                self.ddp = FSDP(model, self.mesh, "dp_shard", replicate)
            self._opt_params = self.ddp.optimizer_params()
            return model
        ddp_cfg = self.config.get("ddp", {})
        data_cfg = self.config["data"]
        local_tokens = data_cfg["micro_batch_size"] * data_cfg["seq_len"] // self.cp_size
        if self.cp_size > 1:
            # every rank of the axis holds two zigzag chunks of each sequence; attention runs as a ring over the axis
            # (on the tcgen05 block-pair kernels when a chunk is a multiple of 128 tokens and head_dim is 128)
            model.cp = (self.mesh, "cp")
            model.cp_kind = self.config.get("cp", {}).get("kind", "ring")
            chunk = data_cfg["seq_len"] // (2 * self.cp_size)
            if chunk % 128 != 0 or model.cp_kind == "ulysses":
                # Ulysses (`cp.kind`: one contiguous chunk per rank, heads exchanged for sequence around attention)
                # runs the module path: its attention between the two all-to-alls is still the tcgen05 kernel
                model.impl = "torch"
        embed_tokens = local_tokens if ddp_cfg.get("early_embedding", True) else 0
        self.ddp = DDP(model, self.mesh, dim=self.grad_axis, bucket_mb=ddp_cfg.get("bucket_mb", 25),
                       fused=ddp_cfg.get("fused"), merge_small=ddp_cfg.get("merge_small", True),
                       comm_sms=ddp_cfg.get("comm_sms", 16), sm_reserve=ddp_cfg.get("sm_reserve", 0),
                       embed_tokens=embed_tokens)
        return model

    def _wire_engine(self) -> None:
        """Let the AdamW kernel refresh the bf16 shadow weights the sm_100a engine computes with."""
        if hasattr(self.ddp, "attach_shadows"):
            self.ddp.attach_shadows(self.optimizer)    # sharded: the shards' shadows are rows of the whole copies
            return
        if not self.on_gpu or getattr(self.model, "impl", "torch") == "torch":
            return
        from torchure_b200 import ops

        if ops.available() and hasattr(self.optimizer, "attach_shadow"):
            for p, shadow in self.model.engine().shadow_pairs():
                self.optimizer.attach_shadow(p, shadow)

    @debug_time
    def _build_dataloader(self):
        data_cfg = dict(self.config["data"])
        data_cfg.setdefault("vocab_size", self.config["model"]["config"]["vocab_size"])
        return build_dataloader(data_cfg, self.tokenizer, self.ignore_index,
                                self.mesh.coordinate(self.data_axis), self.mesh.size(self.data_axis))

    # -- held-out loss ---------------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self) -> torch.Tensor:
        """Mean next-token loss over ``eval.batches`` micro-batches per data-parallel rank of a held-out stream: the
        ``data`` section with the overrides of ``eval.data`` (for the synthetic source the seed defaults to the
        training seed + 1).  The stream starts from its beginning at every call, so successive values are comparable;
        training state (loader position, RNG, optimizer) is untouched.  Not in the reference, whose notes quote a
        held-out perplexity without shipping the loop."""
        ecfg = self.config.get("eval", {})
        assert self.pp_size == 1, "evaluation under pipeline parallelism is not implemented"
        data_cfg = dict(self.config["data"])
        data_cfg.setdefault("vocab_size", self.config["model"]["config"]["vocab_size"])
        data_cfg["seed"] = data_cfg.get("seed", 0) + 1
        data_cfg.update(ecfg.get("data", {}))
        loader = iter(build_dataloader(data_cfg, self.tokenizer, self.ignore_index,
                                       self.mesh.coordinate(self.data_axis), self.mesh.size(self.data_axis)))
        if hasattr(self.ddp, "begin_step"):
            self.ddp.begin_step()      # sharded weights: gather what the last optimizer step changed (idempotent)
        total = torch.zeros((), device=self.device)
        n = int(ecfg.get("batches", 8))
        for _ in range(n):
            batch = {k: v.to(self.device, non_blocking=True) for k, v in next(loader).items()}
            if self.on_gpu:
                with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                    total += self.objective.eval_loss(self.model, batch).float()
            else:
                total += self.objective.eval_loss(self.model, batch).float()
        total /= n
        if self.mesh.size(self.grad_axis) > 1:
            all_reduce(total, self.mesh, self.grad_axis, "avg")
        return total

    def _setup_wandb(self) -> None:
        self.wandb_run = None
        wcfg = self.config.get("wandb", {})
        if not wcfg.get("enabled", False) or self.rank != 0 or self.benchmark:
            return
        assert HAS_WANDB, "wandb.enabled is true but the wandb package is not installed"
        self.wandb_run = wandb.init(project=wcfg.get("project", "torchure_b200"), entity=wcfg.get("entity"),
                                    name=self.run_name, id=self.resume_wandb_id,
                                    resume="must" if self.resume_wandb_id else None, config=self.config)

    # -- device error words ---------------------------------------------------------------------
    def check_device_errors(self) -> None:
        """Raise if any kernel of this process recorded an expired bounded wait (GEMM / attention pipeline waits,
        peer-flag handshakes of the collectives, arrival polls of the fused GEMM+collective kernels).  Such a
        kernel returns early and leaves its output unwritten or unreduced, and the words are sticky, so training
        on would silently diverge.  Reading the words synchronises; it is called where the host synchronises
        anyway: at the logging cadence, before a checkpoint is written and after a timed benchmark region."""
        if not self.on_gpu:
            return
        from torchure_b200 import ops

        if not ops.available():
            return
        from torchure_b200.ops import kernels as K

        K.check_error()
        K.check_comm_error(self.rank)

    # -- checkpoint / resume -------------------------------------------------------------------
    @debug_time
    def checkpoint(self, step: int) -> None:
        """Write the state after `step` completed steps; rank 0 writes replicas, every dp rank its loader."""
        self.check_device_errors()   # never persist the result of a step whose kernels gave up
        self.finish_checkpoint()     # asynchronous writes: the previous step's files first
        if self.sharded:
            # model.pt keeps the reference's unsharded keys (gathered; collective), optimizer state stays sharded:
            # one file per shard coordinate, written by the first replica of that shard
            full = self.ddp.full_state_dict()
            if self.rank == 0:
                self.checkpointer._write(full, step, "model.pt")
            del full
            if "dp_replicate" not in self.mesh.axes() or self.mesh.coordinate("dp_replicate") == 0:
                self.checkpointer.save_optimizer(self.optimizer, step, shard=self.mesh.coordinate("dp_shard"))
        elif self.tp_size > 1 or self.pp_size > 1 or self.ep_size > 1:
            # every tensor-parallel coordinate holds different rows / columns, every pipeline stage different blocks
            # (under the keys of the whole model), every expert-parallel coordinate different experts: one file pair
            # per coordinate, written by the first data-parallel replica
            if self.mesh.coordinate("dp") == 0:
                shard = self.mesh.coordinate(self._split_axis())
                self.checkpointer.save_model(self.model, step, shard=shard)
                self.checkpointer.save_optimizer(self.optimizer, step, shard=shard)
        elif self.rank == 0:
            self.checkpointer.save_model(self.model, step)
            self.checkpointer.save_optimizer(self.optimizer, step)
        if self.rank == 0:
            self.checkpointer.save_scheduler(self.scheduler, step)
            self.checkpointer.save_trainer({
                "step": step,
                "cpu_rng": torch.get_rng_state(),
                "cuda_rng": torch.cuda.get_rng_state(self.device) if self.on_gpu else None,
                "config": self.config,
                "wandb_id": self.wandb_run.id if self.wandb_run else None,
            }, step)
        # the prefetcher knows the position of the first batch that was NOT consumed
        if all(self.mesh.coordinate(a) == 0 for a in ("cp", "pp") if a in self.mesh.axes()):
            # (the ranks of a cp group, and the stages of a pipeline, read the same rows)
            self.checkpointer.save_dataloader(self.prefetcher, step, self.mesh.coordinate(self.data_axis))
        self._unmarked_step = step
        if not self.checkpointer.background:
            self.finish_checkpoint()

    def finish_checkpoint(self) -> None:
        """Mark the last written step complete once EVERY rank's files are on disk.  Synchronous writes: right after
        them.  ``checkpointing.async``: the files are written by a worker thread from host snapshots taken inside
        ``checkpoint()`` while training continues, and this runs before the next checkpoint and when training ends;
        a run that dies in between leaves a step without a marker, which does not exist for ``resume``."""
        if self._unmarked_step is None:
            return
        step, self._unmarked_step = self._unmarked_step, None
        self.checkpointer.wait()
        barrier()
        if self.rank == 0:
            self.checkpointer.mark_complete(step)
            keep = self.config["checkpointing"].get("keep_last")
            if keep:
                self.checkpointer.prune(int(keep))

    def _split_axis(self) -> str:
        """The axis whose coordinates hold different tensors (one checkpoint shard each)."""
        return "tp" if self.tp_size > 1 else ("pp" if self.pp_size > 1 else "ep")

    def _resume(self) -> int:
        if self.resume is None:
            return 0
        if self.resume == "auto":
            step = self.checkpointer.latest()
            if step is None:
                return 0
        elif isinstance(self.resume, int):
            step = self.checkpointer.valid_step(self.resume)
            assert step is not None, f"checkpoint step {self.resume} does not exist or is incomplete"
        else:
            raise ValueError('resume must be null, "auto" or a step number')
        state = self.checkpointer.load_trainer(step)
        assert state["config"]["mesh"] == self.config["mesh"], (
            f"cannot resume across a mesh change: checkpoint {state['config']['mesh']}, config {self.config['mesh']}")
        if self.sharded:
            self.ddp.load_full_state_dict(self.checkpointer._read(step, "model.pt"))
            self.checkpointer.load_optimizer(self.optimizer, step, shard=self.mesh.coordinate("dp_shard"))
        elif self.tp_size > 1 or self.pp_size > 1 or self.ep_size > 1:
            shard = self.mesh.coordinate(self._split_axis())
            self.checkpointer.load_model(self.model, step, shard=shard)
            self.checkpointer.load_optimizer(self.optimizer, step, shard=shard)
        else:
            self.checkpointer.load_model(self.model, step)
            self.checkpointer.load_optimizer(self.optimizer, step)
        if self.resume_scheduler:
            self.checkpointer.load_scheduler(self.scheduler, step)
        else:
            self.scheduler.last_epoch = step
        self.checkpointer.load_dataloader(self.dataloader, step, self.mesh.coordinate(self.data_axis))
        torch.set_rng_state(state["cpu_rng"])
        if self.on_gpu and state.get("cuda_rng") is not None:
            torch.cuda.set_rng_state(state["cuda_rng"], self.device)
        self.resume_wandb_id = state.get("wandb_id")
        return state["step"]

    # -- the step ------------------------------------------------------------------------------
    def micro_train_step(self, batch=None) -> torch.Tensor:
        if batch is None:
            batch = next(self.prefetcher)
        scale = 1.0 / self.microbatches_per_step
        if self.on_gpu:
            with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                loss = self.objective.compute_loss(self.model, batch, loss_scale=scale)
        else:
            loss = self.objective.compute_loss(self.model, batch, loss_scale=scale)
        loss.backward()
        return loss.detach()

    def _device_step(self, batches=None) -> tuple[torch.Tensor, torch.Tensor]:
        """Everything of one optimizer step that runs on the device: micro-batches, gradient reduction, clipping,
        AdamW.  `batches` (one dict per micro-batch) are used instead of the prefetcher when given."""
        if self.pp_size > 1:
            return self._pipeline_step(batches)
        if self.ddp_experts is not None:
            return self._expert_step(batches)
        K = self.microbatches_per_step
        slot = self.ddp.loss_slot() if hasattr(self.ddp, "loss_slot") else None
        if slot is not None:
            slot.zero_()
            loss = slot[0]          # accumulates inside symmetric memory: averaged over the ranks in place below
        else:
            loss = torch.zeros((), device=self.device)
        self._loss_averaged = slot is not None
        if hasattr(self.ddp, "begin_step"):
            self.ddp.begin_step()      # sharded: all-gather the bf16 weights the last optimizer step rewrote
        self.ddp.requires_sync = False
        for i in range(K - 1):
            loss += self.micro_train_step(batches[i] if batches else None)
        self.ddp.requires_sync = True
        loss += self.micro_train_step(batches[K - 1] if batches else None)
        self.ddp.sync()
        if getattr(self.model, "vocab_parallel", None) is not None:
            self._gather_head_rows()
        params = self._opt_params if self._opt_params is not None else [
            p for p in self.model.parameters() if p.requires_grad]
        fused_norm = sq = None
        if self.tp_size == 1 and hasattr(self.ddp, "norm_and_coef") and hasattr(self.optimizer, "set_grad_scale"):
            fused_norm = self.ddp.norm_and_coef(self.max_norm)     # one kernel: partials -> norm and coefficient
        if fused_norm is None:
            sq = self._tp_sq_norm(params) if self.tp_size > 1 else self.ddp.sq_norm()
        if fused_norm is not None:
            grad_norm, coef = fused_norm
            if self.max_norm is not None:
                self.optimizer.set_grad_scale(coef)
        elif sq is not None and hasattr(self.optimizer, "set_grad_scale"):
            grad_norm, coef = grad_norm_and_coef(params, self.mesh, self.max_norm, shard_dims=(), presummed_sq=sq)
            if self.max_norm is not None:
                self.optimizer.set_grad_scale(coef)
        else:
            grad_norm = clip_grad_norm(params, self.mesh, self.max_norm,
                                       shard_dims=getattr(self.ddp, "clip_shard_dims", ()))
        self.optimizer.step()
        if hasattr(self.ddp, "mark_updated"):
            self.ddp.mark_updated()
        self.optimizer.zero_grad()
        if slot is not None:
            self.ddp.reducer.comm.all_reduce_symmetric_(slot, "avg", blocks=1)
            loss = slot[0].clone()
        return loss, grad_norm

    def _pipeline_step(self, batches=None) -> tuple[torch.Tensor, torch.Tensor]:
        """One optimizer step of a pipeline stage: the step's micro-batches run through the schedule
        (``pp.schedule``: "1f1b" or "gpipe"), activations and their gradients moving between neighbouring stages;
        the stage's replicas along "dp" reduce their gradients during the last micro-batch's backward; the two
        holders of a tied embedding / head sum their gradients; the clip norm is taken over all stages."""
        from contextlib import nullcontext

        from torchure_b200.core.grad_helper import _collect, _total_norm
        from torchure_b200.parallel.pipeline import run_schedule

        K = self.microbatches_per_step
        fetched = batches if batches else [next(self.prefetcher) for _ in range(K)]
        micro = [(b["input_ids"], b["labels"]) for b in fetched]
        stage, obj = self.model, self.objective
        fused_ce = getattr(obj, "fused_linear_ce", False)

        def loss_fn(out, label_ids):
            return obj.loss_from_output(out, stage.lm_head.weight, label_ids)

        def last_backward():
            self.ddp.requires_sync = True

        self.ddp.requires_sync = K == 1
        cast = torch.autocast(device_type="cuda", dtype=torch.bfloat16) if self.on_gpu else nullcontext()
        with cast:
            loss = run_schedule(stage, micro, loss_fn, self.config.get("pp", {}).get("schedule", "1f1b"),
                                before_last_backward=last_backward, final_hidden=fused_ce)
        self.ddp.requires_sync = True
        self.ddp.sync()
        stage.sync_tied_grad()
        if loss is None:
            loss = torch.zeros((), device=self.device)
        loss = loss.float().reshape(())
        all_reduce(loss, self.mesh, "pp", "sum")       # the last stage has it; every stage reports it
        grads = _collect(stage.parameters())
        grad_norm = _total_norm(_collect(stage.norm_params()), self.mesh, ("pp",))
        if self.max_norm is not None:
            torch._foreach_mul_(grads, torch.clamp(self.max_norm / (grad_norm + 1e-6), max=1.0))
        self.optimizer.step()
        self.optimizer.zero_grad()
        self._loss_averaged = False
        return loss, grad_norm

    def _expert_step(self, batches=None) -> tuple[torch.Tensor, torch.Tensor]:
        """One optimizer step under expert parallelism.  An expert's gradient collects the tokens of every rank of its
        ep group, each differentiated against that rank's own mean loss: averaging over "dp" and dividing by the size
        of the ep group makes it the gradient of the mean over all ranks, which is what the shared parameters get
        from their average over dp x ep.  The clip norm counts shared tensors once and sums the experts over "ep"."""
        from torchure_b200.core.grad_helper import _collect, _local_sq_norm

        K = self.microbatches_per_step
        wrappers = (self.ddp, self.ddp_experts)
        loss = torch.zeros((), device=self.device)
        for w in wrappers:
            w.requires_sync = False
        for i in range(K - 1):
            loss += self.micro_train_step(batches[i] if batches else None)
        for w in wrappers:
            w.requires_sync = True
        loss += self.micro_train_step(batches[K - 1] if batches else None)
        for w in wrappers:
            w.sync()
        experts = self.model.expert_params()
        mine = {id(p) for p in experts}
        expert_grads = _collect(experts)
        torch._foreach_mul_(expert_grads, 1.0 / self.ep_size)
        shared_grads = _collect([p for p in self.model.parameters() if p.requires_grad and id(p) not in mine])
        sq = _local_sq_norm(expert_grads).reshape(1).clone()
        all_reduce(sq, self.mesh, "ep", "sum")
        grad_norm = (sq + _local_sq_norm(shared_grads).reshape(1)).sqrt().reshape(())
        if self.max_norm is not None:
            torch._foreach_mul_(expert_grads + shared_grads, torch.clamp(self.max_norm / (grad_norm + 1e-6), max=1.0))
        self.optimizer.step()
        self.optimizer.zero_grad()
        self._loss_averaged = False
        return loss, grad_norm

    def _gather_head_rows(self) -> None:
        """Loss-parallel head: every rank of the tp axis computed the head's weight gradient for its own V / tp rows
        (to which the replicated embedding lookup, when the tensor is tied, added the same rows on every rank), so
        the rank's row slice is complete and the other rows are not: each rank's slice replaces those rows
        everywhere."""
        from torchure_b200.core.collective import all_gather
        from torchure_b200.loss.fused_linear_ce import vocab_slice

        grad = self.model.lm_head.weight.grad
        v0, rows = vocab_slice(grad.shape[0], self.mesh, "tp")
        all_gather(grad[v0:v0 + rows].clone(), self.mesh, "tp", output_tensor=grad)

    def _tp_sq_norm(self, params) -> torch.Tensor:
        """Global sum of squared gradients under tensor parallelism: the sharded matrices contribute their own rows /
        columns on every rank (summed over the axis), the replicated tensors are counted once."""
        from torchure_b200.core.grad_helper import _local_sq_norm

        sharded = [p.grad for p in params if p.grad is not None and getattr(p, "_tp_sharded", False)]
        whole = [p.grad for p in params if p.grad is not None and not getattr(p, "_tp_sharded", False)]
        sq = _local_sq_norm(sharded).reshape(1).clone()
        all_reduce(sq, self.mesh, "tp", "sum")
        return (sq + _local_sq_norm(whole).reshape(1)).reshape(())

    def train_step_untimed(self) -> dict[str, torch.Tensor]:
        if self.use_cuda_graph:
            loss, grad_norm = self._graph_step()
        else:
            loss, grad_norm = self._device_step()
        self.scheduler.step()
        if self.mesh.size(self.grad_axis) > 1 and not getattr(self, "_loss_averaged", False):
            all_reduce(loss, self.mesh, self.grad_axis, "avg")
        return {"loss": loss, "grad_norm": grad_norm}

    # -- CUDA-graph replay of the device step ----------------------------------------------------
    def _graph_step(self) -> tuple[torch.Tensor, torch.Tensor]:
        """Replay the whole device step (forward, backward, bucket all-reduces on the communication stream, clip,
        AdamW) from ONE captured CUDA graph.  The first `cuda_graph_warmup` steps run eagerly (they fill the
        tensor-map and pointer-table caches and size the allocator), the next one is captured, and every later step
        copies its batch into the graph's static input tensors, refreshes the device-resident lr / bias-correction
        scalars and replays.  Nothing step-dependent is baked into a node: the clip coefficient and the optimizer
        scalars are read from device memory, and the peer-flag handshakes of the collectives carry no sequence
        numbers."""
        from torchure_b200 import ops

        K = self.microbatches_per_step
        fetched = [next(self.prefetcher) for _ in range(K)]
        if self._graph is None and self._graph_eager_left > 0:
            self._graph_eager_left -= 1
            self.optimizer.enable_device_hyper()
            return self._device_step(fetched)
        if self._graph is None:
            self._static_batches = [{k: v.clone() for k, v in b.items()} for b in fetched]
            snap = self.optimizer.host_state()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = ops.launches()
            with torch.cuda.graph(graph):
                self._static_out = self._device_step(self._static_batches)
            self._graph_launches = ops.launches() - n0
            ops.count_launch(-self._graph_launches)        # capture launched nothing
            self.optimizer.restore_host_state(snap)        # ... and stepped nothing
            self._graph = graph
        else:
            for dst, src in zip(self._static_batches, fetched):
                for k, v in src.items():
                    dst[k].copy_(v, non_blocking=True)
        self.optimizer.host_advance()
        self._graph.replay()
        ops.count_launch(self._graph_launches)
        loss, grad_norm = self._static_out
        return loss.clone(), grad_norm.clone()

    train_step = record_time(train_step_untimed)

    def _line(self, step: int, metrics: dict, seconds: float, tokens_per_step: int) -> str:
        return (f"{step=} || loss={metrics['loss'].item():.4f} || gnorm={metrics['grad_norm'].item():.3f} "
                f"|| lr={self.scheduler.get_last_lr()[0]:.2e} || tps={tokens_per_step / seconds:.0f}")

    @debug_time
    def train_n_step_test(self, n_steps: int) -> list[dict]:
        tokens_per_step = self.config["data"]["seq_len"] * self.global_batch_size
        history = []
        for step in range(n_steps):
            metrics, seconds = self.train_step()
            history.append({"loss": float(metrics["loss"]), "grad_norm": float(metrics["grad_norm"]),
                            "seconds": seconds})
            self.check_device_errors()
            if self.rank == 0:
                print(self._line(step, metrics, seconds, tokens_per_step), flush=True)
        if self.rank == 0 and self.on_gpu:
            print(f"peak cuda mem: {torch.cuda.max_memory_allocated() / 2**30:.2f} GiB")
        return history

    def _mfu(self, tokens_per_step: int, seconds: float) -> float | None:
        """Model FLOPs utilisation against the nominal dense bf16 peak (2.25 PFLOP/s per B200); None off-GPU or when the
        config does not pin the FLOP count (no explicit ffn_dim)."""
        mcfg = self.config["model"]
        if not self.on_gpu or mcfg.get("name") != "qwen3_dense" or "ffn_dim" not in mcfg["config"]:
            return None
        from torchure_b200.models.qwen3 import flops_per_token

        flops = flops_per_token(mcfg["config"], self.config["data"]["seq_len"]) * tokens_per_step
        return flops / seconds / (2.25e15 * self.world_size)

    def _log_metrics(self, metrics: dict, step: int, tokens_per_step: int, seconds: float) -> None:
        jsonl = self.config.get("logging", {}).get("jsonl")
        if jsonl:
            import json

            rec = {"step": step, "loss": metrics["loss"].item(), "grad_norm": metrics["grad_norm"].item(),
                   "lr": self.scheduler.get_last_lr()[0], "tokens": step * tokens_per_step,
                   "tps": tokens_per_step / seconds, "step_time": seconds, "mfu": self._mfu(tokens_per_step, seconds)}
            if "eval_loss" in metrics:
                rec["eval_loss"] = metrics["eval_loss"].item()
            os.makedirs(os.path.dirname(os.path.abspath(jsonl)), exist_ok=True)
            with open(jsonl, "a") as f:
                f.write(json.dumps(rec) + "\n")
        if self.wandb_run is None:
            return
        if "eval_loss" in metrics:
            self.wandb_run.log({"eval/loss": metrics["eval_loss"].item()}, step=step)
        self.wandb_run.log({
            "train/loss": metrics["loss"].item(), "train/grad_norm": metrics["grad_norm"].item(),
            "train/lr": self.scheduler.get_last_lr()[0], "train/tokens": step * tokens_per_step,
            "perf/tps": tokens_per_step / seconds, "perf/step_time": seconds,
            "perf/peak_mem_gib": torch.cuda.max_memory_allocated() / 2**30 if self.on_gpu else 0.0,
        }, step=step)

    # -- preemption ------------------------------------------------------------------------------
    def _watch_signals(self) -> None:
        """``checkpointing.on_signal: true``: SIGTERM / SIGUSR1 (what a scheduler sends before it takes the machines
        away) only set a flag; at the next log cadence the ranks agree on it (one max-reduce of a flag, where every
        rank synchronises anyway), write a checkpoint of the step just completed and leave the loop, so that
        ``resume: "auto"`` continues from there.  A rank is never stopped in the middle of a step or a collective."""
        import signal

        self._stop_requested = False
        if not self.config["checkpointing"].get("on_signal", False):
            return

        def note(signum, frame):
            self._stop_requested = True

        for sig in (signal.SIGTERM, signal.SIGUSR1):
            signal.signal(sig, note)

    def _stop_agreed(self) -> bool:
        if not self.config["checkpointing"].get("on_signal", False):
            return False
        flag = torch.tensor([1.0 if self._stop_requested else 0.0], device=self.device)
        if self.world_size > 1:
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
        return bool(flag.item() > 0)

    def train(self) -> None:
        tokens_per_step = self.config["data"]["seq_len"] * self.global_batch_size
        self._watch_signals()
        try:
            for step in range(self.start_step, self.num_train_steps):
                metrics, seconds = self.train_step()
                done = step + 1
                at_cadence = done % self.log_every == 0 or done == self.num_train_steps
                stop = at_cadence and done != self.num_train_steps and self._stop_agreed()
                if (done % self.save_steps == 0 and step != 0) or done == self.num_train_steps or stop:
                    self.checkpoint(done)
                if at_cadence:
                    self.check_device_errors()   # every rank, at the cadence at which rank 0 reads the loss anyway
                every = int(self.config.get("eval", {}).get("every", 0))
                if every and (done % every == 0 or done == self.num_train_steps):
                    metrics["eval_loss"] = self.evaluate()        # a collective: every rank takes part
                if self.rank == 0:
                    self._log_metrics(metrics, done, tokens_per_step, seconds)
                    if done % self.log_every == 0 or done == self.num_train_steps:
                        print(self._line(step, metrics, seconds, tokens_per_step), flush=True)
                    if "eval_loss" in metrics:
                        print(f"step={step} || eval_loss={metrics['eval_loss'].item():.4f}", flush=True)
                if stop:
                    if self.rank == 0:
                        print(f"stop requested by a signal: checkpoint written after step {done}, leaving", flush=True)
                    break
            if self.rank == 0 and self.on_gpu:
                print(f"peak cuda mem: {torch.cuda.max_memory_allocated() / 2**30:.2f} GiB")
            self.finish_checkpoint()
        finally:
            if self.wandb_run is not None:
                self.wandb_run.finish()
