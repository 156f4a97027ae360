"""Pipeline parallelism: contiguous stages of transformer blocks with GPipe and 1F1B schedules.

Roadmap-only in the reference (directed send/recv as a generalisation of its ring primitive).  A stage owns a slice
of ``model.blocks`` (the first stage also the embedding, the last the final norm and head).  Activations and their
gradients move between neighbouring stages with ``collective.isend`` / ``collective.recv`` (library p2p transport).  Both schedules
run the same per-micro-batch functions and differ only in ordering: GPipe does all forwards then all backwards,
1F1B interleaves them after a warm-up of (stages - stage - 1) forwards, which bounds the live activations.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from torchure_b200.core.collective import isend, recv


def split_layers(num_layers: int, stages: int) -> list[range]:
    base, extra = divmod(num_layers, stages)
    out, at = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append(range(at, at + n))
        at += n
    return out


class PipelineStage(nn.Module):
    def __init__(self, model, mesh, dim: str = "pp"):
        super().__init__()
        self.mesh, self.dim = mesh, dim
        self.stages, self.stage = mesh.size(dim), mesh.coordinate(dim)
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        mine = split_layers(len(model.blocks), self.stages)[self.stage]
        self.blocks = nn.ModuleList(model.blocks[i] for i in mine)
        self.rope = model.rope
        self.token_emb = model.token_emb if self.first else None
        self.norm = model.norm if self.last else None
        self.lm_head = model.lm_head if self.last else None
        self.hidden = model.cfg["emb_dim"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.first:
            x = self.token_emb(x)
        S = x.shape[1]
        cos, sin = self.rope.tables(S, x.device)
        cos, sin = cos[None, None], sin[None, None]
        for b in self.blocks:
            x = b(x, cos, sin)
        if self.last:
            x = self.lm_head(self.norm(x))
        return x


def run_schedule(stage: PipelineStage, micro_inputs, loss_fn, schedule: str = "1f1b"):
    """One optimizer step's forward/backward over `micro_inputs` (list of (ids, labels), identical on every stage).
    Returns the mean loss on the last stage (None elsewhere); parameter grads are accumulated in ``.grad``."""
    mesh, dim, s, n = stage.mesh, stage.dim, stage.stage, stage.stages
    M = len(micro_inputs)
    B, S = micro_inputs[0][0].shape
    dev = next(stage.parameters()).device
    act_shape = (B, S, stage.hidden)
    saved_in: dict[int, torch.Tensor] = {}
    saved_out: dict[int, torch.Tensor] = {}
    losses = []
    sends: list = []  # (work, tensor kept alive): sends are posted and waited for at the end, so a stage never blocks
    #                   on a neighbour that is itself about to send

    def fwd(i):
        ids, labels = micro_inputs[i]
        if stage.first:
            x = ids
        else:
            x = recv(torch.empty(act_shape, device=dev), mesh, dim, s - 1)
            x.requires_grad_()
        out = stage(x)
        saved_in[i] = x
        if stage.last:
            loss = loss_fn(out, labels) / M
            losses.append(loss.detach())
            saved_out[i] = loss
        else:
            payload = out.detach().contiguous()
            sends.append((isend(payload, mesh, dim, s + 1), payload))
            saved_out[i] = out

    def bwd(i):
        out, x = saved_out.pop(i), saved_in.pop(i)
        if stage.last:
            out.backward()
        else:
            out.backward(recv(torch.empty(act_shape, device=dev), mesh, dim, s + 1))
        if not stage.first:
            payload = x.grad.contiguous()
            sends.append((isend(payload, mesh, dim, s - 1), payload))

    if schedule == "gpipe":
        for i in range(M):
            fwd(i)
        for i in range(M):
            bwd(i)
    elif schedule == "1f1b":
        warm = min(M, n - s - 1)
        for i in range(warm):
            fwd(i)
        for i in range(M - warm):
            fwd(warm + i)
            bwd(i)
        for i in range(M - warm, M):
            bwd(i)
    else:
        raise ValueError(f"unknown schedule {schedule!r}")
    for work, _ in sends:
        work.wait()
    return torch.stack(losses).sum() if stage.last else None
