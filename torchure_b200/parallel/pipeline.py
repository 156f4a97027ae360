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

from torchure_b200.core.collective import isend, recv, send_recv


def split_layers(num_layers: int, stages: int) -> list[range]:
    base, extra = divmod(num_layers, stages)
    out, at = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append(range(at, at + n))
        at += n
    return out


class PipelineStage(nn.Module):
    """The part of a decoder that one pipeline stage owns.  Sub-modules keep the names they have in the whole model
    (``blocks.<global index>``, ``token_emb``, ``norm``, ``lm_head``), so a stage's ``state_dict`` is the matching
    subset of the model's and per-stage checkpoint files merge into the unsharded layout by a plain dict union."""

    def __init__(self, model, mesh, dim: str = "pp"):
        super().__init__()
        self.mesh, self.dim = mesh, dim
        self.stages, self.stage = mesh.size(dim), mesh.coordinate(dim)
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        mine = split_layers(len(model.blocks), self.stages)[self.stage]
        self.blocks = nn.ModuleDict({str(i): model.blocks[i] for i in mine})
        self.rope = model.rope
        self.token_emb = model.token_emb if self.first else None
        self.norm = model.norm if self.last else None
        self.lm_head = model.lm_head if self.last else None
        self.hidden = model.cfg["emb_dim"]
        # a tied embedding / head lives on two stages: their gradients are summed and their values kept equal
        self.tied_across = (self.stages > 1 and getattr(model, "lm_head", None) is not None
                            and model.lm_head.weight is model.token_emb.weight)

    def forward(self, x: torch.Tensor, return_final_hidden: bool = False) -> torch.Tensor:
        if self.first:
            x = self.token_emb(x)
        S = x.shape[1]
        cos, sin = self.rope.tables(S, x.device)
        cos, sin = cos[None, None], sin[None, None]
        for b in self.blocks.values():
            x = b(x, cos, sin)
        if self.last:
            x = self.norm(x)
            if not return_final_hidden:
                x = self.lm_head(x)
        return x

    # -- the tied embedding / head across the first and the last stage --------------------------------------------
    def _tied(self):
        if not self.tied_across or not (self.first or self.last):
            return None
        return self.token_emb.weight if self.first else self.lm_head.weight

    def sync_tied_weight(self) -> None:
        """The last stage takes the first stage's embedding values (equal by construction under one seed; this makes
        it so whatever the initialisation did)."""
        w = self._tied()
        if w is None:
            return
        if self.first:
            send_recv(w.detach(), None, self.mesh, self.dim, dst=self.stages - 1)
        else:
            send_recv(None, w.detach(), self.mesh, self.dim, src=0)

    def sync_tied_grad(self) -> None:
        """Both holders end with the SUM of the embedding's and the head's gradient, as the tied tensor of an
        unsplit model has; with the same optimizer state they then apply the same update."""
        w = self._tied()
        if w is None:
            return
        g = w.grad
        if self.first:
            other = send_recv(None, torch.empty_like(g), self.mesh, self.dim, src=self.stages - 1)
            g.add_(other)
            send_recv(g, None, self.mesh, self.dim, dst=self.stages - 1)
        else:
            send_recv(g, None, self.mesh, self.dim, dst=0)
            send_recv(None, g, self.mesh, self.dim, src=0)

    def norm_params(self) -> list:
        """Parameters whose gradients this stage contributes to the global norm: all of its own, except the last
        stage's copy of a tied head (the first stage counts that tensor)."""
        skip = self.lm_head.weight if (self.tied_across and self.last) else None
        return [p for p in self.parameters() if p.requires_grad and p is not skip]


def run_schedule(stage: PipelineStage, micro_inputs, loss_fn, schedule: str = "1f1b", before_last_backward=None,
                 final_hidden: bool = False):
    """One optimizer step's forward/backward over `micro_inputs` (list of (ids, labels), identical on every stage).
    Returns the mean loss on the last stage (None elsewhere); parameter grads are accumulated in ``.grad``.
    `before_last_backward` is called before the backward of the last micro-batch (where a data-parallel wrapper
    switches its gradient reduction on); with `final_hidden` the last stage hands `loss_fn` the normalised hidden
    state instead of logits (for a loss that fuses the head)."""
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
        out = stage(x, return_final_hidden=final_hidden)
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
        if i == M - 1 and before_last_backward is not None:
            before_last_backward()
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
