"""sm_100a execution engine of the decoder: one autograd node per transformer block.

Forward of a block (all bf16 GEMMs on tcgen05, fp32 residual stream)::

    x, h1   = add_rmsnorm(x_in, y_in)            # residual add of the previous sub-layer fused in
    qkv     = h1 @ Wqkv^T                        # q, k, v projections as ONE GEMM (N = (Hq+2Hkv)*hd)
    qk      = qknorm_rope(qkv)                   # per-head RMSNorm + RoPE in one pass
    o       = attention(qk, qkv.v)               # causal GQA flash attention, emits LSE
    y_a     = o @ Wo^T
    x2, h2  = add_rmsnorm(x, y_a)
    gu      = h2 @ [Wgate; Wup]^T                # gate and up as ONE GEMM (N = 2F)
    y_out   = swiglu(gu) @ Wdown^T               # returned unadded: the next block's norm adds it

Each block returns ``(x2, y_out)``; the sum is never materialised on its own.  Backward mirrors it
with dgrad (B operand read MN-major, no transposes) and wgrad (both operands MN-major, fp32 output)
GEMMs.  Weight gradients of the fused projections are returned as row slices of one buffer.

The GEMMs read bf16 *shadow* copies of the fp32 master parameters.  Shadows of q/k/v (and gate/up) are
adjacent rows of one buffer so the fused GEMM sees a single matrix.  The fused AdamW kernel rewrites the
shadows at every step; ``refresh()`` re-casts any parameter whose version counter moved otherwise
(initialisation, ``load_state_dict``, a foreign optimizer).
"""

from __future__ import annotations

import weakref

import torch

from torchure_b200.ops import attention as attn_ops
from torchure_b200.ops import kernels as K

BF16 = torch.bfloat16

_ENGINE_OF_WEIGHT: "weakref.WeakValueDictionary[int, Sm100Engine]" = weakref.WeakValueDictionary()


# value of `engine.pending_tied_grad` when the tied table's bucket was launched by the loss head and the embedding rows
# are to be exchanged through the gradient sink instead of being added locally
EARLY_TABLE = object()


def engine_for_weight(weight: torch.Tensor):
    return _ENGINE_OF_WEIGHT.get(id(weight))


class _LayerShadow:
    """bf16 compute copies of one block's matrices, laid out for the fused GEMMs."""

    def __init__(self, block, device):
        g, f = block.gqa, block.ffn
        D = g.emb_dim
        nq, nkv = g.num_heads * g.head_dim, g.num_kv_heads * g.head_dim
        F_ = f.gate_proj.weight.shape[0]
        self.wqkv = torch.empty(nq + 2 * nkv, D, dtype=BF16, device=device)
        self.wo = torch.empty(D, nq, dtype=BF16, device=device)
        self.wgu = torch.empty(2 * F_, D, dtype=BF16, device=device)
        self.wd = torch.empty(D, F_, dtype=BF16, device=device)
        self.params = dict(w1=block.norm1.weight, wq=g.q_proj.weight, wk=g.k_proj.weight, wv=g.v_proj.weight,
                           wo=g.o_proj.weight, qn=g.q_norm.weight if g.qk_norm else None,
                           kn=g.k_norm.weight if g.qk_norm else None, w2=block.norm2.weight,
                           wg=f.gate_proj.weight, wu=f.up_proj.weight, wd=f.down_proj.weight, table=None)
        self.pairs = [
            (g.q_proj.weight, self.wqkv[:nq]), (g.k_proj.weight, self.wqkv[nq:nq + nkv]),
            (g.v_proj.weight, self.wqkv[nq + nkv:]), (g.o_proj.weight, self.wo),
            (f.gate_proj.weight, self.wgu[:F_]), (f.up_proj.weight, self.wgu[F_:]), (f.down_proj.weight, self.wd),
        ]


class Sm100Engine:
    def __init__(self, model):
        self.model = weakref.proxy(model)
        cfg = model.cfg
        self.cfg = cfg
        dev = model.token_emb.weight.device
        assert cfg["head_dim"] == 128, "the sm_100a engine supports head_dim 128"
        assert cfg["emb_dim"] % 8 == 0 and cfg["ffn_dim"] % 8 == 0
        self.layers = [_LayerShadow(b, dev) for b in model.blocks]
        self.emb_shadow = torch.empty_like(model.token_emb.weight, dtype=BF16)
        self._pairs = [p for layer in self.layers for p in layer.pairs] + [(model.token_emb.weight, self.emb_shadow)]
        self.head_shadow = self.emb_shadow
        if model.lm_head.weight is not model.token_emb.weight:
            self.head_shadow = torch.empty_like(model.lm_head.weight, dtype=BF16)
            self._pairs.append((model.lm_head.weight, self.head_shadow))
        self._versions: dict[int, int] = {}
        self._optimizer_owned = False
        self.tied = model.lm_head.weight is model.token_emb.weight
        self.pending_tied_grad = None      # CE's dW waiting for the embedding backward
        self.expect_tied_grad = False
        _ENGINE_OF_WEIGHT[id(model.lm_head.weight)] = self
        self.dummy = torch.zeros(1, device=dev)
        # hooks of sharded strategies (parallel/fsdp_engine.py): the shadows are maintained outside (no refresh
        # from the fp32 masters), tokens are looked up in the bf16 copy of the table, and `pre_block(i)` runs before
        # block i reads its weights (i = -1: embedding at the bottom, head at the top)
        self.external_shadows = False
        self.bf16_embedding = False
        self.pre_block = None
        # tensor parallelism (parallel/tensor_parallel.py::EngineTP): the projections hold this rank's heads / FFN
        # columns; the partial sums of the row-parallel products and of the column-parallel input gradients are
        # all-reduced over the axis
        self.tp = getattr(model, "tp", None)
        # gain gradients are accumulated by kernels with reductions, into destinations that must start at zero: the
        # backward pass clears all of them with one launch (`prezero_gains`) instead of one fill per gain
        self.gain_params = [p for p in model.parameters() if p.ndim == 1]
        self._prezeroed: set[int] = set()

    def prezero_gains(self, sink) -> None:
        """Called by the first backward function of a pass: zero every gain-gradient destination that starts a new
        sum in this pass (those that continue a running sum are left alone)."""
        from torchure_b200.ops import multi_tensor as MT

        self._prezeroed.clear()
        if sink is None or not MT.available():
            return
        dests = []
        for p in self.gain_params:
            dst, acc = sink.grad_dest(p)
            if not acc:
                dests.append(dst)
                self._prezeroed.add(id(p))
        if dests:
            MT.zero_(dests)

    # -- shadows -----------------------------------------------------------------------------
    def shadow_pairs(self):
        """(fp32 parameter, bf16 shadow) pairs; the fused AdamW writes the shadow while it updates the master."""
        self._optimizer_owned = True
        return list(self._pairs)

    def refresh(self) -> None:
        if self.external_shadows:
            return
        for p, shadow in self._pairs:
            v = p._version
            if self._versions.get(id(p)) != v:
                K.cast_to_bf16(p.detach(), shadow)
                self._versions[id(p)] = v

    def note_optimizer_step(self) -> None:
        """The fused AdamW just rewrote every shadow together with its master."""
        for p, _ in self._pairs:
            self._versions[id(p)] = p._version

    @property
    def cp(self):
        """(mesh, axis) when the model runs under context parallelism: the engine then sees this rank's two zigzag
        chunks of every sequence, rotates by their global positions and runs attention as a ring over the axis."""
        return getattr(self.model, "cp", None)

    def rope_tables(self, S: int, device):
        cp = self.cp
        if cp is None:
            return self.model.rope.tables(S, device)
        return self.model.rope.zigzag_tables(S, cp[0].size(cp[1]), cp[0].coordinate(cp[1]), device)

    # -- forward -----------------------------------------------------------------------------
    def forward_hidden(self, ids: torch.Tensor) -> torch.Tensor:
        m = self.model
        self.refresh()
        B, S = ids.shape
        x, y = None, None
        flat_ids = ids.reshape(-1)
        if self.pre_block is not None:
            self.pre_block(-1)
        for i, (block, sh) in enumerate(zip(m.blocks, self.layers)):
            if self.pre_block is not None:
                self.pre_block(i)
            g = block.gqa
            qn = g.q_norm.weight if g.qk_norm else self.dummy
            kn = g.k_norm.weight if g.qk_norm else self.dummy
            first = i == 0
            x, y = _BlockFn.apply(
                self, sh, i, B, S, flat_ids if first else None,
                m.token_emb.weight if first else None, x, y,
                block.norm1.weight, g.q_proj.weight, g.k_proj.weight, g.v_proj.weight, g.o_proj.weight, qn, kn,
                block.norm2.weight, block.ffn.gate_proj.weight, block.ffn.up_proj.weight, block.ffn.down_proj.weight)
        h = _FinalNormFn.apply(x, y, m.norm.weight, m.norm.eps, self)
        if self.tied and torch.is_grad_enabled() and m.token_emb.weight.requires_grad:
            self.expect_tied_grad = True
        return h.view(B, S, -1)

    def lm_head(self, h: torch.Tensor) -> torch.Tensor:
        m = self.model
        B, S, D = h.shape
        logits = _LinearFn.apply(h.reshape(B * S, D), m.lm_head.weight, self.head_shadow)
        return logits.view(B, S, -1)


class _BlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, eng, sh, layer_idx, B, S, ids, table, x_in, y_in, w1, wq, wk, wv, wo, qn, kn, w2, wg, wu, wd):
        cfg = eng.cfg
        Hq, Hkv, hd, eps = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["norm_eps"]
        use_norm = cfg["qk_norm"]
        cos, sin = eng.rope_tables(S, w1.device)
        if ids is not None:
            x, h1, rstd1 = K.add_rmsnorm(None, None, w1, eps, ids=ids,
                                         table=eng.emb_shadow if eng.bf16_embedding else table)
        else:
            x, h1, rstd1 = K.add_rmsnorm(x_in, y_in, w1, eps)
        qkv = K.linear_fwd(h1, sh.wqkv)
        qk = K.qknorm_rope(qkv, qn, kn, cos, sin, S, Hq, Hkv, eps, use_norm)
        need_grad = any(ctx.needs_input_grad)
        if eng.cp is not None:
            from torchure_b200.parallel.context_parallel import ring_fwd_sm100

            # q is used where it lies in `qk`; K and V travel around the ring, so they get buffers of their own
            k2, v2 = qk[:, Hq * hd:].contiguous(), qkv[:, (Hq + Hkv) * hd:].contiguous()
            o, lse = ring_fwd_sm100(qk, 0, k2, v2, B, S, Hq, Hkv, *eng.cp)
            st = (k2, v2, lse)
        else:
            o, st = attn_ops.attn_fwd(qk, qkv, B, S, Hq, Hkv, hd, need_grad=need_grad)
        y_a = K.linear_fwd(o, sh.wo)
        if eng.tp is not None:
            eng.tp.all_reduce_(y_a)        # row-parallel: sum the partial products of the ranks' heads
        x2, h2, rstd2 = K.add_rmsnorm(x, y_a, w2, eps)
        gu = K.linear_fwd(h2, sh.wgu)
        act = K.swiglu(gu)
        y_out = K.linear_fwd(act, sh.wd)
        if eng.tp is not None:
            eng.tp.all_reduce_(y_out)      # ... and of their FFN columns
        ctx.eng, ctx.sh, ctx.dims = eng, sh, (B, S, Hq, Hkv, hd, eps, use_norm)
        ctx.attn_state = st
        ctx.first = ids is not None
        ctx.save_for_backward(ids, x, h1, rstd1, qkv, qk, o, x2, h2, rstd2, gu, act, w1, qn, kn, w2, cos, sin)
        return x2, y_out

    @staticmethod
    def backward(ctx, dx2, dy):
        ids, x, h1, rstd1, qkv, qk, o, x2, h2, rstd2, gu, act, w1, qn, kn, w2, cos, sin = ctx.saved_tensors
        eng, sh = ctx.eng, ctx.sh
        B, S, Hq, Hkv, hd, eps, use_norm = ctx.dims
        P = dict(sh.params)  # the nn.Parameter objects, which is what a gradient sink is keyed by
        if ctx.first:
            P["table"] = eng.model.token_emb.weight
        out = _GradOut(eng.model._grad_sink, x.device, eng)
        nq, nkv = Hq * hd, Hkv * hd
        # the consumer computed x2 + y_out, so both incoming grads carry the same values
        if dy is None:
            dy = dx2.to(BF16)
        if dx2 is None:
            dx2 = dy.float()
        dy = dy.contiguous()
        # ---- MLP
        d_act = K.linear_dgrad(dy, sh.wd)
        out.wgrad((P["wd"],), dy, act)
        d_gu = K.swiglu_bwd(d_act, gu)
        del d_act
        d_h2 = K.linear_dgrad(d_gu, sh.wgu)
        if eng.tp is not None:
            eng.tp.all_reduce_(d_h2)       # column-parallel input gradient: every rank contributes its columns
        out.wgrad((P["wg"], P["wu"]), d_gu, h2)
        del d_gu
        dw2 = out.small(P["w2"])
        dx1, dx1_b = K.rmsnorm_bwd(d_h2, x2, w2, rstd2, dx2, dw2)
        out.done(P["w2"])
        del d_h2
        # ---- attention
        d_o = K.linear_dgrad(dx1_b, sh.wo)
        out.wgrad((P["wo"],), dx1_b, o)
        if eng.cp is not None:
            from torchure_b200.parallel.context_parallel import ring_bwd_sm100

            k2, v2, lse = ctx.attn_state
            dq_acc, dk, dv = ring_bwd_sm100(qk, 0, k2, v2, o, lse, d_o, B, S, Hq, Hkv, *eng.cp)
            dqkv = torch.empty(B * S, nq + 2 * nkv, dtype=BF16, device=d_o.device)   # q columns: read from dq_acc
            dqkv[:, nq:nq + nkv].copy_(dk.view(B * S, nkv))
            dqkv[:, nq + nkv:].copy_(dv.view(B * S, nkv))
            del k2, v2, lse, dk, dv
        else:
            dqkv, dq_acc = attn_ops.attn_bwd(d_o, qk, qkv, ctx.attn_state, B, S, Hq, Hkv, hd, keep_dq_fp32=True)
        ctx.attn_state = None
        del d_o
        if use_norm:
            dqn, dkn = out.small(P["qn"]), out.small(P["kn"])
        else:
            dqn = dkn = eng.dummy
        if use_norm and eng.tp is not None:
            # the gains are shared by all heads while each rank sees only its own: this backward's contribution is
            # summed over the axis before it joins the (possibly running) destination
            part = torch.zeros(2, dqn.numel(), dtype=torch.float32, device=dqn.device)
            K.qknorm_rope_bwd_(dqkv, qkv, qn, kn, cos, sin, part[0], part[1], S, Hq, Hkv, eps, use_norm, dq_acc=dq_acc)
            eng.tp.all_reduce_(part)
            dqn.add_(part[0])
            dkn.add_(part[1])
        else:
            K.qknorm_rope_bwd_(dqkv, qkv, qn, kn, cos, sin, dqn, dkn, S, Hq, Hkv, eps, use_norm, dq_acc=dq_acc)
        del dq_acc
        if use_norm:
            out.done(P["qn"])
            out.done(P["kn"])
        d_h1 = K.linear_dgrad(dqkv, sh.wqkv)
        if eng.tp is not None:
            eng.tp.all_reduce_(d_h1)
        out.wgrad((P["wq"], P["wk"], P["wv"]), dqkv, h1)
        del dqkv
        dw1 = out.small(P["w1"])
        want_prev = not ctx.first
        early = ctx.first and eng.pending_tied_grad is EARLY_TABLE
        # with the row exchange, dx0 is written where the other ranks can read it
        dx_out = out.sink.embed_rows_dest(x.shape[0], x.shape[1]) if early else None
        dx0, dx0_b = K.rmsnorm_bwd(d_h1, x, w1, rstd1, dx1, dw1, want_bf16=want_prev, dx_out=dx_out)
        out.done(P["w1"])
        if early:
            eng.pending_tied_grad = None
            out.sink.exchange_embedding(ids, P["table"])
        elif ctx.first and ctx.needs_input_grad[6]:
            table = P["table"]
            stash = eng.pending_tied_grad
            eng.pending_tied_grad = None
            if stash is not None:
                d_table = stash  # the head's fp32 dW (possibly the sink's slice); the gather's rows are added to it
            elif out.sink is not None:
                d_table, acc = out.sink.grad_dest(table)
                if not acc:
                    d_table.zero_()
            else:
                d_table = torch.zeros(table.shape, dtype=torch.float32, device=x.device)
            if d_table.is_contiguous() and d_table.shape[1] % 4 == 0:
                K.embedding_scatter_([(ids, dx0)], d_table, ids.numel())   # fixed order of additions, no atomics
            else:
                K.embedding_bwd_(dx0, ids, d_table)
            if out.sink is not None:
                out.sink.grad_written(table)
            else:
                out.grads[table] = d_table
        g = out.grads.get
        return (None, None, None, None, None, None, g(P.get("table")),
                dx0 if want_prev else None, dx0_b if want_prev else None,
                g(P["w1"]), g(P["wq"]), g(P["wk"]), g(P["wv"]), g(P["wo"]),
                g(P["qn"]) if use_norm else None, g(P["kn"]) if use_norm else None,
                g(P["w2"]), g(P["wg"]), g(P["wu"]), g(P["wd"]))


class _GradOut:
    """Where a block's weight gradients go: into the gradient sink (fused DDP buckets) when one is installed,
    otherwise into fresh fp32 tensors handed back to autograd."""

    def __init__(self, sink, device, eng=None):
        self.sink = sink
        self.device = device
        self.eng = eng
        self.grads: dict = {}

    def wgrad(self, params: tuple, dy: torch.Tensor, x: torch.Tensor) -> None:
        """dW[N, K] = dy[M, N]^T x[M, K]; `params` are the parameters whose rows make up N, in order."""
        if self.sink is None:
            rows = [p.shape[0] for p in params]
            dw = K.linear_wgrad(dy, x, out_dtype=torch.float32)
            at = 0
            for p, r in zip(params, rows):
                self.grads[p] = dw[at:at + r]
                at += r
            return
        dests = [self.sink.grad_dest(p) for p in params]
        rows = [d[0].shape[0] for d in dests]   # a sharded strategy may have released the parameter's own storage
        contiguous = all(dests[i][0].data_ptr() + dests[i][0].numel() * 4 == dests[i + 1][0].data_ptr()
                         for i in range(len(dests) - 1))
        same_mode = all(d[1] == dests[0][1] for d in dests)
        if contiguous and same_mode:
            first = dests[0][0]
            whole = torch.as_strided(first, (sum(rows), first.shape[1]), (first.shape[1], 1))
            K.linear_wgrad(dy, x, out=whole, accumulate=dests[0][1])
        else:
            at = 0
            for (dst, acc), r in zip(dests, rows):
                K.linear_wgrad(dy[:, at:at + r], x, out=dst, accumulate=acc)
                at += r
        for p in params:
            self.sink.grad_written(p)

    def small(self, p: torch.Tensor) -> torch.Tensor:
        """Zeroed (or running) fp32 destination for a gain gradient that a kernel accumulates with atomics."""
        if self.sink is None:
            t = torch.zeros(p.shape, dtype=torch.float32, device=self.device)
            self.grads[p] = t
            return t
        dst, acc = self.sink.grad_dest(p)
        if not acc:
            if self.eng is not None and id(p) in self.eng._prezeroed:
                self.eng._prezeroed.discard(id(p))     # cleared with all the others at the start of this pass
            else:
                dst.zero_()
        return dst

    def done(self, p: torch.Tensor) -> None:
        if self.sink is not None:
            self.sink.grad_written(p)


class _FinalNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, w, eps, eng):
        x2, h, rstd = K.add_rmsnorm(x, y, w, eps)
        ctx.save_for_backward(x2, rstd)
        ctx.eng = eng
        return h

    @staticmethod
    def backward(ctx, dh):
        x2, rstd = ctx.saved_tensors
        w = ctx.eng.model.norm.weight
        ctx.eng.prezero_gains(ctx.eng.model._grad_sink)      # this is the first engine function of a backward pass
        out = _GradOut(ctx.eng.model._grad_sink, x2.device, ctx.eng)
        dw = out.small(w)
        dx, dxb = K.rmsnorm_bwd(dh.contiguous().view(x2.shape).to(BF16), x2, w.detach(), rstd, None, dw)
        out.done(w)
        return dx, dxb, out.grads.get(w), None, None


class _LinearFn(torch.autograd.Function):
    """y = x @ w^T on the bf16 shadow of an fp32 weight (lm_head when logits are requested)."""

    @staticmethod
    def forward(ctx, x, weight, shadow):
        ctx.save_for_backward(x, shadow)
        return K.linear_fwd(x.contiguous(), shadow)

    @staticmethod
    def backward(ctx, dy):
        x, shadow = ctx.saved_tensors
        dy = dy.contiguous().to(BF16)
        dx = K.linear_dgrad(dy, shadow) if ctx.needs_input_grad[0] else None
        dw = K.linear_wgrad(dy, x, out_dtype=torch.float32) if ctx.needs_input_grad[1] else None
        return dx, dw, None
