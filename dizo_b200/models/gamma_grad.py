"""d loss / d alpha for the first-order gamma search of DiZO, on the framework's own kernels.

The reference (large_models/trainer.py:714-741, :805-830) deep-copies the model, rewrites every
constrained weight as ``theta_0 + (theta - theta_0) * gamma / ||theta - theta_0||`` under autograd
and calls ``loss.backward()``; only the gamma scalars receive a gradient.  Here the same quantity
is computed without autograd and without a weight gradient:

* forward: the ordinary kernel forward over the blended weights (the sweep stages
  ``theta_0 + alpha (theta - theta_0)`` per layer), keeping per layer the residual-stream inputs,
  the LayerNorm output feeding QKV, the QKV activation, the attention context with its
  log-sum-exp, and the ReLU output;
* backward, layer by layer from the top: data-gradient GEMMs that read the staged weights in
  place (``dz_gemm_bf16_nn``, ReLU backward and gradient accumulation fused in the epilogue),
  the tcgen05 attention backward, LayerNorm input gradients;
* for a constrained tensor W (k_proj / v_proj weight) with ``Y = X W_eff^T``:
  ``d loss / d alpha = <dY, X (theta - theta_0)^T>`` - one extra forward-shaped GEMM and a
  deterministic dot product, never a [out, in] weight gradient.

Supported layout: full-parameter mode, pre-LayerNorm OPT with ``word_embed_proj_dim ==
hidden_size`` and ReLU (every OPT size except 350m); other configurations use the autograd
statement in :mod:`dizo_b200.models.opt_autograd`.  CPU tensors run the same orchestration over
the PyTorch statements of the ops, which is how the CPU suite checks it against autograd.
"""
from __future__ import annotations

import torch

from ..ops import attention as attn_ops
from ..ops import backward as bw
from ..ops import gemm, loss as loss_ops, norm
from .opt import _P, Batch, OPTModel, Transform, layer_prefix


def supported(model: OPTModel) -> bool:
    cfg = model.config
    return (model.mode == "full" and cfg.do_layer_norm_before and cfg.word_embed_proj_dim == cfg.hidden_size
            and cfg.activation_function == "relu" and type(model).hidden_states is OPTModel.hidden_states)


class GammaGrad:
    """``loss_and_grad(batch, alpha)`` -> (loss fp32 [1], d loss / d alpha fp32 [n_slots])."""

    def __init__(self, model: OPTModel):
        assert supported(model), "configuration not covered by the kernel backward"
        self.model = model
        ar = model.arena
        self.slot_of = {n: ar.pieces[ar.index[n]].slot for n in ar.slot_names}
        self.n_slots = len(ar.slot_names)

    # ------------------------------------------------------------------ helpers
    def _stage(self, i: int, tr: Transform, key):
        m = self.model
        lo, hi = m.arena.group_range(i)
        numel = max(m.arena.group_numel(g) for g in m.arena.groups() if g >= 0)
        buf = m._staging_for(("gg", key), numel)
        shift = m._sweep_group(i, tr, buf)
        return m._layer_weights(i, m._resolver(i, tr, buf, shift))

    def _attention(self, qkv, B, L, pad_left):
        """context and the saved statistic (None on CPU: the CPU backward uses autograd)."""
        m = self.model
        H = m.config.num_attention_heads
        if qkv.is_cuda:
            lse = torch.empty((B, H, L), dtype=torch.float32, device=qkv.device)
            ctx = attn_ops.attention(qkv.view(B, L, -1), H, pad_left, lse=lse)
            return ctx, lse
        return attn_ops.attention(qkv.view(B, L, -1), H, pad_left), None

    # ------------------------------------------------------------------ loss tail
    def _tail(self, h2: torch.Tensor, batch: Batch, gget):
        """loss and d loss / d h2 (zero outside ``batch.rows``)."""
        m, cfg = self.model, self.model.config
        d = cfg.hidden_size
        rows = batch.rows
        hr = norm.gather_rows(h2, rows)
        lnw, lnb = gget(_P + "final_layer_norm.weight"), gget(_P + "final_layer_norm.bias")
        x = norm.layernorm(hr, lnw, lnb, cfg.layer_norm_eps)
        table = gget("lm_head.weight") if m.untied else gget(_P + "embed_tokens.weight")
        if batch.cand_ids is not None:
            # a handful of candidate columns: [rows, C] logits, differentiated on the spot
            tc = table[batch.cand_ids.long()].float()
            with torch.enable_grad():
                xf = x.float().requires_grad_(True)
                loss = torch.nn.functional.cross_entropy(xf @ tc.t(), batch.labels.long())
                (dx,) = torch.autograd.grad(loss, xf)
            dx = dx.to(x.dtype)
            loss = loss.detach().reshape(1)
        else:
            lp, lse = _logprobs_lse(x, table, batch.targets)
            # d loss / d lp over [rows] scalars
            with torch.enable_grad():
                lpr = lp.detach().requires_grad_(True)
                loss = _option_loss(lpr, batch)
                (coef,) = torch.autograd.grad(loss, lpr)
            loss = loss.detach().reshape(1)
            dx = torch.empty_like(x)
            step = 4096
            for r0 in range(0, x.shape[0], step):
                r1 = min(x.shape[0], r0 + step)
                logits = gemm.linear(x[r0:r1], table)                       # bf16 [chunk, V]
                bw.softmax_ce_backward_(logits, lse[r0:r1], batch.targets[r0:r1], coef[r0:r1].contiguous())
                dx[r0:r1] = bw.linear_dgrad(logits, table)
        dhr = bw.layernorm_backward(dx, hr, lnw, cfg.layer_norm_eps)
        dh = torch.zeros_like(h2)
        bw.scatter_rows(dhr, rows, dh)
        return loss, dh

    # ------------------------------------------------------------------ main entry
    @torch.no_grad()
    def loss_and_grad(self, batch: Batch, alpha: torch.Tensor):
        m, cfg = self.model, self.model.config
        ar = m.arena
        nl, d = cfg.num_hidden_layers, cfg.hidden_size
        eps = cfg.layer_norm_eps
        B, L = batch.input_ids.shape
        M = B * L
        tr = Transform(seed=0, coef=0.0, alpha=alpha)
        # ---- forward with saves
        g_staged = m._staging_for("globals", ar.group_numel(-1)) if -1 in ar.groups() else None
        g_shift = m._sweep_group(-1, tr, g_staged) if g_staged is not None else 0
        gget = m._resolver(-1, tr, g_staged, g_shift)
        m._gget = gget
        h = norm.embed(batch.input_ids, batch.positions, gget(_P + "embed_tokens.weight"),
                       gget(_P + "embed_positions.weight")).view(M, d)
        saved = []
        for i in range(nl):
            w = self._stage(i, tr, 0)
            x1 = norm.layernorm(h, w.ln1_w, w.ln1_b, eps)
            qkv = gemm.linear(x1, w.qkv_w, w.qkv_b)
            ctx, lse = self._attention(qkv, B, L, batch.pad_left)
            h_mid = gemm.linear(ctx.view(M, d), w.out_w, w.out_b, residual=h)
            x2 = norm.layernorm(h_mid, w.ln2_w, w.ln2_b, eps)
            f = gemm.linear(x2, w.fc1_w, w.fc1_b, act="relu")
            h_out = gemm.linear(f, w.fc2_w, w.fc2_b, residual=h_mid)
            saved.append((h, x1, qkv, ctx, lse, h_mid, f))
            h = h_out
        loss, dh = self._tail(h, batch, gget)
        # ---- backward
        grad = torch.zeros(max(self.n_slots, 1), dtype=torch.float32, device=h.device)
        H = cfg.num_attention_heads
        for i in reversed(range(nl)):
            h_in, x1, qkv, ctx, lse, h_mid, f = saved.pop()
            w = self._stage(i, tr, 1)
            lp = layer_prefix(i)
            # MLP: h_out = h_mid + fc2(relu(fc1(LN2(h_mid))))
            df = bw.linear_dgrad(dh, w.fc2_w, mask=f)                        # [M, F], ReLU backward fused
            dx2 = bw.linear_dgrad(df, w.fc1_w)
            del df
            dh_mid = bw.layernorm_backward(dx2, h_mid, w.ln2_w, eps, add=dh)
            # attention block: h_mid = h_in + out_proj(attn(qkv(LN1(h_in))))
            dctx = bw.linear_dgrad(dh_mid, w.out_w)
            if qkv.is_cuda:
                dqkv = attn_ops.attention_backward(qkv.view(B, L, 3 * d), ctx.view(B, L, d), dctx.view(B, L, d),
                                                   lse, H, batch.pad_left).view(M, 3 * d)
            else:
                dqkv = attn_ops.attention_backward_reference(qkv.view(B, L, 3 * d), dctx.view(B, L, d), H,
                                                             batch.pad_left).view(M, 3 * d)
            # d loss / d alpha of the constrained projections of this layer
            for j, nm in enumerate(("q_proj", "k_proj", "v_proj")):
                full = lp + "self_attn." + nm + ".weight"
                s = self.slot_of.get(full)
                if s is None:
                    continue
                delta = bw.diff(ar.view(full), ar.anchor_view(full))
                t = gemm.linear(x1, delta, out_dtype=torch.float32)          # X (theta - theta_0)^T
                bw.dot(t, dqkv[:, j * d:(j + 1) * d], out=grad[s:s + 1])
                del t, delta
            if i > 0:                     # nothing below the first block depends on a constrained tensor
                dx1 = bw.linear_dgrad(dqkv, w.qkv_w)
                dh = bw.layernorm_backward(dx1, h_in, w.ln1_w, eps, add=dh_mid)
        return loss, grad[:self.n_slots]

def _logprobs_lse(x: torch.Tensor, table: torch.Tensor, targets: torch.Tensor):
    """(log p(target), natural-log log-sum-exp) per row."""
    if not x.is_cuda:
        logits = x.float() @ table.float().t()
        lse = torch.logsumexp(logits, dim=-1)
        return logits.gather(1, targets.long().view(-1, 1)).squeeze(1) - lse, lse
    import ctypes
    from ..ops import _lib
    L = _lib.lib()
    R, K = x.shape
    V = table.shape[0]
    nt = L.dz_gemm_lse_num_tiles(V)
    f = dict(dtype=torch.float32, device=x.device)
    pm, ps = torch.empty((R, nt), **f), torch.empty((R, nt), **f)
    tg, lp, lse = torch.empty(R, **f), torch.empty(R, **f), torch.empty(R, **f)
    ll = ctypes.c_longlong
    rc = L.dz_gemm_bf16_tn_lse(_lib.ptr(x), ll(x.stride(0)), _lib.ptr(table), ll(table.stride(0)),
                               _lib.ptr(targets), _lib.ptr(pm), _lib.ptr(ps), _lib.ptr(tg), R, V, K,
                               ctypes.c_float(1.0), _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm_bf16_tn_lse")
    rc = L.dz_lse_combine(_lib.ptr(pm), _lib.ptr(ps), _lib.ptr(tg), nt, R, _lib.ptr(lp), _lib.ptr(lse),
                          _lib.stream_ptr())
    _lib.check(rc, "dz_lse_combine")
    return lp, lse


def _option_loss(lp: torch.Tensor, batch: Batch) -> torch.Tensor:
    """The loss of ``ops.loss.option_ce`` as a differentiable function of the [rows] log-probs."""
    if not batch.classification:
        return -lp.mean()
    ss = batch.seq_start.tolist()
    seq_lp = torch.stack([lp[ss[i]:ss[i + 1]].mean() for i in range(len(ss) - 1)])
    es = batch.ex_start.tolist()
    labels = batch.labels.tolist()
    losses = [torch.logsumexp(seq_lp[es[e]:es[e + 1]], 0) - seq_lp[es[e] + labels[e]]
              for e in range(len(es) - 1)]
    return torch.stack(losses).mean()
