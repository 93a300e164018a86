"""Differentiable statement of the OPT and LLaMA-family forwards, for the two places that need a backward pass.

1. The first-order gamma search of DiZO (``--enhanced fo``; large_models/trainer.py:714-741,
   :805-830): the loss is differentiated with respect to the per-tensor gamma scalars only.
   The reference deep-copies the whole model every iteration and lets autograd flow through
   ``theta_0 + (theta - theta_0) * gamma / ||theta - theta_0||``; here the blended weight of a
   constrained tensor is built inside a per-layer checkpointed function, so neither a model
   copy nor per-layer activations of more than one layer are kept.
2. Ordinary first-order fine-tuning (``--trainer regular``), the reference's comparison arm
   (large_models/finetune.sh).  The flat arena is the single leaf tensor of an AdamW optimiser.

This path is cold (ten iterations every 50 ZO steps, or a baseline arm); it is written with
PyTorch ops (cuBLAS GEMMs, ``scaled_dot_product_attention``) because it needs autograd, and is
kept numerically aligned with the kernel forward: bf16 storage, fp32 softmax / LayerNorm
statistics / loss.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .opt import _P, Batch, OPTModel, layer_prefix


def _attention(qkv, n_heads, pad_left, prefix_k, prefix_v):
    B, L, d3 = qkv.shape
    d = d3 // 3
    hd = d // n_heads
    q, k, v = qkv.split(d, dim=-1)
    q = q.view(B, L, n_heads, hd).transpose(1, 2)
    k = k.view(B, L, n_heads, hd).transpose(1, 2)
    v = v.view(B, L, n_heads, hd).transpose(1, 2)
    idx = torch.arange(L, device=qkv.device)
    vis = (idx[None, :] <= idx[:, None])[None].expand(B, L, L)
    if pad_left is not None:
        pl = pad_left.view(B, 1, 1).long()
        vis = vis & ((idx.view(1, 1, L) >= pl) | (idx.view(1, 1, L) == idx.view(1, L, 1)))
    if prefix_k is not None:
        P = prefix_k.shape[0]
        pk = prefix_k.view(P, n_heads, hd).permute(1, 0, 2)[None].expand(B, -1, -1, -1)
        pv = prefix_v.view(P, n_heads, hd).permute(1, 0, 2)[None].expand(B, -1, -1, -1)
        k = torch.cat([pk.to(k.dtype), k], dim=2)
        v = torch.cat([pv.to(v.dtype), v], dim=2)
        vis = torch.cat([torch.ones(B, L, P, dtype=torch.bool, device=qkv.device), vis], dim=-1)
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=vis[:, None])
    return o.transpose(1, 2).reshape(B, L, d)


def _ln(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _llama_hidden(model, batch: Batch, W: Callable, use_checkpoint: bool) -> torch.Tensor:
    """Hidden states [B, L, d] of a LLaMA-family model before the final norm (the statement of
    ``LlamaModel._layer_forward``: RMSNorm, rotary q / k with grouped-query head expansion, SwiGLU)."""
    from ..ops.llama import rope_qkv_reference
    cfg = model.config
    ids = batch.input_ids.long()
    B, L = ids.shape
    d, H, Hkv, hd = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    h = F.embedding(ids, W(model.EMBED))

    def layer(i, h):
        lp = model.layer_prefix(i)
        a = lp + "self_attn."
        x = _rms(h, W(lp + "input_layernorm.weight"), cfg.rms_norm_eps)
        qkv = torch.cat([F.linear(x, W(a + "q_proj.weight")), F.linear(x, W(a + "k_proj.weight")),
                         F.linear(x, W(a + "v_proj.weight"))], dim=-1)
        qkv = rope_qkv_reference(qkv.reshape(B * L, -1), L, model.num_prefix, H, Hkv, hd,
                                 cfg.rope_theta).view(B, L, 3 * d)
        if model.use_prefix and model.prefix_reparam:
            emb = W(model.layer_prefix(0) + "self_attn.prefix_input_embeds")

            def mlp(stem):
                mid = torch.tanh(F.linear(emb, W(stem + "0.weight"), W(stem + "0.bias")))
                return F.linear(mid, W(stem + "2.weight"), W(stem + "2.bias"))
            pk, pv = mlp(a + "prefix_mlp_keys."), mlp(a + "prefix_mlp_values.")
        else:
            pk = W(a + "prefix_keys") if model.use_prefix else None
            pv = W(a + "prefix_values") if model.use_prefix else None
        ctx = _attention(qkv, H, batch.pad_left, pk, pv)
        h = h + F.linear(ctx, W(a + "o_proj.weight"))
        x = _rms(h, W(lp + "post_attention_layernorm.weight"), cfg.rms_norm_eps)
        f = F.silu(F.linear(x, W(lp + "mlp.gate_proj.weight"))) * F.linear(x, W(lp + "mlp.up_proj.weight"))
        return h + F.linear(f, W(lp + "mlp.down_proj.weight"))

    for i in range(cfg.num_hidden_layers):
        if use_checkpoint and torch.is_grad_enabled():
            h = checkpoint(layer, i, h, use_reentrant=False)
        else:
            h = layer(i, h)
    return h


def functional_loss(model: OPTModel, batch: Batch, weight_fn: Optional[Callable] = None,
                    use_checkpoint: bool = True) -> torch.Tensor:
    """Scalar loss with autograd.  ``weight_fn(name, tensor)`` may replace any trainable tensor
    by a differentiable function of it (identity when None)."""
    cfg = model.config
    wf = weight_fn or (lambda n, t: t)

    def W(name):
        t = model.param(name)
        return wf(name, t) if model._where[name] is model.arena else t

    if cfg.model_type != "opt":
        B, L = batch.input_ids.shape
        h = _llama_hidden(model, batch, W, use_checkpoint)
        x = _rms(h.reshape(B * L, cfg.hidden_size)[batch.rows.long()], W("model.norm.weight"), cfg.rms_norm_eps)
        return _loss_tail(batch, x, W("lm_head.weight") if model.untied else W(model.EMBED))
    ids = batch.input_ids.long()
    B, L = ids.shape
    d = cfg.hidden_size
    h = F.embedding(ids, W(_P + "embed_tokens.weight"))
    if cfg.word_embed_proj_dim != d:
        h = F.linear(h, W(_P + "project_in.weight"))
    h = h + F.embedding(batch.positions.long(), W(_P + "embed_positions.weight"))
    act = F.relu if cfg.activation_function == "relu" else F.gelu
    pre = cfg.do_layer_norm_before

    def layer(i, h):
        lp = layer_prefix(i)
        a = lp + "self_attn."
        qw, kw, vw = W(a + "q_proj.weight"), W(a + "k_proj.weight"), W(a + "v_proj.weight")
        if model.use_lora:
            s = model.lora_scaling
            qw = qw + s * (W(a + "q_proj.lora_B").float() @ W(a + "q_proj.lora_A").float()).to(qw.dtype)
            vw = vw + s * (W(a + "v_proj.lora_B").float() @ W(a + "v_proj.lora_A").float()).to(vw.dtype)
        x = _ln(h, W(lp + "self_attn_layer_norm.weight"), W(lp + "self_attn_layer_norm.bias"),
                cfg.layer_norm_eps) if pre else h
        qkv = torch.cat([F.linear(x, qw, W(a + "q_proj.bias")), F.linear(x, kw, W(a + "k_proj.bias")),
                         F.linear(x, vw, W(a + "v_proj.bias"))], dim=-1)
        if model.use_prefix and model.prefix_reparam:
            emb = W(layer_prefix(0) + "self_attn.prefix_input_embeds")

            def mlp(stem):
                mid = torch.tanh(F.linear(emb, W(stem + "0.weight"), W(stem + "0.bias")))
                return F.linear(mid, W(stem + "2.weight"), W(stem + "2.bias"))
            pk, pv = mlp(a + "prefix_mlp_keys."), mlp(a + "prefix_mlp_values.")
        else:
            pk = W(a + "prefix_keys") if model.use_prefix else None
            pv = W(a + "prefix_values") if model.use_prefix else None
        ctx = _attention(qkv, cfg.num_attention_heads, batch.pad_left, pk, pv)
        h = h + F.linear(ctx, W(a + "out_proj.weight"), W(a + "out_proj.bias"))
        if not pre:
            h = _ln(h, W(lp + "self_attn_layer_norm.weight"), W(lp + "self_attn_layer_norm.bias"),
                    cfg.layer_norm_eps)
        x = _ln(h, W(lp + "final_layer_norm.weight"), W(lp + "final_layer_norm.bias"),
                cfg.layer_norm_eps) if pre else h
        f = act(F.linear(x, W(lp + "fc1.weight"), W(lp + "fc1.bias")))
        h = h + F.linear(f, W(lp + "fc2.weight"), W(lp + "fc2.bias"))
        if not pre:
            h = _ln(h, W(lp + "final_layer_norm.weight"), W(lp + "final_layer_norm.bias"),
                    cfg.layer_norm_eps)
        return h

    for i in range(cfg.num_hidden_layers):
        if use_checkpoint and torch.is_grad_enabled():
            h = checkpoint(layer, i, h, use_reentrant=False)
        else:
            h = layer(i, h)
    x = h.reshape(B * L, d)[batch.rows.long()]
    if pre:
        x = _ln(x, W(_P + "final_layer_norm.weight"), W(_P + "final_layer_norm.bias"), cfg.layer_norm_eps)
    if cfg.word_embed_proj_dim != d:
        x = F.linear(x, W(_P + "project_out.weight"))
    return _loss_tail(batch, x, W("lm_head.weight") if model.untied else W(_P + "embed_tokens.weight"))


def _loss_tail(batch: Batch, x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """The loss of the rows ``x`` [R, d] (already normalised) under the head ``table`` [V, d]."""
    if batch.cand_ids is not None:
        logits = x.float() @ table[batch.cand_ids.long()].float().t()
        return F.cross_entropy(logits, batch.labels.long())
    logits = (x @ table.t()).float()
    lp = torch.log_softmax(logits, dim=-1).gather(1, batch.targets.long().view(-1, 1)).squeeze(1)
    if not batch.classification:
        return -lp.mean()
    ss = batch.seq_start.tolist()
    seq_lp = torch.stack([lp[ss[i]:ss[i + 1]].mean() for i in range(len(ss) - 1)])
    es = batch.ex_start.tolist()
    labels = batch.labels.tolist()
    losses = [torch.logsumexp(seq_lp[es[e]:es[e + 1]], 0) - seq_lp[es[e] + labels[e]]
              for e in range(len(es) - 1)]
    return torch.stack(losses).mean()


def make_fo_loss(model: OPTModel) -> Callable[[Batch, torch.Tensor], torch.Tensor]:
    """loss(batch, alpha) with autograd through ``theta_0 + alpha_slot * (theta - theta_0)`` for
    the constrained tensors; gradients reach only ``alpha`` (hence gamma)."""
    arena = model.arena
    slot_of = {n: arena.pieces[arena.index[n]].slot for n in arena.slot_names}

    def fo_loss(batch: Batch, alpha: torch.Tensor) -> torch.Tensor:
        def wf(name, t):
            s = slot_of.get(name)
            if s is None:
                return t
            an = arena.anchor_view(name)
            return (an.float() + alpha[s] * (t.float() - an.float())).to(t.dtype)
        return functional_loss(model, batch, wf)

    return fo_loss


def fo_training_step(trainer, inputs) -> torch.Tensor:
    """One AdamW step of ordinary fine-tuning over the trainable arena (``--trainer regular``, the
    reference's comparison arm, large_models/finetune.sh).  ``inputs`` is one batch or a list of
    micro-batches whose gradients are accumulated (mean) before the step; under data parallelism
    the arena gradient is averaged over the ranks."""
    import torch.distributed as dist
    model, a = trainer.model, trainer.args
    micro = inputs if isinstance(inputs, list) else [inputs]
    data = model.arena.data
    if getattr(trainer, "_fo_opt", None) is None:
        data.requires_grad_(True)
        trainer._fo_opt = torch.optim.AdamW([data], lr=a.learning_rate, weight_decay=a.weight_decay)
    for g in trainer._fo_opt.param_groups:
        g["lr"] = trainer._get_learning_rate()
    total = None
    with torch.enable_grad():
        for one in micro:
            loss = functional_loss(model, trainer._to_batch(one)) / len(micro)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
    if trainer._world > 1:
        dist.all_reduce(data.grad, group=trainer.dp_group if trainer.dp_group is not None else None)
        data.grad.div_(trainer._world)
    if a.max_grad_norm and a.max_grad_norm > 0:
        torch.nn.utils.clip_grad_norm_([data], a.max_grad_norm)
    trainer._fo_opt.step()
    trainer._fo_opt.zero_grad(set_to_none=True)
    return total.reshape(1)
