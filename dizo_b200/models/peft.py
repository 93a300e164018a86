"""Parameter-efficient fine-tuning wiring: LoRA, prefix tuning, head tuning.

In this framework the adapters are not modules patched onto a Hugging Face model: they are
extra tensors of the parameter arena (``...self_attn.{q,v}_proj.lora_{A,B}``,
``...self_attn.prefix_{keys,values}``), selected by ``OPTModel(mode=...)``.  The classes below
keep the reference's constructor surface (large_models/lora.py:101-147,
large_models/prefix.py:89-200) as thin descriptions of such a model, and
``init_prefix_by_real_activations`` reproduces the prefix initialisation from the keys/values
of random real tokens (large_models/prefix.py:127-138, :157-162).

Difference kept on purpose: with both ``--lora`` and ``--prefix_tuning`` the reference's LoRA
freeze loop also freezes the prefix tensors (large_models/lora.py:145-147), so only LoRA
trains there; here both sets train.
"""
from __future__ import annotations

import torch

from .opt import OPTModel, layer_prefix, make_batch


class LoRA:
    """Describes LoRA on q_proj and v_proj of every layer: A [r, in] ~ kaiming-uniform(a=sqrt 5),
    B [out, r] = 0, scaling = alpha / r; everything else frozen."""

    def __init__(self, model: OPTModel, r: int = 8, alpha: int = 16, float16: bool = False):
        if not model.use_lora:
            raise ValueError("build the model with mode='lora' (or 'lora+prefix')")
        self.model, self.r, self.alpha = model, r, alpha
        self.scaling = alpha / r
        self.names = [n for n in model.trainable_names if "lora_" in n]


class PrefixTuning:
    """Describes ``num_prefix`` trainable key/value rows per layer, visible to every query."""

    def __init__(self, model: OPTModel, num_prefix: int = 5, reparam: bool = False, embed_dim: int = 512,
                 mid_dim: int = 512, float16: bool = False, init_by_real_act: bool = True, seed: int = 0):
        if reparam:
            raise NotImplementedError("the reparameterisation MLP is unused in the reference "
                                      "(no_reparam defaults to True, large_models/run.py:84)")
        if not model.use_prefix:
            raise ValueError("build the model with mode='prefix' (or 'lora+prefix')")
        self.model, self.num_prefix = model, num_prefix
        self.names = [n for n in model.trainable_names if "prefix_" in n]
        if init_by_real_act:
            init_prefix_by_real_activations(model, seed)


@torch.no_grad()
def init_prefix_by_real_activations(model: OPTModel, seed: int = 0) -> None:
    """prefix_keys/values of layer l <- that layer's K/V projections of ``num_prefix`` random
    vocabulary tokens run through the (prefix-free) model."""
    if not model.use_prefix:
        return
    cfg, P = model.config, model.num_prefix
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab_size, (1, P), generator=g)
    batch = make_batch(ids).to(model.device)
    d = cfg.hidden_size
    model.use_prefix, model.kv_capture = False, []
    try:
        model.hidden_states(batch)
        cap = model.kv_capture
    finally:
        model.use_prefix, model.kv_capture = True, None
    for i, qkv in enumerate(cap):
        q3 = qkv.reshape(P, 3 * d)
        model.param(layer_prefix(i) + "self_attn.prefix_keys").copy_(q3[:, d:2 * d])
        model.param(layer_prefix(i) + "self_attn.prefix_values").copy_(q3[:, 2 * d:])
