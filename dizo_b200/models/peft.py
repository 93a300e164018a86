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

from .opt import OPTModel, make_batch


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
    """Describes ``num_prefix`` trainable key/value rows per layer, visible to every query.  With
    ``reparam`` the rows are produced by a per-layer MLP over shared input embeddings
    (large_models/prefix.py:177-197) and those MLPs and embeddings are what trains."""

    def __init__(self, model: OPTModel, num_prefix: int = 5, reparam: bool = False, embed_dim: int = 512,
                 mid_dim: int = 512, float16: bool = False, init_by_real_act: bool = True, seed: int = 0):
        if not model.use_prefix:
            raise ValueError("build the model with mode='prefix' (or 'lora+prefix')")
        if bool(reparam) != bool(model.prefix_reparam):
            raise ValueError("build the model with prefix_reparam=%r" % bool(reparam))
        self.model, self.num_prefix, self.reparam = model, num_prefix, bool(reparam)
        self.embed_dim, self.mid_dim = embed_dim, mid_dim
        self.names = [n for n in model.trainable_names if "prefix_" in n]
        if init_by_real_act:
            assert not reparam, "real-activation initialisation sets the prefix rows directly (no MLP)"
            init_prefix_by_real_activations(model, seed)


class LoRALinear:
    """A dense layer with a low-rank update, ``y = x W^T + b + s (x A^T) B^T`` with ``s = lora_alpha / r``
    (large_models/lora.py:25-98).  Inside :class:`OPTModel` the adapters are arena tensors folded into the
    QKV operand; this class is the stand-alone form of the same layer over the framework's GEMM kernel,
    for code that adapts a single projection.  ``merge()`` / ``unmerge()`` fold the update into ``weight``
    as the reference's ``train(False)`` / ``train(True)`` do with ``merge_weights``."""

    def __init__(self, in_features: int, out_features: int, r: int = 0, lora_alpha: int = 1,
                 bias: bool = True, device="cpu", dtype=torch.float32, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        bound = (1.0 / in_features) ** 0.5
        self.in_features, self.out_features, self.r, self.lora_alpha = in_features, out_features, r, lora_alpha
        self.weight = ((torch.rand(out_features, in_features, generator=g) * 2 - 1) * bound).to(device, dtype)
        self.bias = ((torch.rand(out_features, generator=g) * 2 - 1) * bound).to(device, dtype) if bias else None
        self.merged = False
        if r > 0:
            self.lora_A = ((torch.rand(r, in_features, generator=g) * 2 - 1) * bound).to(device, dtype)
            self.lora_B = torch.zeros(out_features, r, device=device, dtype=dtype)
            self.scaling = lora_alpha / r

    def trainable(self) -> dict:
        return {"lora_A": self.lora_A, "lora_B": self.lora_B} if self.r > 0 else {}

    def merged_weight(self) -> torch.Tensor:
        from ..ops import peft as peft_ops
        if self.r <= 0 or self.merged:
            return self.weight
        return peft_ops.lora_merge(self.weight, self.lora_A, self.lora_B, self.scaling)

    def merge(self) -> None:
        if self.r > 0 and not self.merged:
            self.weight = self.merged_weight()
            self.merged = True

    def unmerge(self) -> None:
        from ..ops import peft as peft_ops
        if self.r > 0 and self.merged:
            self.weight = peft_ops.lora_merge(self.weight, self.lora_A, self.lora_B, -self.scaling)
            self.merged = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import gemm
        shape = x.shape
        y = gemm.linear(x.reshape(-1, shape[-1]), self.merged_weight(), self.bias)
        return y.view(*shape[:-1], self.out_features)

    __call__ = forward


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
        model.param(model.layer_prefix(i) + "self_attn.prefix_keys").copy_(q3[:, d:2 * d])
        model.param(model.layer_prefix(i) + "self_attn.prefix_values").copy_(q3[:, 2 * d:])
