"""LLaMA-family decoder (LLaMA / LLaMA-2 / LLaMA-3 / Mistral dense models) on the same parameter arena,
transforms and kernels as :class:`dizo_b200.models.opt.OPTModel`.

The reference loads any Hugging Face causal LM (large_models/run.py:167-181) and names the llama modules
where it wires head tuning, prefix tuning and linear probing (large_models/run.py:242-265,
large_models/prefix.py:112-125, large_models/trainer.py:863, :921).  Here the family is a subclass that
changes what differs from OPT and nothing else:

* RMSNorm instead of LayerNorm, no biases, no learned positions;
* rotary position embedding applied to q and k after the fused q | k | v projection; with grouped-query
  attention (fewer key / value heads than query heads) the same kernel repeats the k / v heads, so the
  tcgen05 attention and the decode attention see ordinary multi-head operands;
* SwiGLU feed-forward: one GEMM over the adjacent gate | up weights, ``silu(gate) * up``, down projection
  with the residual fused in the GEMM epilogue;
* an untied ``lm_head.weight``.

Zeroth-order training perturbs every parameter, the token table included: the reference drops the first
named parameter only when it is OPT's ``model.decoder.embed_tokens.weight`` (large_models/trainer.py:1154-1159).
Its DiZO include rule is written against OPT names too and selects nothing for other families; here the same
rule (each layer's k_proj / v_proj weight) applies to the LLaMA names.  Modes: ``full``, ``prefix``,
``head`` (LoRA is OPT-only in the reference as well, large_models/lora.py:114-119).

Positions: a plain forward of the Hugging Face model numbers the columns 0..L-1 whatever the padding, after
the ``num_prefix`` cached prefix rows when prefix tuning is on; rotary attention depends on position
differences only, so left padding needs no per-row positions.  Prefix keys enter unrotated, as rows of the
key cache.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from types import SimpleNamespace

import torch

from ..ops import attention as attn_ops
from ..ops import gemm, norm
from ..ops import llama as llama_ops
from .opt import Batch, OPTModel, _arena_sort_key, adapter_param_specs

_LP = "model."


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int | None = None
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    hidden_act: str = "silu"
    pad_token_id: int | None = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    model_type: str = "llama"

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.pad_token_id is None:
            self.pad_token_id = 0                 # the reference's llama fix-up (large_models/run.py:229-231)

    # names the shared code reads
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def ffn_dim(self) -> int:
        return self.intermediate_size

    @property
    def word_embed_proj_dim(self) -> int:
        return self.hidden_size

    do_layer_norm_before = True
    activation_function = "silu"

    @property
    def layer_norm_eps(self) -> float:
        return self.rms_norm_eps

    @classmethod
    def from_hf(cls, hf) -> "LlamaConfig":
        d = hf if isinstance(hf, dict) else hf.to_dict()
        keys = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in keys}
        rp = d.get("rope_parameters") or {}
        if "rope_theta" not in kw and "rope_theta" in rp:
            kw["rope_theta"] = rp["rope_theta"]
        scaling = d.get("rope_scaling") or (rp if rp.get("rope_type", "default") != "default" else None)
        if scaling and scaling.get("rope_type", scaling.get("type", "default")) != "default":
            raise NotImplementedError(f"rotary scaling {scaling} is not implemented (plain rotary only)")
        if isinstance(kw.get("eos_token_id"), (list, tuple)):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        return cls(**kw)

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        arch = "MistralForCausalLM" if self.model_type == "mistral" else "LlamaForCausalLM"
        d.update(architectures=[arch], attention_bias=False, mlp_bias=False, use_cache=True,
                 head_dim=self.head_dim)
        return d


def _cfg(d, L, h, f, **kw):
    return dict(hidden_size=d, num_hidden_layers=L, num_attention_heads=h, intermediate_size=f, **kw)


PRESETS: dict[str, dict] = {
    "llama-tiny": _cfg(64, 2, 4, 176, vocab_size=512, max_position_embeddings=128),
    "llama-tiny-gqa": _cfg(64, 2, 4, 176, vocab_size=512, max_position_embeddings=128, num_key_value_heads=2),
    "llama-7b": _cfg(4096, 32, 32, 11008, max_position_embeddings=2048, rms_norm_eps=1e-6),
    "llama-13b": _cfg(5120, 40, 40, 13824, max_position_embeddings=2048, rms_norm_eps=1e-6),
    "llama-2-7b": _cfg(4096, 32, 32, 11008),
    "llama-2-13b": _cfg(5120, 40, 40, 13824),
    "llama-2-70b": _cfg(8192, 80, 64, 28672, num_key_value_heads=8),
    "llama-3-8b": _cfg(4096, 32, 32, 14336, num_key_value_heads=8, vocab_size=128256, rope_theta=500000.0,
                       max_position_embeddings=8192, bos_token_id=128000, eos_token_id=128001),
    "mistral-7b": _cfg(4096, 32, 32, 14336, num_key_value_heads=8, max_position_embeddings=32768,
                       model_type="mistral"),
}
for _k in ("llama-2-7b", "llama-2-13b", "llama-2-70b"):
    PRESETS[_k + "-hf"] = PRESETS[_k]
PRESETS["meta-llama-3-8b"] = PRESETS["llama-3-8b"]
PRESETS["mistral-7b-v0.1"] = PRESETS["mistral-7b"]


def preset(name: str, **overrides) -> LlamaConfig:
    key = name.lower().split("/")[-1]
    if key not in PRESETS:
        raise KeyError(f"unknown LLaMA preset {name!r}; known: {sorted(PRESETS)}")
    kw = dict(PRESETS[key])
    kw.update(overrides)
    return LlamaConfig(**kw)


def llama_layer_prefix(i: int) -> str:
    return f"{_LP}layers.{i}."


# order of a layer's tensors inside an arena: the fused operands (q | k | v, gate | up) are adjacent
_LLAMA_ORDER = ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight",
                "input_layernorm.weight", "post_attention_layernorm.weight",
                "self_attn.prefix_keys", "self_attn.prefix_values", "self_attn.prefix_input_embeds"] + \
               [f"self_attn.prefix_mlp_{kv}.{j}.{wb}" for kv in ("keys", "values") for j in (0, 2)
                for wb in ("weight", "bias")]


class LlamaModel(OPTModel):
    """Forward-only LLaMA-family model with trainable / frozen arenas (see the module docstring)."""

    EMBED = _LP + "embed_tokens.weight"
    layer_prefix = staticmethod(llama_layer_prefix)

    def __init__(self, config: LlamaConfig, device="cpu", dtype=torch.float32, mode: str = "full", **kw):
        if "lora" in mode:
            raise NotImplementedError("LoRA is wired for OPT only, as in the reference (large_models/lora.py:114-119)")
        if config.hidden_act != "silu":
            raise NotImplementedError(f"hidden_act {config.hidden_act!r}")
        assert config.head_dim % 4 == 0 and config.num_attention_heads % config.num_key_value_heads == 0
        kw.pop("untie_emb", None)
        super().__init__(config, device, dtype, mode=mode, **kw)

    # ------------------------------------------------------------------ architecture hooks
    def _base_specs(self):
        cfg = self.config
        d, dkv, F, V = cfg.hidden_size, cfg.kv_dim, cfg.intermediate_size, cfg.vocab_size
        specs = [(self.EMBED, (V, d), -1)]
        for i in range(cfg.num_hidden_layers):
            lp = llama_layer_prefix(i)
            specs += [(lp + "self_attn.q_proj.weight", (d, d), i), (lp + "self_attn.k_proj.weight", (dkv, d), i),
                      (lp + "self_attn.v_proj.weight", (dkv, d), i), (lp + "self_attn.o_proj.weight", (d, d), i),
                      (lp + "mlp.gate_proj.weight", (F, d), i), (lp + "mlp.up_proj.weight", (F, d), i),
                      (lp + "mlp.down_proj.weight", (d, F), i), (lp + "input_layernorm.weight", (d,), i),
                      (lp + "post_attention_layernorm.weight", (d,), i)]
        specs.append((_LP + "norm.weight", (d,), -1))
        return specs

    def _adapter_specs(self, lora_r, num_prefix, reparam=False, embed_dim=512, mid_dim=512):
        return adapter_param_specs(self.config, 0, num_prefix, reparam, embed_dim, mid_dim,
                                   layer_prefix=llama_layer_prefix)

    def _sort_key(self, name, group):
        return _arena_sort_key(name, group, _LLAMA_ORDER)

    @staticmethod
    def _is_norm_weight(name: str) -> bool:
        return name.endswith("layernorm.weight") or name.endswith("model.norm.weight")

    def _select_trainable(self):
        if self.mode == "full":
            return list(self.hf_order)            # the token table trains too (see the module docstring)
        return super()._select_trainable()

    def dizo_include_names(self):
        if self.mode == "full":
            return [n for n in self.hf_order if "self_attn.k_proj.weight" in n or "self_attn.v_proj.weight" in n]
        return []

    # ------------------------------------------------------------------ weights of one block
    def _layer_weights(self, i: int, get) -> SimpleNamespace:
        lp = llama_layer_prefix(i)
        a = lp + "self_attn."
        w = SimpleNamespace()
        if self.use_prefix and self.prefix_reparam and i == 0:
            self._prefix_embeds = get(a + "prefix_input_embeds").clone()
        w.qkv_w = self._fused([get(a + "q_proj.weight"), get(a + "k_proj.weight"), get(a + "v_proj.weight")])
        w.out_w = get(a + "o_proj.weight")
        w.gu_w = self._fused([get(lp + "mlp.gate_proj.weight"), get(lp + "mlp.up_proj.weight")])
        w.down_w = get(lp + "mlp.down_proj.weight")
        w.ln1_w, w.ln2_w = get(lp + "input_layernorm.weight"), get(lp + "post_attention_layernorm.weight")
        if self.use_prefix and self.prefix_reparam:
            emb = self._prefix_embeds
            w.prefix_k, w.prefix_v = (self._prefix_mlp(emb, a + f"prefix_mlp_{kv}.", get) for kv in ("keys", "values"))
        else:
            w.prefix_k = get(a + "prefix_keys") if self.use_prefix else None
            w.prefix_v = get(a + "prefix_values") if self.use_prefix else None
        return w

    def _rope(self, qkv_raw: torch.Tensor, L: int, pos0: int) -> torch.Tensor:
        cfg = self.config
        return llama_ops.rope_qkv(qkv_raw, L, pos0 + self.num_prefix, cfg.num_attention_heads,
                                  cfg.num_key_value_heads, cfg.head_dim, cfg.rope_theta)

    def _mlp(self, h: torch.Tensor, w: SimpleNamespace) -> torch.Tensor:
        x = llama_ops.rmsnorm(h, w.ln2_w, self.config.rms_norm_eps)
        f = gemm.linear_swiglu(x, w.gu_w)
        return gemm.linear(f, w.down_w, residual=h)

    # ------------------------------------------------------------------ forward
    def _embed(self, ids, positions, gget):
        return norm.embed(ids, None, gget(self.EMBED), None)

    def _embed_param_names(self):
        return [self.EMBED]

    def _final_norm(self, x, gget):
        return llama_ops.rmsnorm(x, gget(_LP + "norm.weight"), self.config.rms_norm_eps)

    def _layer_forward(self, h: torch.Tensor, w: SimpleNamespace, batch: Batch, rows: torch.Tensor | None = None):
        cfg = self.config
        B, L, d = h.shape
        x = llama_ops.rmsnorm(h, w.ln1_w, cfg.rms_norm_eps)
        qkv = gemm.linear_qkv_rope(x.reshape(B * L, d), w.qkv_w, L, self.num_prefix, cfg.num_attention_heads,
                                   cfg.num_key_value_heads, cfg.head_dim, cfg.rope_theta)
        if self.kv_capture is not None:
            self.kv_capture.append(qkv)
        ctx = attn_ops.attention(qkv.view(B, L, 3 * d), cfg.num_attention_heads, batch.pad_left,
                                 w.prefix_k, w.prefix_v)
        if rows is not None:
            ctx = norm.gather_rows(ctx.reshape(-1, d), rows)
            h = norm.gather_rows(h.reshape(-1, d), rows)
        h = gemm.linear(ctx, w.out_w, residual=h)
        return self._mlp(h, w)

    # ------------------------------------------------------------------ one-token decoding
    def decode_embed(self, tokens, positions, get):
        return norm.embed(tokens.view(-1, 1), None, get(self.EMBED), None).view(-1, self.config.hidden_size)

    def decode_block(self, h, w, k_cache, v_cache, t, pad_left):
        from ..ops import decode as decode_ops
        cfg = self.config
        d = cfg.hidden_size
        x = llama_ops.rmsnorm(h, w.ln1_w, cfg.rms_norm_eps)
        qkv = self._rope(gemm.linear(x, w.qkv_w), 1, t)
        k_cache[:, t].copy_(qkv[:, d:2 * d])
        v_cache[:, t].copy_(qkv[:, 2 * d:])
        ctx = decode_ops.decode_attention(qkv[:, :d], k_cache, v_cache, t + 1, cfg.num_attention_heads, pad_left,
                                          w.prefix_k, w.prefix_v)
        h = gemm.linear(ctx.contiguous(), w.out_w, residual=h)
        return self._mlp(h, w)
