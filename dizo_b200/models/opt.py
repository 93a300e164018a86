"""OPT decoder over flat parameter arenas, forward-only, with in-flight weight transforms.

The graph is the Hugging Face OPT decoder (same parameter names, shapes and numerics
conventions as ``OPTForCausalLM``; the reference carries a copy in
large_models/ht_opt.py:485-1005): token + learned-position embedding (offset 2), pre- or
post-LayerNorm blocks of {QKV, causal attention, out_proj, fc1, activation, fc2}, final
LayerNorm, tied LM head.  What differs is how it is laid out and executed:

* every parameter lives in one of two flat arenas (``arena``: the tensors ZO optimises,
  ``frozen``: the rest), grouped per layer so a layer is one contiguous range;
* q/k/v weights and biases sit back to back and are consumed as one fused [3d, d] GEMM;
* a forward can be run under a :class:`Transform` (``theta + c*z(seed)`` for the two SPSA
  evaluations, ``theta_0 + alpha*(theta - theta_0)`` for the DiZO gamma search): each layer's
  range is swept into a staging buffer on a side stream one layer ahead of the GEMMs that
  consume it, so theta itself is never rewritten for a forward;
* LoRA is merged into the staged q/v weights, prefix rows go straight into the attention
  kernel, and the LM head only sees the rows that predict option tokens.

All math goes through :mod:`dizo_b200.ops`, which runs the sm_100a kernels for CUDA tensors
and PyTorch statements of the same ops for CPU tensors (fp32 oracle).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from types import SimpleNamespace
from typing import Callable, Iterable

import torch

from ..ops import attention as attn_ops
from ..ops import gemm, loss as loss_ops, norm, peft as peft_ops
from ..ops.zo import ParamArena, Piece


@dataclass
class OPTConfig:
    vocab_size: int = 50272
    hidden_size: int = 768
    num_hidden_layers: int = 12
    ffn_dim: int = 3072
    num_attention_heads: int = 12
    max_position_embeddings: int = 2048
    word_embed_proj_dim: int | None = None
    do_layer_norm_before: bool = True
    activation_function: str = "relu"
    pad_token_id: int = 1
    bos_token_id: int = 2
    eos_token_id: int = 2
    tie_word_embeddings: bool = True
    layer_norm_eps: float = 1e-5
    model_type: str = "opt"

    def __post_init__(self):
        if self.word_embed_proj_dim is None:
            self.word_embed_proj_dim = self.hidden_size

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_hf(cls, hf) -> "OPTConfig":
        d = hf if isinstance(hf, dict) else hf.to_dict()
        keys = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in keys})

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d.update(architectures=["OPTForCausalLM"], enable_bias=True,
                 layer_norm_elementwise_affine=True, _remove_final_layer_norm=False,
                 dropout=0.0, attention_dropout=0.0, activation_dropout=0.0, layerdrop=0.0,
                 init_std=0.02, use_cache=True, prefix="</s>")
        return d


def _cfg(d, L, h, f, **kw):
    return dict(hidden_size=d, num_hidden_layers=L, num_attention_heads=h, ffn_dim=f, **kw)


PRESETS: dict[str, dict] = {
    "opt-tiny": _cfg(64, 2, 4, 128, vocab_size=512, max_position_embeddings=128),
    "opt-125m": _cfg(768, 12, 12, 3072),
    "opt-350m": _cfg(1024, 24, 16, 4096, word_embed_proj_dim=512, do_layer_norm_before=False),
    "opt-1.3b": _cfg(2048, 24, 32, 8192),
    "opt-2.7b": _cfg(2560, 32, 32, 10240),
    "opt-6.7b": _cfg(4096, 32, 32, 16384),
    "opt-13b": _cfg(5120, 40, 40, 20480),
    "opt-30b": _cfg(7168, 48, 56, 28672),
    "opt-66b": _cfg(9216, 64, 72, 36864),
}


def preset(name: str, **overrides) -> OPTConfig:
    key = name.lower().split("/")[-1]
    if key not in PRESETS:
        raise KeyError(f"unknown OPT preset {name!r}; known: {sorted(PRESETS)}")
    kw = dict(PRESETS[key])
    kw.update(overrides)
    return OPTConfig(**kw)


# ---------------------------------------------------------------------------- names
_P = "model.decoder."


def layer_prefix(i: int) -> str:
    return f"{_P}layers.{i}."


def base_param_specs(cfg: OPTConfig) -> list[tuple[str, tuple, int]]:
    """(name, shape, group) of every base parameter in Hugging Face ``named_parameters`` order."""
    d, dp, F, V = cfg.hidden_size, cfg.word_embed_proj_dim, cfg.ffn_dim, cfg.vocab_size
    specs: list[tuple[str, tuple, int]] = [
        (_P + "embed_tokens.weight", (V, dp), -1),
        (_P + "embed_positions.weight", (cfg.max_position_embeddings + 2, d), -1),
    ]
    if dp != d:
        specs += [(_P + "project_out.weight", (dp, d), -1), (_P + "project_in.weight", (d, dp), -1)]
    if cfg.do_layer_norm_before:
        specs += [(_P + "final_layer_norm.weight", (d,), -1), (_P + "final_layer_norm.bias", (d,), -1)]
    for i in range(cfg.num_hidden_layers):
        lp = layer_prefix(i)
        for proj in ("k_proj", "v_proj", "q_proj", "out_proj"):
            specs += [(f"{lp}self_attn.{proj}.weight", (d, d), i), (f"{lp}self_attn.{proj}.bias", (d,), i)]
        specs += [(lp + "self_attn_layer_norm.weight", (d,), i), (lp + "self_attn_layer_norm.bias", (d,), i),
                  (lp + "fc1.weight", (F, d), i), (lp + "fc1.bias", (F,), i),
                  (lp + "fc2.weight", (d, F), i), (lp + "fc2.bias", (d,), i),
                  (lp + "final_layer_norm.weight", (d,), i), (lp + "final_layer_norm.bias", (d,), i)]
    return specs


def adapter_param_specs(cfg, lora_r: int, num_prefix: int, reparam: bool = False,
                        embed_dim: int = 512, mid_dim: int = 512, layer_prefix=None,
                        kv_dim: int | None = None) -> list[tuple[str, tuple, int]]:
    """LoRA factors and prefix tensors.  With ``reparam`` the prefix rows are not parameters but the
    output of a per-layer two-layer MLP over shared input embeddings (large_models/prefix.py:177-197):
    ``prefix_input_embeds`` [P, embed_dim] lives with layer 0, every layer owns ``prefix_mlp_keys`` and
    ``prefix_mlp_values`` (Linear(embed, mid) - tanh - Linear(mid, d), names as ``nn.Sequential`` gives)."""
    d = cfg.hidden_size
    layer_prefix = layer_prefix or globals()["layer_prefix"]
    specs = []
    for i in range(cfg.num_hidden_layers):
        lp = layer_prefix(i)
        if lora_r:
            for proj in ("q_proj", "v_proj"):
                specs += [(f"{lp}self_attn.{proj}.lora_A", (lora_r, d), i),
                          (f"{lp}self_attn.{proj}.lora_B", (d, lora_r), i)]
        if num_prefix and not reparam:
            specs += [(lp + "self_attn.prefix_keys", (num_prefix, d), i),
                      (lp + "self_attn.prefix_values", (num_prefix, d), i)]
        if num_prefix and reparam:
            if i == 0:
                specs.append((lp + "self_attn.prefix_input_embeds", (num_prefix, embed_dim), i))
            for kv in ("keys", "values"):
                specs += [(f"{lp}self_attn.prefix_mlp_{kv}.0.weight", (mid_dim, embed_dim), i),
                          (f"{lp}self_attn.prefix_mlp_{kv}.0.bias", (mid_dim,), i),
                          (f"{lp}self_attn.prefix_mlp_{kv}.2.weight", (d, mid_dim), i),
                          (f"{lp}self_attn.prefix_mlp_{kv}.2.bias", (d,), i)]
    return specs


# order of a layer's tensors inside an arena: fused operands are adjacent
_LAYER_ORDER = ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                "self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias",
                "self_attn.out_proj.weight", "self_attn.out_proj.bias",
                "self_attn_layer_norm.weight", "self_attn_layer_norm.bias",
                "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias",
                "final_layer_norm.weight", "final_layer_norm.bias",
                "self_attn.q_proj.lora_A", "self_attn.q_proj.lora_B",
                "self_attn.v_proj.lora_A", "self_attn.v_proj.lora_B",
                "self_attn.prefix_keys", "self_attn.prefix_values", "self_attn.prefix_input_embeds"] + \
               [f"self_attn.prefix_mlp_{kv}.{j}.{wb}" for kv in ("keys", "values") for j in (0, 2)
                for wb in ("weight", "bias")]


def _arena_sort_key(name: str, group: int, order=None):
    if group < 0:
        return (group, 0, name)
    suffix = name.split(f"layers.{group}.", 1)[1]
    return (group, (order or _LAYER_ORDER).index(suffix), name)


@dataclass
class Transform:
    """How a forward reads the trainable tensors: ``blend(theta) + coef * z(seed)``."""
    seed: int = 0
    coef: float = 0.0
    coef_dev: torch.Tensor | None = None
    alpha: torch.Tensor | None = None     # DiZO blend ratios per slot (fp32, on the device)
    seed_dev: torch.Tensor | None = None  # 1-element int64 on the device: overrides ``seed`` (graph replays)


@dataclass
class Batch:
    """One forward's inputs, already on the model's device.

    ``rows``/``targets`` name the (sequence*L + position) hidden rows that predict option
    tokens and the tokens they should predict; ``seq_start`` groups rows into sequences,
    ``ex_start`` groups sequences (candidates) into examples, ``labels`` picks the correct one.
    With ``cand_ids`` set the loss is the verbalizer shortcut on ``rows`` (one row per example)."""
    input_ids: torch.Tensor                 # int32 [B, L]
    pad_left: torch.Tensor | None = None    # int32 [B]
    positions: torch.Tensor | None = None   # int32 [B, L]
    rows: torch.Tensor | None = None        # int32 [R]
    targets: torch.Tensor | None = None     # int32 [R]
    seq_start: torch.Tensor | None = None   # int32 [S+1]
    ex_start: torch.Tensor | None = None    # int32 [E+1]
    labels: torch.Tensor | None = None      # int32 [E]
    cand_ids: torch.Tensor | None = None    # int32 [C]
    classification: bool = True

    def to(self, device, non_blocking: bool = True) -> "Batch":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.to(device, non_blocking=non_blocking) if isinstance(v, torch.Tensor) else v
        return Batch(**kw)

    def pin(self) -> "Batch":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.pin_memory() if isinstance(v, torch.Tensor) and not v.is_cuda else v
        return Batch(**kw)

    def nbytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.__dict__.values()
                   if isinstance(v, torch.Tensor))


class OPTModel:
    """Forward-only OPT with trainable/frozen arenas.

    ``mode``: ``"full"`` (every tensor except the tied embedding, as the reference's ZO set,
    large_models/trainer.py:1147-1160), ``"lora"``, ``"prefix"``, ``"lora+prefix"``, or
    ``"head"`` (LM head only)."""

    def __init__(self, config: OPTConfig, device="cpu", dtype=torch.float32, mode: str = "full",
                 lora_r: int = 8, lora_alpha: int = 16, num_prefix: int = 5, untie_emb: bool = False,
                 overlap_transform: bool = False, prefix_reparam: bool = False, prefix_embed_dim: int = 512,
                 prefix_mid_dim: int = 512):
        self.config = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.mode = mode
        self.use_lora = "lora" in mode
        self.use_prefix = "prefix" in mode
        self.lora_r = lora_r if self.use_lora else 0
        self.lora_scaling = (lora_alpha / lora_r) if self.use_lora else 0.0
        self.num_prefix = num_prefix if self.use_prefix else 0
        self.prefix_reparam = bool(prefix_reparam) and self.use_prefix
        self.untied = untie_emb or mode == "head" or not config.tie_word_embeddings
        self.overlap_transform = overlap_transform and self.device.type == "cuda"

        base = self._base_specs()
        extra = []
        if self.untied:
            extra.append(("lm_head.weight", (config.vocab_size, config.word_embed_proj_dim), -1))
        adapters = self._adapter_specs(self.lora_r, self.num_prefix, self.prefix_reparam,
                                       prefix_embed_dim, prefix_mid_dim)
        # canonical RNG stream ids: independent of mode, sharding and arena order (new kinds of tensors
        # are appended, so the ids of the existing ones never move)
        canon = [n for n, _, _ in base] + ["lm_head.weight"] + \
                [n for n, _, _ in self._adapter_specs(8, 5)] + \
                [n for n, _, _ in self._adapter_specs(0, 5, True)]
        self.tensor_ids = {n: i for i, n in enumerate(canon)}
        self.all_specs = [sp for sp in base + extra + adapters if self.owns(sp[0])]
        self.hf_order = [n for n, _, _ in self.all_specs]
        self.trainable_names = self._select_trainable()
        tset = set(self.trainable_names)

        def mk(specs):
            ps = []
            for n, s, g in specs:
                ls, kw = self.shard_of(n, tuple(s))
                ps.append(Piece(n, ls, self.tensor_ids[n], g, **kw))
            ps.sort(key=lambda p: self._sort_key(p.name, p.group))
            return ps

        self.arena = ParamArena(mk([s for s in self.all_specs if s[0] in tset]), self.device, dtype)
        self.frozen = ParamArena(mk([s for s in self.all_specs if s[0] not in tset]), self.device, dtype)
        self._where = {p.name: self.arena for p in self.arena.pieces}
        self._where.update({p.name: self.frozen for p in self.frozen.pieces})
        self._staging: dict = {}
        self._side = None
        self._merge_buf: dict = {}
        # LoRA: k_proj.weight is frozen, so its copy inside a layer's merged QKV operand stays valid
        self._k_frozen = self.use_lora
        self.kv_capture: list | None = None      # set to [] to record per-layer qkv (generation)

    # ------------------------------------------------------------------ architecture hooks
    EMBED = _P + "embed_tokens.weight"          # the token table (tied LM head)
    layer_prefix = staticmethod(layer_prefix)

    def _base_specs(self) -> list[tuple[str, tuple, int]]:
        return base_param_specs(self.config)

    def _adapter_specs(self, lora_r: int, num_prefix: int, reparam: bool = False, embed_dim: int = 512,
                       mid_dim: int = 512) -> list[tuple[str, tuple, int]]:
        return adapter_param_specs(self.config, lora_r, num_prefix, reparam, embed_dim, mid_dim)

    def _sort_key(self, name: str, group: int):
        return _arena_sort_key(name, group)

    @staticmethod
    def _is_norm_weight(name: str) -> bool:
        return "layer_norm.weight" in name

    # ------------------------------------------------------------------ sharding hooks
    def owns(self, name: str) -> bool:
        """Whether this rank holds parameter ``name`` at all (pipeline stages hold only their own
        blocks; every other layout holds at least a part of every tensor)."""
        return True

    def shard_of(self, name: str, shape: tuple) -> tuple[tuple, dict]:
        """(local shape, Piece keywords) of this rank's part of a parameter.  The base model
        holds every parameter whole; tensor- and fully-sharded-parallel subclasses override."""
        return shape, {}

    def local_slice(self, name: str, full: torch.Tensor) -> torch.Tensor:
        """This rank's part of a full parameter tensor (identity here)."""
        return full

    # ------------------------------------------------------------------ parameter sets
    def _select_trainable(self) -> list[str]:
        names = self.hf_order
        if self.mode == "full":
            out = [n for n in names if n != self.EMBED]
        elif self.mode == "head":
            out = ["lm_head.weight"]
        else:
            out = [n for n in names if ("lora_" in n and self.use_lora) or ("prefix_" in n and self.use_prefix)]
        if not out:
            raise ValueError(f"mode {self.mode!r} selects no trainable tensor")
        return out

    def named_parameters(self) -> Iterable[tuple[str, torch.Tensor]]:
        for n in self.hf_order:
            yield n, self.param(n)

    def param(self, name: str) -> torch.Tensor:
        return self._where[name].view(name)

    def num_parameters(self, trainable_only: bool = False) -> int:
        n = self.arena.trainable_numel()
        return n if trainable_only else n + self.frozen.trainable_numel()

    def dizo_include_names(self) -> list[str]:
        """Tensors that get a DiZO constraint: each layer's k_proj/v_proj weight under full
        fine-tuning, the LoRA factors under LoRA, nothing for prefix-only runs
        (large_models/trainer.py:1147-1160)."""
        if self.mode == "full":
            return [n for n in self.hf_order if n in self._where and self._where[n] is self.arena and
                    ("self_attn.k_proj.weight" in n or "self_attn.v_proj.weight" in n)]
        return [n for n in self.trainable_names if "lora" in n]

    # ------------------------------------------------------------------ init / state dict
    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "OPTModel":
        """Hugging Face style init: N(0, std) matrices and embeddings, zero biases, unit LN."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        for n, shape, _ in self.all_specs:
            t = self.param(n)
            if "lora_A" in n:
                bound = (1.0 / shape[1]) ** 0.5          # kaiming_uniform(a=sqrt(5)) on [r, in]
                v = (torch.rand(shape, generator=g) * 2 - 1) * bound
            elif "lora_B" in n:
                v = torch.zeros(shape)
            elif "prefix_mlp_" in n:
                fan_in = shape[1] if len(shape) == 2 else self._mlp_fan_in(n)
                v = (torch.rand(shape, generator=g) * 2 - 1) * (1.0 / fan_in) ** 0.5     # nn.Linear's default
            elif "prefix_" in n:
                v = torch.randn(shape, generator=g)
            elif self._is_norm_weight(n):
                v = torch.ones(shape)
            elif n.endswith(".bias"):
                v = torch.zeros(shape)
            else:
                v = torch.randn(shape, generator=g) * std
                if n == self.EMBED and self.config.pad_token_id is not None:
                    v[self.config.pad_token_id].zero_()
            t.copy_(self.local_slice(n, v).to(self.dtype))
        if self.untied and self.config.tie_word_embeddings and "lm_head.weight" in self._where:
            self.param("lm_head.weight").copy_(self.param(self.EMBED))       # an untied copy of a tied model
        self._merge_buf = {}                     # cached merged operands hold copies of frozen weights
        return self

    @torch.no_grad()
    def init_random_fast(self, seed: int = 0, std: float = 0.02) -> "OPTModel":
        """Same distributions as :meth:`init_random`, generated on the device (large models)."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        for n, shape, _ in self.all_specs:
            t = self.param(n)
            if "prefix_mlp_" in n:
                fan_in = shape[1] if len(shape) == 2 else self._mlp_fan_in(n)
                t.copy_(((torch.rand(shape, generator=g, device=self.device) * 2 - 1) *
                         (1.0 / fan_in) ** 0.5).to(self.dtype))
            elif "lora_B" in n or n.endswith(".bias"):
                t.zero_()
            elif self._is_norm_weight(n):
                t.fill_(1.0)
            elif "lora_A" in n:
                t.copy_(((torch.rand(shape, generator=g, device=self.device) * 2 - 1) *
                         (1.0 / shape[1]) ** 0.5).to(self.dtype))
            elif "prefix_" in n:
                t.copy_(torch.randn(shape, generator=g, device=self.device).to(self.dtype))
            else:
                # in blocks, so a 50272 x 5120 fp32 temporary never exists for bigger tables
                flat = t.view(-1)
                step = 1 << 26
                for s in range(0, flat.numel(), step):
                    e = min(s + step, flat.numel())
                    flat[s:e].copy_((torch.randn(e - s, generator=g, device=self.device) * std).to(self.dtype))
        if self.untied and self.config.tie_word_embeddings and "lm_head.weight" in self._where:
            self.param("lm_head.weight").copy_(self.param(self.EMBED))       # an untied copy of a tied model
        self._merge_buf = {}                     # cached merged operands hold copies of frozen weights
        return self

    def _mlp_fan_in(self, bias_name: str) -> int:
        return self.param(bias_name[:-len("bias")] + "weight").shape[1]

    def state_dict(self) -> dict[str, torch.Tensor]:
        """Hugging Face OPT names (plus ``lora_A/B`` and ``prefix_keys/values``)."""
        sd = {n: self.param(n).detach().clone() for n in self.hf_order}
        if not self.untied:
            sd["lm_head.weight"] = sd[self.EMBED]
        return sd

    @torch.no_grad()
    def load_state_dict(self, sd: dict[str, torch.Tensor], strict: bool = True) -> list[str]:
        missing = []
        for n in self.hf_order:
            src = sd.get(n)
            if src is None and n.startswith("model."):
                src = sd.get(n[len("model."):])          # OPTModel-prefixed checkpoints
            if src is None:
                if n == "lm_head.weight" and self.EMBED in sd:
                    src = sd[self.EMBED]
                elif "lora_" in n or "prefix_" in n:
                    missing.append(n)
                    continue
                else:
                    missing.append(n)
                    if strict:
                        raise KeyError(f"state dict lacks {n}")
                    continue
            self.param(n).copy_(self.local_slice(n, src).to(self.dtype))
        self._merge_buf = {}                     # cached merged operands hold copies of frozen weights
        return missing

    # ------------------------------------------------------------------ weight resolution
    def _staging_for(self, key, numel: int) -> torch.Tensor:
        buf = self._staging.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(numel, dtype=self.dtype, device=self.device)
            self._staging[key] = buf
        return buf

    def _fused(self, tensors: list[torch.Tensor]) -> torch.Tensor:
        """View adjacent tensors as one (rows stacked) when they are contiguous in memory."""
        t0 = tensors[0]
        esz = t0.element_size()
        ptr = t0.data_ptr()
        ok = True
        for t in tensors:
            if t.data_ptr() != ptr or not t.is_contiguous():
                ok = False
                break
            ptr += t.numel() * esz
        if not ok:
            return torch.cat(tensors, dim=0)
        rows = sum(t.shape[0] for t in tensors)
        shape = (rows,) + tuple(t0.shape[1:])
        return torch.as_strided(t0, shape, t0.stride())

    def _blend_range(self, group: int, transform: Transform | None) -> tuple[int, int] | None:
        """Piece range a transform has to stage for ``group``, or None for the whole group.

        A DiZO blend without perturbation (the gamma-search forwards) changes only the constrained
        tensors.  Under full fine-tuning those are the k/v projection weights, which open every
        block's piece list together with the q weight (one fused QKV operand): staging just these
        three instead of the whole block cuts the sweep traffic of a search forward by 4x.  The
        globals hold no constrained tensor then, so nothing of them is staged."""
        if (transform is None or transform.alpha is None or transform.coef != 0.0
                or transform.coef_dev is not None or self.mode != "full"):
            return None
        lo, hi = self.arena.group_range(group)
        if group < 0:
            return (lo, lo)
        names = [p.name for p in self.arena.pieces[lo:lo + 3]]
        want = ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"]
        if len(names) == 3 and all(n.endswith(w) for n, w in zip(names, want)) and \
                all(p.slot < 0 for p in self.arena.pieces[lo + 3:hi]):
            return (lo, lo + 3)
        return None

    def _resolver(self, group: int, transform: Transform | None, staged: torch.Tensor | None,
                  shift: int) -> Callable[[str], torch.Tensor]:
        only = None
        if staged is not None:
            r = self._blend_range(group, transform)
            if r is not None:
                only = {p.name for p in self.arena.pieces[r[0]:r[1]]}

        def get(name: str) -> torch.Tensor:
            ar = self._where[name]
            if ar is self.arena and staged is not None and (only is None or name in only):
                return ar.view(name, base=staged, shift=shift)
            return ar.view(name)
        return get

    def _sweep_group(self, group: int, transform: Transform, dst: torch.Tensor, small: bool = False,
                     dst2: torch.Tensor | None = None) -> int:
        lo, hi = self.arena.group_range(group)
        r = self._blend_range(group, transform)
        if r is not None:
            lo, hi = r
            if lo == hi:
                return 0
        self.arena.sweep(t_begin=lo, t_end=hi, dst=dst, seed1=transform.seed, c1=transform.coef,
                         c1_dev=transform.coef_dev, seed1_dev=transform.seed_dev, alpha=transform.alpha,
                         small=small, dst2=dst2)
        return self.arena.span(lo, hi)[0]

    def _lora_qkv_buffer(self, i: int, stream: int = 0) -> tuple[torch.Tensor, bool]:
        """The [3d, d] operand that receives W_q + s B_q A_q | W_k | W_v + s B_v A_v of layer ``i`` and
        whether its k section still has to be written.  With room to spare every layer keeps its own
        buffer (two when both streams of a step run side by side), so the frozen k weight is copied once and
        only q and v are re-merged per forward; when memory is short one buffer per stream is shared and k is
        copied along every time."""
        d = self.config.hidden_size
        if self._merge_buf.get("per_layer") is None:
            need = 2 * self.config.num_hidden_layers * 3 * d * d * torch.finfo(self.dtype).bits // 8
            free = torch.cuda.mem_get_info(self.device)[0] if self.device.type == "cuda" else 1 << 62
            self._merge_buf["per_layer"] = free > 4 * need
        if self._merge_buf["per_layer"]:
            buf = self._merge_buf.get((i, stream))
            if buf is None:
                buf = torch.empty((3 * d, d), dtype=self.dtype, device=self.device)
                self._merge_buf[(i, stream)] = buf
                return buf, True
            return buf, not self._k_frozen
        buf = self._merge_buf.get(("qkv", stream))
        if buf is None:
            buf = torch.empty((3 * d, d), dtype=self.dtype, device=self.device)
            self._merge_buf[("qkv", stream)] = buf
        return buf, True

    def _merged_qkv(self, i: int, get: Callable[[str], torch.Tensor], stream: int = 0) -> torch.Tensor:
        """W_q + s B_q A_q | W_k | W_v + s B_v A_v of layer ``i`` with the adapters ``get`` resolves."""
        d = self.config.hidden_size
        a = layer_prefix(i) + "self_attn."
        buf, fresh = self._lora_qkv_buffer(i, stream)
        peft_ops.lora_merge(get(a + "q_proj.weight"), get(a + "q_proj.lora_A"), get(a + "q_proj.lora_B"),
                            self.lora_scaling, out=buf[:d])
        if fresh:
            # the frozen k weight: copied by the merge kernel with a zero scale (W + 0 * B A)
            peft_ops.lora_merge(get(a + "k_proj.weight"), get(a + "q_proj.lora_A"), get(a + "q_proj.lora_B"), 0.0,
                                out=buf[d:2 * d])
        peft_ops.lora_merge(get(a + "v_proj.weight"), get(a + "v_proj.lora_A"), get(a + "v_proj.lora_B"),
                            self.lora_scaling, out=buf[2 * d:])
        return buf

    def _layer_weights(self, i: int, get: Callable[[str], torch.Tensor]) -> SimpleNamespace:
        lp = layer_prefix(i)
        a = lp + "self_attn."
        w = SimpleNamespace()
        if self.use_prefix and self.prefix_reparam and i == 0:
            # the shared embeddings are a tensor of layer 0: read them through layer 0's resolver (so a
            # transform applies) and keep a copy for the layers above, whose staging buffers rotate
            self._prefix_embeds = get(a + "prefix_input_embeds").clone()
        if self.use_lora:
            w.qkv_w = self._merged_qkv(i, get)
        else:
            w.qkv_w = self._fused([get(a + "q_proj.weight"), get(a + "k_proj.weight"), get(a + "v_proj.weight")])
        w.qkv_b = self._fused([get(a + "q_proj.bias"), get(a + "k_proj.bias"), get(a + "v_proj.bias")])
        w.out_w, w.out_b = get(a + "out_proj.weight"), get(a + "out_proj.bias")
        w.ln1_w, w.ln1_b = get(lp + "self_attn_layer_norm.weight"), get(lp + "self_attn_layer_norm.bias")
        w.fc1_w, w.fc1_b = get(lp + "fc1.weight"), get(lp + "fc1.bias")
        w.fc2_w, w.fc2_b = get(lp + "fc2.weight"), get(lp + "fc2.bias")
        w.ln2_w, w.ln2_b = get(lp + "final_layer_norm.weight"), get(lp + "final_layer_norm.bias")
        if self.use_prefix and self.prefix_reparam:
            # prefix rows = MLP(shared input embeddings), recomputed from the (perturbed) MLP parameters
            emb = self._prefix_embeds
            w.prefix_k, w.prefix_v = (self._prefix_mlp(emb, a + f"prefix_mlp_{kv}.", get) for kv in ("keys", "values"))
        else:
            w.prefix_k = get(a + "prefix_keys") if self.use_prefix else None
            w.prefix_v = get(a + "prefix_values") if self.use_prefix else None
        return w

    def _prefix_mlp(self, emb: torch.Tensor, stem: str, get) -> torch.Tensor:
        h = torch.tanh(gemm.linear(emb, get(stem + "0.weight"), get(stem + "0.bias")).float()).to(self.dtype)
        return gemm.linear(h, get(stem + "2.weight"), get(stem + "2.bias"))

    # ------------------------------------------------------------------ forward
    def _layer_forward(self, h: torch.Tensor, w: SimpleNamespace, batch: Batch,
                       rows: torch.Tensor | None = None) -> torch.Tensor:
        """One block.  With ``rows`` (the last block of a loss forward) everything after the attention
        runs on those token rows only and [R, d] is returned: the other rows of the last block's
        out_proj / FFN feed nothing, which saves three quarters of that block's GEMM work."""
        cfg = self.config
        B, L, d = h.shape
        pre = cfg.do_layer_norm_before
        x = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps) if pre else h
        qkv = gemm.linear(x, w.qkv_w, w.qkv_b)
        if self.kv_capture is not None:
            self.kv_capture.append(qkv)
        ctx = attn_ops.attention(qkv.view(B, L, 3 * d), cfg.num_attention_heads, batch.pad_left,
                                 w.prefix_k, w.prefix_v)
        if rows is not None:
            ctx = norm.gather_rows(ctx.reshape(-1, d), rows)
            h = norm.gather_rows(h.reshape(-1, d), rows)
        h = gemm.linear(ctx, w.out_w, w.out_b, residual=h)
        if not pre:
            h = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps)
        x = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps) if pre else h
        f = gemm.linear(x, w.fc1_w, w.fc1_b, act=cfg.activation_function)
        h = gemm.linear(f, w.fc2_w, w.fc2_b, residual=h)
        if not pre:
            h = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps)
        return h

    @torch.no_grad()
    def hidden_states(self, batch: Batch, transform: Transform | None = None,
                      rows: torch.Tensor | None = None) -> torch.Tensor:
        """Decoder output before the final LayerNorm / project_out: [B, L, d], or - with ``rows`` - only
        those (sequence * L + position) rows of it, [R, d] (see :meth:`_layer_forward`)."""
        cfg = self.config
        nl = cfg.num_hidden_layers
        use_t = transform is not None and len(self.arena.pieces) > 0
        has_group = {g: True for g in self.arena.groups()}
        overlap = use_t and self.overlap_transform
        if overlap and self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        # ---- globals
        g_staged, g_shift = None, 0
        if use_t and has_group.get(-1):
            g_staged = self._staging_for("globals", self.arena.group_numel(-1))
            g_shift = self._sweep_group(-1, transform, g_staged)
        self._gget = self._resolver(-1, transform, g_staged, g_shift)
        gget = self._gget
        h = self._embed(batch.input_ids, batch.positions, gget)
        # ---- layers, with the transform of layer i+1 running beside the GEMMs of layer i
        main = torch.cuda.current_stream(self.device) if overlap else None
        ready = [None, None]
        free = [None, None]
        layer_numel = max((self.arena.group_numel(g) for g in self.arena.groups() if g >= 0), default=0)

        def launch_transform(i: int):
            k = i % 2
            buf = self._staging_for(("layer", k), layer_numel)
            if overlap:
                with torch.cuda.stream(self._side):
                    if free[k] is not None:
                        self._side.wait_event(free[k])
                    # the small-footprint sweep: shares the SMs with the previous layer's GEMMs
                    shift = self._sweep_group(i, transform, buf, small=True)
                    ev = torch.cuda.Event()
                    ev.record(self._side)
                ready[k] = ev
            else:
                shift = self._sweep_group(i, transform, buf)
            return buf, shift

        pending = None
        if use_t and nl > 0 and has_group.get(0):
            if overlap:
                start = torch.cuda.Event()
                start.record(main)
                self._side.wait_event(start)
            pending = launch_transform(0)
        for i in range(nl):
            staged, shift = None, 0
            if use_t and has_group.get(i):
                staged, shift = pending
                if overlap:
                    main.wait_event(ready[i % 2])
            # queue the next layer's sweep first: it runs beside this layer's GEMMs
            if use_t and i + 1 < nl and has_group.get(i + 1):
                pending = launch_transform(i + 1)
            w = self._layer_weights(i, self._resolver(i, transform, staged, shift))
            only = rows if (i == nl - 1 and self.kv_capture is None) else None
            h = self._layer_forward(h, w, batch, only)
            if overlap and has_group.get(i):
                ev = torch.cuda.Event()
                ev.record(main)
                free[i % 2] = ev
        if overlap:
            main.wait_stream(self._side)
        if rows is not None and nl == 0:
            h = norm.gather_rows(h.reshape(-1, cfg.hidden_size), rows)
        return h

    def _embed(self, ids: torch.Tensor, positions: torch.Tensor, gget) -> torch.Tensor:
        """Token (+ learned position) embedding of ids / positions [B, L] -> [B, L, d]."""
        cfg = self.config
        tok = gget(self.EMBED)
        pos = gget(_P + "embed_positions.weight")
        if cfg.word_embed_proj_dim != cfg.hidden_size:
            e = norm.embed(ids, None, tok, None)
            e = gemm.linear(e, gget(_P + "project_in.weight"))
            return norm.add_rows(e, positions.reshape(-1), pos)
        return norm.embed(ids, positions, tok, pos)

    def _embed_param_names(self) -> list[str]:
        """The parameters :meth:`_embed` reads."""
        return [self.EMBED, _P + "embed_positions.weight", _P + "project_in.weight"]

    def _final_norm(self, x: torch.Tensor, gget) -> torch.Tensor:
        """What sits between the last block and the LM head: final LayerNorm, project_out."""
        cfg = self.config
        if cfg.do_layer_norm_before:
            x = norm.layernorm(x, gget(_P + "final_layer_norm.weight"),
                               gget(_P + "final_layer_norm.bias"), cfg.layer_norm_eps)
        if cfg.word_embed_proj_dim != cfg.hidden_size:
            x = gemm.linear(x, gget(_P + "project_out.weight"))
        return x

    # ------------------------------------------------------------------ one-token decoding (generation)
    def decode_embed(self, tokens: torch.Tensor, positions: torch.Tensor, get) -> torch.Tensor:
        """tokens, positions: int32 [B] -> [B, d]."""
        return self._embed(tokens.view(-1, 1), positions.view(-1, 1), get).view(-1, self.config.hidden_size)

    def decode_block(self, h: torch.Tensor, w: SimpleNamespace, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     t: int, pad_left: torch.Tensor) -> torch.Tensor:
        """One block on a [B, d] activation: writes this token's K / V at cache column ``t`` and attends to
        columns [0, t]."""
        from ..ops import decode as decode_ops
        cfg = self.config
        d = cfg.hidden_size
        pre = cfg.do_layer_norm_before
        x = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps) if pre else h
        qkv = gemm.linear(x, w.qkv_w, w.qkv_b)
        k_cache[:, t].copy_(qkv[:, d:2 * d])
        v_cache[:, t].copy_(qkv[:, 2 * d:])
        ctx = decode_ops.decode_attention(qkv[:, :d], k_cache, v_cache, t + 1, cfg.num_attention_heads, pad_left,
                                          w.prefix_k, w.prefix_v)
        h = gemm.linear(ctx.contiguous(), w.out_w, w.out_b, residual=h)
        if not pre:
            h = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps)
        x = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps) if pre else h
        f = gemm.linear(x, w.fc1_w, w.fc1_b, act=cfg.activation_function)
        h = gemm.linear(f, w.fc2_w, w.fc2_b, residual=h)
        if not pre:
            h = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps)
        return h

    def _selected(self, batch: Batch, transform: Transform | None) -> torch.Tensor:
        """Final-normalised hidden rows ``batch.rows``.  The replicated model restricts its last block to
        them; sharded layouts (own ``hidden_states``) compute every row and pick afterwards."""
        if type(self).hidden_states is OPTModel.hidden_states:
            return self.final_rows(self.hidden_states(batch, transform, rows=batch.rows), None)
        return self.final_rows(self.hidden_states(batch, transform), batch.rows)

    @torch.no_grad()
    def final_rows(self, h: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        """Final LayerNorm (+ project_out) applied to the selected rows of h only (``rows`` None: h
        already holds just those rows)."""
        cfg = self.config
        d = cfg.hidden_size
        x = h if rows is None else norm.gather_rows(h.reshape(-1, d), rows)
        return self._final_norm(x, self._gget)

    # ------------------------------------------------------------------ both sides of the two-point estimate
    def pair_supported(self) -> bool:
        """Whether :meth:`loss_pair` applies: the unsharded forward, sweeps on the main stream, prefix rows (if
        any) held as parameters."""
        return (type(self).hidden_states is OPTModel.hidden_states and not self.overlap_transform
                and not self.prefix_reparam and len(self.arena.pieces) > 0)

    @torch.no_grad()
    def loss_pair(self, batch: Batch, seed: int, eps: float, seed_dev: torch.Tensor | None = None):
        """(L(theta + eps z), L(theta - eps z)) for z = z(seed).  The two forwards advance block by block: one
        sweep per block draws z once and stages theta + eps z and theta - eps z side by side
        (``ParamArena.sweep(dst2=...)``), then the block runs on each activation stream with its copy.  The staged
        values, the kernels and therefore both losses are the same bit for bit as two separate forwards with
        ``Transform(coef=+eps)`` and ``Transform(coef=-eps)`` (large_models/trainer.py:1570-1595 perturbs, runs a
        forward, perturbs twice the other way, runs the second); what is saved is one of the two draws of z per
        step - a third of the sweep time, which the generator bounds."""
        cfg = self.config
        nl = cfg.num_hidden_layers
        tr = Transform(seed=seed, coef=eps, seed_dev=seed_dev)
        groups = set(self.arena.groups())
        ggets = [self._resolver(-1, None, None, 0)] * 2
        if -1 in groups:
            n = self.arena.group_numel(-1)
            g1, g2 = self._staging_for("globals", n), self._staging_for("globals-", n)
            shift = self._sweep_group(-1, tr, g1, dst2=g2)
            ggets = [self._resolver(-1, tr, g1, shift), self._resolver(-1, tr, g2, shift)]
        # the two streams are one and the same until the first perturbed tensor is read (head tuning: the whole
        # decoder runs once, only the loss tail runs twice)
        same = not any(n in self._where and self._where[n] is self.arena for n in self._embed_param_names())
        h0 = self._embed(batch.input_ids, batch.positions, ggets[0])
        hs = [h0, h0 if same else self._embed(batch.input_ids, batch.positions, ggets[1])]
        layer_numel = max((self.arena.group_numel(g) for g in groups if g >= 0), default=0)
        for i in range(nl):
            only = batch.rows if i == nl - 1 else None
            if i in groups:
                same = False
                b1 = self._staging_for(("layer", i % 2), layer_numel)
                b2 = self._staging_for(("layer-", i % 2), layer_numel)
                shift = self._sweep_group(i, tr, b1, dst2=b2)
                gets = [self._resolver(i, tr, b1, shift), self._resolver(i, tr, b2, shift)]
            else:
                gets = [self._resolver(i, None, None, 0)] * 2
            if same:
                h0 = self._layer_forward(hs[0], self._layer_weights(i, gets[0]), batch, only)
                hs = [h0, h0]
                continue
            if self._shares_block_tail():
                # adapters only (LoRA / prefix): the rest of the block is frozen, so both streams go through its
                # GEMMs together (twice the rows per launch: fuller waves, the weights are read once)
                hs = self._layer_forward_pair(hs, i, gets, batch, only)
                continue
            for s in range(2):
                hs[s] = self._layer_forward(hs[s], self._layer_weights(i, gets[s]), batch, only)
        losses = []
        for s in range(2):
            self._gget = ggets[s]
            h = hs[s]
            if nl == 0:
                h = norm.gather_rows(h.reshape(-1, cfg.hidden_size), batch.rows)
            x = self.final_rows(h, None)
            table = self.lm_head_weight()
            if batch.cand_ids is not None:
                losses.append(loss_ops.verbalizer_ce(x, table, batch.cand_ids, batch.labels)[1])
            else:
                lp = loss_ops.token_logprobs(x, table, batch.targets)
                losses.append(loss_ops.option_ce(lp, batch.seq_start, batch.ex_start, batch.labels,
                                                 batch.classification))
        return losses[0], losses[1]

    def _shares_block_tail(self) -> bool:
        """Adapter-only training (LoRA / prefix rows): between the two streams of a step a block differs in the
        merged QKV operand and the prefix rows at most; LayerNorms, out_proj and the FFN are the same frozen tensors."""
        return (type(self)._layer_forward is OPTModel._layer_forward and not self.prefix_reparam
                and self.mode in ("lora", "prefix", "lora+prefix"))

    @staticmethod
    def _stack2(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """[2 * rows, d] holding a then b, without a copy when they already sit side by side."""
        a2, b2 = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
        if (a2.is_contiguous() and b2.is_contiguous() and
                a2.untyped_storage().data_ptr() == b2.untyped_storage().data_ptr() and
                b2.data_ptr() == a2.data_ptr() + a2.numel() * a2.element_size()):
            return torch.as_strided(a2, (2 * a2.shape[0], a2.shape[1]), a2.stride())
        return torch.cat([a2, b2], dim=0)

    def _layer_forward_pair(self, hs, i: int, gets, batch: Batch, rows: torch.Tensor | None):
        """One block for both streams of the two-point estimate when only adapters are trained: the frozen parts
        (LayerNorms, out_proj, FFN - and the QKV projection without LoRA) run once over both streams' rows, twice
        the rows per launch; the QKV projection runs per stream when LoRA makes its operand differ, attention
        always does (its prefix rows may differ)."""
        cfg = self.config
        B, L, d = hs[0].shape
        M = B * L
        pre = cfg.do_layer_norm_before
        w = self._layer_weights(i, gets[0])
        a = layer_prefix(i) + "self_attn."
        H = self._stack2(hs[0], hs[1])                                   # [2M, d]
        x = norm.layernorm(H, w.ln1_w, w.ln1_b, cfg.layer_norm_eps) if pre else H
        if self.use_lora:
            qkv_w1 = self._merged_qkv(i, gets[1], stream=1)
            qkvs = [gemm.linear(x[:M], w.qkv_w, w.qkv_b), gemm.linear(x[M:], qkv_w1, w.qkv_b)]
        else:
            both = gemm.linear(x, w.qkv_w, w.qkv_b)
            qkvs = [both[:M], both[M:]]
        ctx = torch.empty((2, B, L, d), dtype=H.dtype, device=H.device)
        for s in range(2):
            pk = gets[s](a + "prefix_keys") if self.use_prefix else None
            pv = gets[s](a + "prefix_values") if self.use_prefix else None
            q3 = qkvs[s].view(B, L, 3 * d)
            if q3.is_cuda:
                attn_ops.attention(q3, cfg.num_attention_heads, batch.pad_left, pk, pv, out=ctx[s])
            else:
                ctx[s].copy_(attn_ops.attention(q3, cfg.num_attention_heads, batch.pad_left, pk, pv))
        c = ctx.view(2 * M, d)
        if rows is not None:
            both_rows = torch.cat([rows, rows + M]).to(torch.int32)
            c = norm.gather_rows(c, both_rows)
            H = norm.gather_rows(H, both_rows)
        h = gemm.linear(c, w.out_w, w.out_b, residual=H)
        if not pre:
            h = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps)
        x2 = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps) if pre else h
        f = gemm.linear(x2, w.fc1_w, w.fc1_b, act=cfg.activation_function)
        h = gemm.linear(f, w.fc2_w, w.fc2_b, residual=h)
        if not pre:
            h = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps)
        n = h.shape[0] // 2
        if rows is not None:
            return [h[:n], h[n:]]
        return [h[:n].view(B, L, d), h[n:].view(B, L, d)]

    def lm_head_weight(self) -> torch.Tensor:
        return self._gget("lm_head.weight") if self.untied else self._gget(self.EMBED)

    @torch.no_grad()
    def loss(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        """One fp32 loss (1-element tensor on the device) for the batch."""
        x = self._selected(batch, transform)
        table = self.lm_head_weight()
        if batch.cand_ids is not None:
            _, loss = loss_ops.verbalizer_ce(x, table, batch.cand_ids, batch.labels)
            return loss
        lp = loss_ops.token_logprobs(x, table, batch.targets)
        return loss_ops.option_ce(lp, batch.seq_start, batch.ex_start, batch.labels, batch.classification)

    @torch.no_grad()
    def row_logprobs(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        """log p(target) for every (row, target) pair of the batch (evaluation path)."""
        x = self._selected(batch, transform)
        return loss_ops.token_logprobs(x, self.lm_head_weight(), batch.targets)

    @torch.no_grad()
    def logits(self, batch: Batch, rows: torch.Tensor | None = None) -> torch.Tensor:
        """Full-vocabulary fp32 logits for the selected rows (all rows when ``rows`` is None)."""
        h = self.hidden_states(batch)
        B, L, _ = h.shape
        if rows is None:
            rows = torch.arange(B * L, dtype=torch.int32, device=h.device)
        x = self.final_rows(h, rows)
        return gemm.linear(x, self.lm_head_weight(), out_dtype=torch.float32)


def make_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None, **kw) -> Batch:
    """Build a :class:`Batch` from left-padded ids and a 0/1 mask (positions, pad_left derived)."""
    ids = input_ids.to(torch.int32)
    if attention_mask is None:
        attention_mask = torch.ones_like(ids)
    m = attention_mask.to(torch.int32)
    pad_left = (m.shape[1] - m.sum(dim=1)).to(torch.int32)
    return Batch(input_ids=ids, pad_left=pad_left, positions=norm.opt_positions(m), **kw)
