"""Fully sharded data-parallel OPT for zeroth-order training.

The six weight matrices of every block (q, k, v, out_proj, fc1, fc2 - 99.9 % of the bytes) are
sharded by rows over the ``n`` ranks; biases, LayerNorms and the embeddings stay replicated (a
replicated tensor needs no communication under ZO: every rank regenerates the same z for it
from the shared seed and applies the same update).  Each rank runs its own batch shard.

A forward never gathers a plain weight and then perturbs it.  For every matrix, the owner of a
row shard perturbs it on the way out - theta + c z with z regenerated for the shard's element
indices in the FULL tensor - while its push CTAs store the result into every rank's staged
copy of that matrix over NVLink, and the same launch runs the tcgen05 GEMM that consumes the
previously staged matrix (``FusedComm.fsdp_launch``).  Matrix j+1 therefore travels while
matrix j is being multiplied, nothing of size [N, K] is ever held unperturbed outside its
shard, and nobody regenerates z for somebody else's shard.  Two staging slots alternate:

    launch 0 : push qkv -> A                      (first layer only: nothing to multiply yet)
    launch 1 : GEMM qkv (A)  + push out_proj -> B
    launch 2 : GEMM out (B)  + push fc1 -> A
    launch 3 : GEMM fc1 (A)  + push fc2 -> B
    launch 4 : GEMM fc2 (B)  + push next layer's qkv -> A      ...

Reuse of a slot is guarded by acks (a pusher waits until every rank has finished the GEMM that
read the slot's previous content); all device-side waits are bounded.  Without memory pressure
(OPT-13B is 26 GB of bf16 on a 180 GB B200) replicated data parallelism is faster; this layout is
for models or batch sizes that do not fit otherwise.

The gamma-search forwards of DiZO read theta_0 + alpha (theta - theta_0): that blend is applied
by the ordinary local sweep into the rank's staging area and the pushed rows are taken from
there (coefficient 0 in the push).  The per-tensor norms of the sharded k/v weights are partial
sums reduced by ``FusedComm.norm_allreduce_gamma`` together with the gamma arithmetic.

The reference lists "FSDP + DiZO" as planned only (large_models/README.md:89); its FSDP path
exists for the first-order trainer alone (large_models/finetune_fsdp.sh:59-60).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.opt import _P, Batch, OPTConfig, OPTModel, Transform, layer_prefix
from ..ops import attention as attn_ops
from ..ops import norm
from .fused import FusedComm

_SHARDED = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
            "self_attn.out_proj.weight", "fc1.weight", "fc2.weight")


class FSDPOPTModel(OPTModel):
    def __init__(self, config: OPTConfig, device, dtype=torch.bfloat16, group=None, n_push: int = 16, **kw):
        self.group = group if group is not None else dist.group.WORLD
        self.n = dist.get_world_size(self.group)
        self.r = dist.get_rank(self.group)
        d, F = config.hidden_size, config.ffn_dim
        assert d % (8 * self.n) == 0 and F % (8 * self.n) == 0
        assert config.do_layer_norm_before and config.word_embed_proj_dim == d
        kw.setdefault("mode", "full")
        assert kw["mode"] == "full", "the sharded layout is built for full-parameter ZO"
        super().__init__(config, device, dtype, **kw)
        self.push_perturb_limit = 24 * 1024 * 1024      # shard elements above which the push only copies
        self.comm = FusedComm(self.group, self.device, w_bytes=max(3 * d * d, F * d) * 2, n_push=n_push,
                              norm_slots=max(256, 2 * config.num_hidden_layers))

    # ------------------------------------------------------------------ sharding
    def _sharded(self, name: str) -> bool:
        return any(name.endswith(s) for s in _SHARDED)

    def shard_of(self, name, shape):
        if self._sharded(name):
            rows = shape[0] // self.n
            return (rows, shape[1]), dict(elem_base=self.r * rows * shape[1])
        return shape, {}

    def local_slice(self, name, full):
        if self._sharded(name):
            rows = full.shape[0] // self.n
            return full[self.r * rows:(self.r + 1) * rows]
        return full

    @torch.no_grad()
    def init_random_fast(self, seed: int = 0, std: float = 0.02):
        """Every rank draws the full tensor from the same device generator and keeps its rows."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        for n, shape, _ in self.all_specs:
            t = self.param(n)
            if n.endswith(".bias"):
                t.zero_()
            elif "layer_norm.weight" in n:
                t.fill_(1.0)
            else:
                numel = 1
                for s in shape:
                    numel *= s
                full = torch.empty(numel, dtype=self.dtype, device=self.device)
                step = 1 << 26
                for s0 in range(0, numel, step):
                    e = min(s0 + step, numel)
                    full[s0:e].copy_((torch.randn(e - s0, generator=g, device=self.device) * std).to(self.dtype))
                t.copy_(self.local_slice(n, full.view(shape)))
                del full
        return self

    def gather_full(self, name: str, local: torch.Tensor) -> torch.Tensor:
        """The unsharded tensor ``name`` from every rank's rows ``local`` (cold path, NCCL)."""
        t = local.contiguous()
        if not self._sharded(name):
            return t.clone()
        parts = [torch.empty_like(t) for _ in range(self.n)]
        dist.all_gather(parts, t, group=self.group)
        return torch.cat(parts, dim=0)

    def gather_state_dict(self) -> dict:
        """Full Hugging Face state dict on every rank (cold path: checkpoints, tests; NCCL)."""
        sd = {n: self.gather_full(n, self.param(n)) for n in self.hf_order}
        if not self.untied:
            sd["lm_head.weight"] = sd[_P + "embed_tokens.weight"]
        return sd

    def reduce_norms(self, gs, reinit: bool) -> None:
        self.comm.norm_allreduce_gamma(gs.sq.clone(), gs, reinit)

    # ------------------------------------------------------------------ forward
    def _push_spec(self, i: int, which: str, get, transform: Transform | None):
        """Segments + perturbation of one weight group of layer i (``get`` resolves names to the
        arena shard, or to the locally staged shard when a blend is active)."""
        cfg = self.config
        d, F = cfg.hidden_size, cfg.ffn_dim
        lp = layer_prefix(i)
        names = {"qkv": ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"],
                 "out": ["self_attn.out_proj.weight"], "fc1": ["fc1.weight"], "fc2": ["fc2.weight"]}[which]
        segs = []
        for j, nm in enumerate(names):
            full = lp + nm
            w = get(full)
            rows = w.shape[0]
            piece = self.arena.pieces[self.arena.index[full]]
            block = {"qkv": d, "out": 0, "fc1": 0, "fc2": 0}[which]
            segs.append(dict(w_shard=w, dst_row0=j * block + self.r * rows, tensor_id=piece.tensor_id,
                             elem_base=piece.elem_base))
        N = {"qkv": 3 * d, "out": d, "fc1": F, "fc2": d}[which]
        rows_per_src = segs[0]["w_shard"].shape[0]
        period = d if which == "qkv" else 0
        return segs, N, rows_per_src, period

    @torch.no_grad()
    def hidden_states(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        cfg, fc = self.config, self.comm
        nl, d = cfg.num_hidden_layers, cfg.hidden_size
        B, L = batch.input_ids.shape
        M = B * L
        blend = transform is not None and transform.alpha is not None
        if transform is not None:
            assert transform.coef_dev is None, "the fused push takes its coefficient from the host"
        seed = transform.seed if transform is not None else 0
        coef = transform.coef if (transform is not None and not blend) else 0.0
        # ---- globals (replicated) through the ordinary local sweep
        g_staged, g_shift = None, 0
        if transform is not None:
            g_staged = self._staging_for("globals", self.arena.group_numel(-1))
            g_shift = self._sweep_group(-1, transform, g_staged)
        self._gget = self._resolver(-1, transform, g_staged, g_shift)
        h = norm.embed(batch.input_ids, batch.positions, self._gget(_P + "embed_tokens.weight"),
                       self._gget(_P + "embed_positions.weight")).view(M, d)
        layer_numel = max(self.arena.group_numel(g) for g in self.arena.groups() if g >= 0)
        direct = self._resolver(0, None, None, 0)          # arena shards, unperturbed

        def stage(i):
            """Local sweep of layer i: perturbed / blended replicated vectors (and shards)."""
            if transform is None:
                return self._resolver(i, None, None, 0)
            buf = self._staging_for(("layer", i % 2), layer_numel)
            return self._resolver(i, transform, buf, self._sweep_group(i, transform, buf))

        # The push CTAs regenerate z for the rows they send.  That is the cheapest place while a
        # shard is small (8 ranks: 1/8 of a matrix); with few ranks the shard is large and the few
        # push CTAs would become the bottleneck, so the whole-GPU sweep perturbs the shard into the
        # local staging area first and the push is a plain copy (the path blends always take).
        d_, F_ = cfg.hidden_size, cfg.ffn_dim
        staged_push = blend or (transform is not None and F_ * d_ // self.n > self.push_perturb_limit)

        def push_of(i, which, staged_get):
            segs, N, rps, period = self._push_spec(i, which, staged_get if staged_push else direct, transform)
            return dict(segments=segs, seed=seed, coef=0.0 if staged_push else coef), N, rps, period

        get = stage(0)
        p, N, rps, period = push_of(0, "qkv", get)
        slot, _ = fc.fsdp_launch(push=p)
        pending = (slot, N, rps, period)
        for i in range(nl):
            lp = layer_prefix(i)
            a = lp + "self_attn."
            nget = stage(i + 1) if i + 1 < nl else None
            qkv_b = self._fused([get(a + "q_proj.bias"), get(a + "k_proj.bias"), get(a + "v_proj.bias")])
            x = norm.layernorm(h, get(lp + "self_attn_layer_norm.weight"), get(lp + "self_attn_layer_norm.bias"),
                               cfg.layer_norm_eps)
            # GEMM qkv + push out_proj
            p, N2, rps2, per2 = push_of(i, "out", get)
            slot2, qkv = fc.fsdp_launch(push=p, gemm=dict(slot=pending[0], N=pending[1], x=x, bias=qkv_b,
                                                          rows_per_src=pending[2], src_period=pending[3]))
            if self.kv_capture is not None:
                self.kv_capture.append(qkv)                                  # generation: the prompt's K / V
            ctx = attn_ops.attention(qkv.view(B, L, 3 * d), cfg.num_attention_heads, batch.pad_left)
            # GEMM out_proj (+bias +residual) + push fc1
            p, N3, rps3, per3 = push_of(i, "fc1", get)
            slot3, h = fc.fsdp_launch(push=p, gemm=dict(slot=slot2, N=N2, x=ctx.view(M, d),
                                                        bias=get(a + "out_proj.bias"), residual=h,
                                                        rows_per_src=rps2, src_period=per2))
            x = norm.layernorm(h, get(lp + "final_layer_norm.weight"), get(lp + "final_layer_norm.bias"),
                               cfg.layer_norm_eps)
            # GEMM fc1 (+bias, activation) + push fc2
            p, N4, rps4, per4 = push_of(i, "fc2", get)
            slot4, f = fc.fsdp_launch(push=p, gemm=dict(slot=slot3, N=N3, x=x, bias=get(lp + "fc1.bias"),
                                                        act=cfg.activation_function, rows_per_src=rps3,
                                                        src_period=per3))
            # GEMM fc2 (+bias +residual) + push the next layer's qkv
            g4 = dict(slot=slot4, N=N4, x=f, bias=get(lp + "fc2.bias"), residual=h, rows_per_src=rps4,
                      src_period=per4)
            if nget is not None:
                p, N, rps, period = push_of(i + 1, "qkv", nget)
                slot, h = fc.fsdp_launch(push=p, gemm=g4)
                pending = (slot, N, rps, period)
                get = nget
            else:
                _, h = fc.fsdp_launch(gemm=g4)
        return h.view(B, L, d)
