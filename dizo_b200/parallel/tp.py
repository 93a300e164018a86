"""Tensor-parallel OPT with a sequence-parallel activation layout and fused collectives.

Megatron-style sharding of every block over ``n`` ranks: q/k/v and fc1 are split by output
rows (heads / FFN units), out_proj and fc2 by input columns; LayerNorms, biases of the
row-reduced projections and the embeddings are replicated.  Between blocks the residual stream
is sharded by token rows (each rank holds M/n rows), so LayerNorm and residual memory scale
with 1/n.  The two collectives per projection pair are fused with the GEMMs next to them
(:mod:`dizo_b200.parallel.fused`):

    LN -> [all-gather rows -> QKV GEMM] -> attention over local heads -> [out_proj GEMM ->
    reduce-scatter rows] -> (+bias +residual, LN) -> [all-gather -> fc1 GEMM + ReLU] ->
    [fc2 GEMM -> reduce-scatter] -> (+bias +residual, next LN)

Zeroth-order specifics: every shard regenerates z for its own elements from the shared seed
with the element's index in the FULL tensor (row shards: an element offset; column shards: the
``local_cols / full_cols / col0`` mapping of the sweep kernel), so the perturbed model is
exactly the unsharded perturbed model; replicated tensors are perturbed identically everywhere
without communication.  The DiZO norms of the sharded k/v weights are partial sums that
``FusedComm.norm_allreduce_gamma`` reduces together with the gamma arithmetic.

The reference has no tensor parallelism (only an inherited comment, large_models/ht_opt.py:270-272).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.opt import _P, Batch, OPTConfig, OPTModel, Transform
from ..ops import attention as attn_ops
from ..ops import norm
from .fused import FusedComm

_ROW = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "fc1.weight")
_ROW_BIAS = ("self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias", "fc1.bias")
_COL = ("self_attn.out_proj.weight", "fc2.weight")


class TPOPTModel(OPTModel):
    def __init__(self, config: OPTConfig, device, dtype=torch.bfloat16, group=None, max_tokens: int = 8192,
                 n_push: int = 16, **kw):
        self.group = group if group is not None else dist.group.WORLD
        self.tp = dist.get_world_size(self.group)
        self.tp_rank = dist.get_rank(self.group)
        assert config.num_attention_heads % self.tp == 0 and config.ffn_dim % self.tp == 0
        assert config.do_layer_norm_before and config.word_embed_proj_dim == config.hidden_size
        kw.setdefault("mode", "full")
        assert kw["mode"] == "full", "tensor parallelism is built for full-parameter ZO"
        super().__init__(config, device, dtype, **kw)
        d = config.hidden_size
        self.max_tokens = max_tokens
        self.comm = FusedComm(self.group, self.device, ag_bytes=max_tokens * d * 2,
                              rs_bytes=max_tokens * d * 2, n_push=n_push,
                              norm_slots=max(256, 2 * config.num_hidden_layers))

    # ------------------------------------------------------------------ sharding
    def _kind(self, name: str) -> str:
        if any(name.endswith(s) for s in _ROW):
            return "row"
        if any(name.endswith(s) for s in _ROW_BIAS):
            return "rowvec"
        if any(name.endswith(s) for s in _COL):
            return "col"
        return "rep"

    def shard_of(self, name, shape):
        n, r = self.tp, self.tp_rank
        k = self._kind(name)
        if k == "row":
            rows = shape[0] // n
            return (rows, shape[1]), dict(elem_base=r * rows * shape[1])
        if k == "rowvec":
            rows = shape[0] // n
            return (rows,), dict(elem_base=r * rows)
        if k == "col":
            cols = shape[1] // n
            return (shape[0], cols), dict(local_cols=cols, full_cols=shape[1], col0=r * cols)
        return shape, {}

    def local_slice(self, name, full):
        n, r = self.tp, self.tp_rank
        k = self._kind(name)
        if k in ("row", "rowvec"):
            rows = full.shape[0] // n
            return full[r * rows:(r + 1) * rows]
        if k == "col":
            cols = full.shape[1] // n
            return full[:, r * cols:(r + 1) * cols]
        return full

    @torch.no_grad()
    def init_random_fast(self, seed: int = 0, std: float = 0.02):
        """Every rank draws the FULL tensor from the same device generator and keeps its part, so
        the sharded model equals the unsharded ``init_random_fast`` model."""
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
        """The unsharded tensor ``name`` from every rank's part ``local`` (cold path, NCCL)."""
        k = self._kind(name)
        t = local.contiguous()
        if k == "rep":
            return t.clone()
        parts = [torch.empty_like(t) for _ in range(self.tp)]
        dist.all_gather(parts, t, group=self.group)
        return torch.cat(parts, dim=1 if k == "col" else 0)

    def gather_state_dict(self) -> dict:
        """Full (unsharded) Hugging Face state dict, assembled on every rank (cold path, NCCL)."""
        sd = {n: self.gather_full(n, self.param(n)) for n in self.hf_order}
        if not self.untied:
            sd["lm_head.weight"] = sd[_P + "embed_tokens.weight"]
        return sd

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def hidden_states(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        """Returns this rank's rows of the final residual stream: [M / n, d] (rows = flattened
        (sequence, position), rank r holding rows [r M/n, (r+1) M/n))."""
        cfg, fc = self.config, self.comm
        nl, n, r = cfg.num_hidden_layers, self.tp, self.tp_rank
        d = cfg.hidden_size
        batch = self._fit(batch)
        B, L = batch.input_ids.shape
        M = B * L
        assert M % (n * 128) == 0 and M <= self.max_tokens, "token rows must split into 128-row tiles per rank"
        rows = M // n
        use_t = transform is not None
        # ---- globals (replicated)
        g_staged, g_shift = None, 0
        if use_t:
            g_staged = self._staging_for("globals", self.arena.group_numel(-1))
            g_shift = self._sweep_group(-1, transform, g_staged)
        self._gget = self._resolver(-1, transform, g_staged, g_shift)
        ids = batch.input_ids.reshape(1, M)[:, r * rows:(r + 1) * rows].contiguous()
        pos = batch.positions.reshape(1, M)[:, r * rows:(r + 1) * rows].contiguous()
        h = norm.embed(ids, pos, self._gget(_P + "embed_tokens.weight"),
                       self._gget(_P + "embed_positions.weight")).view(rows, d)
        layer_numel = max(self.arena.group_numel(g) for g in self.arena.groups() if g >= 0)

        def stage(i):
            if not use_t:
                return None, 0
            buf = self._staging_for(("layer", i % 2), layer_numel)
            return buf, self._sweep_group(i, transform, buf)

        cur = stage(0)
        w = self._layer_weights(0, self._resolver(0, transform, *cur))
        x_full, mine = fc.ag_input(M, d)
        norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps, out=mine)
        for i in range(nl):
            nxt_w = None
            if i + 1 < nl:
                nxt = stage(i + 1)
                nxt_w = self._layer_weights(i + 1, self._resolver(i + 1, transform, *nxt))
            qkv = fc.ag_gemm(x_full, w.qkv_w, w.qkv_b)                       # [M, 3 d/n]
            if self.kv_capture is not None:
                self.kv_capture.append(qkv)                                  # this rank's heads (generation)
            ctx = attn_ops.attention(qkv.view(B, L, qkv.shape[1]), cfg.num_attention_heads // n,
                                     batch.pad_left)
            idx = fc.gemm_rs(ctx.view(M, d // n), w.out_w)
            x_full, mine = fc.ag_input(M, d)
            h, _ = fc.rs_reduce_layernorm(idx, h, w.out_b, w.ln2_w, w.ln2_b, cfg.layer_norm_eps, y_out=mine)
            f = fc.ag_gemm(x_full, w.fc1_w, w.fc1_b, act=cfg.activation_function)
            idx = fc.gemm_rs(f, w.fc2_w)
            if nxt_w is not None:
                x_full, mine = fc.ag_input(M, d)
                h, _ = fc.rs_reduce_layernorm(idx, h, w.fc2_b, nxt_w.ln1_w, nxt_w.ln1_b, cfg.layer_norm_eps,
                                              y_out=mine)
                w = nxt_w
            else:
                h, _ = fc.rs_reduce_layernorm(idx, h, w.fc2_b)
        self._rows_local = (r * rows, (r + 1) * rows)
        return h

    def _fit(self, batch: Batch) -> Batch:
        """Pad a batch so that its token rows split into 128-row tiles per rank: the length grows
        on the left to a multiple of 128, and all-padding sequences are appended until the tile count
        divides by the number of ranks.  Row indices of the caller are translated in ``final_rows``."""
        B, L = batch.input_ids.shape
        n = self.tp
        Lp = -(-L // 128) * 128
        Bp = B
        while (Bp * (Lp // 128)) % n:
            Bp += 1
        self._row_map = None
        if Lp == L and Bp == B:
            return batch
        dev = batch.input_ids.device
        ids = torch.ones((Bp, Lp), dtype=batch.input_ids.dtype, device=dev)
        pos = torch.ones((Bp, Lp), dtype=batch.positions.dtype, device=dev)
        ids[:B, Lp - L:] = batch.input_ids
        pos[:B, Lp - L:] = batch.positions
        pad = torch.full((Bp,), Lp, dtype=torch.int32, device=dev)
        old = batch.pad_left if batch.pad_left is not None else torch.zeros(B, dtype=torch.int32, device=dev)
        pad[:B] = old + (Lp - L)
        self._row_map = (L, Lp)
        import dataclasses
        return dataclasses.replace(batch, input_ids=ids, positions=pos, pad_left=pad)

    @torch.no_grad()
    def final_rows(self, h: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Final LayerNorm of the requested global rows, replicated on every rank: each rank fills
        in the rows it owns and one small NCCL all-reduce assembles the rest."""
        cfg = self.config
        lo, hi = self._rows_local
        rows_l = rows.long()
        if self._row_map is not None:                  # indices into the caller's unpadded batch
            L0, Lp = self._row_map
            rows_l = (rows_l // L0) * Lp + rows_l % L0 + (Lp - L0)
        own = (rows_l >= lo) & (rows_l < hi)
        local_idx = torch.where(own, rows_l - lo, torch.zeros_like(rows_l)).to(torch.int32)
        x = norm.gather_rows(h, local_idx)
        x = x * own.view(-1, 1).to(x.dtype)
        dist.all_reduce(x, group=self.group)           # exactly one non-zero contribution per row
        gget = self._gget
        return norm.layernorm(x, gget(_P + "final_layer_norm.weight"), gget(_P + "final_layer_norm.bias"),
                              cfg.layer_norm_eps)

    def reduce_norms(self, gs, reinit: bool) -> None:
        """Sum the per-shard squared distances of the constrained tensors over the ranks and run
        the gamma / alpha arithmetic, in one kernel."""
        self.comm.norm_allreduce_gamma(gs.sq.clone(), gs, reinit)
