"""Pipeline-parallel OPT / LLaMA for zeroth-order training: consecutive blocks on consecutive ranks.

The reference's only multi-GPU placement is ``device_map='auto'`` (large_models/run.py:167-181):
accelerate puts consecutive layers on different GPUs and runs them one after the other, one GPU
busy at a time.  Zeroth-order training is forward-only, so a real pipeline is cheap: rank ``s``
holds blocks ``[lo_s, hi_s)`` (the first stage also the embeddings, the last also the final
LayerNorm and the tied LM-head table), the batch is cut into micro-batches of whole sequences and
every stage receives an activation, runs its blocks and sends the result on while the previous
stage already works on the next micro-batch.  There is no backward, so there are no bubbles beyond
the fill and drain of one forward, and nothing is stashed.

Perturbation needs no communication: every stage regenerates z for its own tensors from the
shared step seed (z depends only on seed, tensor id and element index), so a pipeline step applies
the same perturbation and update as the single-device step (equal up to the summation order of the
last block's small GEMMs, which run per micro-batch here).  The stage's transformed weights
(theta + eps z, or the DiZO blend) are staged once per forward - all owned blocks, not one layer
at a time - because every micro-batch passes through all of them.  The loss is computed on the last
stage and broadcast (one scalar); activations travel by ``torch.distributed`` send / recv (NCCL on
GPUs, gloo on CPU ranks).
"""
from __future__ import annotations

import dataclasses
import re

import torch
import torch.distributed as dist

from ..models.llama import LlamaModel
from ..models.opt import Batch, OPTModel, Transform
from ..ops import loss as loss_ops

_LAYER_RE = re.compile(r"layers\.(\d+)\.")


def stage_bounds(n_layers: int, n_stages: int) -> list[tuple[int, int]]:
    """Contiguous, near-equal block ranges; earlier stages take the remainder."""
    base, rem = divmod(n_layers, n_stages)
    out, lo = [], 0
    for s in range(n_stages):
        hi = lo + base + (1 if s < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


class _Pipeline:
    """The pipeline placement, written against the architecture hooks of :class:`OPTModel` (``EMBED``,
    ``_embed``, ``_embed_param_names``, ``_layer_weights``, ``_layer_forward``, ``final_rows``); mixed into the
    OPT and LLaMA model classes below."""

    def __init__(self, config, device, dtype=torch.bfloat16, group=None, micro_batches: int = 0, **kw):
        self.group = group if group is not None else dist.group.WORLD
        self.n = dist.get_world_size(self.group)
        self.stage = dist.get_rank(self.group)
        assert config.num_hidden_layers >= self.n, "more pipeline stages than blocks"
        self.lo, self.hi = stage_bounds(config.num_hidden_layers, self.n)[self.stage]
        self.micro_batches = micro_batches            # 0 = one micro-batch per stage
        assert getattr(config, "word_embed_proj_dim", config.hidden_size) == config.hidden_size, \
            "project_in/out models are not staged"
        assert not kw.get("prefix_reparam"), "the shared prefix embeddings live with the first block: not staged"
        super().__init__(config, device, dtype, **kw)

    # ------------------------------------------------------------------ ownership
    def owns(self, name: str) -> bool:
        m = _LAYER_RE.search(name)
        if m:
            return self.lo <= int(m.group(1)) < self.hi
        first, last = self.stage == 0, self.stage == self.n - 1
        if name == self.EMBED:
            return first or (last and not self.untied)           # tied LM head reads the table
        if name in self._embed_param_names():
            return first
        return last                                               # final norm, lm_head.weight

    def _rank_of(self, s: int) -> int:
        return dist.get_global_rank(self.group, s) if self.group is not dist.group.WORLD else s

    def gather_state_dict(self) -> dict:
        """Full Hugging Face state dict on every rank (cold path: checkpoints, tests)."""
        parts = [None] * self.n
        dist.all_gather_object(parts, {k: v.cpu() for k, v in self.state_dict().items()}, group=self.group)
        sd = {}
        for p in parts:
            sd.update(p)
        if not self.untied:
            sd["lm_head.weight"] = sd[self.EMBED]
        return sd

    def state_dict(self) -> dict:
        """This stage's tensors only (Hugging Face names)."""
        return {n: self.param(n).detach().clone() for n in self.hf_order}

    def gather_dict(self, local: dict) -> dict:
        """Union of per-stage {name: tensor} dicts on every rank (anchors in checkpoints)."""
        parts = [None] * self.n
        dist.all_gather_object(parts, {k: v.cpu() for k, v in local.items()}, group=self.group)
        out = {}
        for p in parts:
            out.update(p)
        return out

    # ------------------------------------------------------------------ forward
    def _stage_weights(self, transform: Transform | None):
        """Resolvers for the globals and for every owned block, transformed once per forward."""
        ar = self.arena
        groups = ar.groups()
        gets = {}
        for g in [-1] + list(range(self.lo, self.hi)):
            if transform is None or g not in groups:
                gets[g] = self._resolver(g, None, None, 0)
                continue
            buf = self._staging_for(("pp", g), ar.group_numel(g))
            gets[g] = self._resolver(g, transform, buf, self._sweep_group(g, transform, buf))
        return gets

    def _micro(self, batch: Batch) -> list[tuple[int, int]]:
        B = batch.input_ids.shape[0]
        k = self.micro_batches or self.n
        k = max(1, min(k, B))
        step = -(-B // k)
        return [(a, min(B, a + step)) for a in range(0, B, step)]

    @torch.no_grad()
    def hidden_states(self, batch: Batch, transform: Transform | None = None,
                      rows: torch.Tensor | None = None) -> torch.Tensor | None:
        """The last stage returns the final residual stream [B, L, d] (with ``rows``: only those token rows,
        [R, d], the last block running on them alone as in the single-device model); the others None."""
        cfg = self.config
        d = cfg.hidden_size
        B, L = batch.input_ids.shape
        gets = self._stage_weights(transform)
        self._gget = gets[-1]
        first, last = self.stage == 0, self.stage == self.n - 1
        prev_r = self._rank_of(self.stage - 1) if not first else None
        next_r = self._rank_of(self.stage + 1) if not last else None
        weights = [self._layer_weights(i, gets[i]) for i in range(self.lo, self.hi)]
        outs, sends = [], []
        for a, b in self._micro(batch):
            mb = dataclasses.replace(batch, input_ids=batch.input_ids[a:b], positions=batch.positions[a:b],
                                     pad_left=batch.pad_left[a:b] if batch.pad_left is not None else None)
            if first:
                h = self._embed(mb.input_ids, mb.positions, self._gget)
            else:
                h = torch.empty((b - a, L, d), dtype=self.dtype, device=self.device)
                dist.recv(h, src=prev_r, group=self.group)
            for j, w in enumerate(weights):
                only = None
                if last and rows is not None and j == len(weights) - 1:
                    keep = (rows >= a * L) & (rows < b * L)          # this micro-batch's loss rows
                    only = (rows[keep] - a * L).to(torch.int32)
                h = self._layer_forward(h, w, mb, only)
            if last:
                outs.append(h)
            else:
                sends.append((dist.isend(h.contiguous(), dst=next_r, group=self.group), h))
        for req, _ in sends:
            req.wait()
        return torch.cat(outs, dim=0) if last else None

    def _from_last(self, fn, shape) -> torch.Tensor:
        """Run ``fn`` on the last stage and hand its fp32 result of ``shape`` to every stage."""
        last = self.stage == self.n - 1
        out = fn() if last else torch.empty(shape, dtype=torch.float32, device=self.device)
        out = out.reshape(shape).contiguous()
        dist.broadcast(out, src=self._rank_of(self.n - 1), group=self.group)
        return out

    @torch.no_grad()
    def loss(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        h = self.hidden_states(batch, transform, rows=batch.rows)

        def tail():
            x = self.final_rows(h, None)
            table = self.lm_head_weight()
            if batch.cand_ids is not None:
                return loss_ops.verbalizer_ce(x, table, batch.cand_ids, batch.labels)[1]
            lp = loss_ops.token_logprobs(x, table, batch.targets)
            return loss_ops.option_ce(lp, batch.seq_start, batch.ex_start, batch.labels, batch.classification)
        return self._from_last(tail, (1,))

    @torch.no_grad()
    def row_logprobs(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        h = self.hidden_states(batch, transform, rows=batch.rows)
        return self._from_last(lambda: loss_ops.token_logprobs(self.final_rows(h, None),
                                                               self.lm_head_weight(), batch.targets),
                               (batch.targets.numel(),))

    @torch.no_grad()
    def logits(self, batch: Batch, rows: torch.Tensor | None = None) -> torch.Tensor:
        from ..ops import gemm
        h = self.hidden_states(batch)
        B, L = batch.input_ids.shape
        if rows is None:
            rows = torch.arange(B * L, dtype=torch.int32, device=self.device)
        return self._from_last(lambda: gemm.linear(self.final_rows(h, rows), self.lm_head_weight(),
                                                   out_dtype=torch.float32),
                               (rows.numel(), self.config.vocab_size))


class PPOPTModel(_Pipeline, OPTModel):
    """OPT blocks over the ranks of ``group``."""


class PPLlamaModel(_Pipeline, LlamaModel):
    """LLaMA-family blocks over the ranks of ``group`` (every stage builds the rotary table it needs)."""
