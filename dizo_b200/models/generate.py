"""Autoregressive decoding with a KV cache: greedy, temperature / top-k / top-p sampling, beams.

Stands in for the ``model.generate`` calls of the reference (large_models/run.py:277-290,
large_models/trainer.py:1554-1561): same knobs (``do_sample``, ``temperature``, ``num_beams``,
``top_p``, ``top_k``, ``max_new_tokens``, a list of end-of-sequence ids), left-padded batches.
The prompt is one forward through the training kernels with the per-layer QKV activations
captured as the cache; each new token then runs the same GEMM / LayerNorm kernels on a
[batch, d] activation and a small attention over the cache.

Sharded models decode without moving weights.  Tensor parallel: every rank keeps the K / V cache of
its own heads, runs ``decode_attn_kernel`` on them and the row-reduced projections (out_proj, fc2)
are summed with one small all-reduce each.  FSDP: every matrix is sharded by output rows, so a rank
computes its slice of each projection from the replicated [batch, d] activation and the slices are
all-gathered (a few KB per token); attention runs on the full heads on every rank.  All ranks of the
group must call :func:`generate` together (same batch size); the stop test is agreed by all-reduce.
Pipeline parallel: every stage caches the K / V of its own blocks, a token's activation is sent stage to stage
and the last stage's logits are broadcast.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import decode as decode_ops
from ..ops import gemm, norm
from .opt import _P, Batch, OPTModel, layer_prefix, make_batch


def filter_logits(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                  top_p: Optional[float] = None) -> torch.Tensor:
    """Temperature, then top-k, then nucleus filtering (filtered entries become -inf)."""
    if temperature and temperature != 1.0:
        logits = logits / temperature
    if top_k is not None and top_k > 0:
        k = min(int(top_k), logits.shape[-1])
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and 0.0 < top_p < 1.0:
        srt, idx = torch.sort(logits, dim=-1, descending=True)
        cum = torch.softmax(srt, dim=-1).cumsum(dim=-1)
        drop = cum - torch.softmax(srt, dim=-1) >= top_p      # keep the first token that crosses p
        srt = srt.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    return logits


class _Decoder:
    """Per-layer K/V caches and the single-token step."""

    def __init__(self, model: OPTModel, B: int, max_len: int):
        self.m = model
        cfg = model.config
        d = cfg.hidden_size
        dev, dt = model.device, model.dtype
        self.k = [torch.zeros(B, max_len, d, dtype=dt, device=dev) for _ in range(cfg.num_hidden_layers)]
        self.v = [torch.zeros(B, max_len, d, dtype=dt, device=dev) for _ in range(cfg.num_hidden_layers)]
        self.len = 0

    def prefill(self, batch: Batch) -> torch.Tensor:
        m = self.m
        d = m.config.hidden_size
        B, L = batch.input_ids.shape
        m.kv_capture = []
        try:
            h = m.hidden_states(batch)
        finally:
            cap, m.kv_capture = m.kv_capture, None
        for i, qkv in enumerate(cap):
            q3 = qkv.view(B, L, 3 * d)
            self.k[i][:, :L].copy_(q3[:, :, d:2 * d])
            self.v[i][:, :L].copy_(q3[:, :, 2 * d:])
        self.len = L
        return _head_logits(m, h[:, -1, :])                      # left padded: last column is real

    def all_done(self, done: torch.Tensor) -> bool:
        return bool(done.all())

    def reorder(self, index: torch.Tensor) -> None:
        for i in range(len(self.k)):
            self.k[i] = self.k[i].index_select(0, index)
            self.v[i] = self.v[i].index_select(0, index)

    def step(self, tokens: torch.Tensor, positions: torch.Tensor, pad_left: torch.Tensor) -> torch.Tensor:
        """tokens, positions: int32 [B]; returns the next-token logits [B, V] (fp32)."""
        m = self.m
        t = self.len
        h = m.decode_embed(tokens, positions, m._resolver(-1, None, None, 0))
        for i in range(m.config.num_hidden_layers):
            w = m._layer_weights(i, m._resolver(i, None, None, 0))
            h = m.decode_block(h, w, self.k[i], self.v[i], t, pad_left)
        self.len = t + 1
        return _head_logits(m, h)


def _head_logits(model: OPTModel, h_last: torch.Tensor) -> torch.Tensor:
    get = model._resolver(-1, None, None, 0)
    x = model._final_norm(h_last, get)
    table = get("lm_head.weight") if model.untied else get(model.EMBED)
    return gemm.linear(x.contiguous(), table, out_dtype=torch.float32).float()


def _bias_residual(part: torch.Tensor, bias: torch.Tensor, res: torch.Tensor) -> torch.Tensor:
    return (part.float() + bias.float() + res.float()).to(res.dtype)


class _TPDecoder(_Decoder):
    """Tensor parallel: this rank's heads only; the activation [B, d] is replicated."""

    def __init__(self, model, B: int, max_len: int):
        self.m = model
        cfg = model.config
        dl = cfg.hidden_size // model.tp
        dev, dt = model.device, model.dtype
        self.k = [torch.zeros(B, max_len, dl, dtype=dt, device=dev) for _ in range(cfg.num_hidden_layers)]
        self.v = [torch.zeros(B, max_len, dl, dtype=dt, device=dev) for _ in range(cfg.num_hidden_layers)]
        self.len = 0
        self.pad_extra = 0

    def prefill(self, batch: Batch) -> torch.Tensor:
        m = self.m
        dl = m.config.hidden_size // m.tp
        B, L = batch.input_ids.shape
        m.kv_capture = []
        try:
            h = m.hidden_states(batch)                         # pads to whole 128-row tiles per rank
        finally:
            cap, m.kv_capture = m.kv_capture, None
        Lp = m._row_map[1] if m._row_map is not None else L
        for i, qkv in enumerate(cap):
            q3 = qkv.view(-1, Lp, 3 * dl)[:B]
            self.k[i][:, :Lp].copy_(q3[:, :, dl:2 * dl])
            self.v[i][:, :Lp].copy_(q3[:, :, 2 * dl:])
        self.len, self.pad_extra = Lp, Lp - L
        rows = (torch.arange(B, device=h.device, dtype=torch.int32) * L + (L - 1))
        x = m.final_rows(h, rows)                              # final LayerNorm applied, replicated
        return gemm.linear(x.contiguous(), m.lm_head_weight(), out_dtype=torch.float32).float()

    def step(self, tokens, positions, pad_left) -> torch.Tensor:
        m, cfg = self.m, self.m.config
        d, n = cfg.hidden_size, m.tp
        dl = d // n
        get = m._resolver(-1, None, None, 0)
        h = norm.embed(tokens.view(-1, 1), positions.view(-1, 1), get(_P + "embed_tokens.weight"),
                       get(_P + "embed_positions.weight")).view(-1, d)
        t = self.len
        pl = pad_left + self.pad_extra
        for i in range(cfg.num_hidden_layers):
            w = m._layer_weights(i, m._resolver(i, None, None, 0))
            x = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps)
            qkv = gemm.linear(x, w.qkv_w, w.qkv_b)                            # [B, 3 d/n]: own heads
            self.k[i][:, t].copy_(qkv[:, dl:2 * dl])
            self.v[i][:, t].copy_(qkv[:, 2 * dl:])
            ctx = decode_ops.decode_attention(qkv[:, :dl], self.k[i], self.v[i], t + 1,
                                              cfg.num_attention_heads // n, pl)
            part = gemm.linear(ctx.contiguous(), w.out_w, out_dtype=torch.float32)
            dist.all_reduce(part, group=m.group)
            h = _bias_residual(part, w.out_b, h)
            x = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps)
            f = gemm.linear(x, w.fc1_w, w.fc1_b, act=cfg.activation_function)
            part = gemm.linear(f, w.fc2_w, out_dtype=torch.float32)
            dist.all_reduce(part, group=m.group)
            h = _bias_residual(part, w.fc2_b, h)
        self.len = t + 1
        return _head_logits(m, h)

    def all_done(self, done: torch.Tensor) -> bool:
        return bool(done.all())                                # every rank decodes the same batch


class _FSDPDecoder(_Decoder):
    """FSDP: weights sharded by output rows; a rank computes its slice of every projection from the
    replicated activation and the slices are all-gathered."""

    def _gathered(self, x: torch.Tensor, w_shard: torch.Tensor, bias=None, act=None, residual=None):
        m = self.m
        y = gemm.linear(x, w_shard)                                           # [B, out / n]
        parts = torch.empty((m.n,) + tuple(y.shape), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(parts, y.contiguous(), group=m.group)
        full = parts.permute(1, 0, 2).reshape(y.shape[0], -1).float()
        if bias is not None:
            full = full + bias.float()
        if act == "relu":
            full = torch.relu(full)
        elif act == "gelu":
            full = torch.nn.functional.gelu(full)
        if residual is not None:
            full = full + residual.float()
        return full.to(x.dtype)

    def step(self, tokens, positions, pad_left) -> torch.Tensor:
        m, cfg = self.m, self.m.config
        d = cfg.hidden_size
        get = m._resolver(-1, None, None, 0)
        h = norm.embed(tokens.view(-1, 1), positions.view(-1, 1), get(_P + "embed_tokens.weight"),
                       get(_P + "embed_positions.weight")).view(-1, d)
        t = self.len
        for i in range(cfg.num_hidden_layers):
            g = m._resolver(i, None, None, 0)
            lp = layer_prefix(i)
            a = lp + "self_attn."
            x = norm.layernorm(h, g(lp + "self_attn_layer_norm.weight"), g(lp + "self_attn_layer_norm.bias"),
                               cfg.layer_norm_eps)
            q = self._gathered(x, g(a + "q_proj.weight"), g(a + "q_proj.bias"))
            k = self._gathered(x, g(a + "k_proj.weight"), g(a + "k_proj.bias"))
            v = self._gathered(x, g(a + "v_proj.weight"), g(a + "v_proj.bias"))
            self.k[i][:, t].copy_(k)
            self.v[i][:, t].copy_(v)
            ctx = decode_ops.decode_attention(q, self.k[i], self.v[i], t + 1, cfg.num_attention_heads, pad_left)
            h = self._gathered(ctx.contiguous(), g(a + "out_proj.weight"), g(a + "out_proj.bias"), residual=h)
            x = norm.layernorm(h, g(lp + "final_layer_norm.weight"), g(lp + "final_layer_norm.bias"),
                               cfg.layer_norm_eps)
            f = self._gathered(x, g(lp + "fc1.weight"), g(lp + "fc1.bias"), act=cfg.activation_function)
            h = self._gathered(f, g(lp + "fc2.weight"), g(lp + "fc2.bias"), residual=h)
        self.len = t + 1
        return _head_logits(m, h)

    def all_done(self, done: torch.Tensor) -> bool:
        flag = done.all().to(torch.int32).reshape(1)           # ranks decode different batches: agree on the stop
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.m.group)
        return bool(flag.item())


class _PPDecoder(_Decoder):
    """Pipeline parallel: every stage keeps the K / V cache of its own blocks; a token's [B, d] activation
    travels stage to stage and the last stage's logits are broadcast (every rank decodes the same batch)."""

    def __init__(self, model, B: int, max_len: int):
        self.m = model
        cfg = model.config
        d = cfg.hidden_size
        dev, dt = model.device, model.dtype
        self.layers = list(range(model.lo, model.hi))
        self.k = [torch.zeros(B, max_len, d, dtype=dt, device=dev) for _ in self.layers]
        self.v = [torch.zeros(B, max_len, d, dtype=dt, device=dev) for _ in self.layers]
        self.len = 0
        self.B = B

    def prefill(self, batch: Batch) -> torch.Tensor:
        m = self.m
        d = m.config.hidden_size
        B, L = batch.input_ids.shape
        m.kv_capture = []
        try:
            h = m.hidden_states(batch)                         # micro-batches through this stage's blocks
        finally:
            cap, m.kv_capture = m.kv_capture, None
        n_own = len(self.layers)
        row0 = 0
        for j0 in range(0, len(cap), max(n_own, 1)):           # captured per micro-batch, then per block
            rows = cap[j0].numel() // (3 * d * L)
            for j in range(n_own):
                q3 = cap[j0 + j].reshape(rows, L, 3 * d)
                self.k[j][row0:row0 + rows, :L].copy_(q3[:, :, d:2 * d])
                self.v[j][row0:row0 + rows, :L].copy_(q3[:, :, 2 * d:])
            row0 += rows
        self.len = L
        V = m.config.vocab_size
        return m._from_last(lambda: _head_logits(m, h[:, -1, :]), (B, V))

    def step(self, tokens, positions, pad_left) -> torch.Tensor:
        m, cfg = self.m, self.m.config
        d = cfg.hidden_size
        first, last = m.stage == 0, m.stage == m.n - 1
        t = self.len
        if first:
            h = m.decode_embed(tokens, positions, m._resolver(-1, None, None, 0))
        else:
            h = torch.empty((self.B, d), dtype=m.dtype, device=m.device)
            dist.recv(h, src=m._rank_of(m.stage - 1), group=m.group)
        for j, i in enumerate(self.layers):
            w = m._layer_weights(i, m._resolver(i, None, None, 0))
            h = m.decode_block(h, w, self.k[j], self.v[j], t, pad_left)
        if not last:
            dist.send(h.contiguous(), dst=m._rank_of(m.stage + 1), group=m.group)
        self.len = t + 1
        return m._from_last(lambda: _head_logits(m, h), (self.B, cfg.vocab_size))


def _make_decoder(model, B: int, max_len: int) -> _Decoder:
    kind = type(model).__name__
    if type(model).hidden_states is OPTModel.hidden_states:
        return _Decoder(model, B, max_len)
    if kind in ("TPOPTModel", "TPCompositionModel"):
        return _TPDecoder(model, B, max_len)
    if kind in ("FSDPOPTModel", "FSDPCompositionModel"):
        return _FSDPDecoder(model, B, max_len)
    if kind in ("PPOPTModel", "PPLlamaModel"):
        return _PPDecoder(model, B, max_len)
    raise NotImplementedError(f"autoregressive decoding is not built for {kind}")


@torch.no_grad()
def generate(model: OPTModel, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
             max_new_tokens: int = 50, do_sample: bool = False, temperature: float = 1.0,
             top_k: Optional[int] = None, top_p: Optional[float] = None, num_beams: int = 1,
             eos_token_id: Optional[Sequence[int]] = None, pad_token_id: int = 1,
             seed: Optional[int] = None, transform=None) -> List[List[int]]:
    """Returns, per input row, prompt + generated token ids (generation stops at an EOS id,
    which is kept, as Hugging Face does).  ``transform`` is accepted for API symmetry and must
    be None: perturb in place around the call when decoding under a perturbation."""
    assert transform is None, "decode under a perturbation by perturbing in place around generate()"
    dev = model.device
    ids = torch.as_tensor(input_ids).long()
    B0, L0 = ids.shape
    mask = torch.ones_like(ids) if attention_mask is None else torch.as_tensor(attention_mask).long()
    max_new_tokens = max(0, int(max_new_tokens))
    eos = set(int(e) for e in (eos_token_id or []))
    nb = max(1, int(num_beams))
    if nb > 1:
        ids = ids.repeat_interleave(nb, 0)
        mask = mask.repeat_interleave(nb, 0)
    B = ids.shape[0]
    batch = make_batch(ids, mask).to(dev)
    dec = _make_decoder(model, B, L0 + max_new_tokens + 128)   # + room for the tile padding of sharded prefill
    logits = dec.prefill(batch)
    n_real = mask.sum(dim=1).to(dev)
    pad_left = batch.pad_left
    gen = torch.Generator(device=dev)
    if seed is not None:
        gen.manual_seed(seed)
    out = [row[m.bool()].tolist() for row, m in zip(ids, mask)]
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    beam_score = torch.zeros(B, device=dev)
    if nb > 1:
        beam_score.view(B0, nb)[:, 1:] = float("-inf")            # identical beams at step 0
    for t in range(max_new_tokens):
        if nb == 1:
            if do_sample and dev.type != "cuda":
                probs = torch.softmax(filter_logits(logits, temperature, top_k, top_p), dim=-1)
                nxt = torch.multinomial(probs, 1, generator=gen).squeeze(1)
            else:
                nxt = decode_ops.sample(logits.contiguous(), temperature, top_k, top_p, do_sample,
                                        seed=seed or 0, offset=t)
            nxt = torch.where(done, torch.full_like(nxt, pad_token_id), nxt)
        else:
            lp = torch.log_softmax(logits, dim=-1)
            V = lp.shape[-1]
            lp = torch.where(done[:, None], torch.full_like(lp, float("-inf")), lp)
            lp[done, pad_token_id] = 0.0                           # finished beams carry their score
            cand = (beam_score[:, None] + lp).view(B0, nb * V)
            top, flat = cand.topk(nb, dim=-1)
            src = flat // V + (torch.arange(B0, device=dev) * nb)[:, None]
            nxt = (flat % V).reshape(-1)
            src = src.reshape(-1)
            beam_score = top.reshape(-1)
            dec.reorder(src)
            done = done[src]
            n_real = n_real[src]
            pad_left = pad_left[src]
            out = [list(out[i]) for i in src.tolist()]
        toks = nxt.tolist()
        dl = done.tolist()
        for i in range(B):
            if not dl[i]:
                out[i].append(toks[i])
        done = done | torch.tensor([tk in eos for tk in toks], dtype=torch.bool, device=dev)
        if dec.all_done(done) or t + 1 == max_new_tokens:
            break
        pos = (n_real + 2).to(torch.int32)                         # OPT positions: index + 2
        n_real = n_real + 1
        logits = dec.step(nxt.to(torch.int32), pos, pad_left)
    if nb > 1:
        best = beam_score.view(B0, nb).argmax(dim=-1) + torch.arange(B0, device=dev) * nb
        out = [out[i] for i in best.tolist()]
    return out
