"""The sharded forwards written as the plain composition: NCCL collective, then the stand-alone kernels.

These classes compute exactly what :class:`~dizo_b200.parallel.fsdp.FSDPOPTModel` and
:class:`~dizo_b200.parallel.tp.TPOPTModel` compute, with the same sharding, the same sweep and GEMM
kernels and the same z stream, but every collective is a library call placed between kernels:

* FSDP: the local sweep perturbs this rank's row shards into a staging area, ``all_gather_into_tensor``
  (NCCL) assembles each matrix - one matrix ahead, on a communication stream, as a prefetching FSDP
  implementation does - and the two-SM tcgen05 GEMM multiplies the gathered copy;
* tensor parallel: ``all_gather_into_tensor`` of the LayerNorm rows before the QKV / fc1 GEMMs,
  ``reduce_scatter_tensor`` of the out_proj / fc2 partial products, then the stand-alone
  bias + residual add and LayerNorm kernel.

They are the comparison arm of the fused compute+collective kernels (``bench.py`` times both in the
same process) and a second oracle for them in the multi-GPU tests.  The reference has neither layout for
zeroth-order training (its only sharded path is torch FSDP for the first-order trainer,
large_models/finetune_fsdp.sh:51-63).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.opt import _P, Batch, Transform, layer_prefix
from ..ops import attention as attn_ops
from ..ops import gemm, norm
from .fsdp import FSDPOPTModel
from .tp import TPOPTModel


class FSDPCompositionModel(FSDPOPTModel):
    """``FSDPOPTModel`` sharding; forward = local sweep -> NCCL all-gather (prefetched) -> GEMM."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        cfg = self.config
        d, F = cfg.hidden_size, cfg.ffn_dim
        self._wbuf = [torch.empty(max(3 * d * d, F * d), dtype=self.dtype, device=self.device) for _ in range(2)]
        self._comm_stream = torch.cuda.Stream(device=self.device)
        self._n_gather = 0

    def _gather(self, i: int, which: str, get, done: list):
        """Start the all-gather of one weight group of layer ``i`` on the communication stream, into the
        weight buffer that is not in use (``done[k]``: the event after which buffer k may be overwritten).
        Returns (full weight view, event that marks its arrival, buffer index)."""
        cfg = self.config
        d, F = cfg.hidden_size, cfg.ffn_dim
        lp = layer_prefix(i)
        names = {"qkv": ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"],
                 "out": ["self_attn.out_proj.weight"], "fc1": ["fc1.weight"], "fc2": ["fc2.weight"]}[which]
        N, K = {"qkv": (3 * d, d), "out": (d, d), "fc1": (F, d), "fc2": (d, F)}[which]
        k = self._n_gather % 2
        self._n_gather += 1
        full = self._wbuf[k][:N * K].view(N, K)
        cs = self._comm_stream
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        start = torch.cuda.Event()
        start.record(main)                       # the staged shards were written on the main stream
        with torch.cuda.stream(cs):
            cs.wait_event(start)
            if done[k] is not None:
                cs.wait_event(done[k])
            rows = N // len(names)
            for j, nm in enumerate(names):
                shard = get(lp + nm)
                dist.all_gather_into_tensor(full[j * rows:(j + 1) * rows], shard.contiguous(), group=self.group)
            ready.record(cs)
        return full, ready, k

    @torch.no_grad()
    def hidden_states(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        cfg = self.config
        nl, d = cfg.num_hidden_layers, cfg.hidden_size
        B, L = batch.input_ids.shape
        M = B * L
        main = torch.cuda.current_stream(self.device)
        g_staged, g_shift = None, 0
        if transform is not None:
            g_staged = self._staging_for("globals", self.arena.group_numel(-1))
            g_shift = self._sweep_group(-1, transform, g_staged)
        self._gget = self._resolver(-1, transform, g_staged, g_shift)
        h = norm.embed(batch.input_ids, batch.positions, self._gget(_P + "embed_tokens.weight"),
                       self._gget(_P + "embed_positions.weight")).view(M, d)
        layer_numel = max(self.arena.group_numel(g) for g in self.arena.groups() if g >= 0)

        def stage(i):
            if transform is None:
                return self._resolver(i, None, None, 0)
            buf = self._staging_for(("layer", i % 2), layer_numel)
            return self._resolver(i, transform, buf, self._sweep_group(i, transform, buf))

        done = [None, None]                      # per weight buffer: after the GEMM that read it last
        get = stage(0)
        cur = self._gather(0, "qkv", get, done)
        for i in range(nl):
            lp = layer_prefix(i)
            a = lp + "self_attn."
            nget = stage(i + 1) if i + 1 < nl else None
            following = [("out", get, i), ("fc1", get, i), ("fc2", get, i)] + \
                        ([("qkv", nget, i + 1)] if nget is not None else [])
            x = norm.layernorm(h, get(lp + "self_attn_layer_norm.weight"), get(lp + "self_attn_layer_norm.bias"),
                               cfg.layer_norm_eps)
            for step, which in enumerate(("qkv", "out", "fc1", "fc2")):
                # start the next matrix's gather into the other buffer, then multiply the current one
                nxt = None
                if step < len(following):
                    nw, ng, ni = following[step]
                    nxt = self._gather(ni, nw, ng, done)
                w_cur, ev_cur, k_cur = cur
                main.wait_event(ev_cur)
                if which == "qkv":
                    qkv_b = self._fused([get(a + "q_proj.bias"), get(a + "k_proj.bias"), get(a + "v_proj.bias")])
                    qkv = gemm.linear(x, w_cur, qkv_b)
                elif which == "out":
                    h = gemm.linear(ctx.view(M, d), w_cur, get(a + "out_proj.bias"), residual=h)
                elif which == "fc1":
                    f = gemm.linear(x, w_cur, get(lp + "fc1.bias"), act=cfg.activation_function)
                else:
                    h = gemm.linear(f, w_cur, get(lp + "fc2.bias"), residual=h)
                done[k_cur] = torch.cuda.Event()
                done[k_cur].record(main)
                if which == "qkv":
                    ctx = attn_ops.attention(qkv.view(B, L, 3 * d), cfg.num_attention_heads, batch.pad_left)
                elif which == "out":
                    x = norm.layernorm(h, get(lp + "final_layer_norm.weight"), get(lp + "final_layer_norm.bias"),
                                       cfg.layer_norm_eps)
                if nxt is not None:
                    cur = nxt
            if nget is not None:
                get = nget
        main.wait_stream(self._comm_stream)
        return h.view(B, L, d)


class TPCompositionModel(TPOPTModel):
    """``TPOPTModel`` sharding; forward = NCCL all-gather / reduce-scatter between stand-alone kernels."""

    @torch.no_grad()
    def hidden_states(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        cfg = self.config
        nl, n, r = cfg.num_hidden_layers, self.tp, self.tp_rank
        d = cfg.hidden_size
        batch = self._fit(batch)
        B, L = batch.input_ids.shape
        M = B * L
        rows = M // n
        use_t = transform is not None
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
        x_full = torch.empty((M, d), dtype=self.dtype, device=self.device)
        part_rows = torch.empty((rows, d), dtype=self.dtype, device=self.device)

        def stage(i):
            if not use_t:
                return None, 0
            buf = self._staging_for(("layer", i % 2), layer_numel)
            return buf, self._sweep_group(i, transform, buf)

        def gather(x_local):
            dist.all_gather_into_tensor(x_full, x_local, group=self.group)
            return x_full

        def reduce_add(part, bias, res):
            dist.reduce_scatter_tensor(part_rows, part, group=self.group)
            return (part_rows.float() + bias.float() + res.float()).to(self.dtype)

        w = self._layer_weights(0, self._resolver(0, transform, *stage(0)))
        for i in range(nl):
            nxt_w = None
            if i + 1 < nl:
                nxt_w = self._layer_weights(i + 1, self._resolver(i + 1, transform, *stage(i + 1)))
            x = norm.layernorm(h, w.ln1_w, w.ln1_b, cfg.layer_norm_eps)
            qkv = gemm.linear(gather(x), w.qkv_w, w.qkv_b)
            ctx = attn_ops.attention(qkv.view(B, L, qkv.shape[1]), cfg.num_attention_heads // n, batch.pad_left)
            h = reduce_add(gemm.linear(ctx.view(M, d // n), w.out_w), w.out_b, h)
            x = norm.layernorm(h, w.ln2_w, w.ln2_b, cfg.layer_norm_eps)
            f = gemm.linear(gather(x), w.fc1_w, w.fc1_b, act=cfg.activation_function)
            h = reduce_add(gemm.linear(f, w.fc2_w), w.fc2_b, h)
            if nxt_w is not None:
                w = nxt_w
        self._rows_local = (r * rows, (r + 1) * rows)
        return h
