"""d loss / d alpha for the first-order gamma search of DiZO, on the framework's own kernels.

The reference (large_models/trainer.py:714-741, :805-830) deep-copies the model, rewrites every
constrained weight as ``theta_0 + (theta - theta_0) * gamma / ||theta - theta_0||`` under autograd
and calls ``loss.backward()``; only the gamma scalars receive a gradient.  Here the same quantity
is computed without autograd and without a weight gradient:

* forward: the ordinary kernel forward over the blended weights (the sweep stages
  ``theta_0 + alpha (theta - theta_0)`` per layer), keeping per layer the residual-stream inputs,
  the QKV activation, the attention context with its log-sum-exp, and the ReLU output;
* backward, layer by layer from the top: data-gradient GEMMs that read the weights in place
  (``dz_gemm_bf16_nn``, ReLU backward and gradient accumulation fused in the epilogue), the tcgen05
  attention backward, LayerNorm input gradients (pre- and post-LayerNorm blocks, ``project_out``);
* for a constrained weight W (k_proj / v_proj under full fine-tuning) with ``Y = X W_eff^T``:
  ``d loss / d alpha = <dY, X (theta - theta_0)^T>`` - one forward-shaped GEMM and a deterministic
  dot product, never an [out, in] weight gradient;
* for LoRA (the reference constrains the adapter factors, large_models/trainer.py:1154-1155) with
  ``W_eff = W + s B_eff A_eff``:  ``d/d alpha_A = s <dY B_eff, X (A - A_0)^T>`` and
  ``d/d alpha_B = s <dY, (X A_eff^T) (B - B_0)^T>`` - four rank-r GEMMs per adapted projection;
* over FSDP-sharded parameters every weight is assembled by the owners' pushes over NVLink
  (``FusedComm.fsdp_launch``): the forward GEMMs consume the pushed copy in the fused launch, the
  data-gradient GEMMs read the same staging slot after a peer barrier (second gather, in reverse
  layer order), and ``theta - theta_0`` of the k / v shards travels the same way.

* prefix rows (LoRA + prefix; the prefix tensors themselves are never constrained) enter as extra key
  columns of the attention backward: the tiled kernel differentiates the sequence keys with the forward's
  log-sum-exp, which already covers the prefix columns, and a small kernel adds their share of dQ.

Covered: full-parameter, LoRA and LoRA + prefix modes of every OPT size (pre- and post-LayerNorm, with or
without ``project_in/out``, ReLU), replicated or FSDP-sharded (full-parameter).  CPU tensors run the same
orchestration over the PyTorch statements of the ops, which is how the CPU suite checks it against autograd.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch

from ..ops import attention as attn_ops
from ..ops import backward as bw
from ..ops import gemm, norm
from .opt import _P, Batch, OPTModel, Transform, layer_prefix


def _is_fsdp(model) -> bool:
    return type(model).__name__ in ("FSDPOPTModel", "FSDPCompositionModel")


def supported(model: OPTModel) -> bool:
    cfg = model.config
    if cfg.activation_function != "relu":
        return False
    if _is_fsdp(model):
        return model.mode == "full"
    return model.mode in ("full", "lora", "lora+prefix") and type(model).hidden_states is OPTModel.hidden_states


# ---------------------------------------------------------------------------------- weight access
class _Replicated:
    """Whole weights on this rank: GEMMs read the (staged, blended) tensors directly."""

    def __init__(self, model: OPTModel):
        self.m = model
        self.numel = max(model.arena.group_numel(g) for g in model.arena.groups() if g >= 0)

    def stage(self, i: int, tr: Transform, key: int):
        m = self.m
        buf = m._staging_for(("gg", key), self.numel)
        shift = m._sweep_group(i, tr, buf)
        get = m._resolver(i, tr, buf, shift)
        w = m._layer_weights(i, get)
        w.get, w.i = get, i
        return w

    @staticmethod
    def _wb(w, which):
        return {"qkv": (w.qkv_w, w.qkv_b), "out": (w.out_w, w.out_b), "fc1": (w.fc1_w, w.fc1_b),
                "fc2": (w.fc2_w, w.fc2_b)}[which]

    def linear(self, w, which, x, act=None, residual=None):
        W, b = self._wb(w, which)
        return gemm.linear(x, W, b, act=act, residual=residual)

    def dgrad(self, w, which, dy, mask=None, residual=None):
        return bw.linear_dgrad(dy, self._wb(w, which)[0], mask=mask, residual=residual)

    def x_delta(self, w, names, x):
        """X (theta - theta_0)^T for the named constrained [d, d] weights of layer w.i: fp32 [M, d] each."""
        ar = self.m.arena
        return [gemm.linear(x, bw.diff(ar.view(n), ar.anchor_view(n)), out_dtype=torch.float32) for n in names]


class _FSDP:
    """Row-sharded weights: assembled per use by the owners' pushes into a staging slot."""

    def __init__(self, model):
        self.m = model
        self.fc = model.comm
        self.numel = max(model.arena.group_numel(g) for g in model.arena.groups() if g >= 0)

    def stage(self, i: int, tr: Transform, key: int):
        m = self.m
        buf = m._staging_for(("gg", key), self.numel)
        shift = m._sweep_group(i, tr, buf)
        get = m._resolver(i, tr, buf, shift)
        lp = layer_prefix(i)
        a = lp + "self_attn."
        w = SimpleNamespace(get=get, i=i)
        w.qkv_b = m._fused([get(a + "q_proj.bias"), get(a + "k_proj.bias"), get(a + "v_proj.bias")])
        w.out_b, w.fc1_b, w.fc2_b = get(a + "out_proj.bias"), get(lp + "fc1.bias"), get(lp + "fc2.bias")
        w.ln1_w, w.ln1_b = get(lp + "self_attn_layer_norm.weight"), get(lp + "self_attn_layer_norm.bias")
        w.ln2_w, w.ln2_b = get(lp + "final_layer_norm.weight"), get(lp + "final_layer_norm.bias")
        return w

    def linear(self, w, which, x, act=None, residual=None):
        segs, N, rps, period = self.m._push_spec(w.i, which, w.get, None)
        slot, _ = self.fc.fsdp_launch(push=dict(segments=segs, seed=0, coef=0.0))
        bias = {"qkv": w.qkv_b, "out": w.out_b, "fc1": w.fc1_b, "fc2": w.fc2_b}[which]
        _, out = self.fc.fsdp_launch(gemm=dict(slot=slot, N=N, x=x, bias=bias, act=act, residual=residual,
                                               rows_per_src=rps, src_period=period))
        return out

    def _gather(self, segs, N, K):
        """Full [N, K] tensor from every rank's row segments, readable by any kernel: the peers finish
        with the slot (barrier), every owner pushes its rows, the pushes have landed (barrier)."""
        self.fc.barrier()
        slot, _ = self.fc.fsdp_launch(push=dict(segments=segs, seed=0, coef=0.0))
        self.fc.barrier()
        return self.fc.fsdp_weight(slot, N, K)

    def dgrad(self, w, which, dy, mask=None, residual=None):
        segs, N, _, _ = self.m._push_spec(w.i, which, w.get, None)
        K = segs[0]["w_shard"].shape[1]
        return bw.linear_dgrad(dy, self._gather(segs, N, K), mask=mask, residual=residual)

    def x_delta(self, w, names, x):
        m, ar = self.m, self.m.arena
        d = m.config.hidden_size
        segs = []
        for j, n in enumerate(names):
            delta = bw.diff(ar.view(n).contiguous(), ar.anchor_view(n).contiguous())
            segs.append(dict(w_shard=delta, dst_row0=j * d + m.r * delta.shape[0]))
        t = gemm.linear(x, self._gather(segs, len(names) * d, d), out_dtype=torch.float32)
        return [t[:, j * d:(j + 1) * d] for j in range(len(names))]


class GammaGrad:
    """``loss_and_grad(batch, alpha)`` -> (loss fp32 [1], d loss / d alpha fp32 [n_slots])."""

    def __init__(self, model: OPTModel):
        assert supported(model), "configuration not covered by the kernel backward"
        self.model = model
        ar = model.arena
        self.slot_of = {n: ar.pieces[ar.index[n]].slot for n in ar.slot_names}
        self.n_slots = len(ar.slot_names)
        self.prov = _FSDP(model) if _is_fsdp(model) else _Replicated(model)

    # ------------------------------------------------------------------ helpers
    def _attention(self, qkv, B, L, pad_left, w):
        """context and the saved statistic (None on CPU: the CPU backward uses autograd)."""
        H = self.model.config.num_attention_heads
        pk, pv = getattr(w, "prefix_k", None), getattr(w, "prefix_v", None)
        if qkv.is_cuda:
            lse = torch.empty((B, H, L), dtype=torch.float32, device=qkv.device)
            ctx = attn_ops.attention(qkv.view(B, L, -1), H, pad_left, pk, pv, lse=lse)
            return ctx, lse
        return attn_ops.attention(qkv.view(B, L, -1), H, pad_left, pk, pv), None

    # ------------------------------------------------------------------ loss tail
    def _tail(self, h2: torch.Tensor, batch: Batch, gget):
        """loss and d loss / d h2 (zero outside ``batch.rows``)."""
        m, cfg = self.model, self.model.config
        pre = cfg.do_layer_norm_before
        proj = cfg.word_embed_proj_dim != cfg.hidden_size
        rows = batch.rows
        hr = norm.gather_rows(h2, rows)
        x = hr
        if pre:
            lnw, lnb = gget(_P + "final_layer_norm.weight"), gget(_P + "final_layer_norm.bias")
            x = norm.layernorm(hr, lnw, lnb, cfg.layer_norm_eps)
        if proj:
            pw = gget(_P + "project_out.weight")
            x = gemm.linear(x, pw)
        table = gget("lm_head.weight") if m.untied else gget(_P + "embed_tokens.weight")
        if batch.cand_ids is not None:
            # a handful of candidate columns: [rows, C] logits, differentiated on the spot
            tc = table[batch.cand_ids.long()].float()
            with torch.enable_grad():
                xf = x.float().requires_grad_(True)
                loss = torch.nn.functional.cross_entropy(xf @ tc.t(), batch.labels.long())
                (dx,) = torch.autograd.grad(loss, xf)
            dx = dx.to(x.dtype)
            loss = loss.detach().reshape(1)
        else:
            lp, lse = _logprobs_lse(x, table, batch.targets)
            # d loss / d lp over [rows] scalars
            with torch.enable_grad():
                lpr = lp.detach().requires_grad_(True)
                loss = _option_loss(lpr, batch)
                (coef,) = torch.autograd.grad(loss, lpr)
            loss = loss.detach().reshape(1)
            dx = torch.empty_like(x)
            step = 4096
            for r0 in range(0, x.shape[0], step):
                r1 = min(x.shape[0], r0 + step)
                logits = gemm.linear(x[r0:r1], table)                       # bf16 [chunk, V]
                bw.softmax_ce_backward_(logits, lse[r0:r1], batch.targets[r0:r1], coef[r0:r1].contiguous())
                dx[r0:r1] = bw.linear_dgrad(logits, table)
        if proj:
            dx = bw.linear_dgrad(dx, pw)
        dhr = bw.layernorm_backward(dx, hr, lnw, cfg.layer_norm_eps) if pre else dx
        dh = torch.zeros_like(h2)
        bw.scatter_rows(dhr, rows, dh)
        return loss, dh

    # ------------------------------------------------------------------ d loss / d alpha of one layer
    def _alpha_grads(self, w, x1, dqkv, grad):
        m, ar = self.model, self.model.arena
        d = m.config.hidden_size
        lp = layer_prefix(w.i) + "self_attn."
        if m.use_lora:
            s = m.lora_scaling
            for j, nm in ((0, "q_proj"), (2, "v_proj")):
                dy = dqkv[:, j * d:(j + 1) * d]
                na, nb = lp + nm + ".lora_A", lp + nm + ".lora_B"
                sa, sb = self.slot_of.get(na), self.slot_of.get(nb)
                if sa is not None:
                    u = bw.linear_dgrad(dy, w.get(nb))                                  # dY B_eff   [M, r]
                    t = gemm.linear(x1, bw.diff(ar.view(na), ar.anchor_view(na)), out_dtype=torch.float32)
                    bw.dot(t, u, scale=s, out=grad[sa:sa + 1])
                if sb is not None:
                    v = gemm.linear(x1, w.get(na))                                      # X A_eff^T  [M, r]
                    t = gemm.linear(v, bw.diff(ar.view(nb), ar.anchor_view(nb)), out_dtype=torch.float32)
                    bw.dot(t, dy, scale=s, out=grad[sb:sb + 1])
            return
        names, cols = [], []
        for j, nm in enumerate(("q_proj", "k_proj", "v_proj")):
            full = lp + nm + ".weight"
            if full in self.slot_of:
                names.append(full)
                cols.append(j)
        if not names:
            return
        for full, j, t in zip(names, cols, self.prov.x_delta(w, names, x1)):
            s = self.slot_of[full]
            bw.dot(t, dqkv[:, j * d:(j + 1) * d], out=grad[s:s + 1])

    # ------------------------------------------------------------------ main entry
    @torch.no_grad()
    def loss_and_grad(self, batch: Batch, alpha: torch.Tensor):
        m, cfg, P = self.model, self.model.config, self.prov
        ar = m.arena
        nl, d = cfg.num_hidden_layers, cfg.hidden_size
        eps = cfg.layer_norm_eps
        pre = cfg.do_layer_norm_before
        B, L = batch.input_ids.shape
        M = B * L
        tr = Transform(seed=0, coef=0.0, alpha=alpha)
        # ---- forward with saves
        g_staged = m._staging_for("globals", ar.group_numel(-1)) if -1 in ar.groups() else None
        g_shift = m._sweep_group(-1, tr, g_staged) if g_staged is not None else 0
        gget = m._resolver(-1, tr, g_staged, g_shift)
        m._gget = gget
        tok, pos = gget(_P + "embed_tokens.weight"), gget(_P + "embed_positions.weight")
        if cfg.word_embed_proj_dim != d:
            e = gemm.linear(norm.embed(batch.input_ids, None, tok, None), gget(_P + "project_in.weight"))
            h = norm.add_rows(e, batch.positions.reshape(-1), pos).view(M, d)
        else:
            h = norm.embed(batch.input_ids, batch.positions, tok, pos).view(M, d)
        saved = []
        for i in range(nl):
            w = P.stage(i, tr, 0)
            x1 = norm.layernorm(h, w.ln1_w, w.ln1_b, eps) if pre else h
            qkv = P.linear(w, "qkv", x1)
            ctx, lse = self._attention(qkv, B, L, batch.pad_left, w)
            r1 = P.linear(w, "out", ctx.view(M, d), residual=h)
            h_mid = r1 if pre else norm.layernorm(r1, w.ln1_w, w.ln1_b, eps)
            x2 = norm.layernorm(h_mid, w.ln2_w, w.ln2_b, eps) if pre else h_mid
            f = P.linear(w, "fc1", x2, act="relu")
            r2 = P.linear(w, "fc2", f, residual=h_mid)
            h_out = r2 if pre else norm.layernorm(r2, w.ln2_w, w.ln2_b, eps)
            saved.append((h, x1, qkv, ctx, lse, r1, h_mid, f, r2))
            h = h_out
        loss, dh = self._tail(h, batch, gget)
        # ---- backward
        grad = torch.zeros(max(self.n_slots, 1), dtype=torch.float32, device=h.device)
        H = cfg.num_attention_heads
        for i in reversed(range(nl)):
            h_in, x1, qkv, ctx, lse, r1, h_mid, f, r2 = saved.pop()
            w = P.stage(i, tr, 1)
            if pre:
                # h_out = h_mid + fc2(relu(fc1(LN2(h_mid))));  h_mid = h_in + out_proj(attn(qkv(LN1(h_in))))
                df = P.dgrad(w, "fc2", dh, mask=f)                           # ReLU backward fused
                dx2 = P.dgrad(w, "fc1", df)
                del df
                dh_mid = bw.layernorm_backward(dx2, h_mid, w.ln2_w, eps, add=dh)
                dr1 = dh_mid
            else:
                # h_out = LN2(h_mid + fc2(relu(fc1(h_mid))));  h_mid = LN1(h_in + out_proj(attn(qkv(h_in))))
                dr2 = bw.layernorm_backward(dh, r2, w.ln2_w, eps)
                df = P.dgrad(w, "fc2", dr2, mask=f)
                dh_mid = P.dgrad(w, "fc1", df, residual=dr2)
                del df
                dr1 = bw.layernorm_backward(dh_mid, r1, w.ln1_w, eps)
            dctx = P.dgrad(w, "out", dr1)
            pk, pv = getattr(w, "prefix_k", None), getattr(w, "prefix_v", None)
            if qkv.is_cuda:
                dqkv = attn_ops.attention_backward(qkv.view(B, L, 3 * d), ctx.view(B, L, d), dctx.view(B, L, d),
                                                   lse, H, batch.pad_left, prefix_k=pk, prefix_v=pv).view(M, 3 * d)
            else:
                dqkv = attn_ops.attention_backward_reference(qkv.view(B, L, 3 * d), dctx.view(B, L, d), H,
                                                             batch.pad_left, prefix_k=pk, prefix_v=pv).view(M, 3 * d)
            self._alpha_grads(w, x1, dqkv, grad)
            if i > 0:                     # nothing below the first block depends on a constrained tensor
                if pre:
                    dx1 = P.dgrad(w, "qkv", dqkv)
                    dh = bw.layernorm_backward(dx1, h_in, w.ln1_w, eps, add=dr1)
                else:
                    dh = P.dgrad(w, "qkv", dqkv, residual=dr1)
        return loss, grad[:self.n_slots]


def _logprobs_lse(x: torch.Tensor, table: torch.Tensor, targets: torch.Tensor):
    """(log p(target), natural-log log-sum-exp) per row."""
    if not x.is_cuda:
        logits = x.float() @ table.float().t()
        lse = torch.logsumexp(logits, dim=-1)
        return logits.gather(1, targets.long().view(-1, 1)).squeeze(1) - lse, lse
    import ctypes
    from ..ops import _lib
    L = _lib.lib()
    R, K = x.shape
    V = table.shape[0]
    nt = L.dz_gemm_lse_num_tiles(V)
    f = dict(dtype=torch.float32, device=x.device)
    pm, ps = torch.empty((R, nt), **f), torch.empty((R, nt), **f)
    tg, lp, lse = torch.empty(R, **f), torch.empty(R, **f), torch.empty(R, **f)
    ll = ctypes.c_longlong
    rc = L.dz_gemm_bf16_tn_lse(_lib.ptr(x), ll(x.stride(0)), _lib.ptr(table), ll(table.stride(0)),
                               _lib.ptr(targets), _lib.ptr(pm), _lib.ptr(ps), _lib.ptr(tg), R, V, K,
                               ctypes.c_float(1.0), _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm_bf16_tn_lse")
    rc = L.dz_lse_combine(_lib.ptr(pm), _lib.ptr(ps), _lib.ptr(tg), nt, R, _lib.ptr(lp), _lib.ptr(lse),
                          _lib.stream_ptr())
    _lib.check(rc, "dz_lse_combine")
    return lp, lse


def _option_loss(lp: torch.Tensor, batch: Batch) -> torch.Tensor:
    """The loss of ``ops.loss.option_ce`` as a differentiable function of the [rows] log-probs."""
    if not batch.classification:
        return -lp.mean()
    ss = batch.seq_start.tolist()
    seq_lp = torch.stack([lp[ss[i]:ss[i + 1]].mean() for i in range(len(ss) - 1)])
    es = batch.ex_start.tolist()
    labels = batch.labels.tolist()
    losses = [torch.logsumexp(seq_lp[es[e]:es[e + 1]], 0) - seq_lp[es[e] + labels[e]]
              for e in range(len(es) - 1)]
    return torch.stack(losses).mean()
