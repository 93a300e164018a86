"""Causal attention over a fused QKV activation, with left padding and prefix K/V rows.

CUDA: the tcgen05 kernel of ``csrc/attn_sm100.cu``.  CPU (and the oracle for the GPU
tests): a plain PyTorch statement with an explicit mask.  Semantics follow the
reference's eager OPT attention with its additive causal + padding mask
(large_models/ht_opt.py:209-272) and the prefix hook (large_models/prefix.py:23-55).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def attention_reference(qkv: torch.Tensor, n_heads: int, pad_left: torch.Tensor | None = None,
                        prefix_k: torch.Tensor | None = None, prefix_v: torch.Tensor | None = None,
                        scale: float | None = None) -> torch.Tensor:
    """qkv [B, L, 3d] -> context [B, L, d]; fp32 math; returns qkv.dtype."""
    B, L, d3 = qkv.shape
    d = d3 // 3
    hd = d // n_heads
    scale = scale if scale is not None else hd ** -0.5
    q, k, v = qkv.float().split(d, dim=-1)
    q = q.view(B, L, n_heads, hd).transpose(1, 2)
    k = k.view(B, L, n_heads, hd).transpose(1, 2)
    v = v.view(B, L, n_heads, hd).transpose(1, 2)
    idx = torch.arange(L, device=qkv.device)
    vis = idx[None, :] <= idx[:, None]                       # [L(q), L(k)]
    vis = vis[None].expand(B, L, L).clone()
    if pad_left is not None:
        pl = pad_left.to(qkv.device).view(B, 1, 1)
        keep = (idx.view(1, 1, L) >= pl) | (idx.view(1, 1, L) == idx.view(1, L, 1))
        vis &= keep
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    s = s.masked_fill(~vis[:, None], float("-inf"))
    if prefix_k is not None:
        P = prefix_k.shape[0]
        pk = prefix_k.float().view(P, n_heads, hd).permute(1, 0, 2)   # [H, P, hd]
        pv = prefix_v.float().view(P, n_heads, hd).permute(1, 0, 2)
        sp = torch.einsum("bhqd,hkd->bhqk", q, pk) * scale
        s = torch.cat([sp, s], dim=-1)
        v_all = torch.cat([pv[None].expand(B, -1, -1, -1), v], dim=2)
    else:
        v_all = v
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqk,bhkd->bhqd", p, v_all)
    return o.transpose(1, 2).reshape(B, L, d).to(qkv.dtype)


def attention(qkv: torch.Tensor, n_heads: int, pad_left: torch.Tensor | None = None,
              prefix_k: torch.Tensor | None = None, prefix_v: torch.Tensor | None = None,
              scale: float | None = None, out: torch.Tensor | None = None,
              lse: torch.Tensor | None = None) -> torch.Tensor:
    """qkv [B, L, 3d] bf16 (row stride may exceed 3d) -> context [B, L, d] bf16.

    ``lse``: optional fp32 [B, H, L] that receives every query row's log-sum-exp (log2 domain of
    the scaled scores), the statistic :func:`attention_backward` needs."""
    if not qkv.is_cuda:
        assert lse is None, "the CPU statement differentiates through autograd instead"
        return attention_reference(qkv, n_heads, pad_left, prefix_k, prefix_v, scale)
    assert qkv.dtype == torch.bfloat16 and qkv.dim() == 3 and qkv.stride(-1) == 1
    B, L, d3 = qkv.shape
    d = d3 // 3
    hd = d // n_heads
    assert qkv.stride(0) == L * qkv.stride(1), "batch rows must be contiguous"
    scale = scale if scale is not None else hd ** -0.5
    if out is None:
        out = torch.empty((B, L, d), dtype=torch.bfloat16, device=qkv.device)
    npre = 0
    ldp = 0
    if prefix_k is not None:
        assert prefix_k.dtype == torch.bfloat16 and prefix_k.stride(-1) == 1
        npre = prefix_k.shape[0]
        ldp = prefix_k.stride(0)
        assert prefix_v.stride(0) == ldp
    if pad_left is not None:
        assert pad_left.dtype == torch.int32 and pad_left.is_cuda
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.is_contiguous() and lse.shape == (B, n_heads, L)
    rc = _lib.lib().dz_attn_fwd_lse(
        _lib.ptr(qkv), ctypes.c_longlong(qkv.stride(1)), 0, d, 2 * d,
        _lib.ptr(out), ctypes.c_longlong(out.stride(1)), _lib.ptr(pad_left),
        _lib.ptr(prefix_k), _lib.ptr(prefix_v), ctypes.c_longlong(ldp), npre,
        B, L, n_heads, hd, ctypes.c_float(scale), _lib.ptr(lse), _lib.ptr(_lib.err_word(qkv.device)),
        _lib.stream_ptr())
    _lib.check(rc, "dz_attn_fwd_lse")
    return out


def attention_backward_reference(qkv: torch.Tensor, dout: torch.Tensor, n_heads: int,
                                 pad_left: torch.Tensor | None = None, scale: float | None = None,
                                 prefix_k: torch.Tensor | None = None, prefix_v: torch.Tensor | None = None,
                                 d_prefix: tuple | None = None) -> torch.Tensor:
    """d loss / d qkv for d loss / d context = ``dout``: autograd through the fp32 statement.  ``d_prefix``:
    optional pair of fp32 [P, d] tensors that receive the gradients of the prefix keys / values."""
    with torch.enable_grad():
        x = qkv.detach().float().requires_grad_(True)
        leaves = [x]
        pk = pv = None
        if prefix_k is not None:
            pk, pv = prefix_k.detach().float().requires_grad_(True), prefix_v.detach().float().requires_grad_(True)
            leaves += [pk, pv]
        o = attention_reference(x, n_heads, pad_left, pk, pv, scale)
        grads = torch.autograd.grad(o, leaves, dout.float())
    if d_prefix is not None:
        d_prefix[0].copy_(grads[1])
        d_prefix[1].copy_(grads[2])
    return grads[0].to(qkv.dtype)


def attention_backward(qkv: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor,
                       n_heads: int, pad_left: torch.Tensor | None = None, scale: float | None = None,
                       dqkv: torch.Tensor | None = None, prefix_k: torch.Tensor | None = None,
                       prefix_v: torch.Tensor | None = None, d_prefix: tuple | None = None) -> torch.Tensor:
    """Gradient of :func:`attention`: qkv [B, L, 3d], its context ``out`` and ``dout`` [B, L, d] (bf16),
    ``lse`` from the forward -> dqkv [B, L, 3d] bf16 (dQ | dK | dV).  With prefix rows (``prefix_k/v``
    [P, d], the ones the forward saw) their share of dQ is added, and ``d_prefix`` - a pair of zeroed fp32
    [P, d] tensors - receives the gradients of the prefix keys and values when given.

    CUDA: the two tcgen05 passes of ``csrc/attn_bwd_sm100.cu`` over the sequence keys; because the
    forward's log-sum-exp and D = rowsum(dO * O) cover the prefix columns too, those separate exactly and a
    small kernel (``attn_prefix_bwd_kernel``) handles them.  Replaces the autograd pass over the
    reference's eager attention (large_models/ht_opt.py:209-272) in the first-order gamma search
    (large_models/trainer.py:714-741)."""
    if not qkv.is_cuda:
        return attention_backward_reference(qkv, dout, n_heads, pad_left, scale, prefix_k, prefix_v, d_prefix)
    B, L, d3 = qkv.shape
    d = d3 // 3
    hd = d // n_heads
    scale = scale if scale is not None else hd ** -0.5
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and dout.dtype == torch.bfloat16
    assert qkv.stride(-1) == 1 and qkv.stride(0) == L * qkv.stride(1)
    assert out.is_contiguous() and dout.is_contiguous() and out.shape == (B, L, d) == dout.shape
    assert lse.dtype == torch.float32 and lse.is_contiguous() and lse.shape == (B, n_heads, L)
    if dqkv is None:
        dqkv = torch.empty((B, L, 3 * d), dtype=torch.bfloat16, device=qkv.device)
    assert dqkv.stride(-1) == 1 and dqkv.stride(0) == L * dqkv.stride(1)
    dsum = torch.empty((B, n_heads, L), dtype=torch.float32, device=qkv.device)
    ll = ctypes.c_longlong
    rc = _lib.lib().dz_attn_bwd(
        _lib.ptr(qkv), ll(qkv.stride(1)), 0, d, 2 * d,
        _lib.ptr(out), _lib.ptr(dout), ll(d), _lib.ptr(lse), _lib.ptr(dsum),
        _lib.ptr(dqkv), ll(dqkv.stride(1)), _lib.ptr(pad_left),
        B, L, n_heads, hd, ctypes.c_float(scale), _lib.ptr(_lib.err_word(qkv.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_attn_bwd")
    if prefix_k is not None:
        assert prefix_k.dtype == torch.bfloat16 and prefix_k.stride(-1) == 1 and prefix_v.stride(0) == prefix_k.stride(0)
        dpk = dpv = None
        if d_prefix is not None:
            dpk, dpv = d_prefix
            assert dpk.dtype == torch.float32 and dpk.is_contiguous() and dpk.shape == (prefix_k.shape[0], d)
            assert dpv.dtype == torch.float32 and dpv.is_contiguous() and dpv.shape == dpk.shape
        rc = _lib.lib().dz_attn_prefix_bwd(
            _lib.ptr(qkv), ll(qkv.stride(1)), _lib.ptr(dout), ll(d), _lib.ptr(prefix_k), _lib.ptr(prefix_v),
            ll(prefix_k.stride(0)), prefix_k.shape[0], _lib.ptr(lse), _lib.ptr(dsum), _lib.ptr(dqkv),
            ll(dqkv.stride(1)), _lib.ptr(dpk), _lib.ptr(dpv), ll(d), B, L, n_heads, hd, ctypes.c_float(scale),
            _lib.stream_ptr())
        _lib.check(rc, "dz_attn_prefix_bwd")
    return dqkv


def decode_attention_reference(q, k_cache, v_cache, kv_len, n_heads, pad_left=None,
                               prefix_k=None, prefix_v=None, scale=None):
    """One new token per sequence against a KV cache.

    q [B, d]; k_cache, v_cache [B, Lmax, d]; kv_len = number of valid cache rows
    (the new token's K/V already written at kv_len-1)."""
    B, d = q.shape
    hd = d // n_heads
    scale = scale if scale is not None else hd ** -0.5
    qf = q.float().view(B, n_heads, 1, hd)
    k = k_cache[:, :kv_len].float().view(B, kv_len, n_heads, hd).transpose(1, 2)
    v = v_cache[:, :kv_len].float().view(B, kv_len, n_heads, hd).transpose(1, 2)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, k) * scale
    if pad_left is not None:
        idx = torch.arange(kv_len, device=q.device).view(1, 1, 1, kv_len)
        s = s.masked_fill(idx < pad_left.view(B, 1, 1, 1), float("-inf"))
    if prefix_k is not None:
        P = prefix_k.shape[0]
        pk = prefix_k.float().view(P, n_heads, hd).permute(1, 0, 2)
        pv = prefix_v.float().view(P, n_heads, hd).permute(1, 0, 2)
        sp = torch.einsum("bhqd,hkd->bhqk", qf, pk) * scale
        s = torch.cat([sp, s], dim=-1)
        v = torch.cat([pv[None].expand(B, -1, -1, -1), v], dim=2)
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqk,bhkd->bhqd", p, v)
    return o.reshape(B, d).to(q.dtype)
