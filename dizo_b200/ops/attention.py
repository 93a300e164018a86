"""Causal attention over a fused QKV activation, with left padding and prefix K/V rows.

CUDA: the tcgen05 kernel of ``csrc/attn_sm100.cu``.  CPU (and the oracle for the GPU
tests): a plain PyTorch statement with an explicit mask.  Semantics follow the
reference's eager OPT attention with its additive causal + padding mask
(large_models/ht_opt.py:209-272) and the prefix hook (large_models/prefix.py:23-55).
"""
from __future__ import annotations

import ctypes
import math

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
              scale: float | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """qkv [B, L, 3d] bf16 (row stride may exceed 3d) -> context [B, L, d] bf16."""
    if not qkv.is_cuda:
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
    rc = _lib.lib().dz_attn_fwd(
        _lib.ptr(qkv), ctypes.c_longlong(qkv.stride(1)), 0, d, 2 * d,
        _lib.ptr(out), ctypes.c_longlong(out.stride(1)), _lib.ptr(pad_left),
        _lib.ptr(prefix_k), _lib.ptr(prefix_v), ctypes.c_longlong(ldp), npre,
        B, L, n_heads, hd, ctypes.c_float(scale), _lib.ptr(_lib.err_word(qkv.device)),
        _lib.stream_ptr())
    _lib.check(rc, "dz_attn_fwd")
    return out


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
