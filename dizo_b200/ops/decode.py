"""Generation-time ops: single-token attention over a KV cache, token sampling.

CUDA tensors run ``csrc/decode_kernels.cu``; CPU tensors the PyTorch statements
(``attention.decode_attention_reference`` and ``sample_reference`` below)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .attention import decode_attention_reference

ll = ctypes.c_longlong


def decode_attention(q, k_cache, v_cache, kv_len, n_heads, pad_left=None, prefix_k=None, prefix_v=None,
                     scale=None):
    """q [B, d] against k_cache / v_cache [B, Lmax, d] (first ``kv_len`` rows valid) -> [B, d]."""
    if not q.is_cuda:
        return decode_attention_reference(q, k_cache, v_cache, kv_len, n_heads, pad_left, prefix_k, prefix_v, scale)
    B, d = q.shape
    hd = d // n_heads
    scale = scale if scale is not None else hd ** -0.5
    out = torch.empty((B, d), dtype=torch.bfloat16, device=q.device)
    npre = prefix_k.shape[0] if prefix_k is not None else 0
    assert q.stride(-1) == 1 and k_cache.stride(-1) == 1 and v_cache.stride(-1) == 1
    assert k_cache.stride() == v_cache.stride()
    rc = _lib.lib().dz_decode_attn(
        _lib.ptr(q), ll(q.stride(0)), _lib.ptr(k_cache), _lib.ptr(v_cache), ll(k_cache.stride(0)),
        ll(k_cache.stride(1)), _lib.ptr(prefix_k), _lib.ptr(prefix_v),
        ll(prefix_k.stride(0) if prefix_k is not None else 0), npre, _lib.ptr(pad_left), int(kv_len), B,
        n_heads, hd, ctypes.c_float(scale), _lib.ptr(out), ll(out.stride(0)), _lib.stream_ptr())
    _lib.check(rc, "dz_decode_attn")
    return out


def sample_reference(logits, temperature=1.0, top_k=None, top_p=None, do_sample=True, generator=None):
    from ..models.generate import filter_logits
    if not do_sample:
        return logits.argmax(dim=-1)
    probs = torch.softmax(filter_logits(logits.float(), temperature, top_k, top_p), dim=-1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(1)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None,
           top_p: float | None = None, do_sample: bool = True, seed: int = 0, offset: int = 0) -> torch.Tensor:
    """One token id per row of fp32 ``logits`` [B, V] (int64).  ``offset`` distinguishes the
    draws of successive decoding steps under one ``seed``."""
    if not logits.is_cuda:
        g = torch.Generator().manual_seed((seed * 1000003 + offset) & (2 ** 63 - 1))
        return sample_reference(logits, temperature, top_k, top_p, do_sample, g)
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    rc = _lib.lib().dz_sample_topk_topp(
        _lib.ptr(logits), ll(logits.stride(0)), B, V, ctypes.c_float(temperature or 1.0), int(top_k or 0),
        ctypes.c_float(top_p if top_p is not None else 1.0), int(do_sample), ctypes.c_uint64(seed),
        ctypes.c_uint64(offset), _lib.ptr(out), _lib.stream_ptr())
    _lib.check(rc, "dz_sample_topk_topp")
    return out.long()
