"""LayerNorm, OPT embedding (token + learned position), row gather/add.

CUDA tensors run ``csrc/norm_embed.cu``; CPU tensors run the PyTorch statement.
Reference call sites: large_models/ht_opt.py:114-124, :330, :354, :639, :657, :726.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

ll = ctypes.c_longlong


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float = 1e-5,
              out: torch.Tensor | None = None) -> torch.Tensor:
    if not x.is_cuda:
        y = F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, d)
    rc = _lib.lib().dz_layernorm(_lib.ptr(x2), ll(x2.stride(0)), _lib.ptr(w), _lib.ptr(b),
                                 _lib.ptr(o2), ll(o2.stride(0)), ll(x2.shape[0]), d,
                                 ctypes.c_float(eps), _lib.stream_ptr())
    _lib.check(rc, "dz_layernorm")
    return out.reshape(x.shape)


def opt_positions(attention_mask: torch.Tensor, offset: int = 2) -> torch.Tensor:
    """OPT's learned-position indices: cumsum(mask) * mask - 1 + offset (int32)."""
    m = attention_mask.long()
    return ((torch.cumsum(m, dim=1) * m) - 1 + offset).to(torch.int32)


def embed(ids: torch.Tensor, positions: torch.Tensor | None, tok: torch.Tensor,
          pos: torch.Tensor | None) -> torch.Tensor:
    """h = tok[ids] (+ pos[positions]).  ids/positions int32 [B, L]; returns [B, L, d]."""
    B, L = ids.shape
    d = tok.shape[1]
    if not ids.is_cuda:
        h = tok[ids.long()].float()
        if pos is not None:
            h = h + pos[positions.long()].float()
        return h.to(tok.dtype)
    assert ids.dtype == torch.int32 and tok.dtype == torch.bfloat16
    out = torch.empty((B, L, d), dtype=torch.bfloat16, device=tok.device)
    rc = _lib.lib().dz_embed(_lib.ptr(ids), _lib.ptr(positions), _lib.ptr(tok), ll(tok.stride(0)),
                             _lib.ptr(pos), ll(pos.stride(0) if pos is not None else 0),
                             _lib.ptr(out), ll(d), ll(B * L), d, tok.shape[0],
                             pos.shape[0] if pos is not None else 0, _lib.stream_ptr())
    _lib.check(rc, "dz_embed")
    return out


def add_rows(a: torch.Tensor, idx: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """a[m] + table[idx[m]] (used when positions are added after ``project_in``)."""
    d = a.shape[-1]
    a2 = a.reshape(-1, d)
    if not a.is_cuda:
        return (a2.float() + table[idx.reshape(-1).long()].float()).to(a.dtype).reshape(a.shape)
    out = torch.empty_like(a2)
    rc = _lib.lib().dz_add_rows(_lib.ptr(a2), ll(a2.stride(0)), _lib.ptr(idx), _lib.ptr(table),
                                ll(table.stride(0)), _lib.ptr(out), ll(out.stride(0)),
                                ll(a2.shape[0]), d, table.shape[0], _lib.stream_ptr())
    _lib.check(rc, "dz_add_rows")
    return out.reshape(a.shape)


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """src[rows] for a 2-D bf16 ``src`` and int32 ``rows``."""
    if not src.is_cuda:
        return src[rows.long()]
    assert src.dim() == 2 and rows.dtype == torch.int32
    n = rows.numel()
    out = torch.empty((n, src.shape[1]), dtype=src.dtype, device=src.device)
    if n == 0:
        return out
    rc = _lib.lib().dz_gather_rows(_lib.ptr(src), ll(src.stride(0)), _lib.ptr(rows), _lib.ptr(out),
                                   ll(out.stride(0)), ll(n), src.shape[1], ll(src.shape[0]),
                                   _lib.stream_ptr())
    _lib.check(rc, "dz_gather_rows")
    return out
