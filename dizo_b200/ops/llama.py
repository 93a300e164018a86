"""RMSNorm, rotary position embedding (with grouped-query head expansion) and the SwiGLU gate.

CUDA tensors run ``csrc/llama_kernels.cu``; CPU tensors run the PyTorch statement.  These are the
pieces of a LLaMA-family block that the OPT kernels do not cover; the reference reaches such models
through Hugging Face modules (large_models/run.py:167-181, :242-265; large_models/prefix.py:112-125).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

ll = ctypes.c_longlong
_tables: dict = {}


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last dimension."""
    if not x.is_cuda:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    out = torch.empty_like(x2)
    rc = _lib.lib().dz_rmsnorm(_lib.ptr(x2), ll(x2.stride(0)), _lib.ptr(w), _lib.ptr(out), ll(out.stride(0)),
                               ll(x2.shape[0]), d, ctypes.c_float(eps), _lib.stream_ptr())
    _lib.check(rc, "dz_rmsnorm")
    return out.reshape(x.shape)


def rope_table(n_pos: int, hd: int, theta: float, device) -> torch.Tensor:
    """(cos, sin) of position * theta^(-2j/hd): fp32 [n_pos, hd/2, 2], built once per (size, device) in
    float64 so that large angles keep full precision."""
    device = torch.device(device)
    key = (hd, float(theta), str(device))
    t = _tables.get(key)
    if t is None or t.shape[0] < n_pos:
        n = max(n_pos, 2048 if t is None else 2 * t.shape[0])
        inv = theta ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd)
        ang = torch.arange(n, dtype=torch.float64)[:, None] * inv[None, :]
        t = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()
        _tables[key] = t
    return t


def rope_qkv_reference(x: torch.Tensor, L: int, pos0: int, H: int, Hkv: int, hd: int, theta: float) -> torch.Tensor:
    """fp32 statement of :func:`rope_qkv`."""
    M = x.shape[0]
    xf = x.float()
    q = xf[:, :H * hd].view(M, H, hd)
    k = xf[:, H * hd:(H + Hkv) * hd].view(M, Hkv, hd)
    v = xf[:, (H + Hkv) * hd:(H + 2 * Hkv) * hd].view(M, Hkv, hd)
    pos = pos0 + torch.arange(M, device=x.device) % L
    cs = rope_table(int(pos.max()) + 1, hd, theta, x.device)[pos]            # [M, hd/2, 2]
    cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]

    def rot(t):
        a, b = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    rep = H // Hkv
    k, v = rot(k).repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    return torch.cat([rot(q).reshape(M, -1), k.reshape(M, -1), v.reshape(M, -1)], dim=-1).to(x.dtype)


def rope_qkv(x: torch.Tensor, L: int, pos0: int, H: int, Hkv: int, hd: int, theta: float) -> torch.Tensor:
    """x [M, (H + 2 Hkv) hd] = q | k | v of a fused projection -> [M, 3 H hd]: q and k rotated by the row's
    position ``pos0 + m % L`` (pairs (j, j + hd/2), the Hugging Face convention), k and v heads repeated
    ``H / Hkv`` times so that the attention kernels see ordinary multi-head operands."""
    if not x.is_cuda:
        return rope_qkv_reference(x, L, pos0, H, Hkv, hd, theta)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] == (H + 2 * Hkv) * hd
    M = x.shape[0]
    cs = rope_table(pos0 + L, hd, theta, x.device)
    out = torch.empty((M, 3 * H * hd), dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().dz_rope_qkv(_lib.ptr(x), ll(x.stride(0)), _lib.ptr(out), ll(out.stride(0)), _lib.ptr(cs),
                                ll(M), L, pos0, cs.shape[0], H, Hkv, hd, _lib.stream_ptr())
    _lib.check(rc, "dz_rope_qkv")
    return out


def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    """gu [M, 2F] = gate | up  ->  silu(gate) * up  [M, F]."""
    F = gu.shape[-1] // 2
    if not gu.is_cuda:
        g, u = gu[..., :F].float(), gu[..., F:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)
    assert gu.dtype == torch.bfloat16 and gu.stride(-1) == 1
    g2 = gu.reshape(-1, 2 * F)
    out = torch.empty((g2.shape[0], F), dtype=torch.bfloat16, device=gu.device)
    rc = _lib.lib().dz_silu_mul(_lib.ptr(g2), ll(g2.stride(0)), _lib.ptr(out), ll(out.stride(0)),
                                ll(g2.shape[0]), F, _lib.stream_ptr())
    _lib.check(rc, "dz_silu_mul")
    return out.reshape(*gu.shape[:-1], F)
