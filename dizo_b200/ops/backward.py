"""Backward-pass ops for the first-order gamma search of DiZO.

The reference differentiates the loss with respect to the per-tensor gamma scalars by autograd
over a deep copy of the model (large_models/trainer.py:714-741, :805-830).  Only data gradients
are needed for that (no weight gradient is ever materialised: d loss / d alpha of a constrained
tensor W_eff = theta_0 + alpha (theta - theta_0) is the contraction <dY, X (theta - theta_0)^T>),
so the set is: the data-gradient GEMM dX = dY W with the weight read in place as the MN-major
tcgen05 operand (``csrc/gemm_sm100.cu``), the attention backward (``csrc/attn_bwd_sm100.cu``,
bound in :mod:`dizo_b200.ops.attention`) and the memory-bound pieces of ``csrc/bwd_kernels.cu``.
CPU tensors run the plain PyTorch statement of each op (the oracle of the GPU tests).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

ll = ctypes.c_longlong


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, mask: torch.Tensor | None = None,
                 residual: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """dx [M, in] = (dy [M, out] @ w [out, in]), zeroed where ``mask`` <= 0, plus ``residual``.

    ``mask`` is the saved ReLU output of the layer below (its backward fused into the epilogue);
    ``residual`` accumulates a second gradient stream."""
    if not dy.is_cuda:
        y = dy.float() @ w.float()
        if mask is not None:
            y = torch.where(mask.float() > 0, y, torch.zeros_like(y))
        if residual is not None:
            y = y + residual.float()
        return y.to(out_dtype or dy.dtype)
    assert dy.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and dy.dim() == 2 and w.dim() == 2
    M, K = dy.shape
    N = w.shape[1]
    assert w.shape[0] == K and dy.stride(1) == 1 and w.stride(1) == 1
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((M, N), dtype=out_dtype, device=dy.device)
    if mask is not None:
        assert mask.dtype == torch.bfloat16 and mask.shape == (M, N) and mask.stride(1) == 1
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
    rc = _lib.lib().dz_gemm_bf16_nn(
        _lib.ptr(dy), ll(dy.stride(0)), _lib.ptr(w), ll(w.stride(0)), _lib.ptr(out), ll(out.stride(0)),
        _lib.ptr(residual), ll(residual.stride(0) if residual is not None else 0),
        _lib.ptr(mask), ll(mask.stride(0) if mask is not None else 0), M, N, K,
        1 if out_dtype == torch.float32 else 0, _lib.ptr(_lib.err_word(dy.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm_bf16_nn")
    return out


def layernorm_backward(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5,
                       add: torch.Tensor | None = None) -> torch.Tensor:
    """Input gradient of ``layernorm(x, w, b)`` for output gradient ``dy`` (+ ``add``); [rows, d]."""
    d = x.shape[-1]
    if not dy.is_cuda:
        xf, g = x.float(), dy.float() * w.float()
        mean = xf.mean(-1, keepdim=True)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + eps)
        xh = (xf - mean) * rstd
        dx = rstd * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True))
        if add is not None:
            dx = dx + add.float()
        return dx.to(dy.dtype)
    dy2, x2 = dy.reshape(-1, d), x.reshape(-1, d)
    assert dy2.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert dy2.stride(1) == 1 and x2.stride(1) == 1
    out = torch.empty((x2.shape[0], d), dtype=torch.bfloat16, device=dy.device)
    a2 = add.reshape(-1, d) if add is not None else None
    rc = _lib.lib().dz_layernorm_bwd(
        _lib.ptr(dy2), ll(dy2.stride(0)), _lib.ptr(x2), ll(x2.stride(0)), _lib.ptr(w), _lib.ptr(a2),
        ll(a2.stride(0) if a2 is not None else 0), _lib.ptr(out), ll(d), ll(x2.shape[0]), d,
        ctypes.c_float(eps), _lib.stream_ptr())
    _lib.check(rc, "dz_layernorm_bwd")
    return out.view(x.shape)


def softmax_ce_backward_(logits: torch.Tensor, lse: torch.Tensor, targets: torch.Tensor,
                         coef: torch.Tensor) -> torch.Tensor:
    """In place: logits[r, j] <- coef[r] * ((j == targets[r]) - exp(logits[r, j] - lse[r])): the
    gradient of ``sum_r coef[r] * log_softmax(logits)[r, targets[r]]`` with respect to the logits."""
    R, V = logits.shape
    if not logits.is_cuda:
        p = torch.exp(logits.float() - lse.float().view(-1, 1))
        oh = torch.zeros_like(p)
        oh.scatter_(1, targets.long().view(-1, 1), 1.0)
        logits.copy_((coef.float().view(-1, 1) * (oh - p)).to(logits.dtype))
        return logits
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    assert lse.dtype == torch.float32 and coef.dtype == torch.float32 and targets.dtype == torch.int32
    for r0 in range(0, R, 65535):
        r1 = min(R, r0 + 65535)
        rc = _lib.lib().dz_softmax_ce_bwd(_lib.ptr(logits[r0:r1]), ll(logits.stride(0)), _lib.ptr(lse[r0:r1]),
                                          _lib.ptr(targets[r0:r1]), _lib.ptr(coef[r0:r1]), ll(r1 - r0), V,
                                          _lib.stream_ptr())
        _lib.check(rc, "dz_softmax_ce_bwd")
    return logits


def dot(a: torch.Tensor, b: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """scale * sum(a * b): a fp32 [rows, cols], b bf16 [rows, cols] (row strides free); fp32 [1].
    Fixed reduction order (bitwise reproducible)."""
    if not a.is_cuda:
        r = ((a.float() * b.float()).sum() * scale).reshape(1)
        if out is not None:
            out.copy_(r)
            return out
        return r
    assert a.dtype == torch.float32 and b.dtype == torch.bfloat16 and a.shape == b.shape and a.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    L = _lib.lib()
    partials = torch.empty(L.dz_dot_num_partials(), dtype=torch.float32, device=a.device)
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=a.device)
    rc = L.dz_dot_f32_bf16(_lib.ptr(a), ll(a.stride(0)), _lib.ptr(b), ll(b.stride(0)), ll(a.shape[0]),
                           a.shape[1], ctypes.c_float(scale), _lib.ptr(partials), _lib.ptr(out),
                           _lib.stream_ptr())
    _lib.check(rc, "dz_dot_f32_bf16")
    return out


def scatter_rows(src: torch.Tensor, idx: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """dst[idx[r], :] = src[r, :] (rows of ``idx`` distinct)."""
    if not src.is_cuda:
        dst[idx.long()] = src.to(dst.dtype)
        return dst
    assert src.dtype == torch.bfloat16 and dst.dtype == torch.bfloat16 and idx.dtype == torch.int32
    rc = _lib.lib().dz_scatter_rows(_lib.ptr(src), ll(src.stride(0)), _lib.ptr(idx), _lib.ptr(dst),
                                    ll(dst.stride(0)), ll(src.shape[0]), src.shape[1], ll(dst.shape[0]),
                                    _lib.stream_ptr())
    _lib.check(rc, "dz_scatter_rows")
    return dst


def diff(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a - b (bf16, contiguous, a multiple of 8 elements on the kernel path)."""
    if not a.is_cuda or a.numel() % 8 or a.dtype != torch.bfloat16:
        return (a.float() - b.float()).to(a.dtype)
    assert a.is_contiguous() and b.is_contiguous() and b.dtype == torch.bfloat16
    out = torch.empty_like(a)
    rc = _lib.lib().dz_diff_bf16(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), ll(a.numel()), _lib.stream_ptr())
    _lib.check(rc, "dz_diff_bf16")
    return out
