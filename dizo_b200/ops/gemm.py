"""``linear``: out = act((x @ w.T + bias) * scale) + residual.

CUDA tensors run the tcgen05/TMEM kernel in ``csrc/gemm_sm100.cu``; CPU tensors run the
plain PyTorch statement of the same op (the oracle the GPU tests compare against).
Replaces the ``nn.Linear`` calls of the reference's OPT blocks
(large_models/ht_opt.py:178-197, :274, :356-359).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.nn.functional as F

from . import _lib

ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2}
# 0 = choose per shape, 1 = one-SM kernel, 2 = two-SM (cta_group::2) kernel
_VARIANT = int(os.environ.get("DIZO_GEMM_VARIANT", "0"))
# 0: SwiGLU as a GEMM followed by the stand-alone silu_mul kernel (for A/B measurements)
_SWIGLU_FUSED = os.environ.get("DIZO_SWIGLU_FUSED", "1") != "0"
_ROPE_FUSED = os.environ.get("DIZO_ROPE_FUSED", "1") != "0"


def linear_reference(x, w, bias=None, act=None, residual=None, scale: float = 1.0,
                     out_dtype=None):
    """fp32 statement of the op (any device)."""
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if scale != 1.0:
        y = y * scale
    if act == "relu":
        y = torch.relu(y)
    elif act == "gelu":
        y = F.gelu(y)
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ gate.T) * (x @ up.T) for ``w_gate_up`` [2F, K] = gate rows | up rows -> [..., F].

    Where the two-SM kernel runs, each 256-column accumulator tile holds 128 gate columns beside the matching
    128 up columns (the two CTAs of a pair load their halves of the W tile from the two sections) and the
    epilogue writes the product: the [M, 2F] intermediate never reaches memory.  Other shapes go through
    :func:`linear` and the stand-alone ``silu_mul`` kernel."""
    from . import llama as llama_ops
    N, K = w_gate_up.shape
    F = N // 2
    x2 = x.reshape(-1, K)
    M = x2.shape[0]
    fused = (_SWIGLU_FUSED and x.is_cuda and _VARIANT in (0, 2) and N % 256 == 0 and M >= 256
             and ((M + 255) // 256) * (N // 256) >= 48)
    if not fused:
        return llama_ops.silu_mul(linear(x, w_gate_up))
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.stride(-1) == 1
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().dz_gemm2_bf16_tn(
        _lib.ptr(x2), ctypes.c_longlong(x2.stride(0)), _lib.ptr(w_gate_up), ctypes.c_longlong(w_gate_up.stride(0)),
        _lib.ptr(out), ctypes.c_longlong(F), None, None, ctypes.c_longlong(0),
        M, N, K, 3, 0, ctypes.c_float(1.0), _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm2_bf16_tn")
    return out.reshape(*x.shape[:-1], F)


def linear_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, L: int, pos0: int, H: int, Hkv: int, hd: int,
                    theta: float) -> torch.Tensor:
    """Fused q | k | v projection followed by the rotary embedding (and the grouped-query head expansion):
    x [M, K], w_qkv [(H + 2 Hkv) hd, K] -> [M, 3 H hd], row m at position ``pos0 + m % L``.

    With head dim 128 and even head counts the rotation runs in the two-SM GEMM's epilogue (a 256-column
    accumulator tile holds two whole heads, columns j and j + 64 of a head pair up): the raw projection never
    reaches memory.  Other shapes go through :func:`linear` and the stand-alone rotary kernel."""
    from . import llama as llama_ops
    N, K = w_qkv.shape
    x2 = x.reshape(-1, K)
    M = x2.shape[0]
    fused = (_ROPE_FUSED and x.is_cuda and _VARIANT in (0, 2) and hd == 128 and H % 2 == 0 and Hkv % 2 == 0
             and M >= 256 and ((M + 255) // 256) * (N // 256) >= 48)
    if not fused:
        return llama_ops.rope_qkv(linear(x2, w_qkv), L, pos0, H, Hkv, hd, theta)
    assert x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and w_qkv.stride(-1) == 1
    assert N == (H + 2 * Hkv) * hd
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    cs = llama_ops.rope_table(pos0 + L, hd, theta, x.device)
    out = torch.empty((M, 3 * H * hd), dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().dz_gemm2_qkv_rope(
        _lib.ptr(x2), ctypes.c_longlong(x2.stride(0)), _lib.ptr(w_qkv), ctypes.c_longlong(w_qkv.stride(0)),
        _lib.ptr(out), ctypes.c_longlong(out.stride(0)), _lib.ptr(cs), M, K, L, pos0, cs.shape[0], H, Hkv,
        _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm2_qkv_rope")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None,
           residual: torch.Tensor | None = None, scale: float = 1.0,
           out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
           tile_n: int = 0) -> torch.Tensor:
    """x [..., K] (bf16), w [N, K] (bf16) -> [..., N] in ``out_dtype`` (bf16 or fp32).

    ``tile_n``: 0 = choose, 128 / 256 = one-SM kernel with that tile width, 512 = two-SM kernel."""
    if not x.is_cuda:
        y = linear_reference(x, w, bias, act, residual, scale, out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "kernel path is bf16"
    K = x.shape[-1]
    N = w.shape[0]
    assert w.shape[1] == K
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    out_dtype = out_dtype or torch.bfloat16
    assert out_dtype in (torch.bfloat16, torch.float32)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    out2 = out.reshape(-1, N)
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, N)
        assert res2.dtype == torch.bfloat16 and res2.stride(-1) == 1
    assert w.stride(-1) == 1 and out2.stride(-1) == 1
    if M == 0:
        return out.reshape(*x.shape[:-1], N)
    variant = _VARIANT
    if tile_n == 512:
        variant, tile_n = 2, 0
    elif tile_n in (128, 256):
        variant = 1
    if variant == 0:
        # pairs of SMs (256 x 256 tiles) once there is work for most of them
        variant = 2 if (M >= 256 and ((M + 255) // 256) * ((N + 255) // 256) >= 48) else 1
    if variant == 2:
        rc = _lib.lib().dz_gemm2_bf16_tn(
            _lib.ptr(x2), ctypes.c_longlong(x2.stride(0)), _lib.ptr(w), ctypes.c_longlong(w.stride(0)),
            _lib.ptr(out2), ctypes.c_longlong(out2.stride(0)), _lib.ptr(bias), _lib.ptr(res2),
            ctypes.c_longlong(res2.stride(0) if res2 is not None else 0),
            M, N, K, ACT[act], int(out_dtype == torch.float32), ctypes.c_float(scale),
            _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr())
        _lib.check(rc, "dz_gemm2_bf16_tn")
        return out.reshape(*x.shape[:-1], N)
    rc = _lib.lib().dz_gemm_bf16_tn(
        _lib.ptr(x2), ctypes.c_longlong(x2.stride(0)), _lib.ptr(w), ctypes.c_longlong(w.stride(0)),
        _lib.ptr(out2), ctypes.c_longlong(out2.stride(0)), _lib.ptr(bias), _lib.ptr(res2),
        ctypes.c_longlong(res2.stride(0) if res2 is not None else 0),
        M, N, K, ACT[act], int(out_dtype == torch.float32), ctypes.c_float(scale), tile_n,
        _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm_bf16_tn")
    return out.reshape(*x.shape[:-1], N)
