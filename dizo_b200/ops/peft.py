"""LoRA merge: W_eff = W + scaling * B @ A (see ``csrc/peft_kernels.cu``).

Reference forward: ``F.linear(x, W, b) + (x @ A.T @ B.T) * scaling`` (large_models/lora.py:89-98);
merging first is the same function of x and needs one GEMM instead of three.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

ll = ctypes.c_longlong


def lora_merge(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scaling: float,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """w [N, K], a [r, K], b [N, r] -> out [N, K] (same dtype as w)."""
    if not w.is_cuda:
        y = (w.float() + scaling * (b.float() @ a.float())).to(w.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty_like(w)
    N, K = w.shape
    rc = _lib.lib().dz_lora_merge(_lib.ptr(w), ll(w.stride(0)), _lib.ptr(a), ll(a.stride(0)),
                                  _lib.ptr(b), ll(b.stride(0)), _lib.ptr(out), ll(out.stride(0)),
                                  N, K, a.shape[0], ctypes.c_float(scaling), _lib.stream_ptr())
    _lib.check(rc, "dz_lora_merge")
    return out
