"""The allocation-free scoring entry point against the regular one.

Some callers cannot allocate device memory when they need a score (the GPU's memory belongs to
their own pool, or cudaMalloc's implicit synchronisation does not fit their latency budget), so
``dz_token_logprobs_noalloc`` keeps the log-sum-exp partials in a fixed array inside the
library.  It is called here through its exported C symbol, twice in a row with different
inputs (the second call meets the first call's leftovers in the shared scratch), and must agree
with the regular entry points.  This file sorts last on purpose: if it fails, a run that stops
at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

from dizo_b200.ops import _lib
from dizo_b200.ops.loss import token_logprobs

pytestmark = pytest.mark.gpu


def _call(h, table, targets, scale=1.0):
    L = _lib.lib()
    fn = L.dz_token_logprobs_noalloc
    fn.restype = ctypes.c_int
    out = torch.empty(h.shape[0], dtype=torch.float32, device=h.device)
    rc = fn(ctypes.c_void_p(h.data_ptr()), ctypes.c_longlong(h.stride(0)),
            ctypes.c_void_p(table.data_ptr()), ctypes.c_longlong(table.stride(0)),
            ctypes.c_void_p(targets.data_ptr()), ctypes.c_void_p(out.data_ptr()),
            h.shape[0], table.shape[0], h.shape[1], ctypes.c_float(scale),
            ctypes.c_void_p(_lib.err_word(h.device).data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_noalloc_logprobs_match_regular_entry_point_twice():
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(21)
    V, d = 50272, 768
    table = (torch.randn(V, d, device=dev, generator=g) * 0.05).bfloat16()
    for rows in (37, 301):                       # second call: more rows, other data, same scratch
        h = torch.randn(rows, d, device=dev, generator=g).bfloat16()
        tg = torch.randint(0, V, (rows,), device=dev, generator=g, dtype=torch.int32)
        rc, got = _call(h, table, tg)
        assert rc == 0
        want = token_logprobs(h, table, tg)
        torch.cuda.synchronize()
        _lib.check_device_errors()
        assert (got - want).abs().max().item() < 2e-3
        ref = torch.log_softmax(h.float() @ table.float().t(), -1).gather(1, tg.long().view(-1, 1)).squeeze(1)
        assert (got - ref).abs().max().item() < 2e-3


def test_noalloc_rejects_sizes_beyond_its_scratch():
    dev = "cuda"
    h = torch.zeros(513, 64, device=dev, dtype=torch.bfloat16)
    table = torch.zeros(256, 64, device=dev, dtype=torch.bfloat16)
    tg = torch.zeros(513, device=dev, dtype=torch.int32)
    rc, _ = _call(h, table, tg)
    assert rc == 4                                # DZ_ERR_TOO_LARGE
    big = torch.zeros(65536 + 256, 64, device=dev, dtype=torch.bfloat16)
    rc, _ = _call(h[:8], big, tg[:8])
    assert rc == 4
