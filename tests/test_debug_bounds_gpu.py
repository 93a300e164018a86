"""The checked-store build of the kernel library (``-DDZ_DEBUG_BOUNDS``): small-shape runs of the
instrumented kernels record no violation, and a store into memory the host did not register is skipped
and reported instead of being executed.  Runs in a child process because the library variant is chosen
when the package is first imported."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent('''
    import torch
    from dizo_b200.ops import _lib
    assert _lib.DEBUG_BOUNDS and str(_lib._LIB_PATH).endswith("libdizo_b200_dbg.so")
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import DiZOProjector, ZOEngine
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.ops.norm import layernorm
    dev = "cuda"
    cfg = preset("opt-125m", num_hidden_layers=2)
    model = OPTModel(cfg, dev, torch.bfloat16).init_random_fast(0)
    eng = ZOEngine(model, eps=1e-3)
    proj = DiZOProjector(model, max_iters=1)
    b = synthetic_batch(0, 4, 96, cfg.vocab_size).to(dev)
    eng.step(b, 1e-6, seed=3)
    proj.search_zo(lambda: b, seed=1)
    proj.search_fo(lambda: b)
    torch.cuda.synchronize()
    _lib.check_device_errors()                      # also raises on a recorded violation
    assert _lib.debug_violations() == []
    print("CLEAN")
    # a destination the table does not know: the stores are skipped and counted, nothing is written
    x = torch.randn(64, 768, device=dev).bfloat16()
    w = torch.ones(768, device=dev).bfloat16()
    bias = torch.zeros(768, device=dev).bfloat16()
    y = torch.full((64, 768), 7.0, device=dev).bfloat16()
    layernorm(x, w, bias, out=y)                    # registers y, runs normally
    torch.cuda.synchronize()
    assert float(y.float().abs().max()) < 7.0
    y.fill_(7.0)
    _lib.forget(y)
    import ctypes
    rc = _lib.lib().dz_layernorm(ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(768), ctypes.c_void_p(w.data_ptr()),
                                 ctypes.c_void_p(bias.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                 ctypes.c_longlong(768), ctypes.c_longlong(64), 768, ctypes.c_float(1e-5),
                                 _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    bad = _lib.debug_violations()
    assert len(bad) == 1 and bad[0][0] == "norm" and bad[0][1] == 64 * 768 // 8, bad
    assert y.data_ptr() <= bad[0][2] < y.data_ptr() + y.numel() * 2
    assert bool((y.float() == 7.0).all())           # every store was skipped
    torch.zeros(4, device=dev).sum().item()         # the context is still usable
    print("REPORTED", bad)
''')


def test_checked_store_build_reports_and_skips_unregistered_stores():
    env = dict(os.environ, DIZO_DEBUG_BOUNDS="1", PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0 and "CLEAN" in res.stdout and "REPORTED" in res.stdout, \
        (res.stdout[-3000:], res.stderr[-3000:])
