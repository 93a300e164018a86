"""tcgen05 GEMM against an fp32 PyTorch statement of the same op."""
import pytest
import torch

from dizo_b200.ops import _lib
from dizo_b200.ops.gemm import linear, linear_reference

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K,tile_n", [
    (128, 256, 64, 256),
    (128, 128, 128, 128),
    (256, 512, 512, 0),
    (300, 776, 328, 256),      # ragged M, N (multiple of 8), K (multiple of 8, not of 64)
    (77, 200, 72, 128),
    (1000, 2560, 2560, 0),
    (4096, 7680, 2560, 0),
    (256, 256, 64, 512),       # two-SM kernel from here on
    (512, 768, 512, 512),
    (300, 776, 328, 512),
    (77, 200, 72, 512),
    (4096, 7680, 2560, 512),
    (1000, 2560, 10240, 512),
])
def test_gemm_plain(M, N, K, tile_n):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    y = linear(x, w, tile_n=tile_n)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    ref = linear_reference(x, w, out_dtype=torch.float32)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert _rel_err(y, ref) < 6e-3
    assert torch.allclose(y.float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=2e-2)


@pytest.mark.parametrize("act", [None, "relu", "gelu"])
@pytest.mark.parametrize("fp32_out", [False, True])
@pytest.mark.parametrize("tile_n", [0, 512])
def test_gemm_epilogues(act, fp32_out, tile_n):
    M, N, K = 517, 1032, 520
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    od = torch.float32 if fp32_out else torch.bfloat16
    y = linear(x, w, b, act=act, residual=r, scale=0.5, out_dtype=od, tile_n=tile_n)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    ref = linear_reference(x, w, b, act=act, residual=r, scale=0.5, out_dtype=torch.float32)
    tol = 1e-4 if fp32_out else 6e-3
    assert _rel_err(y, ref) < tol


def test_gemm_deterministic():
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(640, 1024, device="cuda", generator=g).bfloat16()
    w = torch.randn(768, 1024, device="cuda", generator=g).bfloat16()
    for tn in (256, 512):
        a = linear(x, w, tile_n=tn)
        b = linear(x, w, tile_n=tn)
        assert torch.equal(a, b)
