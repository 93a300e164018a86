"""Stand-ins for a memory checker: kernels write into views that sit inside canary-filled buffers
(row slack and both ends), with ragged shapes that exercise the edge tiles, and the canaries must
survive; the same launch repeated must give bitwise identical results (a race would not)."""
import pytest
import torch

from dizo_b200.ops import _lib
from dizo_b200.ops import backward as bw
from dizo_b200.ops.attention import attention, attention_backward
from dizo_b200.ops.gemm import linear
from dizo_b200.ops.norm import layernorm
from dizo_b200.ops.zo import ParamArena, Piece

pytestmark = pytest.mark.gpu
DEV = "cuda"
CANARY = -7.0


def _framed(rows, cols, ld, dtype=torch.bfloat16, guard=4096):
    """A [rows, cols] view with row stride ld inside a canary-filled buffer."""
    buf = torch.full((guard + rows * ld + guard,), CANARY, dtype=dtype, device=DEV)
    view = torch.as_strided(buf, (rows, cols), (ld, 1), guard)
    return buf, view


def _canaries_intact(buf, rows, cols, ld, guard=4096):
    assert bool((buf[:guard] == CANARY).all()), "write before the output"
    assert bool((buf[guard + rows * ld:] == CANARY).all()), "write past the output"
    body = buf[guard:guard + rows * ld].view(rows, ld)
    assert bool((body[:, cols:] == CANARY).all()), "write into the row slack"


def _ok():
    torch.cuda.synchronize()
    _lib.check_device_errors()


@pytest.mark.parametrize("M,N,K,tile_n", [(130, 264, 72, 128), (300, 1000, 520, 256), (520, 776, 264, 512),
                                          (1, 8, 8, 0), (257, 50272, 128, 0)])
def test_gemm_stays_inside_its_output(M, N, K, tile_n):
    g = torch.Generator(device=DEV).manual_seed(M + N)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.1).bfloat16()
    b = torch.randn(N, device=DEV, generator=g).bfloat16()
    ld = (N + 8 + 7) // 8 * 8
    buf, out = _framed(M, N, ld)
    linear(x, w, b, act="relu", out=out, tile_n=tile_n)
    _ok()
    _canaries_intact(buf, M, N, ld)
    first = out.clone()
    linear(x, w, b, act="relu", out=out, tile_n=tile_n)
    _ok()
    assert torch.equal(first, out)
    ref = torch.relu(x.float() @ w.float().t() + b.float())
    assert ((out.float() - ref).norm() / ref.norm().clamp_min(1e-6)).item() < 1e-2


def test_attention_forward_and_backward_stay_inside_their_outputs():
    B, L, H, hd = 2, 333, 3, 80
    d = H * hd
    g = torch.Generator(device=DEV).manual_seed(1)
    qkv = torch.randn(B, L, 3 * d, device=DEV, generator=g).bfloat16()
    pad = torch.tensor([0, 41], dtype=torch.int32, device=DEV)
    obuf = torch.full((4096 + B * L * d + 4096,), CANARY, dtype=torch.bfloat16, device=DEV)
    out = obuf[4096:4096 + B * L * d].view(B, L, d)
    lse = torch.empty(B, H, L, dtype=torch.float32, device=DEV)
    attention(qkv, H, pad_left=pad, out=out, lse=lse)
    _ok()
    assert bool((obuf[:4096] == CANARY).all()) and bool((obuf[4096 + B * L * d:] == CANARY).all())
    first = out.clone()
    attention(qkv, H, pad_left=pad, out=out, lse=lse)
    _ok()
    assert torch.equal(first, out)
    dout = torch.randn(B, L, d, device=DEV, generator=g).bfloat16()
    gbuf = torch.full((4096 + B * L * 3 * d + 4096,), CANARY, dtype=torch.bfloat16, device=DEV)
    dqkv = gbuf[4096:4096 + B * L * 3 * d].view(B, L, 3 * d)
    attention_backward(qkv, out, dout, lse, H, pad_left=pad, dqkv=dqkv)
    _ok()
    assert bool((gbuf[:4096] == CANARY).all()) and bool((gbuf[4096 + B * L * 3 * d:] == CANARY).all())
    assert not bool((dqkv == CANARY).all(dim=-1).any()), "a row of the gradient was never written"
    first = dqkv.clone()
    attention_backward(qkv, out, dout, lse, H, pad_left=pad, dqkv=dqkv)
    _ok()
    assert torch.equal(first, dqkv)


def test_layernorm_and_dgrad_are_repeatable_and_bounded():
    g = torch.Generator(device=DEV).manual_seed(2)
    rows, d = 37, 2560
    x = torch.randn(rows, d, device=DEV, generator=g).bfloat16()
    w = torch.randn(d, device=DEV, generator=g).bfloat16()
    b = torch.randn(d, device=DEV, generator=g).bfloat16()
    buf, out = _framed(rows, d, d + 16)
    layernorm(x, w, b, out=out)
    _ok()
    _canaries_intact(buf, rows, d, d + 16)
    dy = torch.randn(300, 520, device=DEV, generator=g).bfloat16()
    wk = (torch.randn(520, 776, device=DEV, generator=g) * 0.1).bfloat16()
    a1, a2 = bw.linear_dgrad(dy, wk), bw.linear_dgrad(dy, wk)
    _ok()
    assert torch.equal(a1, a2)


def test_sweep_stays_inside_its_staging_buffer_and_repeats():
    pieces = [Piece("a", (300, 264), tensor_id=0), Piece("b", (264,), tensor_id=1), Piece("c", (7, 8), tensor_id=2)]
    ar = ParamArena(pieces, DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    ar.data.copy_(torch.randn(ar.data.shape, device=DEV, generator=g).to(ar.data.dtype))
    n = ar.data.numel()
    buf = torch.full((4096 + n + 4096,), CANARY, dtype=ar.data.dtype, device=DEV)
    dst = buf[4096:4096 + n]
    ar.sweep(dst=dst, seed1=11, c1=1e-2)
    _ok()
    assert bool((buf[:4096] == CANARY).all()) and bool((buf[4096 + n:] == CANARY).all())
    first = dst.clone()
    ar.sweep(dst=dst, seed1=11, c1=1e-2)
    _ok()
    assert torch.equal(first, dst)
    assert not torch.equal(dst[:300 * 264], ar.data[:300 * 264])
