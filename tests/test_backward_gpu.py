"""Backward kernels (data-gradient GEMM, attention backward, LayerNorm / softmax gradients, dot,
scatter) against PyTorch fp32 statements / autograd of the same ops."""
import pytest
import torch

from dizo_b200.ops import _lib
from dizo_b200.ops import backward as bw
from dizo_b200.ops.attention import (attention, attention_backward, attention_backward_reference,
                                     attention_reference)

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sync_ok():
    torch.cuda.synchronize()
    _lib.check_device_errors()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("M,K,N", [(300, 512, 768), (1024, 2048, 1000), (64, 50272, 256), (130, 72, 264),
                                   (2048, 1024, 4096)])
def test_linear_dgrad(M, K, N):
    g = torch.Generator(device=DEV).manual_seed(M + K + N)
    dy = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(K, N, device=DEV, generator=g) * 0.05).bfloat16()
    out = bw.linear_dgrad(dy, w)
    _sync_ok()
    ref = dy.float() @ w.float()
    assert _rel(out, ref) < 1e-2
    mask = torch.randn(M, N, device=DEV, generator=g).bfloat16()
    res = torch.randn(M, N, device=DEV, generator=g).bfloat16()
    out2 = bw.linear_dgrad(dy, w, mask=mask, residual=res, out_dtype=torch.float32)
    _sync_ok()
    ref2 = torch.where(mask.float() > 0, ref, torch.zeros_like(ref)) + res.float()
    assert _rel(out2, ref2) < 1e-2
    assert out2.dtype == torch.float32


@pytest.mark.parametrize("B,L,H,hd", [(2, 256, 4, 64), (1, 128, 2, 128), (2, 200, 3, 80), (1, 520, 1, 128),
                                      (3, 384, 2, 128), (1, 64, 2, 64), (1, 1000, 2, 80)])
def test_attention_lse_and_backward(B, L, H, hd):
    g = torch.Generator(device=DEV).manual_seed(B * 1000 + L + hd)
    d = H * hd
    qkv = torch.randn(B, L, 3 * d, device=DEV, generator=g).bfloat16()
    dout = torch.randn(B, L, d, device=DEV, generator=g).bfloat16()
    lse = torch.empty(B, H, L, dtype=torch.float32, device=DEV)
    out = attention(qkv, H, lse=lse)
    _sync_ok()
    # the saved statistic: log2-domain log-sum-exp of the scaled, causally masked scores
    q, k, _ = qkv.float().split(d, dim=-1)
    q = q.view(B, L, H, hd).transpose(1, 2)
    k = k.view(B, L, H, hd).transpose(1, 2)
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * hd ** -0.5
    idx = torch.arange(L, device=DEV)
    s = s.masked_fill(~(idx[None, :] <= idx[:, None]), float("-inf"))
    ref_lse = torch.logsumexp(s, dim=-1) * 1.4426950408889634
    assert (lse - ref_lse).abs().max().item() < 2e-2
    dqkv = attention_backward(qkv, out, dout, lse, H)
    _sync_ok()
    ref = attention_backward_reference(qkv, dout, H)
    for name, sl in (("dq", slice(0, d)), ("dk", slice(d, 2 * d)), ("dv", slice(2 * d, 3 * d))):
        r = _rel(dqkv[..., sl], ref[..., sl])
        assert r < 2e-2, (name, r)


@pytest.mark.parametrize("hd", [64, 80, 128])
def test_attention_backward_left_pad(hd):
    B, L, H = 3, 300, 4
    d = H * hd
    g = torch.Generator(device=DEV).manual_seed(hd)
    qkv = torch.randn(B, L, 3 * d, device=DEV, generator=g).bfloat16()
    pad = torch.tensor([0, 70, 257], dtype=torch.int32, device=DEV)
    dout = torch.randn(B, L, d, device=DEV, generator=g).bfloat16()
    # nothing flows into padding rows in the model; mirror that
    for b in range(B):
        dout[b, :int(pad[b])] = 0
    lse = torch.empty(B, H, L, dtype=torch.float32, device=DEV)
    out = attention(qkv, H, pad_left=pad, lse=lse)
    dqkv = attention_backward(qkv, out, dout, lse, H, pad_left=pad)
    _sync_ok()
    ref = attention_backward_reference(qkv, dout, H, pad_left=pad)
    assert torch.isfinite(dqkv.float()).all()
    assert _rel(dqkv, ref) < 2e-2


@pytest.mark.parametrize("hd", [64, 80, 128])
def test_attention_backward_prefix_rows(hd):
    """Prefix keys / values as extra, unmasked key columns: dQ | dK | dV and the prefix rows' own gradients."""
    B, L, H, P = 2, 200, 4, 5
    d = H * hd
    g = torch.Generator(device=DEV).manual_seed(100 + hd)
    qkv = torch.randn(B, L, 3 * d, device=DEV, generator=g).bfloat16()
    pk = torch.randn(P, d, device=DEV, generator=g).bfloat16()
    pv = torch.randn(P, d, device=DEV, generator=g).bfloat16()
    pad = torch.tensor([0, 33], dtype=torch.int32, device=DEV)
    dout = torch.randn(B, L, d, device=DEV, generator=g).bfloat16()
    dout[1, :33] = 0
    lse = torch.empty(B, H, L, dtype=torch.float32, device=DEV)
    out = attention(qkv, H, pad_left=pad, prefix_k=pk, prefix_v=pv, lse=lse)
    dp = (torch.zeros(P, d, device=DEV), torch.zeros(P, d, device=DEV))
    dqkv = attention_backward(qkv, out, dout, lse, H, pad_left=pad, prefix_k=pk, prefix_v=pv, d_prefix=dp)
    _sync_ok()
    rp = (torch.zeros(P, d, device=DEV), torch.zeros(P, d, device=DEV))
    ref = attention_backward_reference(qkv, dout, H, pad_left=pad, prefix_k=pk, prefix_v=pv, d_prefix=rp)
    for name, sl in (("dq", slice(0, d)), ("dk", slice(d, 2 * d)), ("dv", slice(2 * d, 3 * d))):
        assert _rel(dqkv[..., sl], ref[..., sl]) < 2e-2, (name, _rel(dqkv[..., sl], ref[..., sl]))
    assert _rel(dp[0], rp[0]) < 2e-2 and _rel(dp[1], rp[1]) < 2e-2, (_rel(dp[0], rp[0]), _rel(dp[1], rp[1]))
    # the prefix rows matter: leaving them out of the backward must show
    no_prefix = attention_backward(qkv, out, dout, lse, H, pad_left=pad)
    assert _rel(no_prefix[..., :d], ref[..., :d]) > 5e-2


@pytest.mark.parametrize("rows,d", [(7, 768), (300, 2560), (64, 5120), (5, 9216)])
def test_layernorm_backward(rows, d):
    g = torch.Generator(device=DEV).manual_seed(d)
    x = (torch.randn(rows, d, device=DEV, generator=g) * 2 + 0.5).bfloat16()
    w = torch.randn(d, device=DEV, generator=g).bfloat16()
    dy = torch.randn(rows, d, device=DEV, generator=g).bfloat16()
    add = torch.randn(rows, d, device=DEV, generator=g).bfloat16()
    xf = x.float().requires_grad_(True)
    y = torch.nn.functional.layer_norm(xf, (d,), w.float(), torch.zeros(d, device=DEV), 1e-5)
    (ref,) = torch.autograd.grad(y, xf, dy.float())
    out = bw.layernorm_backward(dy, x, w, 1e-5)
    _sync_ok()
    assert _rel(out, ref) < 1e-2
    out2 = bw.layernorm_backward(dy, x, w, 1e-5, add=add)
    _sync_ok()
    assert _rel(out2, ref + add.float()) < 1e-2


def test_softmax_ce_backward():
    R, V = 37, 50272
    g = torch.Generator(device=DEV).manual_seed(1)
    logits = (torch.randn(R, V, device=DEV, generator=g) * 3).bfloat16()
    targets = torch.randint(0, V, (R,), device=DEV, generator=g, dtype=torch.int32)
    coef = torch.randn(R, device=DEV, generator=g)
    lf = logits.float().requires_grad_(True)
    lp = torch.log_softmax(lf, dim=-1).gather(1, targets.long().view(-1, 1)).squeeze(1)
    (ref,) = torch.autograd.grad((lp * coef).sum(), lf)
    lse = torch.logsumexp(logits.float(), dim=-1)
    out = bw.softmax_ce_backward_(logits.clone(), lse, targets, coef)
    _sync_ok()
    assert (out.float() - ref).abs().max().item() < 2e-2 * coef.abs().max().item()
    assert _rel(out, ref) < 1e-2


def test_dot_scatter_diff():
    g = torch.Generator(device=DEV).manual_seed(2)
    rows, cols = 3000, 640
    a = torch.randn(rows, cols, device=DEV, generator=g)
    big = torch.randn(rows, 3 * cols, device=DEV, generator=g).bfloat16()
    b = big[:, cols:2 * cols]                      # strided rows, as the dK section of a dQKV gradient
    out = bw.dot(a, b, scale=0.5)
    out_again = bw.dot(a, b, scale=0.5)
    _sync_ok()
    ref = 0.5 * (a.double() * b.double()).sum().item()
    assert abs(out.item() - ref) < 1e-3 * max(1.0, abs(ref)) + 0.5
    assert out.item() == out_again.item()          # fixed reduction order
    src = torch.randn(5, 256, device=DEV, generator=g).bfloat16()
    idx = torch.tensor([9, 0, 4, 2, 7], dtype=torch.int32, device=DEV)
    dst = torch.zeros(10, 256, dtype=torch.bfloat16, device=DEV)
    bw.scatter_rows(src, idx, dst)
    x = torch.randn(4096, device=DEV, generator=g).bfloat16()
    y = torch.randn(4096, device=DEV, generator=g).bfloat16()
    df = bw.diff(x, y)
    _sync_ok()
    assert torch.equal(dst[idx.long()], src) and dst[1].abs().sum().item() == 0
    assert torch.equal(df, (x.float() - y.float()).bfloat16())


@pytest.mark.parametrize("kind", ["verbalizer", "lm"])
def test_gamma_grad_kernel_backward_matches_autograd(kind):
    """d loss / d alpha over a 12-layer bf16 model: kernel forward + backward against autograd
    through the PyTorch statement of the same forward."""
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import DiZOProjector
    from dizo_b200.models.gamma_grad import GammaGrad
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.models.opt_autograd import make_fo_loss

    cfg = preset("opt-125m")
    m = OPTModel(cfg, DEV, torch.bfloat16, mode="full").init_random_fast(seed=0)
    proj = DiZOProjector(m)
    g = torch.Generator(device=DEV).manual_seed(3)
    for n in m.arena.slot_names:
        p = m.param(n)
        p.add_((torch.randn(p.shape, device=DEV, generator=g) * 0.02).to(p.dtype))
    b = synthetic_batch(0, 2, 160, cfg.vocab_size, seed=1, pad_left=17).to(DEV)
    if kind == "lm":
        B, L = b.input_ids.shape
        rows = torch.cat([torch.arange(40, L - 1) + i * L for i in range(B)]).to(torch.int32).to(DEV)
        b.rows = rows
        b.targets = b.input_ids.reshape(-1)[(rows + 1).long()].contiguous()
        b.cand_ids = None
        b.classification = False
        b.seq_start = torch.tensor([0, rows.numel()], dtype=torch.int32, device=DEV)
    alpha = torch.rand(proj.n, device=DEV, generator=g) * 0.5 + 0.5
    loss, grad = GammaGrad(m).loss_and_grad(b, alpha)
    _sync_ok()
    a = alpha.clone().requires_grad_(True)
    ref_loss = make_fo_loss(m)(b, a)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 3e-2 * max(1.0, abs(ref_loss.item()))
    cos = torch.nn.functional.cosine_similarity(grad, a.grad.float(), dim=0).item()
    assert cos > 0.98, (cos, grad, a.grad)
    assert _rel(grad, a.grad) < 0.2


@pytest.mark.parametrize("variant", ["lora", "lora+prefix", "post_ln"])
def test_gamma_grad_kernel_backward_other_layouts(variant):
    """The kernel backward for LoRA (the adapter factors are the constrained tensors: rank-8 GEMMs)
    and for the post-LayerNorm layout with project_in / project_out (opt-350m), against autograd."""
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import DiZOProjector
    from dizo_b200.models.gamma_grad import GammaGrad, supported
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.models.opt_autograd import make_fo_loss

    if variant.startswith("lora"):
        cfg = preset("opt-125m", num_hidden_layers=4)
        m = OPTModel(cfg, DEV, torch.bfloat16, mode=variant).init_random_fast(seed=0)
        scale = 0.05
    else:
        cfg = preset("opt-350m", num_hidden_layers=4)
        m = OPTModel(cfg, DEV, torch.bfloat16, mode="full").init_random_fast(seed=0)
        scale = 0.02
    assert supported(m)
    proj = DiZOProjector(m)
    g = torch.Generator(device=DEV).manual_seed(3)
    for n in m.arena.slot_names:
        p = m.param(n)
        p.add_((torch.randn(p.shape, device=DEV, generator=g) * scale).to(p.dtype))
    b = synthetic_batch(0, 2, 160, cfg.vocab_size, seed=1, pad_left=17).to(DEV)
    alpha = torch.rand(proj.n, device=DEV, generator=g) * 0.5 + 0.5
    loss, grad = GammaGrad(m).loss_and_grad(b, alpha)
    _sync_ok()
    a = alpha.clone().requires_grad_(True)
    ref_loss = make_fo_loss(m)(b, a)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 3e-2 * max(1.0, abs(ref_loss.item()))
    cos = torch.nn.functional.cosine_similarity(grad, a.grad.float(), dim=0).item()
    assert cos > 0.97, (cos, grad, a.grad)
