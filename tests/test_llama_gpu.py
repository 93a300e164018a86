"""LLaMA-family kernels (RMSNorm, rotary embedding + head expansion, SwiGLU gate) against their fp32 PyTorch
statements, and the bf16 model on the GPU against the fp32 model on the CPU."""
import pytest
import torch

from dizo_b200.ops import _lib
from dizo_b200.ops import llama as llama_ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sync_ok():
    torch.cuda.synchronize()
    _lib.check_device_errors()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("rows,d", [(7, 64), (300, 4096), (64, 5120), (5, 8192)])
def test_rmsnorm(rows, d):
    g = torch.Generator(device=DEV).manual_seed(d)
    x = (torch.randn(rows, d, device=DEV, generator=g) * 3).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).bfloat16()
    y = llama_ops.rmsnorm(x, w, 1e-5)
    _sync_ok()
    ref = llama_ops.rmsnorm(x.float().cpu(), w.float().cpu(), 1e-5)
    assert _rel(y.cpu(), ref) < 4e-3
    # a strided input (rows of a wider buffer)
    wide = torch.zeros(rows, d + 64, device=DEV, dtype=torch.bfloat16)
    wide[:, :d] = x
    assert torch.equal(llama_ops.rmsnorm(wide[:, :d], w, 1e-5), y)


@pytest.mark.parametrize("H,Hkv,hd,L,pos0", [(4, 4, 64, 33, 0), (8, 2, 128, 100, 5), (6, 3, 80, 17, 4000), (4, 1, 16, 1, 77)])
def test_rope_qkv(H, Hkv, hd, L, pos0):
    B = 3
    g = torch.Generator(device=DEV).manual_seed(hd + L)
    x = torch.randn(B * L, (H + 2 * Hkv) * hd, device=DEV, generator=g).bfloat16()
    y = llama_ops.rope_qkv(x, L, pos0, H, Hkv, hd, 10000.0)
    _sync_ok()
    ref = llama_ops.rope_qkv_reference(x.float().cpu(), L, pos0, H, Hkv, hd, 10000.0)
    assert y.shape == (B * L, 3 * H * hd)
    assert _rel(y.cpu(), ref) < 4e-3
    # v is copied bit for bit, k / v heads are repeated
    d, rep = H * hd, H // Hkv
    v_in = x[:, (H + Hkv) * hd:].view(B * L, Hkv, hd).repeat_interleave(rep, dim=1).reshape(B * L, d)
    assert torch.equal(y[:, 2 * d:], v_in)


@pytest.mark.parametrize("rows,F", [(5, 176), (300, 11008), (64, 13824)])
def test_silu_mul(rows, F):
    g = torch.Generator(device=DEV).manual_seed(F)
    gu = (torch.randn(rows, 2 * F, device=DEV, generator=g) * 2).bfloat16()
    y = llama_ops.silu_mul(gu)
    _sync_ok()
    ref = llama_ops.silu_mul(gu.float().cpu())
    assert _rel(y.cpu(), ref) < 4e-3


@pytest.mark.parametrize("M,K,F", [(2048, 512, 3072), (2000, 1024, 1792), (4096, 256, 11008), (192, 256, 1024)])
def test_gemm_with_swiglu_epilogue(M, K, F):
    """silu(x gate^T) * (x up^T) from the two-SM GEMM's epilogue (the last shape takes the unfused route)."""
    from dizo_b200.ops import gemm
    g = torch.Generator(device=DEV).manual_seed(M + F)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * F, K, device=DEV, generator=g) * K ** -0.5).bfloat16()
    y = gemm.linear_swiglu(x, w)
    _sync_ok()
    assert y.shape == (M, F)
    acc = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(acc[:, :F]) * acc[:, F:]
    assert _rel(y, ref) < 6e-3
    # against the unfused route (bf16 intermediate): same up to that rounding
    unfused = llama_ops.silu_mul(gemm.linear(x, w))
    assert _rel(y, unfused) < 1e-2
    # a view of a wider weight buffer (row pitch larger than K)
    wide = torch.zeros(2 * F, K + 64, device=DEV, dtype=torch.bfloat16)
    wide[:, :K] = w
    assert torch.equal(gemm.linear_swiglu(x, wide[:, :K]), y)
    _sync_ok()


@pytest.mark.parametrize("B,L,K,H,Hkv,pos0", [(8, 256, 512, 8, 8, 0), (8, 250, 1024, 8, 2, 5), (4, 1024, 256, 32, 8, 3),
                                               (2, 64, 256, 8, 8, 0)])
def test_gemm_with_rotary_epilogue(B, L, K, H, Hkv, pos0):
    """q | k | v projection with the rotation (and the grouped-query head expansion) in the two-SM GEMM's epilogue
    against the fp32 statement (the last shape takes the unfused route)."""
    from dizo_b200.ops import gemm
    hd, M = 128, B * L
    g = torch.Generator(device=DEV).manual_seed(M + K + H)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn((H + 2 * Hkv) * hd, K, device=DEV, generator=g) * K ** -0.5).bfloat16()
    y = gemm.linear_qkv_rope(x, w, L, pos0, H, Hkv, hd, 10000.0)
    _sync_ok()
    assert y.shape == (M, 3 * H * hd)
    ref = llama_ops.rope_qkv_reference(x.float() @ w.float().t(), L, pos0, H, Hkv, hd, 10000.0)
    assert _rel(y, ref) < 6e-3
    for sec in range(3):                                   # every section on its own (q, k, v)
        assert _rel(y[:, sec * H * hd:(sec + 1) * H * hd], ref[:, sec * H * hd:(sec + 1) * H * hd]) < 6e-3
    unfused = llama_ops.rope_qkv(gemm.linear(x, w), L, pos0, H, Hkv, hd, 10000.0)
    assert _rel(y, unfused) < 1e-2
    # repeated k / v heads are bit-equal copies
    rep = H // Hkv
    if rep > 1:
        k = y[:, H * hd:2 * H * hd].view(M, Hkv, rep, hd)
        assert torch.equal(k[:, :, 0], k[:, :, rep - 1])
    _sync_ok()


@pytest.mark.parametrize("name", ["llama-tiny", "llama-tiny-gqa"])
def test_model_matches_cpu_statement_and_zo_step_runs(name):
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import ZOEngine
    from dizo_b200.models.generate import generate
    from dizo_b200.models.llama import LlamaModel, preset

    cfg = preset(name, hidden_size=256, num_attention_heads=4, intermediate_size=704, vocab_size=2048,
                 num_key_value_heads=2 if name.endswith("gqa") else 4, max_position_embeddings=512)
    cpu = LlamaModel(cfg, "cpu", torch.float32).init_random(0, std=0.05)
    gpu = LlamaModel(cfg, DEV, torch.bfloat16)
    gpu.load_state_dict(cpu.state_dict())
    # the CPU statement runs on the bf16-rounded weights the GPU holds
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    b = synthetic_batch(0, 3, 160, cfg.vocab_size, seed=1, pad_left=9)
    got = gpu.loss(b.to(DEV))
    _sync_ok()
    want = cpu.loss(b)
    assert abs(got.item() - want.item()) < 3e-2 * max(1.0, abs(want.item())), (got.item(), want.item())
    lg = gpu.logits(b.to(DEV), rows=b.rows.to(DEV))
    lw = cpu.logits(b, rows=b.rows)
    assert _rel(lg.cpu(), lw) < 3e-2
    # decoding: the bf16 kernels pick the same first tokens as the fp32 statement on most rows
    ids = b.input_ids[:, :40].long()
    out_g = generate(gpu, ids, max_new_tokens=4, pad_token_id=0)
    out_c = generate(cpu, ids, max_new_tokens=4, pad_token_id=0)
    assert sum(a[40] == c[40] for a, c in zip(out_g, out_c)) >= 2
    # a ZO step perturbs every tensor (token table included) and moves the loss estimate
    eng = ZOEngine(gpu, eps=1e-3, dp_group=False)
    before = gpu.param(gpu.EMBED).clone()
    l1 = eng.step(b.to(DEV), lr=1e-2, seed=5)
    _sync_ok()
    assert not torch.equal(before, gpu.param(gpu.EMBED))
    assert torch.isfinite(torch.as_tensor(float(l1)))
    # the differentiable statement (first-order gamma search, first-order fine-tuning) on the device in bf16
    from dizo_b200.models.opt_autograd import functional_loss
    with torch.no_grad():
        fl = functional_loss(gpu, b.to(DEV), use_checkpoint=False)
    now = gpu.loss(b.to(DEV))
    _sync_ok()
    assert abs(fl.item() - now.item()) < 5e-2 * max(1.0, abs(now.item())), (fl.item(), now.item())
