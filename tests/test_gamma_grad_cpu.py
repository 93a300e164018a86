"""The kernel-backward orchestration for d loss / d alpha (first-order gamma search) against
autograd through the differentiable statement of the forward, on CPU in fp32."""
import numpy as np
import torch

from dizo_b200.data.batching import batch_from_inputs
from dizo_b200.engine import DiZOProjector
from dizo_b200.models.gamma_grad import GammaGrad, supported
from dizo_b200.models.opt import OPTModel, preset
from dizo_b200.models.opt_autograd import make_fo_loss


def _model():
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32, mode="full").init_random(seed=0, std=0.05)
    proj = DiZOProjector(m)
    g = torch.Generator().manual_seed(3)
    for n in m.arena.slot_names:                       # theta leaves theta_0
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.02)
    return cfg, m, proj


def _inputs(cfg, kind, S=4, L=20):
    rng = np.random.default_rng(5)
    ids = rng.integers(4, cfg.vocab_size, size=(S, L))
    mask = np.ones((S, L), dtype=np.int64)
    mask[1, :6] = 0                                    # left padding
    mask[3, :11] = 0
    ids[mask == 0] = 1
    if kind == "verbalizer":                           # 2 one-token candidates sharing the prompt
        ids[1] = ids[0]; mask[1] = mask[0]
        ids[2] = ids[3]; mask[2] = mask[3]
        ids[[0, 2], -1] = 10
        ids[[1, 3], -1] = 11
        return dict(input_ids=ids, attention_mask=mask, labels=[1, 1, 0, 0], option_len=[1] * S,
                    num_options=[2] * S)
    if kind == "candidates":                           # multi-token options
        return dict(input_ids=ids, attention_mask=mask, labels=[0, 0, 1, 1], option_len=[3, 2, 4, 3],
                    num_options=[2] * S)
    lab = ids.copy()
    return dict(input_ids=ids, attention_mask=mask, labels=lab, option_len=[5, 4, 6, 3])


def test_supported_flags():
    cfg, m, _ = _model()
    assert supported(m)
    assert supported(OPTModel(cfg, "cpu", torch.float32, mode="lora"))
    assert supported(OPTModel(cfg, "cpu", torch.float32, mode="lora+prefix"))
    # GELU has no fused backward mask
    assert not supported(OPTModel(preset("opt-tiny", activation_function="gelu"), "cpu", torch.float32))


def _check_against_autograd(m, proj, cfg):
    gg = GammaGrad(m)
    fo = make_fo_loss(m)
    for kind in ("verbalizer", "candidates", "lm"):
        b = batch_from_inputs(_inputs(cfg, kind), pad_token_id=1)
        alpha = torch.rand(proj.n, generator=torch.Generator().manual_seed(7)) * 0.5 + 0.5
        a = alpha.clone().requires_grad_(True)
        ref_loss = fo(b, a)
        ref_loss.backward()
        loss, g = gg.loss_and_grad(b, alpha)
        assert abs(float(loss) - float(ref_loss.detach())) < 1e-4 * max(1.0, abs(float(ref_loss.detach()))), kind
        scale = a.grad.abs().max().item()
        assert scale > 0
        assert (g - a.grad).abs().max().item() < 2e-3 * scale + 1e-6, (kind, g, a.grad)


def test_lora_factors_gamma_grad_matches_autograd():
    """LoRA: the constrained tensors are the adapter factors; d loss / d alpha comes from rank-r GEMMs."""
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32, mode="lora", lora_r=8).init_random(seed=0, std=0.05)
    proj = DiZOProjector(m)
    assert proj.n == 4 * cfg.num_hidden_layers and supported(m)
    g = torch.Generator().manual_seed(3)
    for n in m.arena.slot_names:                       # A and B leave their anchors (B_0 = 0)
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.05)
    _check_against_autograd(m, proj, cfg)


def test_lora_with_prefix_rows_gamma_grad_matches_autograd():
    """LoRA + prefix: the prefix rows are extra key columns of the attention and of its backward."""
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32, mode="lora+prefix", lora_r=8, num_prefix=3).init_random(seed=0, std=0.05)
    proj = DiZOProjector(m)
    assert proj.n == 4 * cfg.num_hidden_layers and supported(m)
    g = torch.Generator().manual_seed(3)
    for n in m.arena.slot_names:
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.05)
    for n in m.trainable_names:
        if "prefix_" in n:
            m.param(n).copy_(torch.randn(m.param(n).shape, generator=g) * 0.3)
    _check_against_autograd(m, proj, cfg)


def test_post_layernorm_with_projections_gamma_grad_matches_autograd():
    """The opt-350m layout: LayerNorm after the residual add, project_in / project_out around the stack."""
    cfg = preset("opt-tiny", do_layer_norm_before=False, word_embed_proj_dim=32)
    m = OPTModel(cfg, "cpu", torch.float32, mode="full").init_random(seed=0, std=0.05)
    proj = DiZOProjector(m)
    assert supported(m)
    g = torch.Generator().manual_seed(3)
    for n in m.arena.slot_names:
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.02)
    _check_against_autograd(m, proj, cfg)


def test_gamma_grad_matches_autograd():
    cfg, m, proj = _model()
    gg = GammaGrad(m)
    fo = make_fo_loss(m)
    assert proj.n == 2 * cfg.num_hidden_layers
    for kind in ("verbalizer", "candidates", "lm"):
        b = batch_from_inputs(_inputs(cfg, kind), pad_token_id=1)
        assert (b.cand_ids is not None) == (kind == "verbalizer")
        alpha = torch.rand(proj.n, generator=torch.Generator().manual_seed(7)) * 0.5 + 0.5
        a = alpha.clone().requires_grad_(True)
        ref_loss = fo(b, a)
        ref_loss.backward()
        loss, g = gg.loss_and_grad(b, alpha)
        assert abs(float(loss) - float(ref_loss)) < 1e-4 * max(1.0, abs(float(ref_loss))), kind
        scale = a.grad.abs().max().item()
        assert scale > 0
        assert (g - a.grad).abs().max().item() < 2e-3 * scale + 1e-6, (kind, g, a.grad)


def test_search_fo_kernel_backward_equals_autograd_path():
    res = []
    for native in (True, False):
        cfg, m, proj = _model()
        proj.max_iters = 3
        proj.use_kernel_backward = native
        b = batch_from_inputs(_inputs(cfg, "candidates"), pad_token_id=1)
        proj.search_fo(lambda: b, make_fo_loss(m))
        res.append((proj.gs.gamma.clone(), m.arena.data.clone()))
    assert torch.allclose(res[0][0], res[1][0], atol=1e-4, rtol=1e-3)
    assert torch.allclose(res[0][1], res[1][1], atol=1e-5, rtol=1e-4)
