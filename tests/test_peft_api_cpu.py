"""LoRALinear and the prefix re-parameterisation MLP on CPU (fp32) against plain PyTorch statements."""
import torch

from dizo_b200.data.synthetic import synthetic_batch
from dizo_b200.engine import ZOEngine
from dizo_b200.models.opt import OPTModel, Transform, layer_prefix, preset
from dizo_b200.models.opt_autograd import functional_loss
from dizo_b200.models.peft import LoRALinear, PrefixTuning


def test_lora_linear_matches_the_reference_formula():
    lin = LoRALinear(48, 32, r=4, lora_alpha=8, seed=1)
    lin.lora_B.copy_(torch.randn(32, 4, generator=torch.Generator().manual_seed(2)) * 0.1)
    x = torch.randn(5, 7, 48, generator=torch.Generator().manual_seed(3))
    want = torch.nn.functional.linear(x, lin.weight, lin.bias) + (x @ lin.lora_A.t() @ lin.lora_B.t()) * lin.scaling
    assert torch.allclose(lin(x), want, atol=1e-5)
    w0 = lin.weight.clone()
    lin.merge()
    assert lin.merged and torch.allclose(lin(x), want, atol=1e-5)
    lin.unmerge()
    assert not lin.merged and torch.allclose(lin.weight, w0, atol=1e-6)
    assert set(lin.trainable()) == {"lora_A", "lora_B"}
    assert LoRALinear(8, 8).trainable() == {}


def test_prefix_reparameterisation_mlp_trains_the_mlp_and_matches_autograd_forward():
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32, mode="prefix", num_prefix=5, prefix_reparam=True,
                 prefix_embed_dim=16, prefix_mid_dim=24).init_random(0)
    pt = PrefixTuning(m, num_prefix=5, reparam=True, embed_dim=16, mid_dim=24, init_by_real_act=False)
    names = set(pt.names)
    assert layer_prefix(0) + "self_attn.prefix_input_embeds" in names
    assert layer_prefix(1) + "self_attn.prefix_mlp_values.2.weight" in names
    assert not any(n.endswith("prefix_keys") for n in names)
    assert m.param(layer_prefix(1) + "self_attn.prefix_mlp_keys.0.weight").shape == (24, 16)
    b = synthetic_batch(0, 3, 24, cfg.vocab_size, pad_left=4, cand_ids=(17, 29))
    ref = functional_loss(m, b, use_checkpoint=False).item()
    assert abs(m.loss(b).item() - ref) < 1e-4
    # the perturbation reaches the loss through the MLP parameters
    assert abs(m.loss(b, Transform(seed=3, coef=1e-2)).item() - ref) > 1e-6
    eng = ZOEngine(m, eps=1e-3)
    before = m.arena.data.clone()
    eng.step(b, 1e-2, seed=5)
    assert not torch.equal(before, m.arena.data)
    sd = m.state_dict()
    m2 = OPTModel(cfg, "cpu", torch.float32, mode="prefix", num_prefix=5, prefix_reparam=True,
                  prefix_embed_dim=16, prefix_mid_dim=24).init_random(9)
    m2.load_state_dict(sd)
    assert abs(m2.loss(b).item() - m.loss(b).item()) < 1e-6


def test_dizo_module_facade():
    """The reference-shaped DiZO module: constraints / alpha / ts, apply_constraints, perturb_gamma, zo_forward."""
    import torch
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import DiZO
    from dizo_b200.models.opt import OPTModel, preset
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    d = DiZO(m, "l2norm", exclude_list=[m.dizo_include_names()[0]])
    assert len(d.constraints_name) == len(m.dizo_include_names()) - 1 and d.init
    g = torch.Generator().manual_seed(3)
    for n in d.constraints_name:
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.02)
    b = synthetic_batch(0, 4, 16, cfg.vocab_size, cand_ids=(10, 20))
    l0 = float(m.loss(b))
    d.apply_constraints()
    assert not d.init and torch.allclose(d.constraints, d.ts) and torch.allclose(d.alpha, torch.ones_like(d.alpha), atol=1e-6)
    assert abs(float(d.zo_forward(b)) - l0) < 1e-6
    d.perturb_gamma(5, 1.0)
    lp = float(d.zo_forward(b))
    d.perturb_gamma(None, -2.0)
    lm = float(d.zo_forward(b))
    d.perturb_gamma(None, 1.0)
    assert lp != lm and torch.allclose(d.alpha, torch.ones_like(d.alpha), atol=1e-5)
    # apply=True writes the projection into theta: with gamma = 0.5 ts the distance to the anchor halves
    before = (m.param(d.constraints_name[0]) - m.arena.anchor_view(d.constraints_name[0])).norm()
    d.constraints.mul_(0.5)
    d.projector.gs.alpha.copy_(d.constraints / (d.ts + 1e-8))
    d.projector.project()
    after = (m.param(d.constraints_name[0]) - m.arena.anchor_view(d.constraints_name[0])).norm()
    assert abs(float(after / before) - 0.5) < 1e-4


def test_dizo_trainer_constructor():
    """dizo_trainer(model, pgmloader, norm_mode, proj_lr, max_iters, exclude_list): both searches run from it."""
    import torch
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.trainer import dizo_trainer
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    loader = [synthetic_batch(s, 4, 16, cfg.vocab_size, cand_ids=(10, 20)) for s in range(3)]
    t = dizo_trainer(m, loader, "l2norm", 0.1, 2)
    g = torch.Generator().manual_seed(3)
    for n in m.arena.slot_names:
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.02)
    t.dizo_zo_iters()
    t.dizo_iters()
    assert t.i == 2 and t.projector.searches == 2 and torch.isfinite(t.projector.gs.gamma).all()
