"""The framework's ZO / DiZO loop against an independent fp32 oracle on CPU.

The oracle is the stock-PyTorch statement of the reference loop (``baseline/mezo_torch.py``:
Hugging Face ``OPTForCausalLM``, in-place perturb / restore / update, apply-forward-reverse
gamma search) fed with the framework's own z stream, so the two trajectories can be compared
step by step instead of statistically.  Scaled-down version of the CPU configuration
(OPT-125m architecture, eps 1e-3, lr 1e-6, projection by ZO); the full-size run is
``python -m baseline.cpu_oracle``.
"""
import torch
import torch.nn.functional as F

from baseline.mezo_torch import TorchMeZO, build_hf_opt
from dizo_b200.data.synthetic import synthetic_batch
from dizo_b200.engine import DiZOProjector, ZOEngine
from dizo_b200.models.opt import OPTModel, preset
from dizo_b200.ops import philox


def _setup(layers=2, lr=1e-4):
    cfg = preset("opt-125m", num_hidden_layers=layers, vocab_size=2048, max_position_embeddings=128,
                 hidden_size=192, num_attention_heads=6, ffn_dim=512)
    model = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    hf = build_hf_opt(cfg.to_hf_dict(), "cpu", torch.float32)
    hf.load_state_dict(model.state_dict(), strict=False)
    cands = (1099, 372)

    def hf_loss(m, b):
        logits = m(input_ids=b.input_ids.long()).logits[:, -1, :]
        return F.cross_entropy(logits[:, list(cands)], b.labels.long())

    def z_fn(name, p, seed):
        piece = model.arena.pieces[model.arena.index[name]]
        return torch.from_numpy(philox.gaussian(seed, piece.tensor_id, piece.numel)).view(p.shape)

    return cfg, model, hf, cands, hf_loss, z_fn


def test_zo_sgd_tracks_oracle():
    cfg, model, hf, cands, hf_loss, z_fn = _setup()
    seeds = iter([11, 22, 33, 44, 55, 66, 77, 88])
    oracle = TorchMeZO(hf, eps=1e-3, z_fn=z_fn, seed_fn=lambda: next(seeds), loss_fn=hf_loss)
    # same trainable set: everything but the tied token embedding
    assert [n for n, _ in oracle.named] == [n for n in model.hf_order if n in set(model.trainable_names)]
    for mode in ("inflight",):
        eng = ZOEngine(model, eps=1e-3, mode=mode)
        for step, seed in enumerate([11, 22, 33, 44, 55, 66, 77, 88]):
            b = synthetic_batch(step, 8, 32, cfg.vocab_size, cand_ids=cands)
            l_ref = oracle.step(b, lr=1e-4).item()
            l_new = eng.step(b, 1e-4, seed).item()
            assert abs(l_ref - l_new) < 2e-5, (step, l_ref, l_new)
            g_ref = None
        # parameters agree after 8 steps
        sd = dict(hf.named_parameters())
        for n in model.trainable_names:
            assert torch.allclose(model.param(n), sd[n], atol=2e-5), n


def test_inplace_mode_equals_inflight_in_fp32():
    cfg, model, _, cands, _, _ = _setup()
    other = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    a, b = ZOEngine(model, mode="inflight"), ZOEngine(other, mode="inplace")
    for step in range(4):
        batch = synthetic_batch(step, 8, 32, cfg.vocab_size, cand_ids=cands)
        la = a.step(batch, 1e-4, 100 + step).item()
        lb = b.step(batch, 1e-4, 100 + step).item()
        assert abs(la - lb) < 1e-5
    assert torch.allclose(model.arena.data, other.arena.data, atol=1e-6)


def test_dizo_gamma_search_tracks_oracle():
    cfg, model, hf, cands, hf_loss, z_fn = _setup()
    proj = DiZOProjector(model, max_iters=3)
    oracle = TorchMeZO(hf, eps=1e-3, dizo=True, z_fn=z_fn, loss_fn=hf_loss,
                       gamma_z_fn=lambda i, it: philox.scalar_gaussian(5, i, it))
    assert [n for n, _ in oracle.incl] == proj.include          # k_proj / v_proj weights only
    # move both models away from the anchor with a few identical ZO steps
    eng = ZOEngine(model, eps=1e-3)
    seeds = [3, 4, 5]
    it = iter(seeds)
    oracle.seed_fn = lambda: next(it)
    for step, seed in enumerate(seeds):
        b = synthetic_batch(step, 8, 32, cfg.vocab_size, cand_ids=cands)
        oracle.step(b, lr=5e-3)
        eng.step(b, 5e-3, seed)
    batches = [synthetic_batch(10 + i, 8, 32, cfg.vocab_size, cand_ids=cands) for i in range(3)]
    with torch.no_grad():
        oracle.dizo_search(batches)
    bi = iter(batches)
    proj.search_zo(lambda: next(bi), seed=5)
    ref_gamma = torch.cat([g.reshape(1) for g in oracle.gamma])
    assert torch.allclose(proj.gs.gamma, ref_gamma, rtol=2e-3, atol=1e-6), (proj.gs.gamma, ref_gamma)
    ts = proj.gs.ts
    assert (proj.gs.gamma >= 0.8 * ts - 1e-6).all() and (proj.gs.gamma <= 1.2 * ts + 1e-6).all()
    sd = dict(hf.named_parameters())
    for n in proj.include:
        delta = model.param(n) - model.arena.anchor_view(n)
        ref_delta = sd[n] - model.arena.anchor_view(n)
        assert ((delta - ref_delta).norm() / ref_delta.norm()).item() < 5e-3, n


def test_none_and_zo_enhanced_agree_before_first_projection():
    cfg, m1, _, cands, _, _ = _setup()
    m2 = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    DiZOProjector(m2)                                        # anchors taken, no projection yet
    e1, e2 = ZOEngine(m1), ZOEngine(m2)
    for step in range(5):
        b = synthetic_batch(step, 4, 16, cfg.vocab_size, cand_ids=cands)
        assert e1.step(b, 1e-4, step).item() == e2.step(b, 1e-4, step).item()


def test_loss_pair_equals_two_separate_forwards():
    """One sweep per block that stages theta + eps z and theta - eps z from one draw of z, then the block on both
    activation streams: the same two losses, bit for bit, as two forwards with +eps and -eps."""
    import torch
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.models.llama import LlamaModel, preset as llama_preset
    from dizo_b200.models.opt import OPTModel, Transform, preset
    for dtype in (torch.float32, torch.bfloat16):
        models = [OPTModel(preset("opt-tiny"), "cpu", dtype).init_random(0),
                  OPTModel(preset("opt-tiny"), "cpu", dtype, mode="lora+prefix", num_prefix=3).init_random(0),
                  OPTModel(preset("opt-tiny", do_layer_norm_before=False, word_embed_proj_dim=32), "cpu", dtype).init_random(0),
                  LlamaModel(llama_preset("llama-tiny-gqa"), "cpu", dtype).init_random(0)]
        for m in models:
            assert m.pair_supported()
            b = synthetic_batch(3, 4, 24, m.config.vocab_size, cand_ids=(10, 20), pad_left=5)
            l1 = m.loss(b, Transform(seed=77, coef=1e-2))
            l2 = m.loss(b, Transform(seed=77, coef=-1e-2))
            p1, p2 = m.loss_pair(b, 77, 1e-2)
            if m._shares_block_tail():
                # adapter-only training sends both streams through the frozen GEMMs together: on the CPU the BLAS
                # may block twice the rows differently (last bits); the GPU kernels are row-independent (exact
                # equality is asserted there)
                tol = dict(rtol=2e-6, atol=1e-7) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-3)
                assert torch.allclose(l1.reshape(1), p1.reshape(1), **tol) and torch.allclose(l2.reshape(1), p2.reshape(1), **tol)
            else:
                assert torch.equal(l1.reshape(1), p1.reshape(1)) and torch.equal(l2.reshape(1), p2.reshape(1)), (dtype, l1, p1, l2, p2)
            assert not torch.equal(p1.reshape(1), p2.reshape(1))
    assert not OPTModel(preset("opt-tiny"), "cpu", torch.float32, mode="prefix", prefix_reparam=True).pair_supported()
    # head tuning: nothing inside the decoder is perturbed, so the blocks run once for both sides
    for m in (OPTModel(preset("opt-tiny"), "cpu", torch.float32, mode="head").init_random(0),
              LlamaModel(llama_preset("llama-tiny"), "cpu", torch.float32, mode="head").init_random(0)):
        calls = []
        inner = m._layer_forward
        m._layer_forward = lambda *a, **k: (calls.append(1), inner(*a, **k))[1]
        b = synthetic_batch(3, 4, 24, m.config.vocab_size, cand_ids=(10, 20), pad_left=5)
        p1, p2 = m.loss_pair(b, 5, 1e-2)
        assert len(calls) == m.config.num_hidden_layers
        m._layer_forward = inner
        assert torch.equal(p1.reshape(1), m.loss(b, Transform(seed=5, coef=1e-2)).reshape(1))
        assert torch.equal(p2.reshape(1), m.loss(b, Transform(seed=5, coef=-1e-2)).reshape(1))
        assert not torch.equal(p1.reshape(1), p2.reshape(1))
