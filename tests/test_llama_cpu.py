"""LLaMA-family model (RMSNorm, rotary embedding, grouped-query attention, SwiGLU) against the Hugging Face
implementation on CPU in fp32, and through the command line (ZO training, head / prefix modes, checkpoints)."""
import json

import pytest
import torch

from dizo_b200.models.generate import generate
from dizo_b200.models.llama import LlamaConfig, LlamaModel, preset
from dizo_b200.models.opt import Transform, make_batch
from dizo_b200.ops import llama as llama_ops
from dizo_b200.run import main

transformers = pytest.importorskip("transformers")


def _hf(cfg, seed=0):
    torch.manual_seed(seed)
    kw = {k: v for k, v in cfg.to_hf_dict().items() if k != "architectures"}
    return transformers.LlamaForCausalLM(transformers.LlamaConfig(**kw)).eval()


def _inputs(cfg, B=3, L=17):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(3, cfg.vocab_size, (B, L), generator=g)
    mask = torch.ones_like(ids)
    mask[1, :5] = 0
    ids[1, :5] = 0
    return ids, mask


@pytest.mark.parametrize("name", ["llama-tiny", "llama-tiny-gqa"])
def test_logits_equal_hugging_face(name):
    cfg = preset(name)
    hf = _hf(cfg)
    m = LlamaModel(cfg, "cpu", torch.float32)
    assert m.load_state_dict(hf.state_dict()) == []
    assert m.hf_order == [n for n, _ in hf.named_parameters()]
    ids, mask = _inputs(cfg)
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask).logits
    got = m.logits(make_batch(ids, mask)).view(*ids.shape, -1)
    keep = mask.bool()
    assert (got[keep] - ref[keep]).abs().max().item() < 1e-5


def test_greedy_generation_equals_hugging_face():
    cfg = preset("llama-tiny-gqa")
    hf = _hf(cfg)
    m = LlamaModel(cfg, "cpu", torch.float32)
    m.load_state_dict(hf.state_dict())
    ids, mask = _inputs(cfg, L=9)
    ref = hf.generate(input_ids=ids, attention_mask=mask, max_new_tokens=8, do_sample=False, pad_token_id=0,
                      eos_token_id=None)
    got = generate(m, ids, mask, max_new_tokens=8, pad_token_id=0)
    for r, g, mk in zip(ref, got, mask):
        assert r[mk.shape[0] - int(mk.sum()):].tolist() == g


def test_rotary_statement_and_table():
    """rope_qkv's statement against Hugging Face's apply_rotary_pos_emb; head expansion for grouped queries."""
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    H, Hkv, hd, L, B = 4, 2, 16, 7, 2
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B * L, (H + 2 * Hkv) * hd, generator=g)
    out = llama_ops.rope_qkv(x, L, 3, H, Hkv, hd, 10000.0).view(B, L, 3, H, hd)
    pos = (3 + torch.arange(L)).float()
    inv = 10000.0 ** (-torch.arange(0, hd, 2).float() / hd)
    ang = torch.cat([pos[:, None] * inv, pos[:, None] * inv], dim=-1)         # [L, hd]
    cos, sin = ang.cos()[None], ang.sin()[None]
    q = x[:, :H * hd].view(B, L, H, hd).transpose(1, 2)
    k = x[:, H * hd:(H + Hkv) * hd].view(B, L, Hkv, hd).transpose(1, 2)
    v = x[:, (H + Hkv) * hd:].view(B, L, Hkv, hd)
    qr, kr = apply_rotary_pos_emb(q, k, cos, sin)
    assert torch.allclose(out[:, :, 0], qr.transpose(1, 2), atol=1e-5)
    assert torch.allclose(out[:, :, 1], kr.transpose(1, 2).repeat_interleave(H // Hkv, dim=2), atol=1e-5)
    assert torch.equal(out[:, :, 2], v.repeat_interleave(H // Hkv, dim=2))


def test_trainable_sets_and_transform():
    cfg = preset("llama-tiny")
    m = LlamaModel(cfg, "cpu", torch.float32).init_random(0)
    # full fine-tuning perturbs every tensor, the token table included
    assert set(m.trainable_names) == set(m.hf_order) and m.EMBED in m.trainable_names
    assert all("k_proj" in n or "v_proj" in n for n in m.dizo_include_names())
    assert len(m.dizo_include_names()) == 2 * cfg.num_hidden_layers
    head = LlamaModel(cfg, "cpu", torch.float32, mode="head")
    assert head.trainable_names == ["lm_head.weight"]
    pre = LlamaModel(cfg, "cpu", torch.float32, mode="prefix", num_prefix=3)
    assert all("prefix_" in n for n in pre.trainable_names) and len(pre.trainable_names) == 2 * cfg.num_hidden_layers
    with pytest.raises(NotImplementedError):
        LlamaModel(cfg, "cpu", torch.float32, mode="lora")
    # a perturbed forward equals a forward of the explicitly perturbed parameters
    ids, mask = _inputs(cfg)
    b = make_batch(ids, mask, rows=torch.tensor([16, 33, 50], dtype=torch.int32),
                   targets=torch.tensor([5, 6, 7], dtype=torch.int32), seq_start=torch.tensor([0, 1, 2, 3], dtype=torch.int32),
                   ex_start=torch.tensor([0, 3], dtype=torch.int32), labels=torch.tensor([1], dtype=torch.int32))
    tr = Transform(seed=11, coef=1e-2)
    l_t = m.loss(b, tr)
    m.arena.sweep(seed1=11, c1=1e-2)
    l_p = m.loss(b)
    assert abs(float(l_t) - float(l_p)) < 1e-5 and abs(float(l_t) - float(LlamaModel(cfg, "cpu", torch.float32).init_random(0).loss(b))) > 1e-6


def test_prefix_rows_change_the_forward_and_positions_shift():
    cfg = preset("llama-tiny")
    base = LlamaModel(cfg, "cpu", torch.float32).init_random(0)
    pre = LlamaModel(cfg, "cpu", torch.float32, mode="prefix", num_prefix=3).init_random(0)
    pre.load_state_dict(base.state_dict(), strict=False)
    ids, mask = _inputs(cfg)
    a = base.logits(make_batch(ids, mask))
    b = pre.logits(make_batch(ids, mask))
    assert (a - b).abs().max().item() > 1e-4
    # real-activation initialisation: the prefix rows become K / V of random tokens (rotated as cached keys)
    from dizo_b200.models.peft import init_prefix_by_real_activations
    before = pre.param(pre.layer_prefix(0) + "self_attn.prefix_keys").clone()
    init_prefix_by_real_activations(pre, seed=0)
    assert not torch.equal(before, pre.param(pre.layer_prefix(0) + "self_attn.prefix_keys"))


def test_command_line_trains_saves_and_hugging_face_reloads(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    out = tmp_path / "run"
    rc = main(["--task_name", "Synthetic", "--model_name", "llama-tiny", "--random_init", "--trainer", "zo",
               "--num_train", "24", "--num_dev", "8", "--num_eval", "8", "--max_steps", "6", "--learning_rate", "1e-3",
               "--zo_eps", "1e-3", "--per_device_train_batch_size", "4", "--output_dir", str(out), "--save_model",
               "--enhanced", "zo", "--dizo_interval", "3", "--dizo_max_iters", "2", "--train_as_classification",
               "--train_set_seed", "0"])
    assert rc == 0
    with open(out / "config.json") as f:
        assert json.load(f)["model_type"] == "llama"
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(out))
    cfg = LlamaConfig.from_hf(hf.config)
    m = LlamaModel(cfg, "cpu", torch.float32)
    m.load_state_dict(hf.state_dict())
    ids, mask = _inputs(cfg)
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask).logits
    got = m.logits(make_batch(ids, mask)).view(*ids.shape, -1)
    assert (got[mask.bool()] - ref[mask.bool()]).abs().max().item() < 1e-4
    # the saved directory is a checkpoint the loader accepts (config.json with model_type llama)
    rc = main(["--task_name", "Synthetic", "--model_name", str(out), "--num_train", "0", "--num_eval", "4",
               "--output_dir", str(tmp_path / "eval"), "--head_tuning", "--trainer", "none"])
    assert rc == 0


@pytest.mark.parametrize("name,mode", [("llama-tiny-gqa", "full"), ("llama-tiny", "prefix")])
def test_autograd_statement_equals_the_forward_and_differentiates_alpha(name, mode):
    """The differentiable statement used by --enhanced fo / --trainer regular: same loss as the forward of the
    engine, and d loss / d alpha (blend of k / v weights with their anchors) equal to central differences."""
    from dizo_b200.engine import DiZOProjector
    from dizo_b200.models.opt_autograd import functional_loss, make_fo_loss
    cfg = preset(name)
    m = LlamaModel(cfg, "cpu", torch.float32, mode=mode, num_prefix=3).init_random(0)
    ids, mask = _inputs(cfg)
    b = make_batch(ids, mask, rows=torch.tensor([16, 33, 50], dtype=torch.int32),
                   targets=torch.tensor([5, 6, 7], dtype=torch.int32), seq_start=torch.tensor([0, 1, 2, 3], dtype=torch.int32),
                   ex_start=torch.tensor([0, 3], dtype=torch.int32), labels=torch.tensor([1], dtype=torch.int32))
    assert abs(float(functional_loss(m, b, use_checkpoint=False)) - float(m.loss(b))) < 1e-5
    if mode != "full":
        return
    proj = DiZOProjector(m)
    g = torch.Generator().manual_seed(3)
    for n in m.arena.slot_names:
        m.param(n).add_(torch.randn(m.param(n).shape, generator=g) * 0.05)
    fo = make_fo_loss(m)
    alpha = torch.full((proj.n,), 0.8, dtype=torch.float32).requires_grad_(True)
    fo(b, alpha).backward()
    for s in (0, proj.n - 1):
        e = torch.zeros(proj.n)
        e[s] = 1e-2
        with torch.no_grad():
            fd = (float(fo(b, alpha.detach() + e)) - float(fo(b, alpha.detach() - e))) / 2e-2
        assert abs(fd - float(alpha.grad[s])) < 2e-3 * max(1.0, abs(fd)), (s, fd, float(alpha.grad[s]))


@pytest.mark.parametrize("extra", [("--trainer", "zo", "--enhanced", "fo", "--dizo_interval", "2", "--dizo_max_iters", "2"),
                                   ("--trainer", "regular", "--learning_rate", "1e-3")])
def test_command_line_first_order_paths(tmp_path, monkeypatch, extra):
    monkeypatch.chdir(tmp_path)
    rc = main(["--task_name", "Synthetic", "--model_name", "llama-tiny", "--random_init",
               "--num_train", "16", "--num_dev", "4", "--num_eval", "4", "--max_steps", "4",
               "--per_device_train_batch_size", "4", "--output_dir", str(tmp_path / "run"),
               "--train_as_classification", "--train_set_seed", "0", *extra])
    assert rc == 0


def test_fused_projection_entry_points_have_cpu_statements():
    """gemm.linear_swiglu / gemm.linear_qkv_rope (GEMM epilogues on the device) fall back to GEMM + elementwise here."""
    from dizo_b200.ops import gemm
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 32, generator=g)
    w = torch.randn(2 * 48, 32, generator=g) * 0.2
    acc = x @ w.t()
    assert torch.allclose(gemm.linear_swiglu(x, w), torch.nn.functional.silu(acc[:, :48]) * acc[:, 48:], atol=1e-5)
    H, Hkv, hd, L = 4, 2, 16, 3
    wq = torch.randn((H + 2 * Hkv) * hd, 32, generator=g) * 0.2
    got = gemm.linear_qkv_rope(x, wq, L, 2, H, Hkv, hd, 10000.0)
    want = llama_ops.rope_qkv_reference(x @ wq.t(), L, 2, H, Hkv, hd, 10000.0)
    assert got.shape == (6, 3 * H * hd) and torch.allclose(got, want, atol=1e-5)
