"""Trainer loop, evaluation, checkpoints / exact resume, PEFT modes, generation (CPU, tiny model)."""
import json
import os
import random

import numpy as np
import pytest
import torch

from dizo_b200.args import OurArguments
from dizo_b200.data.batching import batch_from_inputs
from dizo_b200.evaluation import Evaluator
from dizo_b200.models.generate import filter_logits, generate
from dizo_b200.models.opt import OPTModel, make_batch, preset
from dizo_b200.models.peft import init_prefix_by_real_activations
from dizo_b200.run import main, result_file_tag
from dizo_b200.tasks import SyntheticDataset
from dizo_b200.trainer import OurTrainer
from dizo_b200.utils import (DataCollatorWithPaddingAndNesting, DataCollatorForTokenClassification,
                             SIGUSR1Callback, StubTokenizer, encode_prompt)
from dizo_b200.utils.checkpoint import (CheckpointError, get_last_checkpoint, load_checkpoint,
                                        save_checkpoint, verify_checkpoint)


def _args(tmp, **kw):
    base = dict(trainer="zo", learning_rate=1e-3, max_steps=8, zo_eps=1e-3, per_device_train_batch_size=4,
                train_as_classification=True, zo_eval_steps=1000, zo_log_steps=4, output_dir=str(tmp),
                save_steps=0, task_name="Synthetic", model_name="opt-tiny", max_length=64, seed=3)
    base.update(kw)
    return OurArguments(**base)


def _trainer(tmp, mode="full", **kw):
    random.seed(0)
    np.random.seed(kw.get("seed", 3))
    args = _args(tmp, **kw)
    task = SyntheticDataset(n_train=64, n_valid=16)
    tok = StubTokenizer(["terrible", "great", "It", "was", "fine", "dull", "film"])
    cfg = preset("opt-tiny")
    model = OPTModel(cfg, "cpu", torch.float32, mode=mode).init_random(0)
    feats = []
    for smp in task.samples["train"]:
        enc, ol = encode_prompt(task, task.get_template(), [], smp, tok, max_length=64)
        gold = smp.candidates.index(smp.correct_candidate)
        if args.train_as_classification:
            feats.append([{"input_ids": enc[i], "labels": gold, "option_len": ol[i], "num_options": 2} for i in range(2)])
        else:
            feats.append({"input_ids": enc[gold], "labels": enc[gold], "option_len": ol[gold]})
    coll = DataCollatorWithPaddingAndNesting(tok, pad_to_multiple_of=8) if args.train_as_classification \
        else DataCollatorForTokenClassification(tok, pad_to_multiple_of=8)
    return OurTrainer(model, args, train_dataset=feats, eval_dataset=task.samples["valid"],
                      processing_class=tok, data_collator=coll, task=task), task, tok


def test_verbalizer_shortcut_equals_general_loss(tmp_path):
    tr, task, tok = _trainer(tmp_path)
    inputs = tr.data_collator(tr.train_dataset[:4])
    short = batch_from_inputs(inputs, tok.pad_token_id)
    full = batch_from_inputs(inputs, tok.pad_token_id, verbalizer_shortcut=False)
    assert short.cand_ids is not None and short.input_ids.shape[0] == 4 and full.input_ids.shape[0] == 8
    assert abs(tr.model.loss(short).item() - tr.model.loss(full).item()) < 1e-5


def test_lm_style_rows_and_pad_handling():
    ids = torch.tensor([[1, 1, 2, 7, 8, 9], [2, 5, 6, 7, 8, 9]])
    mask = (ids != 1).long()
    b = batch_from_inputs({"input_ids": ids, "attention_mask": mask, "labels": ids, "option_len": [2, 3]}, 1,
                          classification=False)
    assert b.rows.tolist() == [3, 4, 6 + 2, 6 + 3, 6 + 4] and b.targets.tolist() == [8, 9, 7, 8, 9]
    assert b.pad_left.tolist() == [2, 0] and b.positions[0].tolist() == [1, 1, 2, 3, 4, 5]


def test_train_logs_lr_schedule_and_reduces_loss(tmp_path):
    tr, _, _ = _trainer(tmp_path, max_steps=40, learning_rate=2e-3)
    tr.train_dataset = tr.train_dataset[:4]          # one fixed batch: the loss must go down
    out = tr.train()
    assert tr.state.global_step == 40 and len(tr.loss_list) == 40
    logs = [r for r in tr.state.log_history if "lr" in r]
    # lr at logged step s is lr0 * (1 - s / (2 * max_steps))
    assert logs[0]["step"] == 4 and logs[0]["lr"] == pytest.approx(2e-3 * (1 - 4 / 80))
    assert np.mean(tr.loss_list[-10:]) < np.mean(tr.loss_list[:10]) - 0.01
    assert out["train_tokens_per_second"] > 0


def test_checkpoint_resume_is_exact(tmp_path):
    a, _, _ = _trainer(tmp_path / "a", max_steps=12, enhanced="zo", dizo_interval=5, dizo_max_iters=2)
    a.train()
    b, _, _ = _trainer(tmp_path / "b", max_steps=12, enhanced="zo", dizo_interval=5, dizo_max_iters=2,
                       save_steps=7)
    from dizo_b200.utils import TrainerCallback

    class StopAt7(TrainerCallback):
        def on_step_end(self, args, state, control, **kw):
            if state.global_step == 7:
                control.should_training_stop = True
    b.add_callback(StopAt7())
    b.train()
    ck = get_last_checkpoint(str(tmp_path / "b"))
    assert ck.endswith("checkpoint-7")
    c, _, _ = _trainer(tmp_path / "b", max_steps=12, enhanced="zo", dizo_interval=5, dizo_max_iters=2)
    np.random.seed(12345)                      # resume must restore the seed stream itself
    c.train(resume_from_checkpoint=ck)
    assert c.state.global_step == 12
    assert torch.equal(c.model.arena.data, a.model.arena.data)
    assert c.loss_list == a.loss_list


def test_corrupted_checkpoint_is_detected(tmp_path):
    tr, _, _ = _trainer(tmp_path)
    out = str(tmp_path / "ck")
    save_checkpoint(out, tr.model, trainer=tr)
    verify_checkpoint(out)
    p = os.path.join(out, "model.safetensors")
    data = open(p, "rb").read()
    open(p, "wb").write(data[:len(data) // 2])
    with pytest.raises(CheckpointError, match="truncated"):
        load_checkpoint(out, tr.model)
    open(p, "wb").write(data[:-1] + bytes([data[-1] ^ 1]))
    with pytest.raises(CheckpointError, match="corrupted"):
        load_checkpoint(out, tr.model)
    os.remove(os.path.join(out, "manifest.json"))
    assert get_last_checkpoint(str(tmp_path)) is None


def test_hf_can_load_saved_checkpoint(tmp_path):
    from transformers import OPTForCausalLM
    tr, _, _ = _trainer(tmp_path)
    tr.save_model(str(tmp_path / "hf"))
    hf = OPTForCausalLM.from_pretrained(str(tmp_path / "hf")).eval()
    ids = torch.randint(4, 500, (2, 12))
    ref = hf(input_ids=ids).logits
    mine = tr.model.logits(make_batch(ids)).view(2, 12, -1)
    assert (ref - mine).abs().max().item() < 1e-4


def test_sharded_checkpoint_layout_loads_in_hf_and_lazily(tmp_path):
    from transformers import OPTForCausalLM
    tr, _, _ = _trainer(tmp_path)
    out = str(tmp_path / "sharded")
    save_checkpoint(out, tr.model, trainer=None, max_shard_bytes=200_000)
    files = sorted(os.listdir(out))
    shards = [f for f in files if f.startswith("model-") and f.endswith(".safetensors")]
    assert len(shards) >= 3 and "model.safetensors.index.json" in files and "model.safetensors" not in files
    assert shards[0] == f"model-00001-of-{len(shards):05d}.safetensors"
    verify_checkpoint(out)
    hf = OPTForCausalLM.from_pretrained(out).eval()
    ids = torch.randint(4, 500, (2, 12))
    assert (hf(input_ids=ids).logits - tr.model.logits(make_batch(ids)).view(2, 12, -1)).abs().max().item() < 1e-4
    m2 = OPTModel(preset("opt-tiny"), "cpu", torch.float32)
    load_checkpoint(out, m2)
    assert torch.equal(m2.arena.data, tr.model.arena.data)


def test_sigusr1_callback_saves_and_stops(tmp_path):
    tr, _, _ = _trainer(tmp_path, max_steps=50)
    cb = SIGUSR1Callback(exit_on_end=False)
    tr.add_callback(cb)
    orig = tr.zo_update

    def hooked(*a, **k):
        orig(*a, **k)
        if tr.state.global_step == 2:
            cb.handle_signal(None, None)
    tr.zo_update = hooked
    tr.train()
    assert tr.state.global_step == 3
    assert get_last_checkpoint(str(tmp_path)).endswith("checkpoint-3")


@pytest.mark.parametrize("mode", ["lora", "prefix", "lora+prefix", "head"])
def test_peft_modes_train_only_their_tensors(tmp_path, mode):
    tr, _, _ = _trainer(tmp_path, mode=mode, max_steps=3)
    m = tr.model
    frozen_before = m.frozen.data.clone()
    before = m.arena.data.clone()
    if "prefix" in mode:
        init_prefix_by_real_activations(m, seed=1)
    tr.train()
    assert torch.equal(m.frozen.data, frozen_before)
    assert not torch.equal(m.arena.data, before)
    names = set(m.trainable_names)
    if mode == "lora+prefix":
        assert any("lora_" in n for n in names) and any("prefix_" in n for n in names)
    if mode == "head":
        assert names == {"lm_head.weight"}
    assert m.num_parameters(True) < m.num_parameters()


def test_evaluator_matches_one_by_one_and_sfc(tmp_path):
    tr, task, tok = _trainer(tmp_path)
    ev = Evaluator(tr.model, tok, task, tr.args)
    samples = task.samples["valid"][:6]
    batched = ev.predict_many([[]], samples)
    single = [ev.one_step_pred([], s) for s in samples]
    assert [p.predicted_candidate for p in batched] == [p.predicted_candidate for p in single]
    demos = task.samples["train"][:2]
    icl = ev.evaluate(demos, samples)
    assert 0.0 <= icl["accuracy"] <= 1.0
    tr.args.sfc = True
    assert len(ev.predict_many([[]], samples)) == 6
    lp = ev.forward(tok.encode("the film It was great"), option_len=1)
    assert lp.shape == (1,) and lp.item() < 0


def test_generation_controls():
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32).init_random(1)
    ids = torch.randint(4, 500, (2, 6))
    greedy = generate(m, ids, max_new_tokens=5)
    again = generate(m, ids, max_new_tokens=5)
    assert greedy == again and all(len(g) == 11 for g in greedy)
    stop = greedy[0][6]
    cut = generate(m, ids[:1], max_new_tokens=5, eos_token_id=[stop])
    assert cut[0] == greedy[0][:7]                          # stops right after the EOS token
    s1 = generate(m, ids, max_new_tokens=5, do_sample=True, top_k=3, temperature=0.8, seed=4)
    s2 = generate(m, ids, max_new_tokens=5, do_sample=True, top_k=3, temperature=0.8, seed=4)
    assert s1 == s2
    lg = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert torch.isinf(filter_logits(lg, top_k=2)[0, :2]).all()
    kept = torch.isfinite(filter_logits(lg, top_p=0.7)[0])
    assert kept.tolist() == [False, False, True, True]


def test_run_main_end_to_end(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    rc = main(["--task_name", "Synthetic", "--model_name", "opt-tiny", "--random_init", "--trainer", "zo", "--num_train", "24",
               "--num_dev", "8", "--num_eval", "8", "--train_set_seed", "0", "--max_steps", "4",
               "--learning_rate", "1e-3", "--per_device_train_batch_size", "4", "--train_as_classification",
               "--enhanced", "zo", "--dizo_interval", "2", "--dizo_max_iters", "1", "--output_dir",
               str(tmp_path / "out"), "--save_steps", "0", "--zo_eval_steps", "2", "--max_length", "64",
               "--metrics_jsonl", str(tmp_path / "metrics.jsonl"), "--zo_log_steps", "2"])
    assert rc == 0
    recs = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    proj = [r for r in recs if "projection" in r]
    assert len(proj) == 2 and all(r["alpha_min"] <= r["alpha_mean"] <= r["alpha_max"] for r in proj)
    assert any("tokens_per_s" in r for r in recs)
    files = os.listdir(tmp_path / "result")
    assert any(f.endswith("trainset0.json") for f in files)
    m = json.load(open(tmp_path / "result" / files[0]))
    assert "accuracy" in m and "dev_accuracy" in m
    assert os.path.exists(tmp_path / "loss_acc" / "Synthetic_zo_ft_enhanced_zo" / "accuracy_seed_42.npy")
    # zero-shot / ICL path: one demonstration set per evaluation sample
    rc = main(["--task_name", "Synthetic", "--model_name", "opt-tiny", "--random_init", "--num_train", "2", "--num_eval", "4",
               "--max_length", "128"])
    assert rc == 0
    assert result_file_tag(OurArguments(task_name="X", model_name="a/b", num_train=3, tag="t")) == "X-b-ntrain3-t"


def test_lazy_weights_over_sharded_checkpoints(tmp_path):
    from safetensors.torch import save_file
    from dizo_b200.utils.checkpoint import LazyWeights, load_weights
    cfg = preset("opt-tiny")
    m = OPTModel(cfg, "cpu", torch.float32).init_random(1)
    sd = {k: v for k, v in m.state_dict().items() if k != "lm_head.weight"}
    names = sorted(sd)
    half = len(names) // 2
    for kind in ("safetensors", "bin"):
        d = tmp_path / kind
        os.makedirs(d)
        parts = {f"part-1.{kind}": names[:half], f"part-2.{kind}": names[half:]}
        for fn, ks in parts.items():
            if kind == "safetensors":
                save_file({k: sd[k].contiguous() for k in ks}, str(d / fn))
            else:
                torch.save({k: sd[k] for k in ks}, d / fn)
        idx = "model.safetensors.index.json" if kind == "safetensors" else "pytorch_model.bin.index.json"
        json.dump({"weight_map": {k: fn for fn, ks in parts.items() for k in ks}}, open(d / idx, "w"))
        lazy = load_weights(str(d), lazy=True)
        assert isinstance(lazy, LazyWeights) and set(lazy.keys()) == set(names) and len(lazy) == len(names)
        m2 = OPTModel(cfg, "cpu", torch.float32)
        assert m2.load_state_dict(lazy, strict=True) == []
        assert torch.equal(m2.arena.data, m.arena.data) and torch.equal(m2.frozen.data, m.frozen.data)
        full = load_weights(str(d))
        assert set(full) == set(names) and torch.equal(full[names[0]], lazy[names[0]])


def test_first_order_trainer_accumulation_equals_large_batch(tmp_path):
    """--trainer regular: two micro-batches of 2 accumulate to the step of one batch of 4; the loss
    falls; evaluation runs at the end of every epoch."""
    tr_a, _, _ = _trainer(tmp_path / "a", trainer="regular", learning_rate=1e-3, max_steps=6,
                          per_device_train_batch_size=4, lr_scheduler_type="constant", max_grad_norm=0.0)
    tr_b, _, _ = _trainer(tmp_path / "b", trainer="regular", learning_rate=1e-3, max_steps=6,
                          per_device_train_batch_size=2, gradient_accumulation_steps=2,
                          lr_scheduler_type="constant", max_grad_norm=0.0)
    ma, mb = tr_a.train(), tr_b.train()
    assert abs(ma["train_loss"] - mb["train_loss"]) < 1e-4
    # AdamW normalises the step, so elements whose gradient is at rounding level may move differently;
    # the trajectories as a whole coincide
    ref = OPTModel(preset("opt-tiny"), "cpu", torch.float32).init_random(0).arena.data
    da, db = tr_a.model.arena.data.detach() - ref, tr_b.model.arena.data.detach() - ref
    assert da.norm() > 0 and ((da - db).norm() / da.norm()).item() < 0.05
    tr_d, _, _ = _trainer(tmp_path / "d", trainer="regular", learning_rate=1e-3, max_steps=12,
                          per_device_train_batch_size=4, lr_scheduler_type="constant")
    tr_d.train_dataset = tr_d.train_dataset[:4]             # the same four examples every step
    tr_d.train()
    assert tr_d.loss_list[-1] < tr_d.loss_list[0] - 0.05
    tr_c, _, _ = _trainer(tmp_path / "c", trainer="regular", learning_rate=1e-3, max_steps=0, num_train_epochs=2,
                          per_device_train_batch_size=16, evaluation_strategy="epoch", zo_eval_steps=10 ** 6)
    tr_c.train()
    assert tr_c.state.global_step == 8 and len(tr_c.accuracy) == 2      # 64 examples / 16 = 4 steps per epoch


def test_linear_probing_end_to_end(tmp_path, monkeypatch):
    """--linear_probing: features from the forward, logistic regression on the host, coefficients
    written into the LM-head rows of the class tokens (large_models/trainer.py:855-957)."""
    monkeypatch.chdir(tmp_path)
    rc = main(["--task_name", "Synthetic", "--model_name", "opt-tiny", "--random_init", "--trainer", "zo", "--linear_probing",
               "--lp_early_stopping", "--num_train", "40", "--num_dev", "8", "--num_eval", "16",
               "--train_set_seed", "0", "--per_device_train_batch_size", "8", "--train_as_classification", "False",
               "--output_dir", str(tmp_path / "out"), "--max_length", "64", "--max_steps", "1"])
    assert rc == 0
    files = [f for f in os.listdir(tmp_path / "result") if f.endswith(".json")]
    assert 0.0 <= json.load(open(tmp_path / "result" / files[0]))["accuracy"] <= 1.0


def test_non_differentiable_objective_end_to_end(tmp_path, monkeypatch):
    """--non_diff on a generation task: the ZO loss is minus the F1 of decoded answers
    (large_models/trainer.py:1544-1568); data from $DIZO_DATA_DIR jsonl files."""
    d = tmp_path / "data" / "squad"
    os.makedirs(d)
    rng = random.Random(0)
    words = ["fine", "dull", "film", "cast", "plot", "warm", "cold", "score"]
    for split, n in (("train", 24), ("validation", 8)):
        with open(d / f"{split}.jsonl", "w") as f:
            for i in range(n):
                ctx = " ".join(rng.choice(words) for _ in range(8))
                ans = ctx.split()[rng.randrange(8)]
                f.write(json.dumps({"id": str(i), "title": "t", "context": ctx, "question": "which word ?",
                                    "answers": {"text": [ans], "answer_start": [0]}}) + "\n")
    monkeypatch.setenv("DIZO_DATA_DIR", str(tmp_path / "data"))
    monkeypatch.chdir(tmp_path)
    rc = main(["--task_name", "SQuAD", "--model_name", "opt-tiny", "--random_init", "--trainer", "zo", "--non_diff",
               "--num_train", "16", "--num_dev", "4", "--num_eval", "4", "--train_set_seed", "0", "--max_steps", "2",
               "--learning_rate", "1e-4", "--per_device_train_batch_size", "4", "--train_as_classification", "False",
               "--output_dir", str(tmp_path / "out"), "--max_length", "96", "--max_new_tokens", "3",
               "--zo_eval_steps", "1000", "--save_steps", "0"])
    assert rc == 0
    files = [f for f in os.listdir(tmp_path / "result") if f.endswith(".json")]
    m = json.load(open(tmp_path / "result" / files[0]))
    assert "f1" in m and 0.0 <= m["f1"] <= 1.0
