"""End-to-end runs of the command-line entry on the GPU: ZO / DiZO (gamma by ZO and by FO),
LoRA + prefix, evaluation, generation, checkpoint round trip."""
import json
import os

import pytest
import torch

from dizo_b200.models.generate import generate
from dizo_b200.models.opt import OPTModel, preset
from dizo_b200.ops import _lib
from dizo_b200.run import main

pytestmark = pytest.mark.gpu


def _common(tmp, *extra):
    return ["--task_name", "Synthetic", "--model_name", "opt-125m", "--random_init", "--trainer", "zo", "--num_train", "32",
            "--num_dev", "8", "--num_eval", "16", "--train_set_seed", "0", "--max_steps", "6",
            "--learning_rate", "1e-5", "--per_device_train_batch_size", "8", "--train_as_classification",
            "--output_dir", str(tmp / "out"), "--save_steps", "0", "--zo_eval_steps", "3", "--max_length", "64",
            "--dizo_interval", "3", "--dizo_max_iters", "2", *extra]


@pytest.mark.parametrize("extra", [
    ("--enhanced", "zo"),
    ("--enhanced", "fo"),
    ("--lora", "--prefix_tuning", "--enhanced", "zo"),
    ("--head_tuning",),
    ("--zo_mode", "inplace", "--zo_stochastic_rounding"),
])
def test_cli_training_runs_on_gpu(tmp_path, monkeypatch, extra):
    monkeypatch.chdir(tmp_path)
    assert main(_common(tmp_path, *extra)) == 0
    torch.cuda.synchronize()
    _lib.check_device_errors()
    res = [f for f in os.listdir(tmp_path / "result") if f.endswith(".json")]
    m = json.load(open(tmp_path / "result" / res[0]))
    assert 0.0 <= m["accuracy"] <= 1.0 and "dev_accuracy" in m


def test_first_order_trainer_runs_on_gpu(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    args = _common(tmp_path, "--gradient_accumulation_steps", "2", "--evaluation_strategy", "steps", "--eval_steps", "3")
    args[args.index("--trainer") + 1] = "regular"
    assert main(args) == 0
    torch.cuda.synchronize()
    _lib.check_device_errors()
    res = [f for f in os.listdir(tmp_path / "result") if f.endswith(".json")]
    assert 0.0 <= json.load(open(tmp_path / "result" / res[0]))["accuracy"] <= 1.0


def test_profiled_steps_report_phase_times(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    mj = tmp_path / "metrics.jsonl"
    assert main(_common(tmp_path, "--enhanced", "zo", "--profile_steps", "1:4", "--metrics_jsonl", str(mj))) == 0
    recs = [json.loads(l) for l in open(mj)]
    prof = [r for r in recs if "forwards_ms" in r]
    assert len(prof) == 3 and all(r["forwards_ms"] > 0 and r["update_ms"] > 0 for r in prof)
    assert any("update_gbs" in r for r in prof) and any("projection" in r for r in recs)


def test_lm_style_training_and_resume_on_gpu(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    args = _common(tmp_path)
    args.remove("--train_as_classification")
    i = args.index("--save_steps")
    args[i + 1] = "4"
    assert main(args) == 0
    assert os.path.isdir(tmp_path / "out" / "checkpoint-4")
    args[args.index("--max_steps") + 1] = "8"
    assert main(args) == 0                      # resumes from checkpoint-4 automatically
    assert os.path.isdir(tmp_path / "out" / "checkpoint-8")


def test_generation_on_gpu_matches_cpu_model():
    cfg = preset("opt-125m", num_hidden_layers=2)
    cpu = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    gpu = OPTModel(cfg, "cuda", torch.bfloat16)
    gpu.load_state_dict(cpu.state_dict())
    cpu.load_state_dict({k: v.float() for k, v in gpu.state_dict().items()})
    ids = torch.randint(4, cfg.vocab_size, (2, 12), generator=torch.Generator().manual_seed(0))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[1, :3] = 0
    a = generate(gpu, ids, mask, max_new_tokens=4)
    b = generate(cpu, ids, mask, max_new_tokens=4)
    # greedy tokens can differ where two logits are within bf16 noise; the first ones must agree
    assert a[0][:13] == b[0][:13] and a[1][:10] == b[1][:10]
    s = generate(gpu, ids, mask, max_new_tokens=4, do_sample=True, top_k=20, top_p=0.9, temperature=0.8, seed=5)
    assert all(len(x) >= 9 for x in s)
    beams = generate(gpu, ids, mask, max_new_tokens=3, num_beams=2)
    assert len(beams) == 2
    torch.cuda.synchronize()
    _lib.check_device_errors()
