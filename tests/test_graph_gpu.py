"""CUDA-graph replay of the ZO step: bitwise identical to the eager step, new seed / batch / learning
rate at every replay; the command-line flag goes through it."""
import json
import os
import time

import pytest
import torch

from dizo_b200.data.synthetic import synthetic_batch
from dizo_b200.engine import GraphedZOStep, ZOEngine
from dizo_b200.models.opt import OPTModel, preset
from dizo_b200.ops import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_graph_replay_equals_eager_steps():
    cfg = preset("opt-125m", num_hidden_layers=4)
    a = OPTModel(cfg, DEV, torch.bfloat16).init_random_fast(0)
    b = OPTModel(cfg, DEV, torch.bfloat16).init_random_fast(0)
    assert torch.equal(a.arena.data, b.arena.data)
    ea, eb = ZOEngine(a, eps=1e-3, dp_group=False), ZOEngine(b, eps=1e-3, dp_group=False)
    batches = [synthetic_batch(s, 4, 64, cfg.vocab_size).to(DEV) for s in range(5)]
    g = GraphedZOStep(eb, batches[0])
    assert torch.equal(a.arena.data, b.arena.data), "warm-up and capture must leave theta untouched"
    for s, bt in enumerate(batches):
        la = ea.step(bt, 1e-3 * (1 - s / 10), seed=100 + s).clone()
        lb = g(bt, 1e-3 * (1 - s / 10), seed=100 + s).clone()
        torch.cuda.synchronize()
        assert la.item() == lb.item(), (s, la, lb)
        assert torch.equal(a.arena.data, b.arena.data), s
    _lib.check_device_errors()
    # launch-bound model: the replay is faster than issuing the launches one by one
    def timed(fn, n=20):
        torch.cuda.synchronize()
        t = time.perf_counter()
        for i in range(n):
            fn(i)
        torch.cuda.synchronize()
        return (time.perf_counter() - t) / n * 1e3
    t_eager = timed(lambda i: ea.step(batches[i % 5], 0.0, seed=i))
    t_graph = timed(lambda i: g(batches[i % 5], 0.0, seed=i))
    print(f"opt-125m/4 layers, 4x64 tokens: eager {t_eager:.2f} ms, graph {t_graph:.2f} ms per step")
    assert t_graph < t_eager * 1.5          # generous: the point is equality above, speed is reported


def test_cli_flag_uses_graph(tmp_path, monkeypatch):
    from dizo_b200.run import main
    monkeypatch.chdir(tmp_path)
    args = ["--task_name", "Synthetic", "--model_name", "opt-125m", "--random_init", "--trainer", "zo", "--num_train", "32",
            "--num_dev", "8", "--num_eval", "16", "--train_set_seed", "0", "--max_steps", "6",
            "--learning_rate", "1e-5", "--per_device_train_batch_size", "8", "--train_as_classification",
            "--save_steps", "0", "--zo_eval_steps", "3", "--max_length", "64", "--enhanced", "zo",
            "--dizo_interval", "3", "--dizo_max_iters", "2"]
    res = {}
    for tag, extra in (("eager", []), ("graph", ["--zo_cuda_graph"])):
        out = tmp_path / tag
        assert main(args + ["--output_dir", str(out), "--tag", tag] + extra) == 0
        f = [x for x in os.listdir(tmp_path / "result") if tag in x][0]
        res[tag] = json.load(open(tmp_path / "result" / f))
    assert res["eager"]["accuracy"] == res["graph"]["accuracy"]
    assert res["eager"]["dev_accuracy"] == res["graph"]["dev_accuracy"]
