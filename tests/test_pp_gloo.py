"""Pipeline parallelism on CPU ranks (gloo): a 3-stage pipeline reproduces the single-process
losses and ZO + DiZO trajectory bit for bit in fp32, and gathers a full state dict."""
import textwrap

from test_dp_gloo import _run_ranks

PP_SCRIPT = textwrap.dedent('''
    import torch, torch.distributed as dist
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import ZOEngine, DiZOProjector
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.parallel.pp import PPOPTModel, stage_bounds
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = preset("opt-tiny", num_hidden_layers=4)
    assert stage_bounds(4, 3) == [(0, 2), (2, 3), (3, 4)]
    solo = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    pp = PPOPTModel(cfg, "cpu", torch.float32, micro_batches=2)
    pp.load_state_dict(solo.state_dict(), strict=False)
    assert pp.num_parameters() < solo.num_parameters()
    def batch(step, pad=0): return synthetic_batch(step, 5, 16, cfg.vocab_size, cand_ids=(10, 20), pad_left=pad)
    # plain and perturbed losses
    from dizo_b200.models.opt import Transform
    for tr in (None, Transform(seed=5, coef=1e-2)):
        a, b = solo.loss(batch(0, 3), tr), pp.loss(batch(0, 3), tr)
        # fp32 on both sides; the last block runs on the loss rows only, per micro-batch in the pipeline and
        # for the whole batch in the single process, so the BLAS sums may differ in the last bits
        assert torch.allclose(a.reshape(1), b.reshape(1), rtol=1e-5, atol=1e-6), (a, b)
    # ZO steps + a gamma search: identical trajectories, no parameter ever communicated
    e1, e2 = ZOEngine(solo, eps=1e-3, dp_group=False), ZOEngine(pp, eps=1e-3, dp_group=False)
    for step in range(4):
        l1 = e1.step(batch(step), 1e-3, seed=100 + step)
        l2 = e2.step(batch(step), 1e-3, seed=100 + step)
        assert abs(float(l1) - float(l2)) < 1e-5, (step, l1, l2)
    full = pp.gather_state_dict()
    ref = solo.state_dict()
    assert set(full) == set(ref)
    for k in ref:
        assert torch.allclose(full[k], ref[k], rtol=0, atol=1e-5), k
    p2 = DiZOProjector(pp, max_iters=2, dp_group=False)
    it = iter(range(100))
    p2.search_zo(lambda: batch(50 + next(it)), seed=9)
    lp = pp.row_logprobs(__import__("dizo_b200.data.batching", fromlist=["x"]).batch_from_inputs(
        dict(input_ids=batch(0).input_ids, labels=batch(0).input_ids.clone(), option_len=[3] * 5), pad_token_id=1))
    assert lp.numel() == 15 and torch.isfinite(lp).all()
    # decoding over the pipeline (every stage caches its own blocks): same tokens as the single process,
    # greedy with left padding and beams
    from dizo_b200.models.generate import generate
    solo2 = OPTModel(cfg, "cpu", torch.float32)
    solo2.load_state_dict(pp.gather_state_dict())
    ids = batch(7).input_ids[:, :9].long()
    mask = torch.ones_like(ids); mask[1, :3] = 0; ids[1, :3] = 1
    for kw in (dict(), dict(num_beams=2)):
        want = generate(solo2, ids, mask, max_new_tokens=5, **kw)
        got = generate(pp, ids, mask, max_new_tokens=5, **kw)
        assert want == got, (kw, want, got)
    print("PP_OK", rank)
''')


PP_LLAMA_SCRIPT = textwrap.dedent('''
    import torch, torch.distributed as dist
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import ZOEngine, DiZOProjector
    from dizo_b200.models.llama import LlamaModel, preset
    from dizo_b200.models.opt import Transform
    from dizo_b200.parallel.pp import PPLlamaModel
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    cfg = preset("llama-tiny-gqa", num_hidden_layers=3)
    for mode in ("full", "prefix"):
        solo = LlamaModel(cfg, "cpu", torch.float32, mode=mode, num_prefix=3).init_random(0)
        pp = PPLlamaModel(cfg, "cpu", torch.float32, micro_batches=2, mode=mode, num_prefix=3)
        pp.load_state_dict(solo.state_dict(), strict=False)
        assert pp.num_parameters() < solo.num_parameters()
        def batch(step, pad=0): return synthetic_batch(step, 5, 16, cfg.vocab_size, cand_ids=(10, 20), pad_left=pad)
        for tr in (None, Transform(seed=5, coef=1e-2)):
            a, b = solo.loss(batch(0, 3), tr), pp.loss(batch(0, 3), tr)
            assert torch.allclose(a.reshape(1), b.reshape(1), rtol=1e-5, atol=1e-6), (mode, a, b)
        e1, e2 = ZOEngine(solo, eps=1e-3, dp_group=False), ZOEngine(pp, eps=1e-3, dp_group=False)
        for step in range(3):
            l1 = e1.step(batch(step), 1e-3, seed=100 + step)
            l2 = e2.step(batch(step), 1e-3, seed=100 + step)
            assert abs(float(l1) - float(l2)) < 1e-5, (mode, step, l1, l2)
        full, ref = pp.gather_state_dict(), solo.state_dict()
        assert set(full) == set(ref)
        for k in ref:
            assert torch.allclose(full[k], ref[k], rtol=0, atol=1e-5), k
    p2 = DiZOProjector(pp, max_iters=2, dp_group=False) if mode == "full" else None
    from dizo_b200.models.generate import generate
    ids = batch(7).input_ids[:, :9].long()
    mask = torch.ones_like(ids); mask[1, :3] = 0; ids[1, :3] = 0
    want = generate(solo, ids, mask, max_new_tokens=5, pad_token_id=0)
    got = generate(pp, ids, mask, max_new_tokens=5, pad_token_id=0)
    assert want == got, (want, got)
    print("PP_OK", rank)
''')


def test_llama_pipeline_matches_single_process():
    outs = _run_ranks(PP_LLAMA_SCRIPT, 2)
    for rc, out in outs:
        assert rc == 0 and "PP_OK" in out, out[-3000:]


def test_pipeline_matches_single_process():
    outs = _run_ranks(PP_SCRIPT, 3)
    for rc, out in outs:
        assert rc == 0 and "PP_OK" in out, out[-3000:]


CLI_SCRIPT = textwrap.dedent('''
    import os, sys, tempfile, torch
    import torch.distributed as dist
    from dizo_b200.run import main
    tmp = os.environ["PP_TMP"]
    os.chdir(tmp)
    rc = main(["--task_name", "Synthetic", "--model_name", "opt-tiny", "--random_init", "--trainer", "zo", "--enhanced", "zo",
               "--num_train", "16", "--num_dev", "4", "--num_eval", "8", "--train_set_seed", "0", "--max_steps", "4",
               "--learning_rate", "1e-4", "--per_device_train_batch_size", "4", "--train_as_classification",
               "--output_dir", os.path.join(tmp, "out"), "--save_steps", "2", "--zo_eval_steps", "2",
               "--max_length", "32", "--dizo_interval", "2", "--dizo_max_iters", "2", "--pp", "2",
               "--load_best_model_at_end"])
    assert rc == 0
    print("CLI_OK", dist.get_rank())
''')


def test_cli_training_over_a_pipeline(tmp_path):
    import os
    outs = _run_ranks(CLI_SCRIPT, 2, extra_env={"PP_TMP": str(tmp_path)})
    for rc, out in outs:
        assert rc == 0 and "CLI_OK" in out, out[-3000:]
    ck = tmp_path / "out" / "checkpoint-4"
    assert (ck / "manifest.json").exists()
    from dizo_b200.utils.checkpoint import load_weights
    sd = load_weights(str(ck))
    assert "model.decoder.layers.0.fc1.weight" in sd and "model.decoder.final_layer_norm.weight" in sd
    # the checkpoint holds full tensors: it loads into a single-process model (another layout) as it is
    import torch
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.utils.checkpoint import load_checkpoint
    solo = OPTModel(preset("opt-tiny"), "cpu", torch.float32)
    missing = solo.load_state_dict(sd, strict=True)
    assert not missing
    load_checkpoint(str(ck), solo)
    assert torch.equal(solo.param("model.decoder.layers.1.fc2.weight"), sd["model.decoder.layers.1.fc2.weight"])
    assert any(f.endswith(".json") for f in os.listdir(tmp_path / "result"))


NONDIFF_SCRIPT = textwrap.dedent('''
    import os, json, torch
    import torch.distributed as dist
    from dizo_b200.run import main
    tmp = os.environ["PP_TMP"]
    os.chdir(tmp)
    rc = main(["--task_name", "SQuAD", "--model_name", "opt-tiny", "--random_init", "--trainer", "zo", "--non_diff",
               "--num_train", "8", "--num_dev", "4", "--num_eval", "4", "--train_set_seed", "0", "--max_steps", "2",
               "--learning_rate", "1e-4", "--per_device_train_batch_size", "4", "--train_as_classification", "False",
               "--output_dir", os.path.join(tmp, "out"), "--max_length", "96", "--max_new_tokens", "3",
               "--zo_eval_steps", "1000", "--save_steps", "0", "--pp", "2"])
    assert rc == 0
    print("NONDIFF_OK", dist.get_rank())
''')


def test_non_differentiable_objective_over_a_pipeline(tmp_path):
    """--non_diff with the blocks spread over two ranks: the ZO loss decodes answers on the sharded model
    (large_models/trainer.py:1544-1568 needs `model.generate`; here every stage caches its own blocks)."""
    import json
    import os
    import random
    d = tmp_path / "data" / "squad"
    os.makedirs(d)
    rng = random.Random(0)
    words = ["fine", "dull", "film", "cast", "plot", "warm", "cold", "score"]
    for split, n in (("train", 16), ("validation", 8)):
        with open(d / f"{split}.jsonl", "w") as f:
            for i in range(n):
                ctx = " ".join(rng.choice(words) for _ in range(8))
                ans = ctx.split()[rng.randrange(8)]
                f.write(json.dumps({"id": str(i), "title": "t", "context": ctx, "question": "which word ?",
                                    "answers": {"text": [ans], "answer_start": [0]}}) + "\n")
    outs = _run_ranks(NONDIFF_SCRIPT, 2, extra_env={"PP_TMP": str(tmp_path), "DIZO_DATA_DIR": str(tmp_path / "data")})
    for rc, out in outs:
        assert rc == 0 and "NONDIFF_OK" in out, out[-3000:]
    files = [f for f in os.listdir(tmp_path / "result") if f.endswith(".json")]
    m = json.load(open(tmp_path / "result" / files[0]))
    assert "f1" in m and 0.0 <= m["f1"] <= 1.0
