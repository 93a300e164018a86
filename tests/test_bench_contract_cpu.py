"""The benchmark's command-line contract and the reference-arm harness, as far as they can be checked
without a GPU: the reference's own hot loop is driven on a tiny CPU model, its files are compared byte for
byte with the source tree when that is present, and the arm answers with one JSON line and exit code 0
where it cannot run (no CUDA device; more than one GPU)."""
import filecmp
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _reference_line(*extra):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "3", *extra], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference"
    return rec


@pytest.mark.skipif(torch.cuda.is_available(), reason="on a GPU box the arm runs the reference instead")
def test_reference_arm_without_a_gpu_says_why():
    rec = _reference_line("--gpus", "1")
    assert "no CUDA device" in rec["unavailable"]


def test_reference_arm_declines_multi_gpu_with_the_reason():
    rec = _reference_line("--gpus", "2")
    assert "single-GPU" in rec["unavailable"] and "run.py:32" in rec["unavailable"]


def _harness():
    from baseline import ref_harness as H
    try:
        ref, shimmed = H.import_reference()
    except H.ReferenceUnavailable as e:
        pytest.skip(str(e))
    return H, ref, shimmed


def test_reference_copy_is_byte_identical_to_the_source_tree():
    H, _, _ = _harness()
    src = os.environ.get("DIZO_REFERENCE_SRC", "/root/reference/large_models")
    if not os.path.isdir(src):
        pytest.skip("no reference source tree on this machine")
    for f in H.REF_FILES:
        assert filecmp.cmp(os.path.join(src, f), os.path.join(H.REF_DIR, f), shallow=False), f


def test_reference_hot_loop_runs_unmodified_on_cpu():
    """zo_step / zo_update of the reference's own OurTrainer move the trainable tensors, keep the token
    embedding fixed (it is dropped from the ZO set), and follow the 0.5-decay LR lambda."""
    H, ref, shimmed = _harness()
    assert "transformers.trainer_pt_utils._get_learning_rate" in shimmed or hasattr(ref.OurTrainer, "_get_learning_rate")
    model = H.build_hf_opt("opt-tiny", "cpu", torch.float32, vocab=512)
    tr = H.make_reference_trainer(ref, model, "cpu", lr=1e-3, max_steps=100, zo_eps=1e-3, enhanced=None)
    assert type(tr).__module__ == "trainer" and type(tr).zo_step.__code__.co_filename.startswith(H.REF_DIR)
    assert all("embed_tokens" not in n for n, _ in tr.named_parameters_to_optim)
    w0 = model.model.decoder.layers[0].fc1.weight.detach().clone()
    e0 = model.model.decoder.embed_tokens.weight.detach().clone()
    np.random.seed(0)
    for s in range(3):
        b = H.reference_batch(s, 4, 16, 512)
        b["input_ids"][:, -1] %= 512
        assert b["input_ids"].shape == (8, 16) and b["num_options"].tolist() == [2] * 8
        loss = float(H.reference_step(tr, b))
        assert np.isfinite(loss)
    assert tr.state.global_step == 3
    assert abs(tr._get_learning_rate() - 1e-3 * (1 - 2 / 200)) < 1e-9
    assert (model.model.decoder.layers[0].fc1.weight - w0).abs().max() > 0
    assert (model.model.decoder.embed_tokens.weight - e0).abs().max() == 0


def test_build_entry_point_compiles_and_imports():
    import importlib.util
    spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(ROOT, "__graft_entry__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()                                   # nvcc cross-compiles for sm_100a without a GPU
    assert os.path.exists(os.path.join(ROOT, "dizo_b200", "ops", "libdizo_b200.so"))
