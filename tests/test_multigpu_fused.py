"""Fused compute+collective kernels on >= 2 GPUs (skipped on smaller boxes)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_collectives_match_nccl_compositions():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(ROOT, "tests", "multigpu_fused_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "FUSED_OK" in res.stdout, (res.stdout[-3000:], res.stderr[-3000:])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_switch_reduction_matches_nccl():
    """multimem.ld_reduce forms (norm all-reduce; GEMM -> reduce-scatter pulled through the switch); the worker
    reports success without checking anything where the symmetric region has no multicast mapping."""
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29536",
           os.path.join(ROOT, "tests", "multigpu_fused_worker.py"), "--multimem"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "FUSED_OK" in res.stdout, (res.stdout[-3000:], res.stderr[-3000:])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_model_matches_unsharded():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29534",
           os.path.join(ROOT, "tests", "multigpu_tp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "TP_OK" in res.stdout, (res.stdout[-3000:], res.stderr[-3000:])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp_model_matches_unsharded():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29535",
           os.path.join(ROOT, "tests", "multigpu_fsdp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "FSDP_OK" in res.stdout, (res.stdout[-3000:], res.stderr[-3000:])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("layout", [("--tp", "2"), ("--fsdp_shard",), ("--pp", "2"), ()])
def test_cli_training_on_two_gpus(tmp_path, layout):
    """The command-line entry under tensor parallelism, FSDP sharding, a pipeline and plain data parallelism:
    DiZO steps, in-loop evaluation, a checkpoint with full (unsharded) tensors, final metrics."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    out = tmp_path / "out"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29537", "-m", "dizo_b200.run",
           "--task_name", "Synthetic", "--model_name", "opt-125m", "--random_init", "--trainer", "zo", "--enhanced", "zo",
           "--num_train", "32", "--num_dev", "8", "--num_eval", "16", "--train_set_seed", "0",
           "--max_steps", "6", "--learning_rate", "1e-5", "--per_device_train_batch_size", "8",
           "--train_as_classification", "--output_dir", str(out), "--save_steps", "4",
           "--zo_eval_steps", "3", "--max_length", "64", "--dizo_interval", "3", "--dizo_max_iters", "2",
           *layout]
    res = subprocess.run(cmd, env=env, cwd=tmp_path, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, (res.stdout[-3000:], res.stderr[-3000:])
    ck = out / "checkpoint-4"
    assert (ck / "manifest.json").exists() and (ck / "zo_state.pt").exists()
    from dizo_b200.utils.checkpoint import load_weights
    sd = load_weights(str(ck))
    assert sd["model.decoder.layers.0.fc1.weight"].shape == (3072, 768)
    assert sd["model.decoder.layers.0.self_attn.k_proj.weight"].shape == (768, 768)
    assert any(f.endswith(".json") for f in os.listdir(tmp_path / "result"))
