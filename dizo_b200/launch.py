"""Environment-variable launchers: ``python -m dizo_b200.launch {dizo,finetune,finetune_fsdp,icl}``.

The reference is driven by four shell scripts that turn environment variables into a ``run.py``
command line (large_models/dizo.sh, finetune.sh, finetune_fsdp.sh, icl.sh): ``MODEL``, ``TASK``,
``MODE`` in {ft, lora, prefix}, ``ENHANCED`` in {None, zo, fo}, ``BS``, ``LR``, ``EPS``, ``SEED``,
``TRAIN`` / ``DEV`` / ``EVAL``, ``STEPS`` / ``EVAL_STEPS`` (ZO) or ``EPOCH`` (first order),
``NUM_GPU``.  This module accepts the same variables with the same defaults and per-task rules
(CB and Copa use 100 dev examples; Copa, ReCoRD, DROP and SQuAD train as language modelling, not
classification; the first-order recipe splits MultiRC / ReCoRD / DROP batches into gradient
accumulation steps), builds the argument list for :mod:`dizo_b200.run` and runs it - in this
process for one GPU, through ``torch.distributed.run`` (one process per GPU, rendezvous on
127.0.0.1) for ``NUM_GPU`` > 1.  Extra command-line arguments are passed through.

Additions: ``PARALLEL`` in {dp, fsdp, tp, pp} selects the multi-GPU layout of the ZO recipes (the
reference has none), and ``finetune_fsdp`` maps to the sharded layout of this framework.
"""
from __future__ import annotations

import os
import subprocess
import sys
from typing import Dict, List, Mapping, Optional

_LM_TASKS = ("Copa", "ReCoRD", "DROP", "SQuAD")
_SMALL_DEV = ("CB", "Copa")
_FO_MICRO_BATCH = {"MultiRC": 2, "ReCoRD": 2, "DROP": 1}      # largest micro-batch of the FO recipe


def _mode_args(mode: str) -> List[str]:
    if mode == "prefix":
        return ["--prefix_tuning", "--num_prefix", "5", "--no_reparam", "--prefix_init_by_real_act"]
    if mode == "lora":
        return ["--lora"]
    if mode == "ft":
        return []
    raise ValueError(f"MODE must be ft, lora or prefix, not {mode!r}")


def build_argv(recipe: str, env: Mapping[str, str]) -> List[str]:
    """Argument list for ``dizo_b200.run`` from the launcher environment."""
    e = lambda k, d: str(env.get(k, d))
    model = e("MODEL", "facebook/opt-13b" if recipe == "icl" else "facebook/opt-1.3b")
    short = model.rstrip("/").split("/")[-1]
    task = env.get("TASK")
    if not task:
        raise ValueError("TASK is not set")
    if recipe == "icl":
        return ["--model_name", model, "--task_name", task, "--output_dir", "result/tmp", "--tag", "icl",
                "--num_train", "32", "--num_eval", "1000", "--load_bfloat16", "--verbose"]
    mode = e("MODE", "ft")
    train, dev, ev = e("TRAIN", 1000), e("DEV", 500), e("EVAL", 1000)
    if task in _SMALL_DEV:
        dev = "100"
    task_args: List[str] = []
    classification = task not in _LM_TASKS
    if recipe == "dizo":
        bs, lr, eps, seed = e("BS", 16), e("LR", "1e-7"), e("EPS", "1e-3"), e("SEED", 26)
        steps, eval_steps = e("STEPS", 20000), e("EVAL_STEPS", 500)
        enhanced = e("ENHANCED", "None")
        tag = f"mezo-{mode}-{steps}-{bs}-{lr}-{eps}-{seed}"
        argv = ["--model_name", model, "--task_name", task, "--output_dir", f"result/{task}-{short}-{tag}",
                "--tag", tag, "--seed", seed, "--train_set_seed", seed, "--num_train", train, "--num_dev", dev,
                "--num_eval", ev, "--logging_steps", "10", "--max_steps", steps, "--trainer", "zo",
                "--load_bfloat16", "--learning_rate", lr, "--zo_eps", eps, "--per_device_train_batch_size", bs,
                "--lr_scheduler_type", "constant", "--load_best_model_at_end", "--evaluation_strategy", "steps",
                "--save_strategy", "steps", "--save_total_limit", "1", "--eval_steps", eval_steps,
                "--save_steps", eval_steps, "--enhanced", enhanced]
        par = e("PARALLEL", "dp")
        n = int(e("NUM_GPU", 1))
        if par == "tp" and n > 1:
            argv += ["--tp", str(n)]
        elif par == "fsdp" and n > 1:
            argv += ["--fsdp_shard"]
        elif par == "pp" and n > 1:
            argv += ["--pp", str(n)]
        elif par != "dp" and n > 1:
            raise ValueError(f"PARALLEL must be dp, fsdp, tp or pp, not {par!r}")
    elif recipe in ("finetune", "finetune_fsdp"):
        fsdp = recipe == "finetune_fsdp"
        epoch, bs, lr, seed = e("EPOCH", 5), int(e("BS", 8)), e("LR", "1e-5"), e("SEED", 0)
        tag = f"{'fsdp' if fsdp else 'ft'}-{mode}-{epoch}-{bs}-{lr}-{seed}"
        micro, accum = bs, 1
        if fsdp:
            micro, accum = 1, bs
        elif task in _FO_MICRO_BATCH:
            micro = min(bs, _FO_MICRO_BATCH[task])
            accum = max(1, bs // micro)
        argv = ["--model_name", model, "--task_name", task, "--output_dir", f"result/{task}-{short}-{tag}",
                "--tag", tag, "--train_set_seed", seed, "--num_train", train, "--num_dev", dev, "--num_eval", ev,
                "--logging_steps", "10", "--trainer", "regular", "--load_bfloat16", "--learning_rate", lr,
                "--num_train_epochs", epoch, "--per_device_train_batch_size", str(micro),
                "--gradient_accumulation_steps", str(accum), "--load_best_model_at_end",
                "--evaluation_strategy", "epoch", "--save_strategy", "epoch", "--save_total_limit", "1"]
        if fsdp:
            argv += ["--no_auto_device"]
    else:
        raise ValueError(f"unknown recipe {recipe!r}")
    argv += ["--train_as_classification"] if classification else ["--train_as_classification", "False"]
    return argv + _mode_args(mode) + task_args


def main(argv: Optional[List[str]] = None, env: Optional[Dict[str, str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    env = dict(os.environ if env is None else env)
    if not argv or argv[0] not in ("dizo", "finetune", "finetune_fsdp", "icl"):
        print(__doc__)
        return 2
    recipe, extra = argv[0], argv[1:]
    run_args = build_argv(recipe, env) + extra
    n = int(env.get("NUM_GPU", "1"))
    print(" ".join(["dizo_b200.run"] + run_args), flush=True)
    if n <= 1:
        from .run import main as run_main
        return int(run_main(run_args) or 0)
    port = str(20000 + os.getpid() % 20000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", port, "-m", "dizo_b200.run"] + run_args
    return subprocess.call(cmd, env=env)


if __name__ == "__main__":
    sys.exit(main())
