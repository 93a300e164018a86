"""Command-line / configuration surface.

Field names and defaults of the first block are those of the reference's ``OurArguments``
(large_models/run.py:35-118); the second block holds the Hugging Face ``TrainingArguments``
names its launch scripts and loop actually use (large_models/dizo.sh:61-73,
large_models/finetune.sh:64-74, large_models/trainer.py:963-1292), re-declared here so the
framework does not depend on ``transformers.Trainer`` or ``accelerate``.  The third block is
new: constants the reference hard-codes, exposed with the reference's values as defaults, and
the parallelism / precision switches of this framework.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
from dataclasses import dataclass, field, fields
from typing import Optional


def _str2bool(v):
    if isinstance(v, bool):
        return v
    s = str(v).lower()
    if s in ("1", "true", "t", "yes", "y"):
        return True
    if s in ("0", "false", "f", "no", "n"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def _opt(kind):
    def conv(v):
        if v is None or str(v).lower() in ("none", "null", ""):
            return None
        return kind(v)
    return conv


@dataclass
class OurArguments:
    # ---- reference block (large_models/run.py:35-118) --------------------------------
    task_name: str = "SST2"
    num_train: int = 0
    num_dev: Optional[int] = None
    num_eval: Optional[int] = None
    num_train_sets: Optional[int] = None
    train_set_seed: Optional[int] = None
    result_file: Optional[str] = None
    model_name: str = "./opt1p3b"
    load_float16: bool = False
    load_bfloat16: bool = False
    load_int8: bool = False
    max_length: int = 2048
    no_auto_device: bool = False
    sfc: bool = False
    icl_sfc: bool = False
    trainer: str = "none"                  # none | regular | zo
    only_train_option: bool = True
    train_as_classification: bool = False
    zo_eps: float = 1e-3
    bits: int = 11                          # parsed, unused (as in the reference)
    rng: int = 8                            # parsed, unused
    pre_gen: bool = False                   # parsed, unused
    handling: bool = False                  # parsed, unused
    size: float = 0.9                       # parsed, unused
    enhanced: Optional[str] = None          # None | zo | fo
    prefix_tuning: bool = False
    num_prefix: int = 5
    no_reparam: bool = True
    prefix_init_by_real_act: bool = True
    lora: bool = False
    lora_alpha: int = 16
    lora_r: int = 8
    sampling: bool = False
    temperature: float = 1.0
    num_beams: int = 1
    top_k: Optional[int] = None
    top_p: float = 0.95
    max_new_tokens: int = 50
    eos_token: str = "\n"
    save_model: bool = False
    no_eval: bool = False
    tag: str = ""
    linear_probing: bool = False
    lp_early_stopping: bool = False
    head_tuning: bool = False
    untie_emb: bool = False
    verbose: bool = False
    non_diff: bool = False
    save_on_interrupt: bool = False

    # ---- Hugging Face TrainingArguments names used by the reference -------------------
    output_dir: str = "result/output"
    overwrite_output_dir: bool = False
    resume_from_checkpoint: Optional[str] = None
    seed: int = 42
    learning_rate: float = 5e-5
    max_steps: int = -1
    num_train_epochs: float = 3.0
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    lr_scheduler_type: str = "linear"
    warmup_steps: int = 0
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    logging_steps: int = 500
    eval_steps: Optional[int] = None
    save_steps: int = 500
    save_total_limit: Optional[int] = None
    evaluation_strategy: str = "no"
    save_strategy: str = "steps"
    load_best_model_at_end: bool = False
    fp16: bool = False
    bf16: bool = False
    fsdp: str = ""
    fsdp_transformer_layer_cls_to_wrap: Optional[str] = None
    local_rank: int = -1
    logging_nan_inf_filter: bool = True
    ignore_data_skip: bool = False
    gradient_checkpointing: bool = False
    report_to: str = "none"

    # ---- new: reference constants as flags, B200 execution switches --------------------
    dizo_interval: int = 50                 # projection period (large_models/trainer.py:1611)
    dizo_max_iters: int = 10                # gamma-search iterations (:1168)
    dizo_proj_lr: float = 0.1               # Adam lr of the FO search (:1168)
    dizo_norm_mode: str = "l2norm"          # (:1168)
    dizo_tau: float = 0.2                   # (:590)
    dizo_zo_eps: float = 0.1                # (:591)
    dizo_step_size: float = 2.0             # (:592)
    dizo_l1: float = 1e-3                   # L1 weight on gamma in the FO search (:739)
    zo_log_steps: int = 50                  # (:1321)
    zo_eval_steps: int = 100                # in-loop dev evaluation period (:1327)
    random_init: bool = False               # build --model_name's shape with random weights (no checkpoint needed)
    zo_mode: str = "inflight"               # inflight (theta never rewritten for a forward) | inplace
    zo_stochastic_rounding: Optional[bool] = None   # unbiased bf16 update; default: on for bf16 parameters
    dp: int = 0                             # data-parallel ranks (0 = WORLD_SIZE)
    tp: int = 1                             # tensor-parallel ranks (1, or the number of ranks)
    tp_max_tokens: int = 32768              # largest batch x padded length a tensor-parallel forward takes
    pp: int = 1                             # pipeline stages (1, or the number of ranks)
    pp_micro_batches: int = 0               # micro-batches per forward (0 = one per stage)
    fsdp_shard: bool = False                # shard parameters over the data-parallel group
    eval_batch_size: int = 16               # candidates scored per forward in evaluation
    synthetic_task: bool = False            # seeded uniform ids + Bernoulli labels (no dataset)
    synthetic_seq_len: int = 64
    heartbeat_timeout: float = 0.0          # > 0: ranks report every step through the store; a silent peer raises PeerLost
    zo_cuda_graph: bool = False             # replay each ZO step as one CUDA graph (launch-bound small models)
    profile_steps: Optional[str] = None     # "a:b": NVTX range + per-phase device timers
    metrics_jsonl: Optional[str] = None

    # -----------------------------------------------------------------------------------
    @property
    def world_size(self) -> int:
        import os
        return int(os.environ.get("WORLD_SIZE", "1"))

    @property
    def process_index(self) -> int:
        import os
        return int(os.environ.get("RANK", "0"))

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True)


def build_parser() -> argparse.ArgumentParser:
    """argparse parser with one ``--name`` option per field; booleans accept a bare flag or
    an explicit value (``--lora`` / ``--train_as_classification False``), as HfArgumentParser."""
    p = argparse.ArgumentParser(description="B200-native zeroth-order fine-tuning (DiZO capabilities)",
                                allow_abbrev=False)
    for f in fields(OurArguments):
        name = "--" + f.name
        default = f.default if f.default is not dataclasses.MISSING else None
        t = f.type if isinstance(f.type, str) else getattr(f.type, "__name__", str(f.type))
        if "bool" in t:
            p.add_argument(name, type=_str2bool, nargs="?", const=True, default=default)
        elif "int" in t:
            p.add_argument(name, type=_opt(int) if "Optional" in t else int, default=default)
        elif "float" in t:
            p.add_argument(name, type=_opt(float) if "Optional" in t else float, default=default)
        else:
            p.add_argument(name, type=_opt(str) if "Optional" in t else str, default=default)
    return p


def parse_args(argv=None) -> OurArguments:
    ns, unknown = build_parser().parse_known_args(argv)
    if unknown:
        import logging
        logging.getLogger(__name__).warning("ignoring unknown arguments: %s", unknown)
    return OurArguments(**vars(ns))
