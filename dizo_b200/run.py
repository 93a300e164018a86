"""Command-line entry: zero-shot / in-context evaluation, ZO / DiZO training, final evaluation.

Same surface and control flow as the reference's ``run.py`` (large_models/run.py:121-580):
``parse_args`` -> ``set_seed`` -> ``get_task`` -> ``Framework`` (model + tokenizer + PEFT wiring)
-> per train set: ``Framework.train`` then ``Framework.evaluate`` on the test split, or
in-context evaluation; results are logged and written as JSON.  Differences by design: no GPU
pinning at import (one process per GPU, rank from the launcher), bf16 as the native precision,
models built over parameter arenas instead of ``AutoModelForCausalLM``.

    python -m dizo_b200.run --model_name facebook/opt-13b --task_name SST2 --trainer zo ...
"""
from __future__ import annotations

import json
import logging
import os
import random
from typing import Optional

import numpy as np
import torch

from .args import OurArguments, parse_args
from .evaluation import Evaluator
from .models import peft as peft_wiring
from .models.opt import OPTConfig, OPTModel, PRESETS, preset
from .tasks import get_task
from .trainer import OurTrainer
from .utils import (DataCollatorForTokenClassification, DataCollatorWithPaddingAndNesting,
                    NondiffCollator, SIGUSR1Callback, StubTokenizer, count_time, encode_prompt,
                    write_metrics_to_file)
from .utils.checkpoint import get_last_checkpoint, load_weights

logging.basicConfig(level=logging.INFO, format="%(asctime)s - %(levelname)s - %(message)s")
logger = logging.getLogger(__name__)


def set_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def _device_and_dist(args: OurArguments):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1 and not torch.distributed.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl" if dev.type == "cuda" else "gloo")
    return dev


class Framework:
    def __init__(self, args: OurArguments, task):
        self.args = args
        self.task = task
        self.device = _device_and_dist(args)
        self.model, self.tokenizer = self.load_model()
        self._evaluator = Evaluator(self.model, self.tokenizer, self.task, self.args)

    # ------------------------------------------------------------------ model / tokenizer
    def _dtype(self) -> torch.dtype:
        a = self.args
        if self.device.type == "cuda":
            # the sm_100a kernels compute in bf16; an fp16 / int8 request is honoured as a one-time
            # conversion of the loaded weights to bf16 (same 16-bit footprint, wider exponent)
            if (a.load_float16 or a.load_int8) and not getattr(Framework, "_told_dtype", False):
                Framework._told_dtype = True
                logger.info("--load_float16 / --load_int8: weights are converted once to bfloat16, the "
                            "precision the sm_100a kernels compute in")
            return torch.bfloat16
        return torch.bfloat16 if a.load_bfloat16 else torch.float32

    @staticmethod
    def resolve_model_dir(name: str) -> Optional[str]:
        """Directory holding ``config.json`` for ``--model_name``: the path itself, or the snapshot of a
        hub id (``facebook/opt-13b``) in the local Hugging Face cache (``HF_HOME``); None if neither
        exists.  Nothing is downloaded."""
        if os.path.isdir(name) and os.path.exists(os.path.join(name, "config.json")):
            return name
        if os.path.isdir(name):
            return None
        try:
            from transformers.utils import cached_file
            cfg = cached_file(name, "config.json", local_files_only=True,
                              _raise_exceptions_for_missing_entries=False,
                              _raise_exceptions_for_connection_errors=False)
        except Exception:  # noqa: BLE001  (malformed ids, cache layout problems)
            cfg = None
        return os.path.dirname(cfg) if cfg else None

    def load_model(self):
        a = self.args
        with count_time("Loading model with FP%d" % (16 if self._dtype() != torch.float32 else 32)):
            state = None
            path = self.resolve_model_dir(a.model_name)
            if path is not None:
                with open(os.path.join(path, "config.json")) as f:
                    raw = json.load(f)
                mtype = raw.get("model_type", "opt")
                if mtype == "opt":
                    cfg = OPTConfig.from_hf(raw)
                elif mtype in ("llama", "mistral"):
                    from .models.llama import LlamaConfig
                    cfg = LlamaConfig.from_hf(raw)
                else:
                    raise NotImplementedError(f"{a.model_name}: model_type {mtype!r}; the kernels implement the "
                                              "OPT and LLaMA (llama, mistral) decoder families")
                if not a.random_init:
                    state = load_weights(path, lazy=True)   # one tensor at a time: every rank keeps its slice
            else:
                # no checkpoint: only an explicit --random_init may train on random weights
                key = os.path.basename(a.model_name.rstrip("/")).lower().replace("opt1p3b", "opt-1.3b")
                if not a.random_init:
                    raise FileNotFoundError(
                        f"--model_name {a.model_name!r} is neither a checkpoint directory nor a model in the "
                        "local Hugging Face cache (nothing is downloaded). Pass --random_init to build a "
                        "randomly initialised model of that shape on purpose.")
                from .models import llama as llama_models
                if key in PRESETS:
                    cfg = preset(key)
                elif key in llama_models.PRESETS:
                    cfg = llama_models.preset(key)
                else:
                    raise KeyError(f"--random_init needs a known shape; {key!r} is not one of "
                                   f"{sorted(PRESETS) + sorted(llama_models.PRESETS)}")
                logger.info("--random_init: %s with random weights", key)
            mode = "full"
            if a.head_tuning:
                mode = "head"
            elif a.lora and a.prefix_tuning:
                mode = "lora+prefix"
            elif a.lora:
                mode = "lora"
            elif a.prefix_tuning:
                mode = "prefix"
            world = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
            self.dp_group = None                      # None: the default group, when there is one
            if cfg.model_type != "opt":
                if a.tp > 1 or a.fsdp_shard:
                    raise NotImplementedError("--tp / --fsdp_shard shard the OPT family; LLaMA-family models run "
                                              "replicated (data parallel) or as a pipeline of blocks (--pp)")
                if a.pp > 1:
                    assert a.pp == world, "--pp must equal the number of ranks (one pipeline)"
                    assert a.enhanced != "fo", "the first-order gamma search is not staged over a pipeline"
                    from .parallel.pp import PPLlamaModel
                    model = PPLlamaModel(cfg, self.device, self._dtype(), micro_batches=a.pp_micro_batches,
                                         mode=mode, num_prefix=a.num_prefix, prefix_reparam=not a.no_reparam)
                    self.dp_group = False
                else:
                    from .models.llama import LlamaModel
                    model = LlamaModel(cfg, self.device, self._dtype(), mode=mode, num_prefix=a.num_prefix,
                                       prefix_reparam=not a.no_reparam)
            elif a.pp > 1:
                # consecutive blocks on consecutive ranks; every rank sees the same batch
                assert a.pp == world, "--pp must equal the number of ranks (one pipeline)"
                assert a.enhanced != "fo", "the first-order gamma search is not staged over a pipeline"
                from .parallel.pp import PPOPTModel
                model = PPOPTModel(cfg, self.device, self._dtype(), micro_batches=a.pp_micro_batches, mode=mode,
                                   lora_r=a.lora_r, lora_alpha=a.lora_alpha, num_prefix=a.num_prefix, prefix_reparam=not a.no_reparam,
                                   untie_emb=a.untie_emb)
                self.dp_group = False
            elif a.tp > 1 or a.fsdp_shard:
                assert a.enhanced != "fo" or (a.fsdp_shard and a.tp <= 1), \
                    "the first-order gamma search runs on replicated or FSDP-sharded parameters"
                # sharded layouts (full-parameter ZO, fused collectives over NVLink peer memory)
                assert mode == "full" and self.device.type == "cuda" and world > 1, \
                    "--tp / --fsdp_shard need full-parameter mode on >= 2 GPUs"
                if a.tp > 1:
                    assert a.tp == world, "--tp must equal the number of ranks (one tensor-parallel group)"
                    from .parallel.tp import TPOPTModel
                    model = TPOPTModel(cfg, self.device, self._dtype(),
                                       max_tokens=a.tp_max_tokens, untie_emb=a.untie_emb)
                    self.dp_group = False             # every rank sees the same batch
                else:
                    from .parallel.fsdp import FSDPOPTModel
                    model = FSDPOPTModel(cfg, self.device, self._dtype(), untie_emb=a.untie_emb)
            else:
                model = OPTModel(cfg, self.device, self._dtype(), mode=mode, lora_r=a.lora_r,
                                 lora_alpha=a.lora_alpha, num_prefix=a.num_prefix, prefix_reparam=not a.no_reparam, untie_emb=a.untie_emb)
            if state is not None:
                model.init_random(a.seed)          # adapters; base weights are overwritten below
                model.load_state_dict(state, strict=False)
            else:
                (model.init_random_fast if self.device.type == "cuda" else model.init_random)(0)
        tokenizer = self._load_tokenizer(path, cfg)
        if a.prefix_tuning and a.prefix_init_by_real_act and a.no_reparam:
            peft_wiring.init_prefix_by_real_activations(model, seed=a.seed)
        return model, tokenizer

    def _load_tokenizer(self, path: Optional[str], cfg: OPTConfig):
        """The checkpoint's tokenizer (``use_fast=False`` as the reference).  The word-level stub stands in
        only for ``--random_init`` models, whose vocabulary has no meaning anyway; a checkpoint whose
        tokenizer does not load is an error, not a silent fallback."""
        a = self.args
        tok = None
        tok_files = ("tokenizer_config.json", "tokenizer.json", "vocab.json", "tokenizer.model")
        if path is not None and any(os.path.exists(os.path.join(path, f)) for f in tok_files):
            try:
                from transformers import AutoTokenizer
                tok = AutoTokenizer.from_pretrained(path, use_fast=False, local_files_only=True)
            except Exception as e:  # noqa: BLE001
                if not a.random_init:
                    raise RuntimeError(f"tokenizer of {path} does not load: {e}. (With --random_init the "
                                       "stub tokenizer is used instead.)") from e
                logger.info("tokenizer of %s does not load (%s): --random_init uses the stub tokenizer", path, e)
        elif path is not None:
            logger.info("%s holds weights but no tokenizer files (a directory written by save_model of a "
                        "stub-tokenizer run): using the stub tokenizer", path)
        if tok is None:
            words = ["terrible", "great", "Yes", "No", "Maybe", "It", "was"]
            tok = StubTokenizer(words, vocab_size=cfg.vocab_size)
        # fix-ups of large_models/run.py:185-231
        if getattr(tok, "pad_token_id", None) is None:
            tok.pad_token_id = 0
        if cfg.model_type == "opt":
            tok.bos_token_id = 0 if not isinstance(tok, StubTokenizer) else tok.bos_token_id
        elif not isinstance(tok, StubTokenizer):
            tok.pad_token_id = 0                     # the llama fix-up of large_models/run.py:229-231
        tok.padding_side = "left"
        return tok

    # ------------------------------------------------------------------ inference API
    def forward(self, input_ids, option_len=None, generation=False):
        return self._evaluator.forward(input_ids, option_len, generation)

    def one_step_pred(self, train_samples, eval_sample, verbose=False):
        return self._evaluator.one_step_pred(train_samples, eval_sample, verbose)

    def evaluate(self, train_samples, eval_samples, one_train_set_per_eval_sample=False):
        return self._evaluator.evaluate(train_samples, eval_samples, one_train_set_per_eval_sample)

    # ------------------------------------------------------------------ training
    def _convert(self, samples) -> list:
        """Samples -> feature dicts (one list of candidate dicts per sample for classification)."""
        a, out = self.args, []
        for sample in samples:
            enc, ol = encode_prompt(self.task, self.task.get_template(), [], sample, self.tokenizer,
                                    max_length=a.max_length, generation=self.task.generation,
                                    generation_with_gold=True, max_new_tokens=a.max_new_tokens)
            if self.task.generation:
                gold_id = 0
            elif isinstance(sample.correct_candidate, list):
                gold_id = sample.candidates.index(sample.correct_candidate[0])
            else:
                gold_id = sample.candidates.index(sample.correct_candidate)
            if a.non_diff:
                enc[gold_id] = enc[gold_id][:-ol[gold_id]]       # no teacher forcing: drop the answer
            if a.train_as_classification:
                out.append([{"input_ids": enc[i], "labels": gold_id, "option_len": ol[i],
                             "num_options": len(sample.candidates)} for i in range(len(enc))])
            elif a.only_train_option:
                d = {"input_ids": enc[gold_id], "labels": enc[gold_id], "option_len": ol[gold_id]}
                if a.non_diff:
                    d["gold"] = sample.correct_candidate
                out.append(d)
            else:
                out.append({"input_ids": enc[gold_id], "labels": enc[gold_id]})
        return out

    def train(self, train_samples, eval_samples):
        a = self.args
        self.tokenizer.padding_side = "left"      # options end up right-aligned
        with count_time("Tokenizing training samples"):
            train_dataset = self._convert(train_samples)
        if a.train_as_classification:
            collator = DataCollatorWithPaddingAndNesting(self.tokenizer, pad_to_multiple_of=8)
        elif a.non_diff:
            collator = NondiffCollator(self.tokenizer, pad_to_multiple_of=8)
        else:
            collator = DataCollatorForTokenClassification(self.tokenizer, pad_to_multiple_of=8)
        trainer = OurTrainer(model=self.model, args=a, train_dataset=train_dataset, eval_dataset=eval_samples,
                             processing_class=self.tokenizer, data_collator=collator, task=self.task,
                             dp_group=getattr(self, "dp_group", None))
        if a.save_on_interrupt:
            trainer.add_callback(SIGUSR1Callback())
        last = None
        if os.path.isdir(a.output_dir) and not a.overwrite_output_dir:
            last = get_last_checkpoint(a.output_dir)
        if last is not None and a.resume_from_checkpoint is None:
            logger.info(f"Checkpoint detected, resuming training at {last}. To avoid this behavior, change "
                        "the `--output_dir` or add `--overwrite_output_dir` to train from scratch.")
        if a.resume_from_checkpoint is not None:
            last = a.resume_from_checkpoint
        metrics = trainer.train(resume_from_checkpoint=last)
        if a.save_model:
            logger.warning("Save model..")
            trainer.save_model()
        self.trainer = trainer
        return metrics


def result_file_tag(args: OurArguments) -> str:
    """File-name tag of a result: task, model, calibration, demos / train set, user tag."""
    save_model_name = args.model_name.split("/")[-1]
    sfc_tag = "-sfc" if args.sfc else ""
    icl_sfc_tag = "-icl_sfc" if args.icl_sfc else ""
    sample_eval_tag = "-sampleeval%d" % args.num_eval if args.num_eval is not None else ""
    sample_train_tag = "-ntrain%d" % args.num_train if args.num_train > 0 else ""
    sample_dev_tag = "-ndev%d" % args.num_dev if args.num_dev is not None else ""
    customized_tag = f"-{args.tag}" if len(args.tag) > 0 else ""
    return f"{args.task_name}-{save_model_name}" + sfc_tag + icl_sfc_tag + sample_eval_tag + \
        sample_train_tag + sample_dev_tag + customized_tag


def main(argv=None):
    args = parse_args(argv)
    set_seed(args.seed)                       # before the task: its subsets use random.sample
    task = get_task(args.task_name)
    framework = Framework(args, task)
    rank = int(os.environ.get("RANK", "0"))

    if args.train_set_seed is not None or args.num_train_sets is not None:
        train_sets = task.sample_train_sets(num_train=args.num_train, num_dev=args.num_dev,
                                            num_eval=args.num_eval, num_train_sets=args.num_train_sets,
                                            seed=args.train_set_seed)
        for set_id, train_samples in enumerate(train_sets):
            set_seed_id = set_id if args.train_set_seed is None else args.train_set_seed
            eval_samples = task.valid_samples if args.num_eval is None else \
                task.sample_subset(data_split="valid", seed=set_seed_id, num=args.num_eval)
            if args.trainer != "none":
                if args.num_dev is not None:
                    dev_samples = train_samples[-args.num_dev:]
                    train_samples = train_samples[:-args.num_dev]
                else:
                    dev_samples = None
                framework.train(train_samples, dev_samples if dev_samples is not None else eval_samples)
                metrics = {} if args.no_eval else framework.evaluate([], eval_samples)
                if dev_samples is not None and not args.no_eval:
                    dev_metrics = framework.evaluate([], dev_samples)
                    for m in dev_metrics:
                        metrics["dev_" + m] = dev_metrics[m]
            else:
                assert args.num_dev is None
                metrics = framework.evaluate(train_samples, eval_samples)
            logger.info("===== Train set %d =====" % set_seed_id)
            logger.info(metrics)
            if rank <= 0:
                os.makedirs("result", exist_ok=True)
                name = result_file_tag(args) + f"-trainset{set_seed_id}.json" if args.result_file is None \
                    else args.result_file
                write_metrics_to_file(metrics, "result/" + name if args.result_file is None else name)
    else:
        assert args.trainer == "none"
        eval_samples = task.valid_samples if args.num_eval is None else \
            task.sample_subset(data_split="valid", seed=0, num=args.num_eval)
        # one demonstration set per evaluation sample (MeZO semantics)
        train_sets = task.sample_train_sets(num_train=args.num_train, num_eval=len(eval_samples))
        metrics = framework.evaluate(train_sets, eval_samples, one_train_set_per_eval_sample=True)
        logger.info(metrics)
        if rank <= 0:
            os.makedirs("result", exist_ok=True)
            name = "result/" + result_file_tag(args) + "-onetrainpereval.json" if args.result_file is None \
                else args.result_file
            write_metrics_to_file(metrics, name)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
