"""Prompt encoding, collators, callbacks and small helpers.

Behavioural counterpart of the reference's ``utils.py``: ``encode_prompt``
(large_models/utils.py:108-175), the nesting / ICL / non-differentiable collators
(:179-288), the SIGUSR1 callback (:291-315), ``Prediction``, ``count_time``, ``temp_seed`` and
the JSON writers (:318-358).  Padding is done here (no ``tokenizer.pad`` dependency), so any
object with ``encode`` / ``decode`` / ``pad_token_id`` / ``padding_side`` works as a tokenizer.
"""
from __future__ import annotations

import contextlib
import json
import logging
import signal
import time
from dataclasses import asdict, dataclass, is_dataclass
from typing import Any, Dict, List, Optional, Union

import numpy as np
import torch

logger = logging.getLogger(__name__)


# --------------------------------------------------------------------------- prompts
def encode_prompt(task, template, train_samples, eval_sample, tokenizer, max_length, sfc=False,
                  icl_sfc=False, generation=False, generation_with_gold=False, max_new_tokens=None):
    """Token ids of the prompt(s) for ``eval_sample`` and the number of option tokens of each.

    Classification / multiple choice: one prompt per candidate, ``option_len`` = tokens of the
    verbalised prompt minus tokens of the prompt without an answer.  Generation: a single
    prompt (``option_len`` 0), or prompt + gold answer when ``generation_with_gold``.
    ``train_samples`` are in-context demonstrations joined by ``task.train_sep``; ``sfc`` /
    ``icl_sfc`` select the calibration variants.  Over-long prompts are truncated on the LEFT
    (demonstrations go first), keeping a leading BOS token."""
    demos = task.train_sep.join(template.verbalize(s, s.correct_candidate).strip() for s in train_samples).strip()
    enc_fn, verb_fn = ((template.encode_sfc, template.verbalize_sfc) if (sfc or icl_sfc)
                       else (template.encode, template.verbalize))
    bare = enc_fn(eval_sample).strip(" ")

    def with_demos(p):
        return (demos + task.train_sep + p).lstrip().strip(" ")

    if not generation:
        full = [verb_fn(eval_sample, c).strip(" ") for c in eval_sample.candidates]
        n_bare = len(tokenizer.encode(bare))
        option_lens = [len(tokenizer.encode(p)) - n_bare for p in full]
        prompts = full if sfc else [with_demos(p) for p in full]
    else:
        assert not sfc and not icl_sfc, "Generation tasks do not support SFC"
        if generation_with_gold:
            full = [verb_fn(eval_sample, eval_sample.correct_candidate)]
            n_bare = len(tokenizer.encode(bare))
            option_lens = [len(tokenizer.encode(p)) - n_bare for p in full]
            prompts = [with_demos(p) for p in full]
        else:
            option_lens = [0]
            prompts = [with_demos(bare)]

    encodings = [tokenizer.encode(p) for p in prompts]
    if generation and max_new_tokens is not None:
        max_length = max_length - max_new_tokens
    if any(len(e) > max_length for e in encodings):
        logger.warning("Exceed max length")
    if getattr(tokenizer, "add_bos_token", False):
        encodings = [e[0:1] + e[1:][-(max_length - 1):] for e in encodings]
    else:
        encodings = [e[-max_length:] for e in encodings]
    return encodings, option_lens


# --------------------------------------------------------------------------- padding / collators
def _pad_len(n: int, multiple: Optional[int]) -> int:
    if multiple:
        return (n + multiple - 1) // multiple * multiple
    return n


def pad_sequences(seqs: List[List[int]], pad_id: int, side: str = "left",
                  pad_to_multiple_of: Optional[int] = None):
    """-> (ids [B, L] int64, attention_mask [B, L] int64)."""
    L = _pad_len(max(len(s) for s in seqs), pad_to_multiple_of)
    ids = torch.full((len(seqs), L), pad_id, dtype=torch.long)
    mask = torch.zeros((len(seqs), L), dtype=torch.long)
    for i, s in enumerate(seqs):
        n = len(s)
        if side == "left":
            ids[i, L - n:] = torch.as_tensor(s, dtype=torch.long)
            mask[i, L - n:] = 1
        else:
            ids[i, :n] = torch.as_tensor(s, dtype=torch.long)
            mask[i, :n] = 1
    return ids, mask


@dataclass
class DataCollatorWithPaddingAndNesting:
    """Flattens a list of per-example candidate lists into one padded batch."""
    tokenizer: Any
    padding: Union[bool, str] = True
    max_length: Optional[int] = None
    pad_to_multiple_of: Optional[int] = None
    return_tensors: str = "pt"

    def __call__(self, features: List[List[Dict[str, Any]]]) -> Dict[str, Any]:
        flat = [ff for f in features for ff in f]
        side = getattr(self.tokenizer, "padding_side", "left")
        ids, mask = pad_sequences([f["input_ids"] for f in flat], self.tokenizer.pad_token_id, side,
                                  self.pad_to_multiple_of)
        batch: Dict[str, Any] = {"input_ids": ids, "attention_mask": mask}
        for k in flat[0]:
            if k in ("input_ids", "attention_mask"):
                continue
            key = "labels" if k in ("label", "label_ids") else k
            batch[key] = torch.as_tensor([f[k] for f in flat])
        return batch


@dataclass
class DataCollatorForTokenClassification:
    """LM-style features (``labels`` = token ids): pads ids with pad and labels with -100."""
    tokenizer: Any
    padding: Union[bool, str] = True
    max_length: Optional[int] = None
    pad_to_multiple_of: Optional[int] = None
    label_pad_token_id: int = -100
    return_tensors: str = "pt"

    def __call__(self, features: List[Dict[str, Any]]) -> Dict[str, Any]:
        side = getattr(self.tokenizer, "padding_side", "left")
        ids, mask = pad_sequences([f["input_ids"] for f in features], self.tokenizer.pad_token_id, side,
                                  self.pad_to_multiple_of)
        batch: Dict[str, Any] = {"input_ids": ids, "attention_mask": mask}
        if "labels" in features[0]:
            lab, _ = pad_sequences([list(f["labels"]) for f in features], self.label_pad_token_id, side,
                                   self.pad_to_multiple_of)
            batch["labels"] = lab
        for k in features[0]:
            if k in ("input_ids", "attention_mask", "labels", "gold"):
                continue
            batch[k] = torch.as_tensor([f[k] for f in features])
        if "gold" in features[0]:
            batch["gold"] = [f["gold"] for f in features]
        return batch


@dataclass
class NondiffCollator(DataCollatorForTokenClassification):
    """Collator for non-differentiable objectives: keeps the ``gold`` answers as a list."""


@dataclass
class ICLCollator:
    """Right-pads every key of the features (ids with pad, masks with 0)."""
    tokenizer: Any

    def __call__(self, features: List[Dict[str, Any]]) -> Dict[str, Any]:
        if not isinstance(features[0], dict):
            features = [vars(f) for f in features]
        pad_id = self.tokenizer.pad_token_id
        fill = {"input_ids": pad_id, "attention_mask": 0, "sfc_input_ids": pad_id,
                "sfc_attention_mask": 0, "labels": pad_id}
        batch = {}
        for key in features[0]:
            n = max(len(f[key]) for f in features)
            arr = np.stack([np.pad(np.asarray(f[key]), (0, n - len(f[key])), "constant",
                                   constant_values=(0, fill[key])) for f in features])
            batch[key] = torch.from_numpy(arr).long()
        return batch


# --------------------------------------------------------------------------- callbacks
class TrainerControl:
    def __init__(self):
        self.should_save = False
        self.should_training_stop = False
        self.should_evaluate = False
        self.should_log = False


class TrainerCallback:
    def on_train_begin(self, args, state, control, **kw): ...
    def on_step_end(self, args, state, control, **kw): ...
    def on_train_end(self, args, state, control, **kw): ...
    def on_log(self, args, state, control, logs=None, **kw): ...
    def on_save(self, args, state, control, **kw): ...


class SIGUSR1Callback(TrainerCallback):
    """On SIGUSR1 (SLURM pre-emption) or SIGINT: ask for a checkpoint at the next step boundary
    and stop.  Unlike the reference, whose loop never acts on ``should_save``
    (large_models/utils.py:291-315 vs large_models/trainer.py:1319-1358), the trainer here
    honours it with a real checkpoint."""

    def __init__(self, exit_on_end: bool = True) -> None:
        self.signal_received = False
        self.exit_on_end = exit_on_end
        signal.signal(signal.SIGUSR1, self.handle_signal)
        signal.signal(signal.SIGINT, self.handle_signal)
        logger.warning("Handler registered")

    def handle_signal(self, signum, frame):
        self.signal_received = True
        logger.warning("Signal received")

    def on_step_end(self, args, state, control, **kwargs):
        if self.signal_received:
            control.should_save = True
            control.should_training_stop = True

    def on_train_end(self, args, state, control, **kwargs):
        if self.signal_received and self.exit_on_end:
            raise SystemExit(0)


# --------------------------------------------------------------------------- misc
@dataclass
class Prediction:
    correct_candidate: Union[int, str, list]
    predicted_candidate: Union[int, str]


@contextlib.contextmanager
def count_time(name):
    logger.info("%s..." % name)
    t0 = time.time()
    try:
        yield
    finally:
        logger.info("Done with %.2fs" % (time.time() - t0))


@contextlib.contextmanager
def temp_seed(seed):
    state = np.random.get_state()
    np.random.seed(seed)
    try:
        yield
    finally:
        np.random.set_state(state)


class EnhancedJSONEncoder(json.JSONEncoder):
    def default(self, o):
        if is_dataclass(o):
            return asdict(o)
        if isinstance(o, (np.integer,)):
            return int(o)
        if isinstance(o, (np.floating,)):
            return float(o)
        return super().default(o)


def write_predictions_to_file(final_preds, output):
    with open(output, "w") as f:
        for pred in final_preds:
            f.write(json.dumps(pred, cls=EnhancedJSONEncoder) + "\n")


def write_metrics_to_file(metrics, output):
    with open(output, "w") as f:
        json.dump(metrics, f, cls=EnhancedJSONEncoder, indent=4)


class StubTokenizer:
    """Whitespace / character tokenizer for offline tests and the synthetic task.

    Words seen at construction get their own ids; everything else falls back to characters.
    A space before a word is part of the word token (GPT-2 style), so ``"It was great"`` and
    ``"It was"`` differ by exactly the tokens of ``" great"``."""
    padding_side = "left"
    add_bos_token = True

    def __init__(self, words: Optional[List[str]] = None, vocab_size: int = 512):
        self.pad_token_id, self.bos_token_id, self.eos_token_id = 1, 2, 2
        self.vocab: Dict[str, int] = {}
        self.inv: Dict[int, str] = {}
        self.vocab_size = vocab_size
        nxt = 4
        for ch in [chr(c) for c in range(32, 127)] + ["\n"]:
            self.vocab[ch] = nxt
            self.inv[nxt] = ch
            nxt += 1
        for w in words or []:
            for form in (w, " " + w):
                if form not in self.vocab and nxt < vocab_size:
                    self.vocab[form] = nxt
                    self.inv[nxt] = form
                    nxt += 1

    def _pieces(self, text: str):
        i, n = 0, len(text)
        while i < n:
            j = i + 1 if text[i] == " " else i
            k = j
            while k < n and text[k] not in " \n":
                k += 1
            word = text[i:k]
            if k > j and word in self.vocab:
                yield word
                i = k
            else:
                yield text[i]
                i += 1

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        ids = [self.vocab.get(p, self.vocab["?"]) for p in self._pieces(text)]
        return ([self.bos_token_id] if add_special_tokens and self.add_bos_token else []) + ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out = []
        for i in ids:
            i = int(i)
            if skip_special_tokens and i in (self.pad_token_id, self.bos_token_id):
                continue
            out.append(self.inv.get(i, ""))
        return "".join(out)
