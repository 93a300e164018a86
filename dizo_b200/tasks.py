"""Task registry: ``get_task("Name[__sub]")`` -> a dataset object with train/valid/test samples.

Mirrors the reference's task layer (large_models/tasks.py:19-481): ``Sample`` records, a
``Dataset`` base with ``sample_train_sets`` / ``sample_subset`` for in-context demonstrations,
and eleven datasets (SST2, Copa, BoolQ, MultiRC, CB, WIC, WSC, ReCoRD, RTE, SQuAD, DROP), each
drawing 1000 training and at most 500 validation examples with ``random.sample`` (so the
subset depends on the global seed set before the task is built) and using the validation
subset as the test set.

Examples come from Hugging Face ``datasets`` when that is importable and the data are
cached; otherwise from JSON-lines files ``$DIZO_DATA_DIR/<key>/{train,validation}.jsonl``
with the same field names.  ``Synthetic`` is an offline task with the same interface.
"""
from __future__ import annotations

import json
import logging
import os
import random
import sys
from dataclasses import dataclass
from typing import Callable, List, Optional, Union

import numpy as np

from . import templates as T
from .utils import temp_seed

logger = logging.getLogger(__name__)


def get_task(task_name: str):
    """``"SST2"`` -> ``SST2Dataset()``; ``"Group__sub"`` passes ``sub`` as the subtask."""
    parts = task_name.split("__")
    group, subtask = (parts[0], parts[1]) if len(parts) == 2 else (parts[0], None)
    cls = getattr(sys.modules[__name__], f"{group}Dataset")
    return cls(subtask)


@dataclass
class Sample:
    id: Optional[int] = None
    data: Optional[dict] = None
    correct_candidate: Union[str, int, List[str], None] = None
    candidates: Optional[list] = None


def load_split(hf_args: tuple, key: str, split: str) -> list[dict]:
    """Rows of one split, from ``datasets`` or from ``$DIZO_DATA_DIR/<key>/<split>.jsonl``."""
    root = os.environ.get("DIZO_DATA_DIR")
    if root:
        path = os.path.join(root, key, f"{split}.jsonl")
        if os.path.exists(path):
            with open(path) as f:
                return [json.loads(line) for line in f if line.strip()]
    try:
        from datasets import load_dataset
    except ImportError as e:  # pragma: no cover - depends on the image
        raise RuntimeError(f"task data for {key!r} not found: install `datasets` with a local cache, "
                           f"or put {split}.jsonl under $DIZO_DATA_DIR/{key}/") from e
    return list(load_dataset(*hf_args)[split])


class Dataset:
    mixed_set = False
    train_sep = "\n\n"
    generation = False
    metric_name = "accuracy"
    samples: dict

    def __init__(self, subtask=None, **kwargs) -> None:
        self.subtask = subtask

    def get_task_name(self):
        return self.subtask

    def load_dataset(self, *a, **k):
        raise NotImplementedError

    def get_template(self, template_version=0):
        return T.Template()

    def build_sample(self, example):
        return None

    def sample_train_sets(self, num_train=32, num_dev=None, num_eval=None, num_train_sets=None, seed=None):
        """Demonstration / training sets: one for ``seed``, or ``num_train_sets`` (seeds 0..n-1),
        or one per evaluation sample (seeds drawn under ``temp_seed(0)``)."""
        if seed is not None:
            seeds = [seed]
        elif num_train_sets is not None:
            seeds = list(range(num_train_sets))
        else:
            assert num_dev is None, "a dev split needs --train_set_seed or --num_train_sets"
            n = len(self.samples["valid"]) if num_eval is None else num_eval
            with temp_seed(0):
                seeds = np.random.randint(0, 10000, n)
        out = []
        for i, s in enumerate(seeds):
            if self.mixed_set:
                raise NotImplementedError
            want = num_train + (num_dev or 0)        # dev samples ride at the end of the train set
            if num_dev is not None and want > len(self.samples["train"]):
                logger.warning("num_train + num_dev > available training examples")
            out.append(self.sample_subset(data_split="train", seed=int(s), num=want))
            if num_dev is not None:
                logger.info(f"Sample train set {len(out[-1])}/{len(self.samples['train'])}")
                logger.info(f"... including dev set {num_dev} samples")
        return out

    def sample_subset(self, data_split="train", seed=0, num=100, exclude=None):
        with temp_seed(seed):
            pool = self.samples[data_split]
            order = np.random.permutation(len(pool)).tolist()[:num if exclude is None else num + 1]
            if exclude is not None and exclude in order:
                order.remove(exclude)
            else:
                order = order[:num]
            return [pool[i] for i in order]

    @property
    def valid_samples(self):
        return self.samples["valid"]


class _TableDataset(Dataset):
    """A dataset described by class attributes: where the rows come from, how a row becomes a
    :class:`Sample`, which template versions exist."""
    hf_args: tuple = ()
    key: str = ""
    train_cap = 1000
    valid_cap = 500
    templates: dict = {}
    default_template = 0

    def __init__(self, subtask=None, **kwargs) -> None:
        self.subtask = subtask
        self.load_dataset(subtask, **kwargs)

    def load_dataset(self, path=None, **kwargs):
        train = [self.build_sample(e, i) for i, e in enumerate(load_split(self.hf_args, self.key, "train"))]
        valid = [self.build_sample(e, i) for i, e in enumerate(load_split(self.hf_args, self.key, "validation"))]
        train = random.sample(train, min(self.train_cap, len(train)))
        valid = random.sample(valid, min(self.valid_cap, len(valid)))
        self.samples = {"train": train, "valid": valid, "test": valid}

    def build_sample(self, example, idx=None) -> Sample:  # type: ignore[override]
        raise NotImplementedError

    def get_template(self, template_version=None):
        v = self.default_template if template_version is None else template_version
        return self.templates[v]()


def _label_task(name, hf_args, key, templates, n_labels, label_field="label", default_template=0,
                candidates=None, correct: Callable | None = None, doc=""):
    def build_sample(self, example, idx=None):
        cands = list(range(n_labels)) if candidates is None else candidates
        gold = correct(example) if correct else int(example[label_field])
        return Sample(id=example.get("idx", idx), data=example, correct_candidate=gold, candidates=cands)
    return type(name, (_TableDataset,), dict(hf_args=hf_args, key=key, templates=templates,
                                             default_template=default_template,
                                             build_sample=build_sample, __doc__=doc))


SST2Dataset = _label_task("SST2Dataset", ("glue", "sst2"), "sst2", {0: T.SST2Template}, 2)
BoolQDataset = _label_task(
    "BoolQDataset", ("boolq",), "boolq",
    {0: T.BoolQTemplate, 1: T.BoolQTemplateV2, 2: T.BoolQTemplateV3}, 2, default_template=2,
    candidates=["Yes", "No"], correct=lambda e: "Yes" if e["answer"] else "No")
MultiRCDataset = _label_task("MultiRCDataset", ("super_glue", "multirc"), "multirc", {0: T.MultiRCTemplate}, 2)
CBDataset = _label_task("CBDataset", ("super_glue", "cb"), "cb", {0: T.CBTemplate}, 3)
WICDataset = _label_task("WICDataset", ("super_glue", "wic"), "wic", {0: T.WICTemplate}, 2)
WSCDataset = _label_task("WSCDataset", ("super_glue", "wsc.fixed"), "wsc", {0: T.WSCTemplate}, 2)
RTEDataset = _label_task("RTEDataset", ("super_glue", "rte"), "rte", {0: T.RTETemplate}, 2)


class CopaDataset(_TableDataset):
    hf_args, key, templates = ("super_glue", "copa"), "copa", {0: T.CopaTemplate}

    def build_sample(self, example, idx=None):
        return Sample(id=example.get("idx", idx), data=example,
                      candidates=[example["choice1"], example["choice2"]],
                      correct_candidate=example[f"choice{example['label'] + 1}"])


class ReCoRDDataset(_TableDataset):
    hf_args, key, templates = ("super_glue", "record"), "record", {0: T.ReCoRDTemplateGPT3}

    def build_sample(self, example, idx=None):
        return Sample(id=example.get("idx", idx), data=example, candidates=example["entities"],
                      correct_candidate=example["answers"])


class SQuADDataset(_TableDataset):
    hf_args, key, templates = ("squad",), "squad", {0: T.SQuADv2Template}
    metric_name = "f1"
    generation = True

    def build_sample(self, example, idx=None):
        answers = example["answers"]["text"] if isinstance(example["answers"], dict) else example["answers"]
        assert len(answers) > 0
        return Sample(id=idx, data={"title": example.get("title", ""), "context": example["context"],
                                    "question": example["question"], "answers": answers},
                      candidates=None, correct_candidate=answers)


class DROPDataset(_TableDataset):
    hf_args, key, templates = ("drop",), "drop", {0: T.DROPTemplate}
    metric_name = "f1"
    generation = True

    def build_sample(self, example, idx=None):
        spans = example.get("answers_spans")
        answers = spans["spans"] if isinstance(spans, dict) else example["answers"]
        assert len(answers) > 0
        return Sample(id=idx, data={"context": example.get("passage", example.get("context")),
                                    "question": example["question"], "answers": answers},
                      candidates=None, correct_candidate=answers)


class SyntheticDataset(Dataset):
    """Offline sentiment-like task: sentences of random "words", the label decides which of
    two marker words dominates.  Same interface as the real tasks; template = SST-2's."""

    def __init__(self, subtask=None, n_train=1000, n_valid=200, **kwargs):
        self.subtask = subtask
        rng = random.Random(0 if subtask is None else hash(subtask) & 0xFFFF)
        good = ["fine", "bright", "warm", "glad"]
        bad = ["dull", "cold", "grim", "sour"]
        filler = ["the", "film", "was", "and", "very", "quite", "plot", "cast", "score", "it"]

        def make(i):
            label = rng.randint(0, 1)
            words = [rng.choice(filler) for _ in range(rng.randint(4, 9))]
            for _ in range(rng.randint(1, 3)):
                words.insert(rng.randint(0, len(words)), rng.choice(good if label else bad))
            return Sample(id=i, data={"sentence": " ".join(words), "label": label, "idx": i},
                          correct_candidate=label, candidates=[0, 1])
        train = [make(i) for i in range(n_train)]
        valid = [make(n_train + i) for i in range(n_valid)]
        self.samples = {"train": train, "valid": valid, "test": valid}

    def get_template(self, template_version=0):
        return T.SST2Template()
