"""Templates, tasks, prompt encoding, collators, metrics, argument surface (CPU)."""
import json
import random

import numpy as np
import pytest

from dizo_b200 import templates as T
from dizo_b200.args import OurArguments, parse_args
from dizo_b200.metrics import calculate_metric, f1, normalize_answer
from dizo_b200.tasks import Sample, SyntheticDataset, get_task
from dizo_b200.utils import (DataCollatorForTokenClassification, DataCollatorWithPaddingAndNesting,
                             ICLCollator, Prediction, StubTokenizer, encode_prompt, temp_seed)


def S(**data):
    return Sample(id=0, data=data, correct_candidate=None, candidates=None)


def test_template_strings():
    s = S(sentence=" a fine film ")
    t = T.SST2Template()
    assert t.encode(s) == "a fine film It was"
    assert t.verbalize(s, 1) == "a fine film It was great"
    assert t.verbalize(s, 0) == "a fine film It was terrible"
    assert t.encode_sfc(s) == " It was" and t.verbalize_sfc(s, 1) == " It was great"

    c = S(premise="The man broke his toe.", question="cause", choice1="He got a hole in his sock.",
          choice2="He dropped a hammer on his foot.", label=1)
    ct = T.CopaTemplate()
    assert ct.encode(c) == "The man broke his toe because "
    assert ct.verbalize(c, c.data["choice2"]) == "The man broke his toe because he dropped a hammer on his foot."
    assert ct.verbalize(c, "I left.") == "The man broke his toe because I left."
    assert ct.encode_sfc(c) == "because" and ct.verbalize_sfc(c, "He ran.") == "because he ran."
    c.data["question"] = "effect"
    assert ct.encode(c).endswith(" so ")

    b = S(passage="P.", question="is it so")
    assert T.BoolQTemplate().verbalize(b, "Yes") == "P. Is it so? Yes"
    assert T.BoolQTemplateV2().encode(b) == "P. Is it so?\\n\\n"
    assert T.BoolQTemplateV3().verbalize(b, "No") == "P. Is it so?\nNo"
    assert T.BoolQTemplateV3().encode_sfc(b) == "" and T.BoolQTemplateV3().verbalize_sfc(b, "No") == "No"

    m = S(paragraph="Par", question="Q", answer="A")
    assert T.MultiRCTemplate().verbalize(m, 1) == \
        'Par\nQuestion: Q\nI found this answer "A". Is that correct? Yes or No?\nYes'
    n = S(premise="P", hypothesis="H")
    assert T.CBTemplate().verbalize(n, 2) == 'Suppose P Can we infer that "H"? Yes, No, or Maybe?\nMaybe'
    assert T.MNLITemplate().encode(n) == T.CBTemplate().encode(n)
    assert T.RTETemplate().verbalize(n, 0) == 'P\nDoes this mean that "H" is true? Yes or No?\nYes'
    w = S(word="bank", sentence1="s1", sentence2="s2")
    assert T.WICTemplate().verbalize(w, 0) == \
        'Does the word "bank" have the same meaning in these two sentences? Yes, No?\ns1\ns2\nNo'
    ws = S(text="T", span1_text="Bob", span2_text="He")
    assert T.WSCTemplate().encode(ws) == \
        'T\nIn the previous sentence, does the pronoun "he" refer to Bob? Yes or No?\n'
    r = S(passage="Text\n@highlight\nFact", query="X met @placeholder", entities=["A", "B"], answers=["A"])
    assert T.ReCoRDTemplateGPT3().encode(r) == "Text\n- Fact\n-"
    assert T.ReCoRDTemplateGPT3().verbalize(r, ["A"]) == "Text\n- Fact\n- X met A"
    assert T.ReCoRDTemplate().verbalize(r, "B").endswith('Question: what is the "@placeholder"\nAnswer: B')
    q = S(title="Ti", context="C", question=" Q? ", answers=["a1", "a2"])
    assert T.SQuADv2Template().encode(q) == "Title: Ti\nContext: C\nQuestion: Q?\nAnswer:"
    assert T.SQuADv2Template().verbalize(q, None) == "Title: Ti\nContext: C\nQuestion: Q?\nAnswer: a1\n"
    assert T.DROPTemplate().encode(q) == "Passage: C\nQuestion: Q?\nAnswer:"
    with pytest.raises(NotImplementedError):
        T.DROPTemplate().encode_sfc(q)


def test_metrics():
    assert normalize_answer("The  Cat, sat!") == "cat sat"
    assert f1("the cat sat", ["cat sat down"]) == pytest.approx(0.8)
    assert f1("x", ["CANNOTANSWER"]) == 0 and f1("cannotanswer", ["CANNOTANSWER"]) == 1
    preds = [Prediction(1, 1), Prediction(0, 1)]
    assert calculate_metric(preds, "accuracy") == 0.5
    assert calculate_metric([Prediction([0, 2], 2)], "accuracy") == 1.0
    assert calculate_metric([Prediction(["A cat"], "cat")], "em") == 1.0
    assert calculate_metric([Prediction(["cat sat down"], "the cat sat")], "f1") == pytest.approx(0.8)


def test_args_surface_and_parsing():
    a = OurArguments()
    ref_defaults = dict(task_name="SST2", num_train=0, max_length=2048, trainer="none", only_train_option=True,
                        train_as_classification=False, zo_eps=1e-3, bits=11, rng=8, size=0.9, enhanced=None,
                        num_prefix=5, no_reparam=True, prefix_init_by_real_act=True, lora_alpha=16, lora_r=8,
                        top_p=0.95, max_new_tokens=50, eos_token="\n", model_name="./opt1p3b")
    for k, v in ref_defaults.items():
        assert getattr(a, k) == v, k
    assert (a.dizo_interval, a.dizo_max_iters, a.dizo_tau, a.dizo_zo_eps, a.dizo_step_size) == (50, 10, 0.2, 0.1, 2.0)
    p = parse_args(["--task_name", "RTE", "--trainer", "zo", "--lora", "--train_as_classification", "False",
                    "--learning_rate", "1e-6", "--enhanced", "zo", "--num_dev", "500", "--top_k", "None",
                    "--max_steps", "4000", "--load_float16", "--lr_scheduler_type", "constant"])
    assert p.task_name == "RTE" and p.lora is True and p.train_as_classification is False
    assert p.learning_rate == 1e-6 and p.enhanced == "zo" and p.num_dev == 500 and p.top_k is None
    assert p.load_float16 is True and p.max_steps == 4000


def test_task_sampling_and_registry():
    random.seed(0)
    task = get_task("Synthetic")
    assert isinstance(task, SyntheticDataset) and len(task.samples["train"]) == 1000
    sets = task.sample_train_sets(num_train=8, num_train_sets=3)
    assert len(sets) == 3 and all(len(s) == 8 for s in sets)
    again = task.sample_train_sets(num_train=8, num_train_sets=3)
    assert [x.id for x in sets[1]] == [x.id for x in again[1]]
    one = task.sample_train_sets(num_train=4, num_dev=2, seed=7)
    assert len(one) == 1 and len(one[0]) == 6
    per_eval = task.sample_train_sets(num_train=2, num_eval=5)
    assert len(per_eval) == 5
    sub = task.sample_subset("valid", seed=1, num=10, exclude=3)
    assert len(sub) == 10


def test_task_from_jsonl(tmp_path, monkeypatch):
    d = tmp_path / "rte"
    d.mkdir()
    rows = [{"premise": f"p{i}", "hypothesis": f"h{i}", "label": i % 2, "idx": i} for i in range(30)]
    for split in ("train", "validation"):
        (d / f"{split}.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    monkeypatch.setenv("DIZO_DATA_DIR", str(tmp_path))
    random.seed(1)
    task = get_task("RTE")
    assert len(task.samples["train"]) == 30 and task.samples["test"] is task.samples["valid"]
    s = task.samples["train"][0]
    assert s.candidates == [0, 1] and s.correct_candidate in (0, 1)
    assert "Does this mean that" in task.get_template().encode(s)


def test_encode_prompt_and_collators():
    tok = StubTokenizer(["terrible", "great", "It", "was"])
    task = SyntheticDataset()
    tpl = task.get_template()
    smp = task.samples["valid"][0]
    enc, ol = encode_prompt(task, tpl, [], smp, tok, max_length=64)
    assert len(enc) == 2 and ol == [1, 1]
    assert enc[0][:-1] == enc[1][:-1] and enc[0][-1] != enc[1][-1] and enc[0][0] == tok.bos_token_id
    demos = task.samples["train"][:3]
    enc_icl, _ = encode_prompt(task, tpl, demos, smp, tok, max_length=4096)
    text = tok.decode(enc_icl[0])
    assert text.count("It was") == 4 and "\n\n" in text
    # left truncation keeps BOS and the answer end
    enc_t, _ = encode_prompt(task, tpl, demos, smp, tok, max_length=20)
    assert len(enc_t[0]) == 20 and enc_t[0][0] == tok.bos_token_id and enc_t[0][-1] == enc[0][-1]
    sfc, sol = encode_prompt(task, tpl, demos, smp, tok, max_length=64, sfc=True)
    assert tok.decode(sfc[1]).strip() == "It was great" and sol == [1, 1]

    feats = [[{"input_ids": enc[i], "labels": 1, "option_len": ol[i], "num_options": 2} for i in range(2)],
             [{"input_ids": enc[i][:-3] + enc[i][-1:], "labels": 0, "option_len": 1, "num_options": 2} for i in range(2)]]
    batch = DataCollatorWithPaddingAndNesting(tok, pad_to_multiple_of=8)(feats)
    assert batch["input_ids"].shape[0] == 4 and batch["input_ids"].shape[1] % 8 == 0
    assert batch["attention_mask"][2, 0] == 0 and batch["attention_mask"][2, -1] == 1      # left padded
    assert batch["labels"].tolist() == [1, 1, 0, 0] and batch["num_options"].tolist() == [2, 2, 2, 2]
    lm = DataCollatorForTokenClassification(tok, pad_to_multiple_of=8)(
        [{"input_ids": enc[0], "labels": enc[0], "option_len": 1}, {"input_ids": enc[1][2:], "labels": enc[1][2:], "option_len": 1}])
    assert lm["labels"][1, 0] == -100 and lm["input_ids"][1, 0] == tok.pad_token_id
    icl = ICLCollator(tok)([{"input_ids": [2, 5, 6], "attention_mask": [1, 1, 1]}, {"input_ids": [2, 5], "attention_mask": [1, 1]}])
    assert icl["input_ids"][1].tolist() == [2, 5, tok.pad_token_id] and icl["attention_mask"][1].tolist() == [1, 1, 0]


def test_temp_seed_restores_state():
    np.random.seed(5)
    a = np.random.rand()
    np.random.seed(5)
    with temp_seed(99):
        np.random.rand()
    assert np.random.rand() == a
