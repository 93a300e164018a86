"""Scoring and prediction: candidate log-likelihoods, SFC calibration, generation, ICL.

Reference behaviour: ``Framework.forward`` / ``one_step_pred`` / ``evaluate``
(large_models/run.py:269-371; duplicated in large_models/trainer.py:1701-1766) score one
candidate per forward with a full-vocabulary ``log_softmax`` and a host sync each.  Here all
candidates of a group of samples go through one batched forward that only sends the option
rows to the LM head.  Generation tasks decode and are scored by the task's metric (the
reference's fork never reaches its generation branch from ``one_step_pred``; this builds the
intended behaviour).
"""
from __future__ import annotations

import logging
from typing import List, Optional

import numpy as np
import torch

from .data.batching import batch_from_inputs
from .metrics import calculate_metric
from .models.opt import OPTModel
from .utils import Prediction, encode_prompt, pad_sequences

logger = logging.getLogger(__name__)


class Evaluator:
    def __init__(self, model: OPTModel, tokenizer, task, args):
        self.model, self.tokenizer, self.task, self.args = model, tokenizer, task, args

    # ------------------------------------------------------------------ scoring
    def score_sequences(self, seqs: List[List[int]], option_lens: List[int]) -> List[torch.Tensor]:
        """Per sequence, the log-probabilities of its last ``option_len`` tokens (CPU fp32)."""
        out: List[Optional[torch.Tensor]] = [None] * len(seqs)
        bs = max(1, int(getattr(self.args, "eval_batch_size", 16)))
        order = sorted(range(len(seqs)), key=lambda i: len(seqs[i]))
        for s in range(0, len(order), bs):
            idx = order[s:s + bs]
            ids, mask = pad_sequences([seqs[i] for i in idx], self.tokenizer.pad_token_id, "left", 8)
            inputs = {"input_ids": ids, "attention_mask": mask, "labels": ids,
                      "option_len": [max(1, option_lens[i]) for i in idx]}
            b = batch_from_inputs(inputs, pad_token_id=-1, classification=False).to(self.model.device)
            lp = self.model.row_logprobs(b).float().cpu()
            ss = b.seq_start.cpu().tolist()
            for j, i in enumerate(idx):
                out[i] = lp[ss[j]:ss[j + 1]]
        return out  # type: ignore[return-value]

    def forward(self, input_ids: List[int], option_len: Optional[int] = None, generation: bool = False):
        """Single-sequence API of the reference: option-token log-probabilities, or the decoded
        continuation when ``generation``."""
        if generation:
            return self.generate_text(input_ids)
        return self.score_sequences([input_ids], [option_len or 1])[0]

    def generate_text(self, input_ids: List[int]) -> str:
        from .models.generate import generate
        a = self.args
        eos = [self.tokenizer.eos_token_id]
        extra = self.tokenizer.encode(a.eos_token, add_special_tokens=False)
        if extra:
            eos.append(extra[-1])
        ids = torch.tensor([input_ids], dtype=torch.long)
        out = generate(self.model, ids, max_new_tokens=min(a.max_new_tokens, a.max_length - len(input_ids)),
                       do_sample=a.sampling, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                       num_beams=a.num_beams, eos_token_id=eos, pad_token_id=self.tokenizer.pad_token_id)
        return self.tokenizer.decode(out[0][len(input_ids):], skip_special_tokens=True).strip()

    # ------------------------------------------------------------------ prediction
    def one_step_pred(self, train_samples, eval_sample, verbose: bool = False) -> Prediction:
        return self.predict_many([train_samples], [eval_sample], verbose=verbose)[0]

    def predict_many(self, train_sets, eval_samples, verbose: bool = False) -> List[Prediction]:
        """``train_sets[i]`` are the in-context demonstrations for ``eval_samples[i]`` (a single
        set is shared when ``len(train_sets) == 1``)."""
        a, task, tok = self.args, self.task, self.tokenizer
        verbose = verbose or getattr(a, "verbose", False)
        template = task.get_template()
        preds: List[Prediction] = []
        if task.generation:
            for i, smp in enumerate(eval_samples):
                demos = train_sets[i if len(train_sets) > 1 else 0]
                enc, _ = encode_prompt(task, template, demos, smp, tok, max_length=a.max_length,
                                       generation=True, max_new_tokens=a.max_new_tokens)
                text = self.generate_text(enc[0])
                if verbose:
                    logger.info("=== Prompt ===\n%s\nOutput: %s", tok.decode(enc[0]), text)
                preds.append(Prediction(correct_candidate=smp.correct_candidate, predicted_candidate=text))
            return preds

        seqs, lens, owner = [], [], []
        sfc_seqs, sfc_lens = [], []
        for i, smp in enumerate(eval_samples):
            demos = train_sets[i if len(train_sets) > 1 else 0]
            enc, ol = encode_prompt(task, template, demos, smp, tok, max_length=a.max_length)
            for c in range(len(enc)):
                seqs.append(enc[c]); lens.append(ol[c]); owner.append(i)
            if a.sfc or a.icl_sfc:
                senc, sol = encode_prompt(task, template, demos, smp, tok, max_length=a.max_length,
                                          sfc=a.sfc, icl_sfc=a.icl_sfc)
                sfc_seqs += senc; sfc_lens += sol
        lps = self.score_sequences(seqs, lens)
        sfc_lps = self.score_sequences(sfc_seqs, sfc_lens) if sfc_seqs else None
        k = 0
        for i, smp in enumerate(eval_samples):
            n = len(smp.candidates)
            if sfc_lps is not None:
                # calibrated: mean over option tokens of (log p - log p_sfc)
                scores = [(lps[k + c] - sfc_lps[k + c]).mean().item() for c in range(n)]
            else:
                scores = [lps[k + c].mean().item() for c in range(n)]
            if verbose:
                logger.info("Candidates %s scores %s", smp.candidates, scores)
            k += n
            if isinstance(smp.correct_candidate, list):
                gold = [smp.candidates.index(c) for c in smp.correct_candidate]
            else:
                gold = smp.candidates.index(smp.correct_candidate)
            preds.append(Prediction(correct_candidate=gold, predicted_candidate=int(np.argmax(scores))))
        return preds

    def evaluate(self, train_samples, eval_samples, one_train_set_per_eval_sample: bool = False,
                 chunk: int = 32) -> dict:
        """Metric over ``eval_samples``; ``train_samples`` are ICL demonstrations (one shared set,
        or one set per evaluation sample)."""
        if one_train_set_per_eval_sample:
            logger.info(f"There are {len(eval_samples)} validation samples and one train set per eval sample")
        else:
            logger.info(f"There are {len(train_samples)} training samples and {len(eval_samples)} validation samples")
        preds: List[Prediction] = []
        for s in range(0, len(eval_samples), chunk):
            part = eval_samples[s:s + chunk]
            sets = [train_samples[s + j] for j in range(len(part))] if one_train_set_per_eval_sample \
                else [train_samples]
            preds += self.predict_many(sets, part)
        name = getattr(self.task, "metric_name", "accuracy")
        return {name: calculate_metric(preds, name)}
