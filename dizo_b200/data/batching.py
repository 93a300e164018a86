"""Collated inputs -> :class:`dizo_b200.models.opt.Batch`.

The reference's loss wrapper (large_models/trainer.py:1446-1522) shifts the full logits, masks
everything except the last ``option_len`` tokens of every sequence, averages their
log-probabilities per candidate and takes a cross entropy over each example's candidates (or a
token cross entropy when not training as classification).  The same objective is described
here by index tensors built once on the host: which hidden rows predict option tokens, which
token each must predict, how rows group into sequences and sequences into examples.  Only those
rows ever reach the LM head.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..models.opt import Batch
from ..ops.norm import opt_positions


def batch_from_inputs(inputs: Dict[str, Any], pad_token_id: int, classification: Optional[bool] = None,
                      only_train_option: bool = True, verbalizer_shortcut: bool = True) -> Batch:
    """``inputs``: ``input_ids`` [S, L] (left padded), ``attention_mask``, and either
    (``labels`` [S] = index of the correct candidate, ``option_len`` [S], ``num_options`` [S])
    for classification, or (``labels`` [S, L] token ids, optional ``option_len``) for LM-style
    training.  Returns a CPU batch."""
    ids = torch.as_tensor(inputs["input_ids"]).to(torch.int32)
    S, L = ids.shape
    mask = inputs.get("attention_mask")
    mask = torch.ones_like(ids) if mask is None else torch.as_tensor(mask).to(torch.int32)
    pad_left = (L - mask.sum(dim=1)).to(torch.int32)
    positions = opt_positions(mask)
    if classification is None:
        classification = "num_options" in inputs
    opt_len = inputs.get("option_len")
    if opt_len is not None:
        opt_len = [int(x) for x in torch.as_tensor(opt_len).tolist()]
    n_real = mask.sum(dim=1).tolist()

    if classification:
        num_options = [int(x) for x in torch.as_tensor(inputs["num_options"]).tolist()]
        cand_label = [int(x) for x in torch.as_tensor(inputs["labels"]).tolist()]
        ex_start, labels, i = [0], [], 0
        while i < S:
            n = num_options[i]
            labels.append(cand_label[i])
            i += n
            ex_start.append(i)
        if verbalizer_shortcut:
            short = _try_verbalizer_shortcut(ids, pad_left, positions, opt_len, ex_start, labels, L)
            if short is not None:
                return short
    rows, targets, seq_start = [], [], [0]
    ids_l = ids.tolist()
    for s in range(S):
        if opt_len is not None and (only_train_option or classification):
            ol = min(opt_len[s], n_real[s] - 1)
        else:
            ol = n_real[s] - 1                      # every real token after the first
        for pos in range(L - ol, L):
            tok = ids_l[s][pos]
            if tok == pad_token_id:
                continue                             # pad labels are ignored, as in the reference
            rows.append(s * L + pos - 1)
            targets.append(tok)
        seq_start.append(len(rows))
    b = Batch(input_ids=ids, pad_left=pad_left, positions=positions,
              rows=torch.tensor(rows, dtype=torch.int32), targets=torch.tensor(targets, dtype=torch.int32),
              seq_start=torch.tensor(seq_start, dtype=torch.int32), classification=bool(classification))
    if classification:
        b.ex_start = torch.tensor(ex_start, dtype=torch.int32)
        b.labels = torch.tensor(labels, dtype=torch.int32)
    return b


def _try_verbalizer_shortcut(ids, pad_left, positions, opt_len, ex_start, labels, L) -> Optional[Batch]:
    """If every candidate is a single token, the candidates of an example share their prompt and
    all examples use the same candidate tokens, the candidate cross entropy equals a cross
    entropy over those tokens' logits at the last prompt position (the softmax normaliser
    cancels): forward one sequence per example instead of one per candidate."""
    if opt_len is None or any(o != 1 for o in opt_len):
        return None
    E = len(ex_start) - 1
    cand = None
    keep = []
    for e in range(E):
        a, b = ex_start[e], ex_start[e + 1]
        if b - a < 2:
            return None
        block = ids[a:b]
        if not bool((block[:, :-1] == block[0:1, :-1]).all()) or not bool((pad_left[a:b] == pad_left[a]).all()):
            return None
        c = block[:, -1].tolist()
        if cand is None:
            cand = c
        elif c != cand:
            return None
        keep.append(a)
    keep_t = torch.tensor(keep, dtype=torch.long)
    rows = torch.arange(E, dtype=torch.int32) * L + (L - 2)
    return Batch(input_ids=ids[keep_t].contiguous(), pad_left=pad_left[keep_t].contiguous(),
                 positions=positions[keep_t].contiguous(), rows=rows,
                 labels=torch.tensor(labels, dtype=torch.int32),
                 cand_ids=torch.tensor(cand, dtype=torch.int32), classification=True)
