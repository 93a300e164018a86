"""Synthetic verbalizer task: seeded uniform token ids, Bernoulli(0.5) labels.

Every prompt is ``seq_len`` ids drawn uniformly from [4, vocab) and the label picks one of
``cand_ids`` (fixed verbalizer tokens); the loss is the cross entropy over the last-position
logits of those candidate ids.  Batches are a pure function of (seed, rank, step), so every
process can build its own shard and a resumed run sees the same data.
"""
from __future__ import annotations

import numpy as np
import torch

from ..models.opt import Batch

DEFAULT_CANDS = (1099, 372)     # two fixed token ids standing in for "great" / "terrible"


def synthetic_batch(step: int, n_prompts: int, seq_len: int, vocab: int, seed: int = 1,
                    rank: int = 0, cand_ids=DEFAULT_CANDS, pad_left: int = 0,
                    pin: bool = False) -> Batch:
    """CPU batch for ``step`` (optionally in pinned memory, ready for an async H2D copy)."""
    rng = np.random.Generator(np.random.Philox(key=[seed, (rank << 32) | (step & 0xFFFFFFFF)]))
    ids = rng.integers(4, vocab, size=(n_prompts, seq_len), dtype=np.int64).astype(np.int32)
    labels = (rng.random(n_prompts) < 0.5).astype(np.int32)
    ids_t = torch.from_numpy(ids)
    pl = torch.full((n_prompts,), pad_left, dtype=torch.int32)
    mask = torch.ones(n_prompts, seq_len, dtype=torch.int32)
    if pad_left:
        mask[:, :pad_left] = 0
        ids_t[:, :pad_left] = 1
    pos = (torch.cumsum(mask, 1) * mask - 1 + 2).to(torch.int32)
    rows = (torch.arange(n_prompts, dtype=torch.int32) * seq_len + (seq_len - 1))
    b = Batch(input_ids=ids_t, pad_left=pl, positions=pos, rows=rows,
              labels=torch.from_numpy(labels), cand_ids=torch.tensor(cand_ids, dtype=torch.int32),
              classification=True)
    return b.pin() if pin else b
