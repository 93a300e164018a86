"""Loss tail: option-row log-probabilities, candidate cross entropy, verbalizer shortcut.

The reference's ``forward_wrap_with_option_len`` (large_models/trainer.py:1446-1522,
large_models/utils.py:31-105) computes full [B, L, V] logits, a full-vocabulary
log_softmax, gathers the gold tokens, averages the last ``option_len`` per candidate and
applies a cross entropy over candidates (or token CE).  Here only the rows that predict
option tokens reach the LM head, and the log-sum-exp is fused into the GEMM epilogue.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

ll = ctypes.c_longlong


def token_logprobs(h_rows: torch.Tensor, table: torch.Tensor, targets: torch.Tensor,
                   scale: float = 1.0) -> torch.Tensor:
    """log softmax(h_rows @ table.T * scale)[r, targets[r]] for every row (fp32 [R])."""
    if not h_rows.is_cuda:
        logits = (h_rows.float() @ table.float().t()) * scale
        lp = torch.log_softmax(logits, dim=-1)
        return lp.gather(1, targets.long().view(-1, 1)).squeeze(1)
    L = _lib.lib()
    R, K = h_rows.shape
    V = table.shape[0]
    nt = L.dz_gemm_lse_num_tiles(V)
    f = dict(dtype=torch.float32, device=h_rows.device)
    pm = torch.empty((R, nt), **f)
    ps = torch.empty((R, nt), **f)
    tg = torch.empty(R, **f)
    out = torch.empty(R, **f)
    assert targets.dtype == torch.int32
    rc = L.dz_gemm_bf16_tn_lse(_lib.ptr(h_rows), ll(h_rows.stride(0)), _lib.ptr(table),
                               ll(table.stride(0)), _lib.ptr(targets), _lib.ptr(pm), _lib.ptr(ps),
                               _lib.ptr(tg), R, V, K, ctypes.c_float(scale),
                               _lib.ptr(_lib.err_word(h_rows.device)), _lib.stream_ptr())
    _lib.check(rc, "dz_gemm_bf16_tn_lse")
    rc = L.dz_lse_combine(_lib.ptr(pm), _lib.ptr(ps), _lib.ptr(tg), nt, R, _lib.ptr(out), None,
                          _lib.stream_ptr())
    _lib.check(rc, "dz_lse_combine")
    return out


def option_ce(logprob: torch.Tensor, seq_start: torch.Tensor, ex_start: torch.Tensor | None,
              labels: torch.Tensor | None, classification: bool) -> torch.Tensor:
    """One fp32 loss from per-row log-probabilities.

    ``seq_start`` [S+1]: rows of sequence s are [seq_start[s], seq_start[s+1]).
    classification: sequences are candidates; ``ex_start`` [E+1] groups them into examples and
    ``labels`` [E] is the index of the correct candidate: loss = mean_e CE(mean-logprob per
    candidate).  Otherwise: token cross entropy, mean over all rows."""
    n_seq = seq_start.numel() - 1
    if not logprob.is_cuda:
        if not classification:
            return -logprob.float().mean().reshape(1)
        ss = seq_start.tolist()
        seq_lp = torch.stack([logprob[ss[i]:ss[i + 1]].float().mean() for i in range(n_seq)])
        es = ex_start.tolist()
        losses = []
        for e in range(len(es) - 1):
            c = seq_lp[es[e]:es[e + 1]]
            losses.append(torch.logsumexp(c, 0) - c[int(labels[e])])
        return torch.stack(losses).mean().reshape(1)
    out = torch.empty(1, dtype=torch.float32, device=logprob.device)
    seq_lp = torch.empty(max(n_seq, 1), dtype=torch.float32, device=logprob.device)
    n_ex = (ex_start.numel() - 1) if classification else 0
    rc = _lib.lib().dz_option_ce(_lib.ptr(logprob), _lib.ptr(seq_start), n_seq, _lib.ptr(ex_start),
                                 _lib.ptr(labels), n_ex, 0 if classification else 1,
                                 _lib.ptr(seq_lp), _lib.ptr(out), _lib.stream_ptr())
    _lib.check(rc, "dz_option_ce")
    return out


def verbalizer_ce(h_last: torch.Tensor, table: torch.Tensor, cand_ids: torch.Tensor,
                  labels: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """Logits of the candidate ids at the last position and their mean cross entropy.

    Equals the candidate-CE of the general path when every candidate is one token and the
    candidates of an example share the prompt (the log-softmax normaliser cancels)."""
    E = h_last.shape[0]
    C = cand_ids.numel()
    if not h_last.is_cuda:
        logits = h_last.float() @ table[cand_ids.long()].float().t()
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits, labels.long()).reshape(1)
        return logits, loss
    logits = torch.empty((E, C), dtype=torch.float32, device=h_last.device)
    loss = torch.empty(1, dtype=torch.float32, device=h_last.device) if labels is not None else None
    rc = _lib.lib().dz_verbalizer_ce(_lib.ptr(h_last), ll(h_last.stride(0)), _lib.ptr(table),
                                     ll(table.stride(0)), _lib.ptr(cand_ids), C, _lib.ptr(labels), E,
                                     h_last.shape[1], _lib.ptr(logits), _lib.ptr(loss),
                                     _lib.stream_ptr())
    _lib.check(rc, "dz_verbalizer_ce")
    return logits, loss
