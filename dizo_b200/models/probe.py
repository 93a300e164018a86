"""Linear probing: fit a logistic regression on the LM-head input features of the option
tokens and write its coefficients into the LM-head rows of the class tokens.

Same procedure as the reference (large_models/trainer.py:855-957): features are the final
hidden states (after the last LayerNorm) at the positions that predict option tokens, targets
are those tokens, the classifier is scikit-learn's ``LogisticRegressionCV`` without intercept
(OPT's LM head has no bias), a two-class fit is expanded to (-w/2, +w/2).  The features come
from the kernel forward; the regression itself stays on the host.
"""
from __future__ import annotations

import logging

import torch


logger = logging.getLogger(__name__)


@torch.no_grad()
def collect_features(trainer, max_batches: int | None = None):
    model, a = trainer.model, trainer.args
    assert not a.train_as_classification and a.only_train_option, \
        "linear probing uses LM-style features (train_as_classification False, only_train_option True)"
    feats, targs = [], []
    n = len(trainer.train_dataset)
    bs = a.per_device_train_batch_size
    for s in range(0, n, bs):
        if max_batches is not None and s // bs >= max_batches:
            break
        inputs = trainer.data_collator([trainer.train_dataset[i] for i in range(s, min(n, s + bs))])
        b = trainer._to_batch(inputs)
        h = model.hidden_states(b)
        x = model.final_rows(h, b.rows)
        feats.append(x.float().cpu())
        targs.append(b.targets.cpu())
    return torch.cat(feats).numpy(), torch.cat(targs).numpy()


def linear_probe(trainer):
    from sklearn.linear_model import LogisticRegressionCV
    model, a = trainer.model, trainer.args
    logger.info("Linear probing")
    logger.info("Starting to get features for training dataset")
    features, targets = collect_features(trainer)
    logger.info("Finished getting features for training dataset")
    tol = 0.01 if a.lp_early_stopping else 1e-4
    max_iter = 1000 if a.lp_early_stopping else 5000
    logger.info("Fitting logistic regression...")
    reg = LogisticRegressionCV(max_iter=max_iter, fit_intercept=False, random_state=0, tol=tol,
                               n_jobs=-1).fit(features, targets)
    logger.info("Done")
    coef = torch.tensor(reg.coef_, dtype=torch.float32)
    if coef.shape[0] == 1:                      # two classes: one weight vector
        assert len(reg.classes_) == 2
        coef = torch.cat([-coef / 2, coef / 2], dim=0)
    name = "lm_head.weight" if model.untied else model.EMBED
    head = model.param(name)
    logger.info("Assigning weights to model")
    for i, token_id in enumerate(reg.classes_):
        head[int(token_id)].copy_(coef[i].to(head.dtype))
    return {"linear_probing_classes": [int(c) for c in reg.classes_]}
