"""Stock-PyTorch statement of the reference's ZO hot loop (the same-box baseline).

The reference cannot be imported with the installed ``transformers`` (its trainer module needs
symbols that no longer exist), so this file restates, with library calls only, exactly what
its training step does on the GPU:

* perturb / restore / update: ``torch.manual_seed(seed)`` then, per trainable tensor,
  ``z = torch.normal(0, 1, size)`` materialised in the parameter dtype and an out-of-place
  ``param + scale * z * eps`` (large_models/trainer.py:1429-1444, :1597-1608) - four sweeps over
  the parameters per step;
* forward: Hugging Face ``OPTForCausalLM`` (cuBLAS GEMMs, the installed attention backend),
  full [B, L, V] logits, shift, full-vocabulary ``log_softmax``, gather of the gold tokens,
  mean over the last ``option_len`` tokens per candidate, cross entropy over candidates
  (large_models/trainer.py:1446-1522);
* DiZO gamma search by ZO: per-tensor norms, apply / forward / reverse twice per iteration,
  ten iterations, final apply (large_models/trainer.py:545-614, :782-803).

Nothing of the framework's kernels or engine is used here.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


def build_hf_opt(cfg_dict: dict, device, dtype, seed: int = 0):
    from transformers import OPTConfig, OPTForCausalLM
    skip = ("model_type", "architectures")
    hc = OPTConfig(**{k: v for k, v in cfg_dict.items() if k not in skip})
    torch.manual_seed(seed)
    with torch.device(device):
        model = OPTForCausalLM(hc).to(dtype)
    return model.eval()


def loss_with_option_len(model, input_ids, attention_mask, option_len, num_options, labels, pad_id=1):
    """Candidate log-likelihood classification loss, as the reference computes it."""
    logits = model(input_ids=input_ids, attention_mask=attention_mask).logits
    shift_logits = logits[..., :-1, :].contiguous()
    shift_labels = torch.clone(input_ids)[..., 1:].contiguous()
    shift_labels[shift_labels == pad_id] = -100
    for i, ol in enumerate(option_len):
        shift_labels[i, :-ol] = -100
    log_probs = F.log_softmax(shift_logits, dim=-1)
    mask = shift_labels != -100
    shift_labels[~mask] = 0
    selected = torch.gather(log_probs, dim=-1, index=shift_labels.unsqueeze(-1)).squeeze(-1)
    selected = (selected * mask).sum(-1) / mask.sum(-1)
    n = num_options[0]
    selected = selected.view(-1, n)
    return F.cross_entropy(selected, labels.view(-1, n)[:, 0])


class TorchMeZO:
    """Reference-pattern ZO-SGD (+ optional DiZO gamma search by ZO) on a HF model."""

    def __init__(self, model, eps=1e-3, dizo=False, z_fn=None, seed_fn=None, gamma_z_fn=None, loss_fn=None):
        """``z_fn(name, param, seed)``, ``seed_fn()``, ``gamma_z_fn(index, iteration)`` and
        ``loss_fn(model, batch)`` let a test feed this loop the framework's random streams and
        loss; by default it draws from torch / NumPy exactly as the reference does."""
        self.model = model
        self.eps = eps
        self.z_fn = z_fn
        self.seed_fn = seed_fn or (lambda: int(np.random.randint(1_000_000_000)))
        self.gamma_z_fn = gamma_z_fn
        self.loss_fn = loss_fn or (lambda m, b: loss_with_option_len(m, **b))
        self.named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        # the reference drops the (tied) token embedding from the ZO set in full fine-tuning
        if self.named and self.named[0][0] == "model.decoder.embed_tokens.weight":
            self.named = self.named[1:]
        self.random_vector = {}
        self.dizo = dizo
        if dizo:
            self.incl = [(n, p) for n, p in self.named
                         if "self_attn.k_proj.weight" in n or "self_attn.v_proj.weight" in n]
            self.anchor = {n: p.detach().clone() for n, p in self.incl}
            self.gamma = [torch.zeros(1, device=p.device, dtype=p.dtype) for _, p in self.incl]

    def _z(self, name, p, seed):
        if self.z_fn is not None:
            return self.z_fn(name, p, seed).to(p.dtype)
        return torch.normal(mean=0, std=1, size=p.data.size(), device=p.data.device, dtype=p.data.dtype)

    def perturb(self, seed, scaling):
        torch.manual_seed(seed)
        for name, p in self.named:
            z = self._z(name, p, seed)
            p.data = p.data + scaling * z * self.eps
            self.random_vector[name] = z

    @torch.inference_mode()
    def step(self, batch, lr):
        seed = self.seed_fn()
        self.perturb(seed, 1)
        l1 = self.loss_fn(self.model, batch)
        self.perturb(seed, -2)
        l2 = self.loss_fn(self.model, batch)
        g = ((l1 - l2) / (2 * self.eps)).item()
        self.perturb(seed, 1)
        torch.manual_seed(seed)
        for name, p in self.named:
            z = self._z(name, p, seed)
            p.data = p.data - lr * (g * z)
        return l1

    # ---- DiZO gamma search by ZO (apply -> forward -> reverse, twice per iteration)
    def _apply(self, alphas):
        for (n, p), a in zip(self.incl, alphas):
            an = self.anchor[n]
            p.copy_((p.detach() - an) * a + an)

    def _reverse(self, alphas):
        for (n, p), a in zip(self.incl, alphas):
            an = self.anchor[n]
            p.copy_((p.detach() - an) / a + an)

    def _ratios(self):
        return [g / (torch.norm(p.data - self.anchor[n]) + 1e-8) for (n, p), g in zip(self.incl, self.gamma)]

    @torch.no_grad()
    def dizo_search(self, batches, tau=0.2, zo_eps=0.1, step_size=2):
        init = True
        for it, batch in enumerate(batches):
            ts = [torch.norm(p.data - self.anchor[n]) for n, p in self.incl]
            if init:
                self.gamma = [t.clone().reshape(1) for t in ts]
                init = False
            zs = []
            for i, g in enumerate(self.gamma):
                if self.gamma_z_fn is not None:
                    z = torch.tensor([self.gamma_z_fn(i, it)], device=g.device, dtype=g.dtype)
                else:
                    z = torch.normal(0, 1, size=(1,), device=g.device, dtype=g.dtype)
                z = torch.clip(z, (-tau / zo_eps) * ts[i], (tau / zo_eps) * ts[i])
                zs.append(z)
                self.gamma[i] = g + z * zo_eps
            al = self._ratios(); self._apply(al)
            l1 = self.loss_fn(self.model, batch)
            self._reverse(al)
            for i in range(len(self.gamma)):
                self.gamma[i] = self.gamma[i] - 2 * zs[i] * zo_eps
            al = self._ratios(); self._apply(al)
            l2 = self.loss_fn(self.model, batch)
            self._reverse(al)
            grad = (l1 - l2) / (2 * zo_eps)
            for i in range(len(self.gamma)):
                g = self.gamma[i] + zs[i] * zo_eps
                self.gamma[i] = torch.clip(g - step_size * ts[i] * grad * zs[i], (1 - tau) * ts[i], (1 + tau) * ts[i])
        self._apply(self._ratios())


def synthetic_reference_batch(step, n_prompts, seq_len, vocab, seed, rank, cand_ids, device, candidates=2):
    """The framework's synthetic prompts in the reference's input format: every prompt becomes
    ``candidates`` sequences (prompt[:-1] + candidate token), option_len 1."""
    rng = np.random.Generator(np.random.Philox(key=[seed, (rank << 32) | (step & 0xFFFFFFFF)]))
    ids = rng.integers(4, vocab, size=(n_prompts, seq_len), dtype=np.int64)
    labels = (rng.random(n_prompts) < 0.5).astype(np.int64)
    seqs, labs = [], []
    for b in range(n_prompts):
        for c in range(candidates):
            s = ids[b].copy()
            s[-1] = cand_ids[c % len(cand_ids)]
            seqs.append(s)
            labs.append(labels[b] % candidates)
    x = torch.from_numpy(np.stack(seqs)).to(device)
    return dict(input_ids=x, attention_mask=torch.ones_like(x),
                option_len=[1] * len(seqs), num_options=[candidates] * len(seqs),
                labels=torch.tensor(labs, device=device))
