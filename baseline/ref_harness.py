"""Harness that drives the UNMODIFIED reference (luozoupi/DiZO, ``large_models/*.py``) for the benchmark.

The reference is a flat script directory (no ``setup.py`` / ``pyproject.toml``), so it is used as a
byte-identical copy of its ``large_models/*.py`` under ``baseline/_ref/``.  Its ``trainer.py``
imports ten names that the installed ``transformers`` 5.x / ``huggingface_hub`` no longer export
(large_models/trainer.py:45-58, :80, :88, :93-113, :141-156, :834).  None of them is called on the
zeroth-order path, so this module installs inert stand-ins for them *into the library modules*
before the import - the reference files stay untouched.  ``_get_learning_rate`` is the one name
the hot loop calls (large_models/trainer.py:1608); it is bound to the implementation the library
itself still ships as ``transformers.Trainer._get_learning_rate``.

``transformers.Trainer.__init__`` needs ``accelerate``, which is not installed, so the reference's
``OurTrainer`` object is created with ``__new__`` and given exactly the attributes its own training
loop sets up before the hot loop (large_models/trainer.py:1100-1102 LR lambda, :1147-1171 trainable
set, DiZO include rule, anchor copy, ``dizo_trainer``).  From there on every line that runs is the
reference's: ``OurTrainer.zo_step`` (:1570-1595), ``zo_perturb_parameters`` (:1429-1444),
``zo_forward`` + ``forward_wrap_with_option_len`` (:1446-1542), ``zo_update`` (:1597-1617) and
``dizo_trainer.dizo_zo_iters`` / ``DiZO.zo_forward`` (:564-614, :782-803) on a Hugging Face
``OPTForCausalLM``.  Nothing of this repository's package, kernels or engine is imported here.
"""
from __future__ import annotations

import importlib
import os
import shutil
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_FILES = ("dataset.py", "enhanced_model_support.py", "ht_opt.py", "lora.py", "metrics.py", "prefix.py",
             "processors.py", "run.py", "tasks.py", "templates.py", "test.py", "trainer.py", "utils.py")

# (module, name): names the reference imports that the installed libraries no longer have
MISSING_NAMES = (
    ("transformers.integrations", "is_sigopt_available"),
    ("transformers.integrations", "run_hp_search_sigopt"),
    ("huggingface_hub", "Repository"),
    ("transformers.modeling_utils", "load_sharded_checkpoint"),
    ("transformers.trainer_pt_utils", "DistributedTensorGatherer"),
    ("transformers.trainer_pt_utils", "SequentialDistributedSampler"),
    ("transformers.utils", "get_full_repo_name"),
    ("transformers.utils", "is_ipex_available"),
    ("transformers.utils", "is_torchdynamo_available"),
    ("transformers.trainer_pt_utils", "_get_learning_rate"),
)

# OPT shapes (Hugging Face config fields) for the models the benchmark names
OPT_SHAPES = {
    "opt-tiny": dict(num_hidden_layers=2, hidden_size=128, num_attention_heads=2, ffn_dim=512),
    "opt-125m": dict(num_hidden_layers=12, hidden_size=768, num_attention_heads=12, ffn_dim=3072),
    "opt-1.3b": dict(num_hidden_layers=24, hidden_size=2048, num_attention_heads=32, ffn_dim=8192),
    "opt-2.7b": dict(num_hidden_layers=32, hidden_size=2560, num_attention_heads=32, ffn_dim=10240),
    "opt-6.7b": dict(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, ffn_dim=16384),
    "opt-13b": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, ffn_dim=20480),
}
VERBALIZER_IDS = (1099, 372)      # the two fixed candidate token ids of the synthetic task


class ReferenceUnavailable(RuntimeError):
    pass


def ensure_reference_copy(src: str | None = None) -> str:
    """Make sure ``baseline/_ref`` holds the reference's files; copy them if a source tree is at hand."""
    have = os.path.isdir(REF_DIR) and all(os.path.exists(os.path.join(REF_DIR, f)) for f in ("trainer.py", "utils.py"))
    if have:
        return REF_DIR
    cands = [src, os.environ.get("DIZO_REFERENCE_SRC"), "/root/reference/large_models"]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "trainer.py")):
            os.makedirs(REF_DIR, exist_ok=True)
            for f in REF_FILES:
                if os.path.exists(os.path.join(c, f)):
                    shutil.copyfile(os.path.join(c, f), os.path.join(REF_DIR, f))
            return REF_DIR
    raise ReferenceUnavailable("baseline/_ref is empty and no reference source tree is present to copy from")


def install_missing_names() -> list[str]:
    """Give the library modules the ten names the reference imports and they no longer export."""
    import transformers
    done = []
    for mod_name, name in MISSING_NAMES:
        mod = importlib.import_module(mod_name)
        if hasattr(mod, name):
            continue
        if name == "_get_learning_rate":
            stand_in = transformers.Trainer._get_learning_rate        # the library's own implementation
        elif name.startswith("is_"):
            stand_in = lambda *a, **k: False                          # noqa: E731  "feature not available"
        elif name[0].isupper():
            stand_in = type(name, (), {"__doc__": "placeholder for a class removed from the library"})
        else:
            def stand_in(*a, _n=name, **k):
                raise NotImplementedError(f"{_n} was removed from the installed library")
        setattr(mod, name, stand_in)
        done.append(f"{mod_name}.{name}")
    return done


def import_reference():
    """Import the reference's ``trainer`` module from the untouched copy. Returns (module, shimmed names)."""
    ensure_reference_copy()
    shimmed = install_missing_names()
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)          # the reference uses flat imports: ``from utils import ...``
    try:
        mod = importlib.import_module("trainer")
    except Exception as e:                                             # noqa: BLE001
        raise ReferenceUnavailable(f"import of the reference trainer fails: {type(e).__name__}: {e}"[:300]) from e
    if os.path.dirname(os.path.abspath(mod.__file__)) != REF_DIR:
        raise ReferenceUnavailable(f"'trainer' resolved to {mod.__file__}, not the reference copy")
    return mod, shimmed


def build_hf_opt(model_name: str, device, dtype, seed: int = 0, vocab: int = 50272):
    """Random-init Hugging Face ``OPTForCausalLM`` of the named shape (no hub access)."""
    from transformers import OPTConfig, OPTForCausalLM
    shp = OPT_SHAPES[model_name]
    cfg = OPTConfig(vocab_size=vocab, max_position_embeddings=2048, word_embed_proj_dim=shp["hidden_size"],
                    do_layer_norm_before=True, activation_function="relu", dropout=0.0, **shp)
    torch.manual_seed(seed)
    with torch.device(device):
        model = OPTForCausalLM(cfg).to(dtype)
    return model.eval()


def reference_batch(step: int, n_prompts: int, seq_len: int, vocab: int, seed: int = 1, rank: int = 0,
                    candidates: int = 2, pin: bool = False) -> dict:
    """One synthetic batch in the layout the reference's nesting collator hands to ``zo_step``
    (large_models/utils.py:206-233, large_models/run.py:415-419): every prompt becomes ``candidates``
    sequences ending in a verbalizer token; ``labels`` repeats the gold candidate index,
    ``option_len`` and ``num_options`` are int64 tensors (``tokenizer.pad(..., return_tensors='pt')``).
    Same token ids and labels as the framework's synthetic task for (seed, rank, step)."""
    rng = np.random.Generator(np.random.Philox(key=[seed, (rank << 32) | (step & 0xFFFFFFFF)]))
    ids = rng.integers(4, vocab, size=(n_prompts, seq_len), dtype=np.int64)
    labels = (rng.random(n_prompts) < 0.5).astype(np.int64)
    seqs = np.repeat(ids, candidates, axis=0)
    for c in range(candidates):
        seqs[c::candidates, -1] = VERBALIZER_IDS[c % len(VERBALIZER_IDS)]
    n = n_prompts * candidates
    b = {"input_ids": torch.from_numpy(seqs),
         "attention_mask": torch.ones(n, seq_len, dtype=torch.int64),
         "labels": torch.from_numpy(np.repeat(labels % candidates, candidates)),
         "option_len": torch.ones(n, dtype=torch.int64),
         "num_options": torch.full((n,), candidates, dtype=torch.int64)}
    if pin:
        b = {k: v.pin_memory() for k, v in b.items()}
    return b


def batch_nbytes(b: dict) -> int:
    return sum(v.numel() * v.element_size() for v in b.values() if torch.is_tensor(v))


def make_reference_trainer(ref, model, device, *, lr: float, max_steps: int, zo_eps: float,
                           enhanced: str | None, search_batches=None):
    """An ``OurTrainer`` of the reference in the state its loop has right before the first step.

    Restates only set-up lines of ``_inner_training_loop`` (the loop itself needs ``accelerate``):
    :1025 optimizer (never stepped on the ZO path), :1100-1102 LR lambda, :1147-1160 trainable set and
    DiZO exclude list, :1163-1171 anchor copy + ``dizo_trainer``."""
    import copy
    from torch.optim.lr_scheduler import LambdaLR
    from transformers.trainer_callback import TrainerState

    tr = ref.OurTrainer.__new__(ref.OurTrainer)
    args = types.SimpleNamespace(
        zo_eps=zo_eps, non_diff=False, n_gpu=1, gradient_accumulation_steps=1, enhanced=enhanced,
        max_steps=max_steps, learning_rate=lr, device=torch.device(device), past_index=-1, trainer="zo",
        task_name="Synthetic")
    tr.args = args
    tr.model = model
    tr.is_deepspeed_enabled = False
    tr.state = TrainerState()
    tr.optimizer = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=lr)
    tr.lr_scheduler = LambdaLR(tr.optimizer, lambda step: 1 - tr.state.global_step / (2 * args.max_steps))

    tr.named_parameters_to_optim = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    if tr.named_parameters_to_optim[0][0] != "model.decoder.embed_tokens.weight":
        tr.exclude_list = [k for k in model.state_dict().keys() if "lora" not in k]
    else:
        tr.exclude_list = ["model.decoder.embed_tokens.weight"] + [
            n for n, _ in tr.named_parameters_to_optim
            if "self_attn.v_proj.weight" not in n and "self_attn.k_proj.weight" not in n]
        tr.named_parameters_to_optim = tr.named_parameters_to_optim[1:]
    if enhanced in ("zo", "fo"):
        tr.base_model = copy.deepcopy(model)
        for name, param in tr.base_model.named_parameters():
            if name in tr.exclude_list:
                param.data = param.data.to("cpu")
        tr.dizo_trainer = ref.dizo_trainer(tr.base_model, list(search_batches or []), "l2norm", 0.1, 10,
                                           tr.exclude_list)
    else:
        args.enhanced = None
    tr.loss_list = []
    tr.random_vector = {}
    return tr


def reference_step(tr, inputs) -> torch.Tensor:
    """One iteration of the reference loop body on the ZO path (large_models/trainer.py:1224-1225,
    :1264-1265, :1313): ``zo_step``, ``zo_update``, ``global_step += 1``.  The 50-step gamma search that
    ``zo_update`` would trigger is timed separately by the benchmark, so ``global_step`` is kept off
    its multiples here."""
    loss = tr.zo_step(tr.model, inputs)
    tr.zo_update(tr.args, tr.model)
    tr.state.global_step += 1
    if (tr.state.global_step + 1) % 50 == 0:
        tr.state.global_step += 1
    return loss
