"""Checkpoints: Hugging Face compatible weights + everything needed to resume a ZO run exactly.

A checkpoint directory holds
  * ``model.safetensors`` (``pytorch_model.bin`` when safetensors is missing) with Hugging Face
    OPT parameter names, plus ``lora_A/B`` and ``prefix_keys/values`` entries, and ``config.json``
    - loadable by ``transformers.OPTForCausalLM.from_pretrained`` for full fine-tuning runs;
  * ``trainer_state.json`` (step, epoch, log history, best metric);
  * ``zo_state.pt``: NumPy global RNG state (the per-step seeds are drawn from it, so restoring
    it replays the same z stream), loss / accuracy curves, the DiZO gamma vector with its
    first-order Adam moments, the projection seed generator, and the anchor theta_0 of the
    constrained tensors;
  * ``manifest.json``: byte sizes and SHA-256 of every file, checked on load, so a truncated or
    corrupted checkpoint is detected instead of silently resumed.
The reference only discovers checkpoints (large_models/run.py:466-479) and reloads
``trainer_state.json`` (large_models/trainer.py:1072-1094); its ZO loop never writes any.
"""
from __future__ import annotations

import hashlib
import json
import logging
import os
import re
from typing import Optional

import numpy as np
import torch

logger = logging.getLogger(__name__)


class CheckpointError(RuntimeError):
    pass


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for blk in iter(lambda: f.read(1 << 22), b""):
            h.update(blk)
    return h.hexdigest()


def _write_manifest(out: str) -> None:
    files = {}
    for name in sorted(os.listdir(out)):
        p = os.path.join(out, name)
        if name != "manifest.json" and os.path.isfile(p):
            files[name] = {"bytes": os.path.getsize(p), "sha256": _sha256(p)}
    with open(os.path.join(out, "manifest.json"), "w") as f:
        json.dump(files, f, indent=2)


def verify_checkpoint(path: str) -> None:
    man = os.path.join(path, "manifest.json")
    if not os.path.exists(man):
        raise CheckpointError(f"{path}: no manifest.json (incomplete checkpoint)")
    with open(man) as f:
        files = json.load(f)
    for name, meta in files.items():
        p = os.path.join(path, name)
        if not os.path.exists(p):
            raise CheckpointError(f"{path}: {name} is missing")
        if os.path.getsize(p) != meta["bytes"]:
            raise CheckpointError(f"{path}: {name} is truncated ({os.path.getsize(p)} of {meta['bytes']} bytes)")
        if _sha256(p) != meta["sha256"]:
            raise CheckpointError(f"{path}: {name} is corrupted (checksum mismatch)")


def iter_full_tensors(model):
    """(name, full tensor) pairs in Hugging Face order.  For sharded models each tensor is gathered
    on its own (a collective: every rank of the model's group iterates), so nothing larger than one
    full tensor exists on a device at a time."""
    if hasattr(model, "gather_full"):                      # tensor parallel / FSDP
        tied = None
        for n in model.hf_order:
            t = model.gather_full(n, model.param(n))
            if n == "model.decoder.embed_tokens.weight":
                tied = t
            yield n, t
        if not model.untied and tied is not None:
            yield "lm_head.weight", tied
    elif hasattr(model, "gather_state_dict"):              # pipeline stages
        yield from model.gather_state_dict().items()
    else:
        yield from model.state_dict().items()


def save_weights_sharded(out: str, items, write: bool = True, max_shard_bytes: int = 8 << 30) -> list[str]:
    """Stream (name, tensor) pairs into safetensors files of at most ``max_shard_bytes``: one
    ``model.safetensors`` when everything fits, otherwise ``model-0000i-of-0000n.safetensors`` plus
    ``model.safetensors.index.json`` (the Hugging Face sharded layout).  Tensors are moved to the
    host one at a time; with ``write`` False the pairs are only consumed (the gathers behind them
    are collective)."""
    from safetensors.torch import save_file
    if write:
        os.makedirs(out, exist_ok=True)
    shards: list[tuple[str, list[str]]] = []
    cur: dict = {}
    cur_bytes = 0
    total = 0
    embed_ptr = None

    def flush():
        nonlocal cur, cur_bytes
        if cur:
            tmp = f"model-part{len(shards) + 1:05d}.safetensors"
            save_file(cur, os.path.join(out, tmp), metadata={"format": "pt"})
            shards.append((tmp, list(cur)))
            cur, cur_bytes = {}, 0

    for name, t in items:
        if not write:
            continue
        if name == "lm_head.weight" and embed_ptr is not None and t.data_ptr() == embed_ptr:
            continue                                        # tied: stored once, as Hugging Face does
        if name == "model.decoder.embed_tokens.weight":
            embed_ptr = t.data_ptr()
        c = t.detach().to("cpu").contiguous()
        if c.data_ptr() == t.data_ptr():
            c = c.clone()
        nb = c.numel() * c.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            flush()
        cur[name] = c
        cur_bytes += nb
        total += nb
    if not write:
        return []
    flush()
    if len(shards) == 1:
        os.replace(os.path.join(out, shards[0][0]), os.path.join(out, "model.safetensors"))
        return ["model.safetensors"]
    weight_map, names = {}, []
    for i, (tmp, keys) in enumerate(shards):
        final = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        os.replace(os.path.join(out, tmp), os.path.join(out, final))
        names.append(final)
        for k in keys:
            weight_map[k] = final
    with open(os.path.join(out, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    return names


def save_weights(out: str, state_dict: dict) -> str:
    os.makedirs(out, exist_ok=True)
    sd = {k: v.detach().cpu().contiguous() for k, v in state_dict.items()}
    try:
        from safetensors.torch import save_file
        # tied tensors may not share storage inside a safetensors file
        if "lm_head.weight" in sd and "model.decoder.embed_tokens.weight" in sd and \
                sd["lm_head.weight"].data_ptr() == sd["model.decoder.embed_tokens.weight"].data_ptr():
            sd = {k: v for k, v in sd.items() if k != "lm_head.weight"}
        p = os.path.join(out, "model.safetensors")
        save_file(sd, p, metadata={"format": "pt"})
    except ImportError:  # pragma: no cover
        p = os.path.join(out, "pytorch_model.bin")
        torch.save(sd, p)
    return p


class LazyWeights:
    """Read-only mapping name -> tensor over a Hugging Face checkpoint directory that materialises one
    tensor (safetensors) or one shard (``.bin``) at a time, so loading OPT-66B on eight ranks does not
    hold eight full state dicts in host memory: every rank pulls a tensor, keeps its slice, drops it."""

    def __init__(self, path: str):
        self.path = path
        self._where: dict[str, str] = {}
        self._safe = True
        self._bin_cache: tuple[str, dict] | None = None
        st, sti = os.path.join(path, "model.safetensors"), os.path.join(path, "model.safetensors.index.json")
        pb, pbi = os.path.join(path, "pytorch_model.bin"), os.path.join(path, "pytorch_model.bin.index.json")
        if os.path.exists(st):
            from safetensors import safe_open
            with safe_open(st, "pt") as f:
                self._where = {k: "model.safetensors" for k in f.keys()}
        elif os.path.exists(sti):
            with open(sti) as f:
                self._where = dict(json.load(f)["weight_map"])
        elif os.path.exists(pbi):
            self._safe = False
            with open(pbi) as f:
                self._where = dict(json.load(f)["weight_map"])
        elif os.path.exists(pb):
            self._safe = False
            self._bin_cache = ("pytorch_model.bin", torch.load(pb, map_location="cpu", weights_only=True))
            self._where = {k: "pytorch_model.bin" for k in self._bin_cache[1]}
        else:
            raise CheckpointError(f"{path}: no model.safetensors / pytorch_model.bin")

    def __contains__(self, name) -> bool:
        return name in self._where

    def keys(self):
        return self._where.keys()

    def __iter__(self):
        return iter(self._where)

    def __len__(self) -> int:
        return len(self._where)

    def __getitem__(self, name: str) -> torch.Tensor:
        shard = self._where[name]
        if self._safe:
            from safetensors import safe_open
            with safe_open(os.path.join(self.path, shard), "pt") as f:
                return f.get_tensor(name)
        if self._bin_cache is None or self._bin_cache[0] != shard:
            self._bin_cache = (shard, torch.load(os.path.join(self.path, shard), map_location="cpu",
                                                 weights_only=True))
        return self._bin_cache[1][name]

    def get(self, name: str, default=None):
        return self[name] if name in self._where else default

    def items(self):
        for k in self._where:
            yield k, self[k]


def load_weights(path: str, lazy: bool = False):
    """The checkpoint's state dict; ``lazy`` returns a :class:`LazyWeights` view instead of reading
    every tensor up front."""
    if lazy:
        return LazyWeights(path)
    st = os.path.join(path, "model.safetensors")
    if os.path.exists(st):
        from safetensors.torch import load_file
        return load_file(st)
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        from safetensors.torch import load_file
        with open(idx) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        sd = {}
        for s in shards:
            sd.update(load_file(os.path.join(path, s)))
        return sd
    for name in ("pytorch_model.bin",):
        p = os.path.join(path, name)
        if os.path.exists(p):
            return torch.load(p, map_location="cpu", weights_only=True)
    idx = os.path.join(path, "pytorch_model.bin.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        sd = {}
        for s in shards:
            sd.update(torch.load(os.path.join(path, s), map_location="cpu", weights_only=True))
        return sd
    raise CheckpointError(f"{path}: no model.safetensors / pytorch_model.bin")


def full_state_dict(model) -> dict:
    """Unsharded Hugging Face state dict.  Sharded models (tensor parallel, FSDP) assemble it with
    collectives: every rank of the model's group must call this."""
    if hasattr(model, "gather_state_dict"):
        return model.gather_state_dict()
    return model.state_dict()


def save_checkpoint(out: str, model, trainer=None, write: bool = True, max_shard_bytes: int = 8 << 30) -> None:
    """Write a checkpoint directory.  With a sharded model every rank calls this (the gathers are
    collective) and only the rank with ``write`` touches the file system; the files hold full
    tensors (streamed one at a time into safetensors shards), so a checkpoint can be resumed under
    a different parallel layout."""
    ar = model.arena
    anchor = None
    if trainer is not None and trainer.dizo_trainer is not None:
        gather = getattr(model, "gather_full", None)
        anchor = {n: (gather(n, ar.anchor_view(n)) if gather else ar.anchor_view(n)).detach().cpu().clone()
                  for n in ar.slot_names}
        if hasattr(model, "gather_dict"):              # pipeline stages hold disjoint sets of tensors
            anchor = model.gather_dict(anchor)
    save_weights_sharded(out, iter_full_tensors(model), write=write, max_shard_bytes=max_shard_bytes)
    if not write:
        return
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(model.config.to_hf_dict(), f, indent=2)
    if trainer is not None:
        trainer.state.save_to_json(os.path.join(out, "trainer_state.json"))
        zo = {"numpy_rng": np.random.get_state(), "loss_list": list(trainer.loss_list),
              "accuracy": list(trainer.accuracy), "objective": trainer.objective,
              "args": trainer.args.to_dict()}
        if trainer.dizo_trainer is not None:
            zo["dizo"] = trainer.dizo_trainer.projector.state_dict()
            zo["dizo_i"] = trainer.dizo_trainer.i
            zo["pgm_count"] = trainer._pgm_count
            zo["dizo_seed_rng"] = trainer._dizo_seed_rng.get_state()
            zo["anchor"] = anchor
        torch.save(zo, os.path.join(out, "zo_state.pt"))
    _write_manifest(out)


def load_checkpoint(path: str, model, trainer=None, verify: bool = True) -> None:
    if verify:
        verify_checkpoint(path)
    model.load_state_dict(load_weights(path, lazy=True), strict=False)
    if trainer is None:
        return
    from ..trainer import TrainerState
    ts = os.path.join(path, "trainer_state.json")
    if os.path.exists(ts):
        keep_max = trainer.state.max_steps
        trainer.state = TrainerState.load_from_json(ts)
        trainer.state.max_steps = keep_max or trainer.state.max_steps
    zp = os.path.join(path, "zo_state.pt")
    if os.path.exists(zp):
        zo = torch.load(zp, map_location="cpu", weights_only=False)
        np.random.set_state(zo["numpy_rng"])
        trainer.loss_list = list(zo.get("loss_list", []))
        trainer.accuracy = list(zo.get("accuracy", []))
        trainer.objective = zo.get("objective", 0.0)
        if "dizo" in zo and trainer.dizo_trainer is not None:
            trainer.dizo_trainer.projector.load_state_dict(zo["dizo"])
            trainer.dizo_trainer.i = zo.get("dizo_i", 0)
            trainer._pgm_count = zo.get("pgm_count", 0)
            trainer._pgm_iter = None
            trainer._dizo_seed_rng.set_state(zo["dizo_seed_rng"])
            ar = model.arena
            for n, t in zo.get("anchor", {}).items():
                if n in ar.index:                      # a pipeline stage restores its own tensors only
                    ar.anchor_view(n).copy_(model.local_slice(n, t).to(ar.dtype))


_CKPT_RE = re.compile(r"^checkpoint-(\d+)$")


def get_last_checkpoint(folder: str) -> Optional[str]:
    """Highest-numbered complete ``checkpoint-N`` directory under ``folder`` (or None)."""
    if not os.path.isdir(folder):
        return None
    best = None
    for name in os.listdir(folder):
        m = _CKPT_RE.match(name)
        p = os.path.join(folder, name)
        if m and os.path.isdir(p) and os.path.exists(os.path.join(p, "manifest.json")):
            if best is None or int(m.group(1)) > best[0]:
                best = (int(m.group(1)), p)
    return best[1] if best else None
