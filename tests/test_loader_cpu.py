"""Model / tokenizer resolution of the command-line entry: a checkpoint directory, a hub id found in the
local Hugging Face cache, an explicit ``--random_init``, and the loud failure otherwise."""
import json
import os

import pytest
import torch

from dizo_b200.args import OurArguments
from dizo_b200.models.opt import OPTModel, preset
from dizo_b200.run import Framework
from dizo_b200.tasks import get_task
from dizo_b200.utils.checkpoint import save_checkpoint


def _args(**kw):
    base = dict(task_name="Synthetic", trainer="none", num_train=0, num_eval=2, max_length=64)
    base.update(kw)
    return OurArguments(**base)


def _write_checkpoint(path):
    model = OPTModel(preset("opt-tiny"), "cpu", torch.float32).init_random(7)
    save_checkpoint(str(path), model)
    return model


def test_missing_checkpoint_fails_loudly_without_random_init():
    with pytest.raises(FileNotFoundError, match="random_init"):
        Framework(_args(model_name="facebook/opt-tiny"), get_task("Synthetic"))


def test_random_init_is_explicit():
    fw = Framework(_args(model_name="facebook/opt-tiny", random_init=True), get_task("Synthetic"))
    assert fw.model.config.hidden_size == preset("opt-tiny").hidden_size
    with pytest.raises(KeyError):
        Framework(_args(model_name="facebook/not-a-shape", random_init=True), get_task("Synthetic"))


def test_checkpoint_directory_loads_its_weights(tmp_path):
    ref = _write_checkpoint(tmp_path / "ckpt")
    fw = Framework(_args(model_name=str(tmp_path / "ckpt")), get_task("Synthetic"))
    name = "model.decoder.layers.1.fc1.weight"
    assert torch.equal(fw.model.param(name), ref.param(name))


def test_hub_id_resolves_through_the_local_cache(tmp_path, monkeypatch):
    snap = tmp_path / "hub" / "models--facebook--opt-tiny" / "snapshots" / "0123abcd"
    ref = _write_checkpoint(snap)
    refs = tmp_path / "hub" / "models--facebook--opt-tiny" / "refs"
    refs.mkdir(parents=True)
    (refs / "main").write_text("0123abcd")
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path / "hub"))
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    import huggingface_hub.constants as hc
    monkeypatch.setattr(hc, "HF_HUB_CACHE", str(tmp_path / "hub"), raising=False)
    monkeypatch.setattr(hc, "HUGGINGFACE_HUB_CACHE", str(tmp_path / "hub"), raising=False)
    path = Framework.resolve_model_dir("facebook/opt-tiny")
    assert path is not None and os.path.exists(os.path.join(path, "config.json")), path
    fw = Framework(_args(model_name="facebook/opt-tiny"), get_task("Synthetic"))
    name = "model.decoder.layers.0.self_attn.k_proj.weight"
    assert torch.equal(fw.model.param(name), ref.param(name))


def test_broken_tokenizer_files_are_an_error_not_a_stub(tmp_path):
    _write_checkpoint(tmp_path / "ckpt")
    (tmp_path / "ckpt" / "tokenizer_config.json").write_text("{ this is not json")
    with pytest.raises(RuntimeError, match="tokenizer"):
        Framework(_args(model_name=str(tmp_path / "ckpt")), get_task("Synthetic"))


def test_float16_request_is_converted_once_not_warned_every_run(caplog):
    import logging
    fw = Framework(_args(model_name="opt-tiny", random_init=True, load_float16=True), get_task("Synthetic"))
    assert fw.model.dtype in (torch.float32, torch.bfloat16)
    assert not [r for r in caplog.records if r.levelno >= logging.WARNING and "fp16" in r.getMessage()]
