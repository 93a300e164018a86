"""Launcher recipes: environment variables -> run.py argument lists that parse."""
import pytest

from dizo_b200.args import parse_args
from dizo_b200.launch import build_argv


def test_dizo_recipe_defaults_and_task_rules():
    argv = build_argv("dizo", {"TASK": "SST2", "ENHANCED": "zo"})
    a = parse_args(argv)
    assert a.trainer == "zo" and a.enhanced == "zo" and a.train_as_classification
    assert a.per_device_train_batch_size == 16 and a.max_steps == 20000 and a.zo_eps == 1e-3
    assert a.num_dev == 500 and a.seed == 26 and a.train_set_seed == 26 and a.save_steps == 500
    a = parse_args(build_argv("dizo", {"TASK": "Copa", "MODE": "lora"}))
    assert a.num_dev == 100 and not a.train_as_classification and a.lora and a.enhanced in (None, "None")
    a = parse_args(build_argv("dizo", {"TASK": "SQuAD", "MODE": "prefix", "NUM_GPU": "8", "PARALLEL": "tp"}))
    assert a.prefix_tuning and a.num_prefix == 5 and a.prefix_init_by_real_act and a.tp == 8
    a = parse_args(build_argv("dizo", {"TASK": "RTE", "NUM_GPU": "4", "PARALLEL": "fsdp"}))
    assert a.fsdp_shard and a.tp == 1


def test_first_order_and_icl_recipes():
    a = parse_args(build_argv("finetune", {"TASK": "DROP", "BS": "8"}))
    assert a.trainer == "regular" and a.per_device_train_batch_size == 1
    assert a.gradient_accumulation_steps == 8 and not a.train_as_classification
    a = parse_args(build_argv("finetune", {"TASK": "MultiRC", "BS": "8"}))
    assert a.per_device_train_batch_size == 2 and a.gradient_accumulation_steps == 4
    a = parse_args(build_argv("finetune_fsdp", {"TASK": "SST2"}))
    assert a.no_auto_device and a.per_device_train_batch_size == 1 and a.gradient_accumulation_steps == 8
    a = parse_args(build_argv("icl", {"TASK": "CB"}))
    assert a.num_train == 32 and a.num_eval == 1000 and a.trainer == "none" and a.verbose
    with pytest.raises(ValueError):
        build_argv("dizo", {})


def test_tensor_parallel_batch_fitting():
    """Token rows are padded to 128-row tiles per rank; caller row indices are translated."""
    import types
    import torch
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.parallel.tp import TPOPTModel
    dummy = types.SimpleNamespace(tp=8)
    b = synthetic_batch(0, 3, 40, 1000, pad_left=5)
    fitted = TPOPTModel._fit(dummy, b)
    Bp, Lp = fitted.input_ids.shape
    assert Lp == 128 and (Bp * (Lp // 128)) % 8 == 0 and Bp >= 3
    assert torch.equal(fitted.input_ids[:3, Lp - 40:], b.input_ids)
    assert (fitted.input_ids[:3, :Lp - 40] == 1).all() and (fitted.input_ids[3:] == 1).all()
    assert fitted.pad_left[:3].tolist() == [5 + Lp - 40] * 3 and fitted.pad_left[3:].tolist() == [Lp] * (Bp - 3)
    L0, Lp2 = dummy._row_map
    rows = b.rows.long()
    mapped = (rows // L0) * Lp2 + rows % L0 + (Lp2 - L0)
    assert torch.equal(fitted.input_ids.reshape(-1)[mapped], b.input_ids.reshape(-1)[rows])
    # already fitting batches pass through untouched
    dummy2 = types.SimpleNamespace(tp=2)
    b2 = synthetic_batch(0, 2, 128, 1000)
    assert TPOPTModel._fit(dummy2, b2) is b2 and dummy2._row_map is None
