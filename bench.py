"""Headline benchmark: zeroth-order (DiZO) training throughput of OPT-13B in bf16.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference ...                     # the unmodified reference, if installable
    python bench.py --impl baseline ...                      # stock-PyTorch statement of the reference loop

Metric: ZO training tokens/s = (prompts per rank x sequence length x ranks) / step time.  A
step is two forward passes (theta + eps z, theta - eps z), the scalar all-reduce of the
projected gradient under data parallelism, and the parameter update; the DiZO gamma search
(20 forwards + norms + projection, every 50 steps) is timed in the same run and charged to
every step as 1/50 of its cost.  Data are synthetic (seeded uniform ids, Bernoulli labels),
weights are random-init OPT-13B.  All times are CUDA-event times on the launching stream,
max over ranks.  For N > 1 launch under ``python -m torch.distributed.run``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_PUBLISHED = None  # the reference publishes no tokens/s figure


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--model", default="opt-13b")
    ap.add_argument("--prompts", type=int, default=8, help="prompts per rank")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--mode", default="full", help="full | lora | prefix | lora+prefix")
    ap.add_argument("--zo-mode", default="inflight", choices=["inflight", "inplace"])
    ap.add_argument("--enhanced", default="zo", choices=["none", "zo", "fo"],
                    help="DiZO gamma search: zeroth-order (the headline), first-order, or off (plain MeZO)")
    ap.add_argument("--overlap", action="store_true", help="sweep the next layer on a side stream")
    ap.add_argument("--parallelism", default="dp", choices=["dp", "fsdp", "tp", "pp"],
                    help="dp: replicated parameters, per-rank batches (default); fsdp: row-sharded weights, "
                         "fused gather+perturb+GEMM; tp: tensor parallel with fused AG->GEMM / GEMM->RS "
                         "(one global batch of --prompts x --seq)")
    ap.add_argument("--baseline-candidates", type=int, default=2)
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-sharded", action="store_true",
                    help="N >= 2: do not time the FSDP / tensor-parallel steps (fused kernels vs NCCL composition)")
    ap.add_argument("--sharded-steps", type=int, default=3)
    return ap.parse_args()


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        quiet_nccl()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "samples": len(sm), "reasons": sorted(reasons)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


# ------------------------------------------------------------------------------- ours
def quiet_nccl():
    """NCCL prints its version banner to stdout under NCCL_DEBUG=VERSION; the bench prints one JSON line."""
    if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"


def run_ours(a, world, rank, local):
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import DiZOProjector, ZOEngine
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.ops import _lib

    dev = torch.device("cuda", local)
    from dizo_b200.models import llama as llama_models
    is_llama = a.model.lower() in llama_models.PRESETS
    cfg = llama_models.preset(a.model) if is_llama else preset(a.model)
    par = a.parallelism if world > 1 else "dp"
    if is_llama and (par != "dp" or a.enhanced == "fo"):
        raise SystemExit("LLaMA-family models run replicated (--parallelism dp) with --enhanced zo | none")
    if par in ("tp", "pp") and a.enhanced == "fo":
        raise SystemExit("--enhanced fo runs on replicated or FSDP-sharded parameters (--parallelism dp | fsdp)")
    if par == "fsdp":
        from dizo_b200.parallel.fsdp import FSDPOPTModel
        model = FSDPOPTModel(cfg, dev)
    elif par == "tp":
        from dizo_b200.parallel.tp import TPOPTModel
        model = TPOPTModel(cfg, dev, max_tokens=a.prompts * a.seq)
    elif par == "pp":
        from dizo_b200.parallel.pp import PPOPTModel
        model = PPOPTModel(cfg, dev)
    elif is_llama:
        model = llama_models.LlamaModel(cfg, dev, torch.bfloat16, mode=a.mode, overlap_transform=a.overlap)
    else:
        model = OPTModel(cfg, dev, torch.bfloat16, mode=a.mode, overlap_transform=a.overlap)
    model.init_random_fast(seed=0)
    dp_group = False if par in ("tp", "pp") else None
    engine = ZOEngine(model, eps=1e-3, mode=a.zo_mode, dp_group=dp_group)
    projector = DiZOProjector(model, dp_group=dp_group) if a.enhanced != "none" else None
    data_rank = 0 if par in ("tp", "pp") else rank   # tensor / pipeline parallel: one global batch
    lr0, max_steps = 1e-6, 20000
    V = cfg.vocab_size

    def host_batch(step):
        return synthetic_batch(step, a.prompts, a.seq, V, seed=1, rank=data_rank, pin=True)

    def lr_at(k):
        return lr0 * (1 - k / (2 * max_steps))

    # ---- device-timed region: inputs already resident
    n_res = a.warmup + a.steps
    resident = [host_batch(s).to(dev) for s in range(n_res)]
    torch.cuda.synchronize()
    for s in range(a.warmup):
        engine.step(resident[s], lr_at(s), seed=1000 + s)
    barrier(world)
    _lib.check_device_errors()
    sampler = ClockSampler(physical_gpu_index(local))
    if rank == 0:
        sampler.start()
    l0 = _lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    e0.record()
    for s in range(a.warmup, a.warmup + a.steps):
        engine.step(resident[s], lr_at(s), seed=1000 + s)
    e1.record()
    barrier(world)
    launches = _lib.launch_count - l0
    step_ms = max_over_ranks(e0.elapsed_time(e1) / a.steps, world)

    # ---- the gamma search (every 50 steps in training), timed once
    search_ms = 0.0
    if projector is not None:
        it = iter(range(10 ** 9))
        nb = lambda: resident[next(it) % n_res]
        search = (lambda sd: projector.search_zo(nb, seed=sd)) if a.enhanced == "zo" else \
                 (lambda sd: projector.search_fo(nb))
        search(7)                                # warm
        barrier(world)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        search(8)
        s1.record()
        barrier(world)
        search_ms = max_over_ranks(s0.elapsed_time(s1), world)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_device_errors()
    ms = step_ms + search_ms / 50.0
    tokens = a.prompts * a.seq * (1 if par in ("tp", "pp") else world)

    # ---- end to end through the public trainer call: pinned H2D of each step's inputs,
    #      the step, D2H read of its loss
    e2e = None
    if not a.skip_e2e:
        from dizo_b200.trainer import OurTrainer
        from dizo_b200.args import OurArguments
        targs = OurArguments(trainer="zo", learning_rate=lr0, max_steps=max_steps, zo_eps=1e-3,
                             enhanced=None, zo_mode=a.zo_mode)
        tr = OurTrainer(model=model, args=targs, engine=engine, dp_group=dp_group)
        hb = [host_batch(10_000 + s) for s in range(a.steps + 2)]
        for s in range(2):
            tr.training_step(hb[s])
        barrier(world)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        last = 0.0
        for s in range(2, 2 + a.steps):
            last = tr.training_step(hb[s])        # float: includes the device->host read
        t1.record()
        barrier(world)
        e2e_ms = max_over_ranks(t0.elapsed_time(t1) / a.steps, world) + search_ms / 50.0
        e2e = {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": hb[0].nbytes(), "d2h_bytes_per_step": 4, "last_loss": last}

    nparam = model.arena.trainable_numel()
    # ---- perturb bandwidth: one pass of the in-flight perturbation over every parameter group
    #      (theta + eps z into the per-layer staging buffer, z regenerated), as each forward does;
    #      bytes = parameters read + staged copy written.  The update sweep is the same kernel in place.
    # ---- perturb + update bandwidth: the sweeps of one step, timed on their own - the staging pass over every
    #      parameter group as the forwards issue it (theta + eps z and theta - eps z side by side from one draw of
    #      z where the model pairs the forwards: 2 B read + 4 B written per parameter; otherwise one side: 2 + 2)
    #      and the update pass (stochastic rounding as in training; 2 + 2 B).  z is regenerated in every pass.
    sweep_gbs, sweep_detail = None, None
    if par == "dp" and model.arena.trainable_numel() > 0:
        from dizo_b200.models.opt import Transform
        groups = model.arena.groups()
        biggest = max(model.arena.group_numel(g) for g in groups)
        paired = bool(getattr(model, "pair_supported", lambda: False)()) and a.zo_mode == "inflight"

        def staging_pass(seed):
            tr = Transform(seed=seed, coef=1e-3)
            for k, g in enumerate(groups):
                b1 = model._staging_for(("bench", k % 2), biggest)
                b2 = model._staging_for(("bench-", k % 2), biggest) if paired else None
                model._sweep_group(g, tr, b1, dst2=b2)

        def update_pass(seed):
            engine.projected_grad.fill_(1e-9)            # lr * g far below a bf16 step: theta stays where it is
            engine.update(seed, 1e-6)

        def timed(fn):
            fn(1)
            w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            w0.record()
            for i in range(3):
                fn(2 + i)
            w1.record()
            torch.cuda.synchronize()
            return max_over_ranks(w0.elapsed_time(w1) / 3, world)
        stage_ms, update_ms = timed(staging_pass), timed(update_pass)
        esz = model.arena.data.element_size()
        pbytes = model.arena.trainable_numel() * esz
        stage_b, update_b = (3 if paired else 2) * pbytes, 2 * pbytes
        sweep_gbs = (stage_b + update_b) / (stage_ms + update_ms) / 1e6
        sweep_detail = {"staging_ms": stage_ms, "staging_gbs": stage_b / stage_ms / 1e6, "two_sided": paired,
                        "update_ms": update_ms, "update_gbs": update_b / update_ms / 1e6,
                        "bytes_per_param_per_step": (stage_b * (1 if paired else 2) + update_b) / pbytes * esz}
    out = {
        "metric": "zo_train_tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform ids, Bernoulli labels); random-init weights",
        "impl": "ours",
        "config": {"model": a.model, "global_batch": a.prompts * (1 if par == "tp" else world), "seq_len": a.seq,
                   "parallelism": f"{par}{world}", "trainable": a.mode, "zo_mode": a.zo_mode,
                   "forwards_per_step": 2, "enhanced": a.enhanced,
                   "zo_step_ms": step_ms, "gamma_search_ms": search_ms, "gamma_search_period": 50,
                   "l2_policy": "per-step working set (parameters) far exceeds L2; no flush needed",
                   "trainable_params": nparam},
        "perturb_update_gbs": sweep_gbs, "perturb_update": sweep_detail,
        "gpu_launches": launches, "clocks": clocks, "e2e": e2e,
    }
    if world > 1 and par == "dp" and a.mode == "full" and not a.skip_sharded:
        # free the replicated model first: the sharded models need the memory
        del engine, projector, model, resident
        if not a.skip_e2e:
            del tr, hb
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        out["extra"] = run_sharded_extras(a, world, rank, local)
    return out


# ------------------------------------------------------------------------------- sharded layouts
NVLINK_GBS = 770.0            # measured peer copy rate per direction per GPU on this pool (900 nominal)


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def run_sharded_extras(a, world, rank, local):
    """The communication-bound layouts under the same clock as the headline (N >= 2 only): one full ZO
    step (two forwards, scalar all-reduce, update sweep) of

    * OPT-13B, parameters row-sharded over the N ranks (FSDP), 8 prompts x 1024 tokens per rank: the
      fused gather + perturb + GEMM launches against the composition perturb -> NCCL all-gather
      (prefetched on a second stream) -> GEMM;
    * at N = 8, OPT-66B tensor parallel over the 8 ranks, 16 prompts x 512 tokens in total: fused
      all-gather -> GEMM and GEMM -> reduce-scatter -> LayerNorm against NCCL all-gather /
      reduce-scatter between the stand-alone kernels.

    Both arms use this repository's sweep, GEMM and attention kernels; only the collectives differ.
    Roofline of a step = the slower of (GEMM FLOPs per rank / measured sustained bf16 rate) and (bytes a
    rank receives over NVLink / 770 GB/s)."""
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import ZOEngine
    from dizo_b200.models.opt import preset
    from dizo_b200.ops import _lib
    from dizo_b200.parallel.composition import FSDPCompositionModel, TPCompositionModel
    from dizo_b200.parallel.fsdp import FSDPOPTModel
    from dizo_b200.parallel.tp import TPOPTModel
    import gc

    dev = torch.device("cuda", local)
    peaks, peak_kind = _peaks()
    flops_rate = peaks["bf16_tflops_sustained"] * 1e12
    K, W = max(1, a.sharded_steps), 2
    out = {"peaks": peak_kind, "nvlink_gbs": NVLINK_GBS, "steps": K, "warmup": W}

    def time_model(build, prompts, seq, vocab, data_rank, dp_group):
        model = build()
        model.init_random_fast(seed=0)
        eng = ZOEngine(model, eps=1e-3, dp_group=dp_group)
        bs = [synthetic_batch(s, prompts, seq, vocab, seed=1, rank=data_rank).to(dev) for s in range(W + K)]
        for s in range(W):
            eng.step(bs[s], 1e-6, seed=500 + s)
        barrier(world)
        _lib.check_device_errors()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(W, W + K):
            eng.step(bs[s], 1e-6, seed=500 + s)
        e1.record()
        barrier(world)
        _lib.check_device_errors()
        ms = max_over_ranks(e0.elapsed_time(e1) / K, world)
        loss = float(eng.loss1.item())
        del eng, model, bs
        gc.collect()
        torch.cuda.empty_cache()
        return ms, loss

    def record(key, cfg, prompts, seq, arms, tokens, flops_per_rank, nvlink_bytes_per_rank, data_rank, dp_group):
        rec = {"model": key, "tokens_per_step": tokens}
        for arm, build in arms:
            try:
                ms, loss = time_model(build, prompts, seq, cfg.vocab_size, data_rank, dp_group)
                rec[f"{arm}_ms"] = ms
                rec[f"{arm}_loss"] = loss
            except Exception as e:  # noqa: BLE001  (the headline number must survive a failure here)
                rec[f"{arm}_error"] = f"{type(e).__name__}: {e}"[:300]
        roof_ms = max(flops_per_rank / flops_rate, nvlink_bytes_per_rank / (NVLINK_GBS * 1e9)) * 1e3
        rec["roofline_ms"] = roof_ms
        if "fused_ms" in rec:
            rec["fused_of_roofline"] = roof_ms / rec["fused_ms"]
            rec["fused_tokens_per_sec"] = tokens / (rec["fused_ms"] / 1e3)
        if "fused_ms" in rec and "composition_ms" in rec:
            rec["fused_over_composition"] = rec["composition_ms"] / rec["fused_ms"]
        return rec

    # ---- FSDP, OPT-13B, 8 x 1024 per rank
    cfg = preset("opt-13b")
    d, F, nl = cfg.hidden_size, cfg.ffn_dim, cfg.num_hidden_layers
    mat_params = nl * (4 * d * d + 2 * d * F)
    tokens_rank = 8 * 1024
    out["fsdp"] = record(
        "opt-13b", cfg, 8, 1024,
        [("fused", lambda: FSDPOPTModel(cfg, dev)), ("composition", lambda: FSDPCompositionModel(cfg, dev))],
        tokens=tokens_rank * world, flops_per_rank=2 * 2.0 * mat_params * tokens_rank,
        nvlink_bytes_per_rank=2 * 2.0 * mat_params * (world - 1) / world, data_rank=rank, dp_group=None)
    out["fsdp"]["parallelism"] = f"fsdp{world}"

    # ---- tensor parallel, OPT-66B, 16 x 512 in total (8 GPUs)
    if world == 8:
        cfg = preset("opt-66b")
        d, F, nl = cfg.hidden_size, cfg.ffn_dim, cfg.num_hidden_layers
        mat_params = nl * (4 * d * d + 2 * d * F)
        tokens = 16 * 512
        out["tp"] = record(
            "opt-66b", cfg, 16, 512,
            [("fused", lambda: TPOPTModel(cfg, dev, max_tokens=tokens)),
             ("composition", lambda: TPCompositionModel(cfg, dev, max_tokens=tokens))],
            tokens=tokens, flops_per_rank=2 * 2.0 * mat_params * tokens / world,
            nvlink_bytes_per_rank=2 * nl * 4 * (tokens * d * 2.0) * (world - 1) / world,
            data_rank=0, dp_group=False)
        out["tp"]["parallelism"] = f"tp{world}"
    return out


# ------------------------------------------------------------------------------- baseline
def run_baseline(a, world, rank, local):
    """Reference algorithm in stock PyTorch (HF model, torch.normal sweeps, full-vocab loss)."""
    import numpy as np
    from baseline.mezo_torch import TorchMeZO, build_hf_opt, synthetic_reference_batch
    from dizo_b200.data.synthetic import DEFAULT_CANDS
    from dizo_b200.models.opt import preset
    dev = torch.device("cuda", local)
    cfg = preset(a.model)
    model = build_hf_opt(cfg.to_hf_dict(), dev, torch.bfloat16)
    opt = TorchMeZO(model, eps=1e-3, dizo=(a.enhanced == "zo"))
    np.random.seed(0)
    mk = lambda s: synthetic_reference_batch(s, a.prompts, a.seq, cfg.vocab_size, 1, rank,
                                             DEFAULT_CANDS, dev, a.baseline_candidates)
    batches = [mk(s) for s in range(a.warmup + a.steps)]

    def step(s):
        l = opt.step(batches[s], 1e-6)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(l)
    for s in range(a.warmup):
        step(s)
    barrier(world)
    sampler = ClockSampler(physical_gpu_index(local))
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(a.warmup, a.warmup + a.steps):
        step(s)
    e1.record()
    barrier(world)
    step_ms = max_over_ranks(e0.elapsed_time(e1) / a.steps, world)
    search_ms = 0.0
    if a.enhanced == "zo":
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        opt.dizo_search([batches[i % len(batches)] for i in range(10)])
        s1.record()
        barrier(world)
        search_ms = max_over_ranks(s0.elapsed_time(s1), world)
    clocks = sampler.stop() if rank == 0 else None
    ms = step_ms + search_ms / 50.0
    tokens = a.prompts * a.seq * world
    return {"metric": "zo_train_tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "baseline",
            "config": {"model": a.model, "global_batch": a.prompts * world, "seq_len": a.seq,
                       "parallelism": f"dp{world}", "candidates_per_prompt": a.baseline_candidates,
                       "zo_step_ms": step_ms, "gamma_search_ms": search_ms},
            "clocks": clocks}


# ------------------------------------------------------------------------------- reference
REFERENCE_MULTI_GPU_REASON = (
    "the reference's zeroth-order path is single-GPU only: large_models/run.py:32 pins "
    "CUDA_VISIBLE_DEVICES=0 and zo_step / zo_update (large_models/trainer.py:1570-1617) contain no "
    "collective, so there is no N-GPU reference job to time")


def run_reference(a):
    """Time the unmodified reference (``baseline/_ref``) on the same metric and configuration.

    The reference's own ``OurTrainer.zo_step`` / ``zo_update`` and ``dizo_trainer.dizo_zo_iters`` run on a
    random-init Hugging Face OPT model of the named shape in bf16 (its ``--load_bfloat16`` dtype), fed
    the synthetic batches in the layout of its nesting collator: one sequence per candidate, two
    candidates per prompt, as its classification path does (large_models/run.py:415-419).  Nothing of
    this repository's package is imported on this path."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if world > 1 or a.gpus > 1:
        return unavailable(REFERENCE_MULTI_GPU_REASON)
    if a.parallelism != "dp" or a.mode != "full":
        return unavailable("the reference arm times full-parameter ZO on one GPU only")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device in this process; the reference's DiZO module allocates on 'cuda' "
                           "(large_models/trainer.py:389)")
    from baseline import ref_harness as H
    try:
        ref, shimmed = H.import_reference()
    except H.ReferenceUnavailable as e:
        return unavailable(str(e))
    if a.model not in H.OPT_SHAPES:
        return unavailable(f"no shape table entry for {a.model}")
    import numpy as np
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    enhanced = None if a.enhanced == "none" else a.enhanced
    if enhanced == "fo":
        return unavailable("the reference arm times the zeroth-order gamma search (the headline configuration)")
    V, cands = 50272, a.baseline_candidates
    model = H.build_hf_opt(a.model, dev, torch.bfloat16)
    lr0, max_steps = 1e-6, 20000
    n_res = a.warmup + a.steps
    resident = [{k: v.to(dev) for k, v in H.reference_batch(s, a.prompts, a.seq, V, candidates=cands).items()}
                for s in range(n_res)]
    search_batches = [{k: v.to(dev) for k, v in H.reference_batch(5000 + s, a.prompts, a.seq, V,
                                                                 candidates=cands).items()} for s in range(10)]
    tr = H.make_reference_trainer(ref, model, dev, lr=lr0, max_steps=max_steps, zo_eps=1e-3,
                                  enhanced=enhanced, search_batches=search_batches)
    np.random.seed(0)
    torch.cuda.synchronize()
    for s in range(a.warmup):
        H.reference_step(tr, resident[s])
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(a.warmup, n_res):
        H.reference_step(tr, resident[s])
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / a.steps

    search_ms = 0.0
    if enhanced == "zo":
        tr.dizo_trainer.dizo_zo_iters(tr.model, base_model=tr.base_model)      # warm, as the other arms do
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        tr.dizo_trainer.dizo_zo_iters(tr.model, base_model=tr.base_model)
        s1.record()
        torch.cuda.synchronize()
        search_ms = s0.elapsed_time(s1)
    clocks = sampler.stop()
    ms = step_ms + search_ms / 50.0
    tokens = a.prompts * a.seq

    e2e = None
    if not a.skip_e2e:
        hb = [H.reference_batch(10_000 + s, a.prompts, a.seq, V, candidates=cands, pin=True)
              for s in range(a.steps + 2)]
        for s in range(2):
            float(H.reference_step(tr, hb[s]))
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        last = 0.0
        for s in range(2, 2 + a.steps):
            # zo_forward moves the pinned host batch to the device itself (_prepare_inputs, once per
            # forward); the loss and the projected gradient are read back on the host
            last = float(H.reference_step(tr, hb[s]))
        t1.record()
        torch.cuda.synchronize()
        e2e_ms = t0.elapsed_time(t1) / a.steps + search_ms / 50.0
        e2e = {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 2 * H.batch_nbytes(hb[0]),
               # bf16 loss + bf16 projected gradient, and per forward the loss wrapper's host reads of
               # option_len (8 B) and of the num_options comparison (1 B) for every sequence
               "d2h_bytes_per_step": 2 + 2 + 2 * 9 * a.prompts * cands,
               "last_loss": last}
    print(json.dumps({
        "metric": "zo_train_tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform ids, Bernoulli labels); random-init weights",
        "impl": "reference",
        "config": {"model": a.model, "global_batch": a.prompts, "seq_len": a.seq, "parallelism": "dp1",
                   "trainable": "full", "forwards_per_step": 2, "enhanced": a.enhanced,
                   "candidates_per_prompt": cands, "sequences_per_forward": a.prompts * cands,
                   "zo_step_ms": step_ms, "gamma_search_ms": search_ms, "gamma_search_period": 50,
                   "l2_policy": "per-step working set (parameters) far exceeds L2; no flush needed",
                   "reference_entry_points": "OurTrainer.zo_step, zo_update, dizo_trainer.dizo_zo_iters",
                   "library_names_stubbed": shimmed},
        "gpu_launches": None, "clocks": clocks, "e2e": e2e}))
    return 0


def main():
    a = parse()
    # Libraries write banners to stdout (NCCL prints its version there); the contract is ONE JSON line.  File
    # descriptor 1 points at stderr while the benchmark runs and is restored for the result line.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(*args, **kw):
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        _print(*args, **kw)
        sys.stdout.flush()
        os.dup2(2, 1)
    import builtins
    _print = builtins.print
    globals()["print"] = emit           # every print of this module is a result line
    if a.impl == "reference":
        return run_reference(a)
    world, rank, local = dist_setup()
    out = run_ours(a, world, rank, local) if a.impl == "ours" else run_baseline(a, world, rank, local)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
