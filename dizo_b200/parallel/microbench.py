"""Timing of the fused compute+collective kernels against the NCCL + GEMM composition.

    python -m torch.distributed.run --nproc-per-node N -m dizo_b200.parallel.microbench \
        [--rows 8192 --hidden 9216 --ffn-dim 36864] [--iters 10] [--push-ctas N --push-share F] [--switch-reduce]

For every path, device time (CUDA events, max over ranks) of the fused launch and of the
composition it replaces (NCCL all-gather or reduce-scatter plus the framework's own GEMM), and
the achieved fraction of the roofline: max(FLOPs / measured bf16 peak, NVLink bytes per rank /
770 GB/s) divided by the measured time.  One JSON line per path on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import linear
from ..ops.microbench import _peaks
from .fused import FusedComm

NVLINK_GBS = 770.0       # measured peer copy per direction on this pool


def timed(fn, iters, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", dest="m", type=int, default=8192, help="token rows (global for TP, per rank for FSDP)")
    ap.add_argument("--hidden", dest="d", type=int, default=9216)
    ap.add_argument("--ffn-dim", dest="ffn", type=int, default=36864)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--push-ctas", dest="n_push", type=int, default=0,
                    help="CTAs whose push warps are active (0 = the default policy for this number of ranks)")
    ap.add_argument("--switch-reduce", action="store_true",
                    help="also time GEMM -> reduce-scatter with the sum taken inside the switch (multimem.ld_reduce)")
    ap.add_argument("--one-sm", action="store_true", help="keep the fused launches on the one-SM tile kernel")
    ap.add_argument("--push-share", type=float, default=0.0,
                    help="output tiles of a pushing CTA relative to the others (0 = it only pushes)")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    peaks = _peaks()
    M, d, F = a.m, a.d, a.ffn
    Fl, rows = F // world, M // world
    fc = FusedComm(ag_bytes=M * d * 2, rs_bytes=M * d * 2, w_bytes=F * d * 2)
    fc.push_ctas, fc.push_share, fc.two_sm = a.n_push, a.push_share, not a.one_sm
    g = torch.Generator(device=dev).manual_seed(1)
    x_local = torch.randn(rows, d, device=dev, generator=g).bfloat16()
    w1 = (torch.randn(Fl, d, device=dev, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(d, Fl, device=dev, generator=g) * 0.02).bfloat16()
    y = torch.empty(M, Fl, device=dev, dtype=torch.bfloat16)
    x_gather = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
    part = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
    rs_out = torch.empty(rows, d, device=dev, dtype=torch.bfloat16)
    peak = peaks["bf16_tflops_sustained"] * 1e12
    out = []

    def report(name, fused_ms, base_ms, flops, nvlink_bytes):
        floor_ms = max(flops / peak, nvlink_bytes / (NVLINK_GBS * 1e9)) * 1e3
        out.append({"path": name, "world": world, "fused_ms": fused_ms, "nccl_composition_ms": base_ms,
                    "speedup": base_ms / fused_ms, "roofline_ms": floor_ms,
                    "fraction_of_roofline": floor_ms / fused_ms,
                    "tflops_per_gpu": flops / fused_ms / 1e9, "hidden": d,
                    "push_ctas": a.n_push or ("all" if world <= 2 else 16), "push_share": a.push_share,
                    "tile_kernel": "one-SM" if a.one_sm else "two-SM"})

    # ---- TP: all-gather -> GEMM (fc1 shape)
    def fused_ag():
        x_full, mine = fc.ag_input(M, d)
        mine.copy_(x_local)
        fc.ag_gemm(x_full, w1, out=y)

    def base_ag():
        dist.all_gather_into_tensor(x_gather, x_local)
        linear(x_gather, w1, out=y)
    report("tp_ag_gemm", timed(fused_ag, a.iters, world), timed(base_ag, a.iters, world),
           2.0 * M * Fl * d, (world - 1) * rows * d * 2)

    # ---- TP: GEMM -> reduce-scatter (fc2 shape)
    lnw = torch.ones(d, device=dev, dtype=torch.bfloat16)
    lnb = torch.zeros(d, device=dev, dtype=torch.bfloat16)

    def fused_rs():
        idx = fc.gemm_rs(y, w2)
        fc.rs_reduce_layernorm(idx, x_local, lnb, lnw, lnb)

    def base_rs():
        linear(y, w2, out=part)
        dist.reduce_scatter_tensor(rs_out, part)
        torch.nn.functional.layer_norm(rs_out + x_local, (d,), lnw, lnb)
    t_base_rs = timed(base_rs, a.iters, world)
    report("tp_gemm_rs_ln", timed(fused_rs, a.iters, world), t_base_rs,
           2.0 * M * d * Fl, (world - 1) * rows * d * 2)
    if a.switch_reduce and fc.has_multicast:
        # pull form: local GEMM, barrier, the switch adds the ranks' copies while the owner reads its rows
        def pull_rs():
            idx = fc.gemm_rs_pull(y, w2)
            fc.rs_reduce_layernorm(idx, x_local, lnb, lnw, lnb)
        report("tp_gemm_rs_ln_switch_reduce", timed(pull_rs, a.iters, world), t_base_rs,
               2.0 * M * d * Fl, (world - 1) * rows * d * 2)

    # ---- FSDP: shard push + perturbation + GEMM (fc1 of the full width, per-rank tokens)
    xs = torch.randn(M, d, device=dev, generator=g).bfloat16()
    shard = (torch.randn(Fl, d, device=dev, generator=g) * 0.02).bfloat16()
    w_full = torch.empty(F, d, device=dev, dtype=torch.bfloat16)
    yf = torch.empty(M, F, device=dev, dtype=torch.bfloat16)
    seg = [dict(w_shard=shard, dst_row0=rank * Fl, tensor_id=3, elem_base=rank * Fl * d)]
    state = {"slot": None}

    from ..ops.zo import ParamArena, Piece
    ar = ParamArena([Piece("w", (Fl, d), tensor_id=3, elem_base=rank * Fl * d)], dev)
    ar.view("w").copy_(shard)
    stage = torch.empty_like(ar.data)
    # the model's policy (FSDPOPTModel.push_perturb_limit): a small shard is perturbed by the push CTAs on
    # its way out; a large one is perturbed by the whole-GPU sweep first and pushed as a plain copy
    staged_push = Fl * d > 24 * 1024 * 1024
    seg_staged = [dict(w_shard=stage[:Fl * d].view(Fl, d), dst_row0=rank * Fl, tensor_id=3,
                       elem_base=rank * Fl * d)]

    def push_spec():
        if staged_push:
            ar.sweep(dst=stage, seed1=9, c1=1e-3)
            return dict(segments=seg_staged, seed=9, coef=0.0)
        return dict(segments=seg, seed=9, coef=1e-3)

    def fused_fsdp():
        # steady state of the pipeline: this launch multiplies the weight pushed by the previous one
        if state["slot"] is None:
            state["slot"], _ = fc.fsdp_launch(push=push_spec())
        prev = state["slot"]
        state["slot"], _ = fc.fsdp_launch(push=push_spec(),
                                          gemm=dict(slot=prev, N=F, x=xs, rows_per_src=Fl, out=yf))

    def base_fsdp():
        ar.sweep(dst=stage, seed1=9, c1=1e-3)                     # perturb the shard
        dist.all_gather_into_tensor(w_full, stage[:Fl * d].view(Fl, d))
        linear(xs, w_full, out=yf)
    report("fsdp_gather_perturb_gemm", timed(fused_fsdp, a.iters, world), timed(base_fsdp, a.iters, world),
           2.0 * M * F * d, (world - 1) * Fl * d * 2)

    torch.cuda.synchronize()
    _lib.check_device_errors()
    if rank == 0:
        for o in out:
            print(json.dumps(o))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
