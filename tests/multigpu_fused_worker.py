"""Worker for tests/test_multigpu_fused.py: run under torchrun on >= 2 GPUs.

Checks every fused compute+collective path against the composition of an NCCL collective and
the single-GPU kernels.  NVLS is off and the kernels use plain peer stores; with ``--multimem`` only the two
paths that reduce inside the switch run (multimem.ld_reduce on the symmetric region's multicast address)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dizo_b200.ops import _lib, philox  # noqa: E402
from dizo_b200.ops.zo import perturb_reference  # noqa: E402
from dizo_b200.ops.gemm import linear  # noqa: E402
from dizo_b200.ops.norm import layernorm  # noqa: E402
from dizo_b200.ops.zo import GammaState  # noqa: E402
from dizo_b200.parallel.fused import FusedComm  # noqa: E402


def switch_reduction(fc, dev, rank, world, g):
    """Norm all-reduce and GEMM -> reduce-scatter -> LayerNorm with the sum taken inside the switch."""
    if not fc.has_multicast:
        if rank == 0:
            print("FUSED_OK (no multicast mapping on this box: nothing to check)")
        return dist.destroy_process_group()
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
    gs = GammaState(6, dev)
    for rep in range(3):
        part = torch.arange(1, 7, device=dev, dtype=torch.float32) * (rank + 1) * (rep + 1)
        fc.norm_allreduce_gamma(part, gs, reinit=True, use_multimem=True)
        want = part.clone()
        dist.all_reduce(want)
        torch.cuda.synchronize()
        assert torch.allclose(gs.sq, want), (gs.sq, want)
    M, d, Fl = 1024 * world, 2560, 1280
    rows = M // world
    y = torch.randn(M, Fl, device=dev, generator=g).bfloat16()
    w2_l = (torch.randn(d, Fl * world, device=dev, generator=g) * 0.03).bfloat16()[:, rank * Fl:(rank + 1) * Fl].contiguous()
    b2 = torch.randn(d, device=dev, generator=g).bfloat16()
    lnw = torch.randn(d, device=dev, generator=g).bfloat16()
    lnb = torch.randn(d, device=dev, generator=g).bfloat16()
    resid_all = torch.randn(M, d, device=dev, generator=g).bfloat16()
    for rep in range(4):                                    # both buffers twice: reuse after the barrier
        y_rep = (y.float() * (1 + 0.25 * rep)).bfloat16()
        resid = resid_all[rank * rows:(rank + 1) * rows]
        idx = fc.gemm_rs_pull(y_rep, w2_l)
        h, z = fc.rs_reduce_layernorm(idx, resid, b2, lnw, lnb)
        part_ref = linear(y_rep, w2_l, out_dtype=torch.float32)
        dist.all_reduce(part_ref)
        h_ref = (part_ref[rank * rows:(rank + 1) * rows] + b2.float() + resid.float()).bfloat16()
        z_ref = layernorm(h_ref, lnw, lnb)
        torch.cuda.synchronize()
        assert rel(h, h_ref) < 6e-3, ("gemm_rs_pull", rep, rel(h, h_ref))
        assert rel(z, z_ref) < 1e-2, ("rs_pull_ln", rep, rel(z, z_ref))
    _lib.check_device_errors()
    dist.barrier()
    if rank == 0:
        print("FUSED_OK switch reduction")
    dist.destroy_process_group()


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    # two shape sets: a small one (one-SM tile kernel) and one with enough 256 x 256 tiles and 256-row ownership
    # blocks for the two-SM kernel (cta_group::2) to take every fused launch
    cases = [(256 * world, 1024, 2048, 384, 640), (1024 * world, 2560, 2560 * world, 1024, 2560)]
    Mx, dx, Fx = cases[-1][:3]
    fc = FusedComm(ag_bytes=Mx * dx * 2, rs_bytes=Mx * dx * 2, w_bytes=max(Fx, 3 * cases[-1][4]) * dx * 2, n_push=8)
    g = torch.Generator(device=dev).manual_seed(1234)          # same stream on every rank
    if "--multimem" in sys.argv:
        return switch_reduction(fc, dev, rank, world, g)

    # ---- barrier + norm all-reduce fused with the gamma arithmetic
    fc.barrier()
    gs = GammaState(6, dev)
    part = torch.arange(1, 7, device=dev, dtype=torch.float32) * (rank + 1)
    for rep in range(2):
        fc.norm_allreduce_gamma(part, gs, reinit=True)
        want = part.clone()
        dist.all_reduce(want)
        torch.cuda.synchronize()
        assert torch.allclose(gs.sq, want), (gs.sq, want)
        assert torch.allclose(gs.ts, want.sqrt()) and torch.allclose(gs.gamma, want.sqrt())
        assert torch.allclose(gs.alpha, torch.ones_like(gs.alpha), atol=1e-6)

    L = _lib.lib()
    for case, (M, d, F, xs_rows, dq) in enumerate(cases):
        two = [L.dz_comm_gemm_two_sm(M, F // world, 1, M // world, 0), L.dz_comm_gemm_two_sm(M, d, 0, 0, 0),
               L.dz_comm_gemm_two_sm(xs_rows, F, 2, F // world, 0)]
        assert two == ([0, 0, 0] if case == 0 else [1, 1, 1]), (case, two)
        run_case(fc, g, dev, rank, world, M, d, F, xs_rows, dq)
    # the policies used with more than two ranks, on both tile kernels: sixteen CTAs that only push, and CTAs
    # that push and keep a part of a normal CTA's tiles
    for ctas, share in ((16, 0.0), (32, 0.5)):
        fc.push_ctas, fc.push_share = ctas, share
        for M, d, F, xs_rows, dq in cases:
            run_case(fc, g, dev, rank, world, M, d, F, xs_rows, dq)
    fc.push_ctas, fc.push_share = 0, 0.0

    torch.cuda.synchronize()
    _lib.check_device_errors()
    dist.barrier()
    report = fc.protocol_report()            # every ready / ack / partial-sum word agrees with the launches issued
    assert not report, report
    if rank == 0:
        print("FUSED_OK world", world)
    dist.destroy_process_group()


def run_case(fc, g, dev, rank, world, M, d, F, xs_rows, dq):
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
    # ---- tensor parallel: all-gather -> GEMM, GEMM -> reduce-scatter (+ residual + LayerNorm)
    x_all = torch.randn(M, d, device=dev, generator=g).bfloat16()
    w1 = (torch.randn(F, d, device=dev, generator=g) * 0.03).bfloat16()      # fc1, rows sharded
    b1 = torch.randn(F, device=dev, generator=g).bfloat16()
    w2 = (torch.randn(d, F, device=dev, generator=g) * 0.03).bfloat16()      # fc2, columns sharded
    b2 = torch.randn(d, device=dev, generator=g).bfloat16()
    lnw = torch.randn(d, device=dev, generator=g).bfloat16()
    lnb = torch.randn(d, device=dev, generator=g).bfloat16()
    rows, Fl = M // world, F // world
    w1_l, b1_l = w1[rank * Fl:(rank + 1) * Fl].contiguous(), b1[rank * Fl:(rank + 1) * Fl].contiguous()
    w2_l = w2[:, rank * Fl:(rank + 1) * Fl].contiguous()
    for rep in range(3):
        x_rep = (x_all.float() * (1 + 0.1 * rep)).bfloat16()
        x_full, mine = fc.ag_input(M, d)
        mine.copy_(x_rep[rank * rows:(rank + 1) * rows])
        y = fc.ag_gemm(x_full, w1_l, b1_l, act="relu")                       # [M, F/world]
        ref = linear(x_rep, w1_l, b1_l, act="relu")
        torch.cuda.synchronize()
        assert rel(y, ref) < 1e-3, ("ag_gemm", rep, rel(y, ref))
        idx = fc.gemm_rs(y, w2_l)                                            # partial [M, d] -> owners
        resid = x_rep[rank * rows:(rank + 1) * rows]
        h, z = fc.rs_reduce_layernorm(idx, resid, b2, lnw, lnb)
        part_ref = linear(ref, w2_l, out_dtype=torch.float32)
        dist.all_reduce(part_ref)
        h_ref = (part_ref[rank * rows:(rank + 1) * rows] + b2.float() + resid.float()).bfloat16()
        z_ref = layernorm(h_ref, lnw, lnb)
        torch.cuda.synchronize()
        assert rel(h, h_ref) < 6e-3, ("gemm_rs", rep, rel(h, h_ref))
        assert rel(z, z_ref) < 1e-2, ("rs_ln", rep, rel(z, z_ref))

    # ---- FSDP: shard push fused with the perturbation and the consuming GEMM
    xs = torch.randn(xs_rows, d, device=dev, generator=g).bfloat16()
    shard = w1[rank * Fl:(rank + 1) * Fl].contiguous()
    z_full = torch.from_numpy(philox.gaussian(77, 9, F * d)).view(F, d).to(dev)
    w_pert = perturb_reference(w1, 1e-2, z_full)
    seg = lambda: [dict(w_shard=shard, dst_row0=rank * Fl, tensor_id=9, elem_base=rank * Fl * d)]
    for rep in range(3):
        nxt = fc._calls["w"] % 2
        if rep < 2:      # push and consume in the same launch
            slot, out = fc.fsdp_launch(push=dict(segments=seg(), seed=77, coef=1e-2),
                                       gemm=dict(slot=nxt, N=F, x=xs, bias=b1, rows_per_src=Fl))
        else:            # prefetch style: push first, consume in the next launch (with another push)
            slot, _ = fc.fsdp_launch(push=dict(segments=seg(), seed=77, coef=1e-2))
            _, out = fc.fsdp_launch(push=dict(segments=seg(), seed=77, coef=0.0),
                                    gemm=dict(slot=slot, N=F, x=xs, bias=b1, rows_per_src=Fl))
        torch.cuda.synchronize()
        ref = linear(xs, w_pert, b1)
        got = fc.fsdp_weight(slot, F, d)
        # the pushed shard is the packed bf16 fma of the staging sweep: equal to the host statement bit for bit
        assert torch.equal(got, w_pert), ("fsdp gather+perturb", rep)
        assert rel(out, ref) < 1e-3, ("fsdp_gemm", rep, rel(out, ref))
    # fused q|k|v: three segments in one push, ownership repeating every dq rows, tiles that
    # straddle two owners (rows_per_src = dq / world need not be a multiple of the 256-row tile)
    wq = [(torch.randn(dq, d, device=dev, generator=g) * 0.03).bfloat16() for _ in range(3)]
    rq = dq // world
    segs = [dict(w_shard=wq[j][rank * rq:(rank + 1) * rq].contiguous(), dst_row0=j * dq + rank * rq,
                 tensor_id=20 + j, elem_base=rank * rq * d) for j in range(3)]
    nxt = fc._calls["w"] % 2
    slot, out = fc.fsdp_launch(push=dict(segments=segs, seed=5, coef=-1e-2),
                               gemm=dict(slot=nxt, N=3 * dq, x=xs, rows_per_src=rq, src_period=dq))
    torch.cuda.synchronize()
    zq = [torch.from_numpy(philox.gaussian(5, 20 + j, dq * d)).view(dq, d).to(dev) for j in range(3)]
    w_qkv = torch.cat([perturb_reference(wq[j], -1e-2, zq[j]) for j in range(3)])
    assert torch.equal(fc.fsdp_weight(slot, 3 * dq, d), w_qkv)
    assert rel(out, linear(xs, w_qkv)) < 2e-3, rel(out, linear(xs, w_qkv))


if __name__ == "__main__":
    main()
