"""Worker for tests/test_multigpu_fused.py: FSDP-sharded OPT vs the unsharded model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dizo_b200.data.synthetic import synthetic_batch  # noqa: E402
from dizo_b200.engine import DiZOProjector, ZOEngine  # noqa: E402
from dizo_b200.models.opt import OPTModel, Transform, preset  # noqa: E402
from dizo_b200.ops import _lib  # noqa: E402
from dizo_b200.parallel.composition import FSDPCompositionModel  # noqa: E402
from dizo_b200.parallel.fsdp import FSDPOPTModel  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = preset("opt-125m", num_hidden_layers=3, hidden_size=640, num_attention_heads=8, ffn_dim=1280,
                 vocab_size=4096, max_position_embeddings=512)      # hd 80, shards of 320 rows
    fs = FSDPOPTModel(cfg, dev, n_push=8).init_random_fast(0)
    ref = OPTModel(cfg, dev, torch.bfloat16).init_random_fast(0)
    sd = fs.gather_state_dict()
    for n, t in ref.state_dict().items():
        assert torch.equal(sd[n], t), n
    # every rank has its own batch shard; the reference sees this rank's shard too
    b = synthetic_batch(0, 4, 192, cfg.vocab_size, rank=rank, cand_ids=(17, 29)).to(dev)
    # the NCCL composition (sweep -> all-gather -> GEMM) of the same sharded model
    comp = FSDPCompositionModel(cfg, dev, n_push=8).init_random_fast(0)
    assert torch.equal(comp.arena.data, fs.arena.data)
    for t in (None, Transform(seed=5, coef=1e-2), Transform(seed=5, coef=-1e-2)):
        l_fs, l_ref, l_comp = fs.loss(b, t).item(), ref.loss(b, t).item(), comp.loss(b, t).item()
        assert abs(l_fs - l_ref) < 2e-2, (t, l_fs, l_ref)
        # same perturbed bits, same GEMM tiles up to the kernel variant: the two sharded arms agree closely
        assert abs(l_fs - l_comp) < 5e-3, (t, l_fs, l_comp)
    del comp
    # autoregressive decoding without moving weights: next-token logits of the prompt and of two more
    # steps against the replicated model, then a whole generate() call
    from dizo_b200.models.generate import _make_decoder, generate
    from dizo_b200.models.opt import make_batch
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(4, cfg.vocab_size, (3, 37), generator=gen)
    mask = torch.ones_like(ids)
    mask[1, :9] = 0
    ids[1, :9] = 1
    gb = make_batch(ids, mask).to(dev)
    d_sh, d_ref = _make_decoder(fs, 3, 37 + 8 + 128), _make_decoder(ref, 3, 37 + 8 + 128)
    l_sh, l_ref = d_sh.prefill(gb), d_ref.prefill(gb)
    n_real = mask.sum(1).to(dev)
    for stepi in range(3):
        assert (l_sh - l_ref).abs().max().item() < 0.15, (stepi, (l_sh - l_ref).abs().max().item())
        nxt = l_ref.argmax(-1).to(torch.int32)
        pos = (n_real + 2).to(torch.int32)
        n_real = n_real + 1
        l_sh, l_ref = d_sh.step(nxt, pos, gb.pad_left), d_ref.step(nxt, pos, gb.pad_left)
    out = generate(fs, ids, attention_mask=mask, max_new_tokens=6, eos_token_id=[2])
    assert len(out) == 3 and all(len(o) >= int(m.sum()) + 1 for o, m in zip(out, mask))
    # data-parallel ZO steps over sharded parameters: g is all-reduced, shards updated locally
    e_fs = ZOEngine(fs, eps=1e-2)
    for step in range(3):
        e_fs.step(b, 1e-3, seed=40 + step)
    g_fs = e_fs.projected_grad.item()
    # same steps on the unsharded model with the all-reduced g (emulated: average of per-rank g)
    e_ref = ZOEngine(ref, eps=1e-2)
    for step in range(3):
        e_ref.step(b, 1e-3, seed=40 + step)
    sd = fs.gather_state_dict()
    worst = max((sd[n].float() - t.float()).abs().max().item() for n, t in ref.state_dict().items())
    assert worst < 2e-2, worst
    assert abs(g_fs - e_ref.projected_grad.item()) < 0.5
    # DiZO over shards: reduced norms + a gamma search through blended pushes
    p_fs, p_ref = DiZOProjector(fs, max_iters=1), DiZOProjector(ref, max_iters=1)
    fs.arena.sweep(seed1=3, c1=5e-3)
    ref.arena.sweep(seed1=3, c1=5e-3)
    p_fs.measure(); p_fs._begin(True)
    p_ref.measure(); p_ref._begin(True)
    torch.cuda.synchronize()
    assert torch.allclose(p_fs.gs.ts, p_ref.gs.ts, rtol=1e-3), (p_fs.gs.ts, p_ref.gs.ts)
    al = torch.full_like(p_fs.gs.alpha, 0.9)
    l_fs, l_ref = fs.loss(b, Transform(alpha=al)).item(), ref.loss(b, Transform(alpha=al)).item()
    assert abs(l_fs - l_ref) < 2e-2, (l_fs, l_ref)
    # first-order gamma search over the shards: the kernel backward with every weight (and theta - theta_0 of
    # the k / v shards) assembled by pushes equals the replicated kernel backward on the same batch
    from dizo_b200.models.gamma_grad import GammaGrad, supported
    assert supported(fs)
    g = torch.Generator(device=dev).manual_seed(11)
    al = torch.rand(p_fs.n, device=dev, generator=g) * 0.5 + 0.6
    lf, gf = GammaGrad(fs).loss_and_grad(b, al.clone())
    lr_, gr = GammaGrad(ref).loss_and_grad(b, al.clone())
    torch.cuda.synchronize()
    _lib.check_device_errors()
    assert abs(lf.item() - lr_.item()) < 2e-2, (lf, lr_)
    cos = torch.nn.functional.cosine_similarity(gf, gr, dim=0).item()
    assert cos > 0.98 and 0.8 < (gf.norm() / gr.norm()).item() < 1.25, (cos, gf, gr)
    p_fs.max_iters = 2
    p_fs.search_fo(lambda: b)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    p_fs.search_zo(lambda: b, seed=1)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    dist.barrier()
    report = fs.comm.protocol_report()            # every ready / ack / partial-sum word agrees with the launches issued
    assert not report, report
    if rank == 0:
        print("FSDP_OK world", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
