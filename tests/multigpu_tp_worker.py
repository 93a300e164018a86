"""Worker for tests/test_multigpu_fused.py: tensor-parallel OPT vs the unsharded model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dizo_b200.data.synthetic import synthetic_batch  # noqa: E402
from dizo_b200.engine import DiZOProjector, ZOEngine  # noqa: E402
from dizo_b200.models.opt import OPTModel, Transform, preset  # noqa: E402
from dizo_b200.ops import _lib  # noqa: E402
from dizo_b200.parallel.composition import TPCompositionModel  # noqa: E402
from dizo_b200.parallel.tp import TPOPTModel  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = preset("opt-125m", num_hidden_layers=2, hidden_size=1024, num_attention_heads=8, ffn_dim=2048,
                 vocab_size=4096, max_position_embeddings=512)
    tp = TPOPTModel(cfg, dev, max_tokens=1024, n_push=8).init_random_fast(0)
    ref = OPTModel(cfg, dev, torch.bfloat16).init_random_fast(0)
    sd = tp.gather_state_dict()
    for n, t in ref.state_dict().items():
        assert torch.equal(sd[n], t), n
    b = synthetic_batch(0, 4, 256, cfg.vocab_size, cand_ids=(17, 29)).to(dev)     # 1024 token rows
    # the NCCL composition (all-gather / reduce-scatter between the stand-alone kernels)
    comp = TPCompositionModel(cfg, dev, max_tokens=1024, n_push=8).init_random_fast(0)
    assert torch.equal(comp.arena.data, tp.arena.data)
    for t in (None, Transform(seed=5, coef=1e-2), Transform(seed=5, coef=-1e-2)):
        l_tp, l_ref, l_comp = tp.loss(b, t).item(), ref.loss(b, t).item(), comp.loss(b, t).item()
        assert abs(l_tp - l_ref) < 2e-2, (t, l_tp, l_ref)
        assert abs(l_tp - l_comp) < 2e-2, (t, l_tp, l_comp)
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
    d_sh, d_ref = _make_decoder(tp, 3, 37 + 8 + 128), _make_decoder(ref, 3, 37 + 8 + 128)
    l_sh, l_ref = d_sh.prefill(gb), d_ref.prefill(gb)
    n_real = mask.sum(1).to(dev)
    for stepi in range(3):
        assert (l_sh - l_ref).abs().max().item() < 0.15, (stepi, (l_sh - l_ref).abs().max().item())
        nxt = l_ref.argmax(-1).to(torch.int32)
        pos = (n_real + 2).to(torch.int32)
        n_real = n_real + 1
        l_sh, l_ref = d_sh.step(nxt, pos, gb.pad_left), d_ref.step(nxt, pos, gb.pad_left)
    out = generate(tp, ids, attention_mask=mask, max_new_tokens=6, eos_token_id=[2])
    assert len(out) == 3 and all(len(o) >= int(m.sum()) + 1 for o, m in zip(out, mask))
    # ZO steps: same z on shards as on the full tensors
    e_tp, e_ref = ZOEngine(tp, eps=1e-2, dp_group=False), ZOEngine(ref, eps=1e-2, dp_group=False)
    for step in range(3):
        e_tp.step(b, 1e-3, seed=40 + step)
        e_ref.step(b, 1e-3, seed=40 + step)
    sd = tp.gather_state_dict()
    worst = max((sd[n].float() - t.float()).abs().max().item() for n, t in ref.state_dict().items())
    assert worst < 2e-2, worst
    # DiZO: sharded norms reduced + gamma arithmetic in the fused kernel
    p_tp, p_ref = DiZOProjector(tp, max_iters=1, dp_group=False), DiZOProjector(ref, max_iters=1, dp_group=False)
    tp.arena.sweep(seed1=3, c1=5e-3)
    ref.arena.sweep(seed1=3, c1=5e-3)
    p_tp.measure(); p_tp._begin(True)
    p_ref.measure(); p_ref._begin(True)
    torch.cuda.synchronize()
    assert torch.allclose(p_tp.gs.ts, p_ref.gs.ts, rtol=1e-3), (p_tp.gs.ts, p_ref.gs.ts)
    p_tp.search_zo(lambda: b, seed=1)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    dist.barrier()
    report = tp.comm.protocol_report()            # every ready / ack / partial-sum word agrees with the launches issued
    assert not report, report
    if rank == 0:
        print("TP_OK world", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
