"""sm_100a kernels (attention, LayerNorm, embedding, loss tail, ZO sweeps) against PyTorch
fp32 statements of the same ops."""
import numpy as np
import pytest
import torch

from dizo_b200.ops import _lib, philox
from dizo_b200.ops.attention import attention, attention_reference
from dizo_b200.ops.loss import option_ce, token_logprobs, verbalizer_ce
from dizo_b200.ops.norm import add_rows, embed, gather_rows, layernorm, opt_positions
from dizo_b200.ops.zo import CHUNK, GammaState, ParamArena, Piece, fill_z, perturb_reference, scalar_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sync_ok():
    torch.cuda.synchronize()
    _lib.check_device_errors()


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("B,L,H,hd", [
    (2, 256, 4, 64), (1, 128, 2, 128), (2, 200, 3, 80), (1, 64, 2, 64), (3, 384, 2, 128),
    (1, 1000, 2, 80), (2, 24, 12, 64), (1, 520, 1, 128),
])
def test_attention_causal(B, L, H, hd):
    g = torch.Generator(device=DEV).manual_seed(B * 1000 + L + hd)
    qkv = torch.randn(B, L, 3 * H * hd, device=DEV, generator=g).bfloat16()
    out = attention(qkv, H)
    _sync_ok()
    ref = attention_reference(qkv.float(), H)
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2


@pytest.mark.parametrize("hd", [64, 80, 128])
def test_attention_left_pad_and_prefix(hd):
    B, L, H = 3, 300, 4
    g = torch.Generator(device=DEV).manual_seed(hd)
    qkv = torch.randn(B, L, 3 * H * hd, device=DEV, generator=g).bfloat16()
    pad = torch.tensor([0, 70, 257], dtype=torch.int32, device=DEV)
    pk = torch.randn(5, H * hd, device=DEV, generator=g).bfloat16()
    pv = torch.randn(5, H * hd, device=DEV, generator=g).bfloat16()
    for use_prefix in (False, True):
        out = attention(qkv, H, pad_left=pad, prefix_k=pk if use_prefix else None,
                        prefix_v=pv if use_prefix else None)
        _sync_ok()
        ref = attention_reference(qkv.float(), H, pad_left=pad,
                                  prefix_k=pk.float() if use_prefix else None,
                                  prefix_v=pv.float() if use_prefix else None)
        # compare real (non-padding) query rows only
        for b in range(B):
            p = int(pad[b])
            d = (out[b, p:].float() - ref[b, p:]).abs().max().item()
            assert d < 3e-2, (use_prefix, b, d)
        assert torch.isfinite(out.float()).all()


def test_attention_large_scores_rescale():
    # big logits force the lazily-raised running maximum to be corrected
    B, L, H, hd = 1, 512, 2, 64
    g = torch.Generator(device=DEV).manual_seed(3)
    qkv = (torch.randn(B, L, 3 * H * hd, device=DEV, generator=g) * 4).bfloat16()
    out = attention(qkv, H)
    _sync_ok()
    ref = attention_reference(qkv.float(), H)
    assert (out.float() - ref).abs().max().item() < 0.15
    assert ((out.float() - ref).norm() / ref.norm()).item() < 2e-2


# ------------------------------------------------------------------ norm / embed
@pytest.mark.parametrize("rows,d", [(7, 768), (300, 2560), (64, 5120), (5, 9216), (3, 64)])
def test_layernorm(rows, d):
    g = torch.Generator(device=DEV).manual_seed(d)
    x = (torch.randn(rows, d, device=DEV, generator=g) * 2 + 0.5).bfloat16()
    w = torch.randn(d, device=DEV, generator=g).bfloat16()
    b = torch.randn(d, device=DEV, generator=g).bfloat16()
    y = layernorm(x, w, b)
    ref = torch.nn.functional.layer_norm(x.float(), (d,), w.float(), b.float(), 1e-5)
    assert (y.float() - ref).abs().max().item() < 4e-2


def test_embed_gather_add():
    V, d, B, L = 1000, 256, 3, 17
    g = torch.Generator(device=DEV).manual_seed(1)
    tok = torch.randn(V, d, device=DEV, generator=g).bfloat16()
    pos = torch.randn(64, d, device=DEV, generator=g).bfloat16()
    ids = torch.randint(0, V, (B, L), device=DEV, generator=g, dtype=torch.int32)
    mask = torch.ones(B, L, device=DEV, dtype=torch.int32)
    mask[1, :5] = 0
    p = opt_positions(mask)
    assert p[1, 4].item() == 1 and p[1, 5].item() == 2 and p[0, 0].item() == 2
    h = embed(ids, p, tok, pos)
    ref = (tok[ids.long()].float() + pos[p.long()].float())
    assert (h.float() - ref).abs().max().item() < 4e-2
    rows = torch.tensor([5, 0, 44], dtype=torch.int32, device=DEV)
    assert torch.equal(gather_rows(h.view(-1, d), rows), h.view(-1, d)[rows.long()])
    a = add_rows(h, p.view(-1), pos)
    assert (a.float() - (h.float() + pos[p.view(-1).long()].float().view(B, L, d))).abs().max() < 7e-2


# ------------------------------------------------------------------ loss tail
def test_token_logprobs_and_option_ce():
    R, d, V = 37, 512, 50272
    g = torch.Generator(device=DEV).manual_seed(9)
    h = torch.randn(R, d, device=DEV, generator=g).bfloat16()
    table = (torch.randn(V, d, device=DEV, generator=g) * 0.05).bfloat16()
    tg = torch.randint(0, V, (R,), device=DEV, generator=g, dtype=torch.int32)
    tg[0] = V - 1
    tg[1] = 0
    lp = token_logprobs(h, table, tg)
    _sync_ok()
    ref = torch.log_softmax(h.float() @ table.float().t(), -1).gather(1, tg.long().view(-1, 1)).squeeze(1)
    assert (lp - ref).abs().max().item() < 2e-3
    # 6 examples: 2+3+2+2+3+2 = 14 candidates over the 37 rows
    seq_len = [3, 2, 4, 1, 2, 3, 3, 2, 2, 4, 3, 2, 3, 3]
    seq_start = torch.tensor(np.concatenate([[0], np.cumsum(seq_len)]), dtype=torch.int32, device=DEV)
    ex_start = torch.tensor([0, 2, 5, 7, 9, 12, 14], dtype=torch.int32, device=DEV)
    labels = torch.tensor([1, 2, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    loss = option_ce(lp, seq_start, ex_start, labels, True)
    ref_loss = option_ce(ref.cpu(), seq_start.cpu(), ex_start.cpu(), labels.cpu(), True)
    assert abs(loss.item() - ref_loss.item()) < 2e-3
    lm = option_ce(lp, seq_start, None, None, False)
    assert abs(lm.item() + ref.mean().item()) < 2e-3


def test_verbalizer_ce():
    E, d, V = 16, 768, 50272
    g = torch.Generator(device=DEV).manual_seed(2)
    h = torch.randn(E, d, device=DEV, generator=g).bfloat16()
    table = (torch.randn(V, d, device=DEV, generator=g) * 0.05).bfloat16()
    cand = torch.tensor([1099, 372], dtype=torch.int32, device=DEV)
    labels = torch.randint(0, 2, (E,), device=DEV, generator=g, dtype=torch.int32)
    logits, loss = verbalizer_ce(h, table, cand, labels)
    ref_logits = h.float() @ table[cand.long()].float().t()
    assert (logits - ref_logits).abs().max().item() < 1e-3
    ref_loss = torch.nn.functional.cross_entropy(ref_logits, labels.long())
    assert abs(loss.item() - ref_loss.item()) < 1e-4


# ------------------------------------------------------------------ ZO sweeps
def _arena(device, dtype=torch.bfloat16):
    pieces = [Piece("g.pos", (50, 64), tensor_id=1, group=-1),
              Piece("l0.k", (64, 64), tensor_id=2, group=0),
              Piece("l0.v", (64, 64), tensor_id=3, group=0),
              Piece("l0.b", (100,), tensor_id=4, group=0),          # ragged: not a multiple of 8... 100 = 12*8+4
              Piece("l1.k", (96, 128), tensor_id=5, group=1),
              Piece("l1.v", (3000,), tensor_id=6, group=1)]
    a = ParamArena(pieces, device, dtype)
    g = torch.Generator().manual_seed(0)
    for p in a.pieces:
        a.view(p.name).copy_((torch.randn(p.shape, generator=g) * 0.02).to(dtype))
    return a


def test_z_matches_numpy():
    z = fill_z(10000, seed=99, tensor_id=5, device=DEV).cpu().numpy()
    ref = philox.gaussian(99, 5, 10000)
    assert np.abs(z - ref).max() < 2e-5
    z2 = fill_z(1024, seed=99, tensor_id=5, device=DEV, elem_base=4096).cpu().numpy()
    assert np.abs(z2 - philox.gaussian(99, 5, 8192)[4096:5120]).max() < 2e-5


def test_sweep_matches_cpu_oracle():
    ga, ca = _arena(DEV), _arena("cpu")
    assert torch.equal(ga.data.cpu(), ca.data)
    for a in (ga, ca):
        a.sweep(seed1=5, c1=1e-3)
    # the plain perturbation is a packed bf16 fma (exact product and sum, one rounding): the host
    # statement reproduces it bit for bit
    assert torch.equal(ga.data.cpu(), ca.data)
    # padding between pieces is never touched
    p = ga.pieces[3]
    assert ga.data[p.offset + p.numel: p.offset + CHUNK].abs().sum().item() == 0


def test_sweep_staging_range_and_two_terms():
    ga, ca = _arena(DEV), _arena("cpu")
    lo, hi = ga.group_range(1)
    n = ga.group_numel(1)
    sg = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    sc = torch.zeros(n, dtype=torch.bfloat16)
    coef = torch.tensor([2.0], dtype=torch.float32)
    before = ga.data.clone()
    ga.sweep(t_begin=lo, t_end=hi, dst=sg, seed1=5, c1=1e-3, seed2=6, c2=-0.5e-3, c2_dev=coef.to(DEV))
    ca.sweep(t_begin=lo, t_end=hi, dst=sc, seed1=5, c1=1e-3, seed2=6, c2=-0.5e-3, c2_dev=coef)
    assert torch.equal(ga.data, before)                      # theta untouched
    d = (sg.cpu().float() - sc.float()).abs()
    assert d.max().item() <= 2.5e-4 and (d > 0).float().mean().item() < 0.01
    k = ga.view("l1.k", base=sg, shift=ga.span(lo, hi)[0])
    zk = torch.from_numpy(philox.gaussian(5, 5, 96 * 128)).view(96, 128)
    zk2 = torch.from_numpy(philox.gaussian(6, 5, 96 * 128)).view(96, 128)
    want = ca.view("l1.k").float() + 1e-3 * zk - 1e-3 * zk2
    assert (k.cpu().float() - want).abs().max().item() < 3e-4


def test_small_footprint_sweep_equals_the_regular_one():
    """The variant that shares SMs with a GEMM (4 KB table, 512 threads) writes the same bits."""
    ga = _arena(DEV)
    ga.set_dizo(["l0.k", "l0.v", "l1.k", "l1.v"])
    ga.sweep(seed1=1, c1=5e-3)
    lo, hi = ga.group_range(1)
    n = ga.group_numel(1)
    alpha = torch.tensor([0.8, 1.2, 1.0, 0.9], dtype=torch.float32, device=DEV)
    for kw in (dict(seed1=5, c1=1e-3), dict(seed1=5, c1=-1e-3), dict(alpha=alpha), dict(seed1=7, c1=1e-3, alpha=alpha)):
        a = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
        b = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
        ga.sweep(t_begin=lo, t_end=hi, dst=a, **kw)
        ga.sweep(t_begin=lo, t_end=hi, dst=b, small=True, **kw)
        _sync_ok()
        assert torch.equal(a, b), kw


def test_two_sided_sweep_equals_two_sweeps():
    """theta + c z and theta - c z staged from one draw of z: the same bits as two sweeps with +c and -c, for
    every group (ragged tensor tails included), in both kernel variants and with a device-side seed."""
    ga = _arena(DEV)
    seed_dev = torch.tensor([91], dtype=torch.int64, device=DEV)
    for g in ga.groups():
        lo, hi = ga.group_range(g)
        n = ga.group_numel(g)
        for kw in (dict(seed1=5, c1=1e-3), dict(seed1=5, c1=1e-3, small=True), dict(seed1_dev=seed_dev, c1=2e-3)):
            plus = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
            minus = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
            a = torch.full((n,), 7.0, dtype=torch.bfloat16, device=DEV)
            b = torch.full((n,), 7.0, dtype=torch.bfloat16, device=DEV)
            ga.sweep(t_begin=lo, t_end=hi, dst=plus, **kw)
            ga.sweep(t_begin=lo, t_end=hi, dst=minus, **{**kw, "c1": -kw["c1"]})
            ga.sweep(t_begin=lo, t_end=hi, dst=a, dst2=b, **kw)
            _sync_ok()
            # compare what the sweeps write (the padding between pieces keeps the buffer's old content)
            for i in range(lo, hi):
                p_ = ga.pieces[i]
                o = p_.offset - ga.span(lo, hi)[0]
                assert torch.equal(a[o:o + p_.numel], plus[o:o + p_.numel]), (g, kw, p_.name)
                assert torch.equal(b[o:o + p_.numel], minus[o:o + p_.numel]), (g, kw, p_.name)
                assert not torch.equal(a[o:o + p_.numel], b[o:o + p_.numel])


def test_perturb_restore_replay_and_update():
    a = _arena(DEV)
    ref = a.data.clone()
    a.sweep(seed1=42, c1=1e-3)
    a.sweep(seed1=42, c1=-2e-3)
    a.sweep(seed1=42, c1=1e-3)
    # bf16 round trips: at most one ulp away from where it started (ulp(0.06) ~ 4.9e-4)
    assert (a.data.float() - ref.float()).abs().max().item() <= 5e-4
    g_dev = torch.tensor([3.0], dtype=torch.float32, device=DEV)
    b = _arena(DEV)
    b.sweep(seed1=42, c1=-1e-2, c1_dev=g_dev)
    z = fill_z(64 * 64, 42, 2, DEV).view(64, 64)
    want = perturb_reference(_arena("cpu").view("l0.k"), -3e-2, z.cpu())
    assert torch.equal(b.view("l0.k").cpu(), want)


def test_dizo_blend_norm_project():
    ga, ca = _arena(DEV), _arena("cpu")
    names = ["l0.k", "l0.v", "l1.k", "l1.v"]
    for a in (ga, ca):
        a.set_dizo(names)
        a.sweep(seed1=1, c1=5e-3)                      # move away from the anchor
    sqg = torch.zeros(4, dtype=torch.float32, device=DEV)
    sqc = torch.zeros(4, dtype=torch.float32)
    ga.sweep(sq_out=sqg)                                # in-place identity + norms
    ca.sweep(sq_out=sqc)
    for i, n in enumerate(names):
        want = ((ga.view(n).float() - ga.anchor_view(n).float()) ** 2).sum().item()
        assert abs(sqg[i].item() - want) / want < 1e-4
    assert torch.allclose(sqg.cpu(), sqc, rtol=2e-2)
    alpha = torch.tensor([0.8, 1.2, 1.0, 0.9], dtype=torch.float32)
    before = {n: ga.view(n).clone() for n in names}
    gpos_before = ga.view("g.pos").clone()
    ga.sweep(alpha=alpha.to(DEV), sq_out=sqg)           # projection + new norms in one pass
    for i, n in enumerate(names):
        an = ga.anchor_view(n).float()
        want = an + alpha[i].item() * (before[n].float() - an)
        assert (ga.view(n).float() - want).abs().max().item() < 3e-4
    # pieces without a slot are untouched by the blend
    assert torch.equal(ga.view("g.pos"), gpos_before)
    # deterministic norms
    sq2 = torch.zeros_like(sqg)
    ga.sweep(sq_out=sq2)
    sq3 = torch.zeros_like(sqg)
    ga.sweep(sq_out=sq3)
    assert torch.equal(sq2, sq3)


def test_stochastic_rounding_is_unbiased_and_matches_cpu():
    pieces = [Piece("w", (512, 512), tensor_id=0)]
    ga, ca = ParamArena(pieces, DEV), ParamArena([Piece("w", (512, 512), tensor_id=0)], "cpu")
    for a in (ga, ca):
        a.view("w").fill_(0.0302734375)                 # exactly representable in bf16
    # an update far below half an ulp (ulp here = 2^-13 ~ 1.2e-4) vanishes without SR
    ga.sweep(seed1=3, c1=0.0, seed2=0, c2=0.0)
    upd = 1e-5
    gb = ParamArena([Piece("w", (512, 512), tensor_id=0)], DEV)
    gb.view("w").fill_(0.0302734375)
    gb.sweep(seed1=3, c1=upd)
    z = fill_z(512 * 512, 3, 0, DEV)
    moved_rn = (gb.data.float() - 0.0302734375)
    ga.sweep(seed1=3, c1=upd, stochastic_round_seed=77)
    ca.sweep(seed1=3, c1=upd, stochastic_round_seed=77)
    moved_sr = (ga.data.float() - 0.0302734375)
    want = upd * z
    # correlation of the realised move with the wanted move: SR keeps the signal
    def corr(a, b):
        return (a * b).sum().item() / (a.norm().item() * b.norm().item() + 1e-30)
    assert corr(moved_sr, want) > 0.2
    assert abs(moved_sr.mean().item() - want.mean().item()) < 3e-6
    assert corr(moved_rn, want) < corr(moved_sr, want)
    assert (ga.data.cpu().float() - ca.data.float()).abs().max().item() <= 1.3e-4
    assert ((ga.data.cpu() != ca.data).float().mean().item()) < 0.01


def test_gamma_state_matches_cpu():
    n = 6
    gs, cs = GammaState(n, DEV), GammaState(n, "cpu")
    sq = torch.tensor([1.0, 4.0, 0.25, 9.0, 2.0, 0.5])
    gs.sq.copy_(sq)
    cs.sq.copy_(sq)
    for s in (gs, cs):
        s.begin(reinit=True)
        s.perturb(+1.0, seed=17, it=0)
    assert torch.allclose(gs.gamma.cpu(), cs.gamma, atol=1e-5)
    assert torch.allclose(gs.alpha.cpu(), cs.alpha, atol=1e-5)
    l1 = torch.tensor([0.71]); l2 = torch.tensor([0.69])
    for s, dev in ((gs, DEV), (cs, "cpu")):
        s.perturb(-2.0)
        s.perturb(+1.0)
        s.step(l1.to(dev), l2.to(dev))
    assert torch.allclose(gs.gamma.cpu(), cs.gamma, atol=1e-5)
    ts = sq.sqrt()
    assert (gs.gamma.cpu() >= 0.8 * ts - 1e-6).all() and (gs.gamma.cpu() <= 1.2 * ts + 1e-6).all()
    out = torch.zeros(1, device=DEV)
    scalar_diff(l1.to(DEV), l2.to(DEV), 500.0, out)
    assert abs(out.item() - 10.0) < 1e-3


# ------------------------------------------------------------------ bounded waits
def test_peer_wait_times_out_with_error_status_instead_of_hanging():
    """A flag that nothing ever sets: the kernel gives up after its time limit, records
    ERR_WAIT_PEER in the error word and returns; the context stays usable."""
    import ctypes
    import time
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)          # "rank 1" never writes flags[1]
    ptrs = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64, device=DEV)
    t0 = time.time()
    rc = _lib.lib().dz_peer_barrier(_lib.ptr(ptrs), 0, 2, ctypes.c_uint(1), _lib.ptr(_lib.err_word(DEV)),
                                    _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 10.0
    with pytest.raises(_lib.KernelError, match="peer"):
        _lib.check_device_errors()
    # the device still works and the error word is clear again
    x = torch.ones(8, device=DEV)
    assert x.sum().item() == 8
    _lib.check_device_errors()


# ------------------------------------------------------------------ decoding
def test_decode_attention_matches_reference():
    from dizo_b200.ops.attention import decode_attention_reference
    from dizo_b200.ops.decode import decode_attention
    for H, hd, Lmax, kv_len in ((12, 64, 96, 70), (32, 80, 300, 300), (40, 128, 64, 1)):
        B, d = 3, H * hd
        g = torch.Generator(device=DEV).manual_seed(hd)
        q = torch.randn(B, d, device=DEV, generator=g).bfloat16()
        kc = torch.randn(B, Lmax, d, device=DEV, generator=g).bfloat16()
        vc = torch.randn(B, Lmax, d, device=DEV, generator=g).bfloat16()
        pad = torch.tensor([0, min(5, kv_len - 1), 0], dtype=torch.int32, device=DEV)
        pk = torch.randn(5, d, device=DEV, generator=g).bfloat16()
        pv = torch.randn(5, d, device=DEV, generator=g).bfloat16()
        for pre in (False, True):
            out = decode_attention(q, kc, vc, kv_len, H, pad, pk if pre else None, pv if pre else None)
            ref = decode_attention_reference(q.float(), kc.float(), vc.float(), kv_len, H, pad,
                                             pk.float() if pre else None, pv.float() if pre else None)
            assert (out.float() - ref).abs().max().item() < 3e-2


def test_sampling_kernel_distribution_and_filters():
    from dizo_b200.ops.decode import sample
    V = 1000
    g = torch.Generator(device=DEV).manual_seed(0)
    logits = torch.randn(1, V, device=DEV, generator=g) * 2
    assert sample(logits, do_sample=False).item() == logits.argmax().item()
    big = logits.repeat(4096, 1).contiguous()
    # top-k: only the k most likely tokens may appear
    toks = sample(big, temperature=0.7, top_k=5, top_p=1.0, seed=3)
    top5 = set(logits[0].topk(5).indices.tolist())
    assert set(toks.tolist()) <= top5 and len(set(toks.tolist())) >= 3
    # nucleus: the sampled set is the smallest prefix of the sorted distribution reaching p
    p = torch.softmax(logits[0].float(), -1)
    srt, idx = p.sort(descending=True)
    n_keep = int((srt.cumsum(0) < 0.5).sum().item()) + 1
    toks = sample(big, top_p=0.5, seed=4)
    assert set(toks.tolist()) <= set(idx[:n_keep].tolist())
    # frequencies follow the renormalised probabilities
    counts = torch.bincount(toks, minlength=V).float() / toks.numel()
    want = torch.zeros(V, device=DEV)
    want[idx[:n_keep]] = srt[:n_keep] / srt[:n_keep].sum()
    assert (counts - want).abs().max().item() < 0.04
    # different steps draw differently, same (seed, offset) repeats
    a, b, c = sample(big, seed=9, offset=0), sample(big, seed=9, offset=0), sample(big, seed=9, offset=1)
    assert torch.equal(a, b) and not torch.equal(a, c)
