"""Kernel micro-benchmarks: CUDA-event timing of one kernel on one shape, against the library
call it replaces, as a burst (best of N after warm-up) or sustained (back to back for some
seconds, which is what a long training step sees under the power cap).

    python -m dizo_b200.ops.microbench gemm --m 8192 --n 15360 --k 5120 [--seconds 3]
    python -m dizo_b200.ops.microbench attn --batch 8 --seq 1024 --heads 40 --hd 128
    python -m dizo_b200.ops.microbench sweep --mib 2048 [--flags z2,blend,norm,sr,dual]
    python -m dizo_b200.ops.microbench layernorm --rows 8192 --d 5120
    python -m dizo_b200.ops.microbench dgrad --m 8192 --n 5120 --k 20480      # dX = dY W, W [k, n]
    python -m dizo_b200.ops.microbench attn_bwd --batch 8 --seq 1024 --heads 40 --hd 128
    python -m dizo_b200.ops.microbench lnbwd --rows 8192 --d 5120
    python -m dizo_b200.ops.microbench lmhead --rows 4096 --d 5120 --n 50272   # log-sum-exp fused LM head
    python -m dizo_b200.ops.microbench decode --batch 8 --seq 1024 --heads 40 --hd 128

Each run prints one JSON line with achieved TFLOP/s or GB/s and the fraction of the measured
peak found in MEASURED_PEAKS.json at the repository root (if present).  ``--only ours`` skips the
library call (used for profiler captures of a single kernel).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch

from . import _lib
from .attention import attention
from .gemm import linear
from .norm import layernorm
from .zo import ParamArena, Piece


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                     "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "fallback": True}


def time_fn(fn, iters=20, warmup=3, seconds=0.0, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if seconds > 0:
        n = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        while time.time() - t0 < seconds:
            for _ in range(10):
                fn()
            n += 10
            torch.cuda.current_stream().synchronize() if n % 200 == 0 else None
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    best = float("inf")
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "dgrad", "attn", "attn_bwd", "sweep", "layernorm", "lnbwd", "lmhead", "decode"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--mib", type=int, default=2048)
    ap.add_argument("--flags", default="")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--d", type=int, default=5120)
    ap.add_argument("--seconds", type=float, default=0.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="both", choices=["both", "ours", "lib"])
    a = ap.parse_args()
    peaks = _peaks()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.seconds == 0 else None
    out = {"kernel": a.kernel, "mode": "sustained" if a.seconds else "burst"}
    if a.kernel == "gemm":
        x = torch.randn(a.m, a.k, device=dev, generator=g).bfloat16()
        w = (torch.randn(a.n, a.k, device=dev, generator=g) * 0.02).bfloat16()
        y = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * a.m * a.n * a.k
        peak = peaks["bf16_tflops_sustained" if a.seconds else "bf16_tflops"]
        out.update(shape=[a.m, a.n, a.k])
        if a.flags in ("swiglu", "rope"):
            # fused epilogues of the LLaMA block: n = 2F (gate | up) or (H + 2 Hkv) * 128 (q | k | v, H = Hkv);
            # the alternative is the plain GEMM followed by the stand-alone kernel
            from . import gemm as gemm_mod
            from . import llama as llama_ops
            H = a.n // (3 * 128)
            L = a.seq
            fused = (lambda: gemm_mod.linear_swiglu(x, w)) if a.flags == "swiglu" else \
                (lambda: gemm_mod.linear_qkv_rope(x, w, L, 0, H, H, 128, 10000.0))
            plain = (lambda: llama_ops.silu_mul(linear(x, w, out=y))) if a.flags == "swiglu" else \
                (lambda: llama_ops.rope_qkv(linear(x, w, out=y), L, 0, H, H, 128, 10000.0))
            ms = time_fn(fused, a.iters, seconds=a.seconds, flush=flush)
            out.update(epilogue=a.flags, ours_ms=ms, ours_tflops=fl / ms / 1e9,
                       ours_frac_of_measured=fl / ms / 1e9 / peak)
            ms = time_fn(plain, a.iters, seconds=a.seconds, flush=flush)
            out.update(unfused_ms=ms, unfused_tflops=fl / ms / 1e9)
            print(json.dumps(out))
            return
        if a.only != "lib":
            ms = time_fn(lambda: linear(x, w, out=y, tile_n=a.tile_n), a.iters, seconds=a.seconds, flush=flush)
            out.update(ours_ms=ms, ours_tflops=fl / ms / 1e9, ours_frac_of_measured=fl / ms / 1e9 / peak)
        if a.only != "ours":
            ms = time_fn(lambda: torch.matmul(x, w.t(), out=y), a.iters, seconds=a.seconds, flush=flush)
            out.update(lib_ms=ms, lib_tflops=fl / ms / 1e9)
    elif a.kernel == "dgrad":
        from .backward import linear_dgrad
        dy = torch.randn(a.m, a.k, device=dev, generator=g).bfloat16()
        w = (torch.randn(a.k, a.n, device=dev, generator=g) * 0.02).bfloat16()
        fl = 2.0 * a.m * a.n * a.k
        peak = peaks["bf16_tflops_sustained" if a.seconds else "bf16_tflops"]
        out.update(shape=[a.m, a.n, a.k])
        if a.only != "lib":
            ms = time_fn(lambda: linear_dgrad(dy, w), a.iters, seconds=a.seconds, flush=flush)
            out.update(ours_ms=ms, ours_tflops=fl / ms / 1e9, ours_frac_of_measured=fl / ms / 1e9 / peak)
        if a.only != "ours":
            ms = time_fn(lambda: torch.matmul(dy, w), a.iters, seconds=a.seconds, flush=flush)
            out.update(lib_ms=ms, lib_tflops=fl / ms / 1e9)
    elif a.kernel == "attn_bwd":
        from .attention import attention_backward
        d = a.heads * a.hd
        qkv = torch.randn(a.batch, a.seq, 3 * d, device=dev, generator=g).bfloat16()
        do = torch.randn(a.batch, a.seq, d, device=dev, generator=g).bfloat16()
        lse = torch.empty(a.batch, a.heads, a.seq, dtype=torch.float32, device=dev)
        o = attention(qkv, a.heads, lse=lse)
        dqkv = torch.empty_like(qkv)
        # useful work: 5 GEMM-shaped products over the causal half (the two-pass kernel executes 7)
        fl = 10.0 * a.batch * a.heads * a.seq * a.seq * a.hd / 2
        out.update(shape=[a.batch, a.seq, a.heads, a.hd])
        if a.only != "lib":
            ms = time_fn(lambda: attention_backward(qkv, o, do, lse, a.heads, dqkv=dqkv), a.iters,
                         seconds=a.seconds, flush=flush)
            out.update(ours_ms=ms, ours_tflops=fl / ms / 1e9,
                       ours_frac_of_measured=fl / ms / 1e9 / peaks["bf16_tflops"])
        if a.only != "ours":
            q, k, v = (t.view(a.batch, a.seq, a.heads, a.hd).transpose(1, 2).detach().requires_grad_(True)
                       for t in qkv.split(d, dim=-1))
            with torch.enable_grad():
                so = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            gso = do.view(a.batch, a.seq, a.heads, a.hd).transpose(1, 2)
            ms = time_fn(lambda: torch.autograd.grad(so, (q, k, v), gso, retain_graph=True), a.iters,
                         seconds=a.seconds, flush=flush)
            out.update(lib_ms=ms, lib_tflops=fl / ms / 1e9)
    elif a.kernel == "lnbwd":
        from .backward import layernorm_backward
        x = torch.randn(a.rows, a.d, device=dev, generator=g).bfloat16()
        dy = torch.randn(a.rows, a.d, device=dev, generator=g).bfloat16()
        w = torch.randn(a.d, device=dev, generator=g).bfloat16()
        nbytes = 6.0 * a.rows * a.d                      # read x and dy, write dx
        ms = time_fn(lambda: layernorm_backward(dy, x, w), a.iters, seconds=a.seconds, flush=flush)
        out.update(shape=[a.rows, a.d], ours_ms=ms, ours_gbs=nbytes / ms / 1e6,
                   ours_frac_of_measured=nbytes / ms / 1e6 / peaks["hbm_gbs"])
    elif a.kernel == "lmhead":
        from .loss import token_logprobs
        x = torch.randn(a.rows, a.d, device=dev, generator=g).bfloat16()
        table = (torch.randn(a.n, a.d, device=dev, generator=g) * 0.02).bfloat16()
        tg = torch.randint(0, a.n, (a.rows,), device=dev, generator=g, dtype=torch.int32)
        fl = 2.0 * a.rows * a.n * a.d
        out.update(shape=[a.rows, a.n, a.d])
        if a.only != "lib":
            ms = time_fn(lambda: token_logprobs(x, table, tg), a.iters, seconds=a.seconds, flush=flush)
            out.update(ours_ms=ms, ours_tflops=fl / ms / 1e9, ours_frac_of_measured=fl / ms / 1e9 / peaks["bf16_tflops"],
                       logits_bytes_avoided=2.0 * a.rows * a.n)
        if a.only != "ours":
            def ref():
                lg = torch.matmul(x, table.t()).float()
                return torch.log_softmax(lg, dim=-1).gather(1, tg.long().view(-1, 1))
            ms = time_fn(ref, a.iters, seconds=a.seconds, flush=flush)
            out.update(lib_ms=ms, lib_tflops=fl / ms / 1e9)
    elif a.kernel == "decode":
        from .decode import decode_attention
        d = a.heads * a.hd
        q = torch.randn(a.batch, d, device=dev, generator=g).bfloat16()
        kc = torch.randn(a.batch, a.seq, d, device=dev, generator=g).bfloat16()
        vc = torch.randn(a.batch, a.seq, d, device=dev, generator=g).bfloat16()
        nbytes = 4.0 * a.batch * a.seq * d               # the K and V cache rows read once
        ms = time_fn(lambda: decode_attention(q, kc, vc, a.seq, a.heads), a.iters, seconds=a.seconds, flush=flush)
        out.update(shape=[a.batch, a.seq, a.heads, a.hd], ours_ms=ms, ours_gbs=nbytes / ms / 1e6,
                   ours_frac_of_measured=nbytes / ms / 1e6 / peaks["hbm_gbs"])
    elif a.kernel == "attn":
        d = a.heads * a.hd
        qkv = torch.randn(a.batch, a.seq, 3 * d, device=dev, generator=g).bfloat16()
        o = torch.empty(a.batch, a.seq, d, device=dev, dtype=torch.bfloat16)
        fl = 4.0 * a.batch * a.heads * a.seq * a.seq * a.hd / 2
        out.update(shape=[a.batch, a.seq, a.heads, a.hd])
        if a.only != "lib":
            ms = time_fn(lambda: attention(qkv, a.heads, out=o), a.iters, seconds=a.seconds, flush=flush)
            out.update(ours_ms=ms, ours_tflops=fl / ms / 1e9)
        if a.only != "ours":
            q, k, v = [t.view(a.batch, a.seq, a.heads, a.hd).transpose(1, 2) for t in qkv.split(d, -1)]
            ms = time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True),
                         a.iters, seconds=a.seconds, flush=flush)
            out.update(lib_ms=ms, lib_tflops=fl / ms / 1e9)
    elif a.kernel == "sweep":
        n = a.mib * (1 << 20) // 2
        per = 1 << 24
        pieces = [Piece(f"t{i}", (min(per, n - i * per),), tensor_id=i, group=0) for i in range((n + per - 1) // per)]
        ar = ParamArena(pieces, dev)
        ar.data.normal_(0, 0.02, generator=g)
        fl = set(x for x in a.flags.split(",") if x)
        kw = dict(seed1=1, c1=1e-3)
        if "z2" in fl:
            kw.update(seed2=2, c2=1e-3)
        if "blend" in fl or "norm" in fl:
            ar.set_dizo([p.name for p in pieces])
        if "blend" in fl:
            kw.update(alpha=torch.ones(ar.n_slots, device=dev))
        if "norm" in fl:
            kw.update(sq_out=torch.zeros(ar.n_slots, device=dev))
        if "sr" in fl:
            kw.update(stochastic_round_seed=5)
        if "dual" in fl:
            # the two-sided staging sweep: theta + c z and theta - c z from one draw of z (2 B read, 4 B written)
            kw.update(dst=torch.empty(ar.data.numel(), dtype=torch.bfloat16, device=dev),
                      dst2=torch.empty(ar.data.numel(), dtype=torch.bfloat16, device=dev))
        nbytes = 4.0 * n * (1.5 if ("blend" in fl or "norm" in fl or "dual" in fl) else 1.0)
        ms = time_fn(lambda: ar.sweep(**kw), a.iters, seconds=a.seconds, flush=flush)
        out.update(elements=n, flags=sorted(fl), ours_ms=ms, ours_gbs=nbytes / ms / 1e6,
                   ours_frac_of_measured=nbytes / ms / 1e6 / peaks["hbm_gbs"])
        if a.only != "ours":
            # the reference pattern: materialised z + three elementwise passes, per tensor
            def ref():
                for p in pieces:
                    t = ar.view(p.name)
                    z = torch.normal(0, 1, size=t.shape, device=dev, dtype=t.dtype)
                    t.data = t.data + 1.0 * z * 1e-3
            ms = time_fn(ref, max(3, a.iters // 4), seconds=a.seconds, flush=flush)
            out.update(lib_ms=ms, lib_effective_gbs=nbytes / ms / 1e6)
    else:
        x = torch.randn(a.rows, a.d, device=dev, generator=g).bfloat16()
        w = torch.randn(a.d, device=dev, generator=g).bfloat16()
        b = torch.randn(a.d, device=dev, generator=g).bfloat16()
        y = torch.empty_like(x)
        nbytes = 4.0 * a.rows * a.d
        if a.flags == "rms":
            # RMSNorm of the LLaMA block (same traffic: one read, one write)
            from . import llama as llama_ops
            ms = time_fn(lambda: llama_ops.rmsnorm(x, w, 1e-5), a.iters, seconds=a.seconds, flush=flush)
            out.update(kernel="rmsnorm", shape=[a.rows, a.d], ours_ms=ms, ours_gbs=nbytes / ms / 1e6,
                       ours_frac_of_measured=nbytes / ms / 1e6 / peaks["hbm_gbs"])
            print(json.dumps(out))
            return
        ms = time_fn(lambda: layernorm(x, w, b, out=y), a.iters, seconds=a.seconds, flush=flush)
        out.update(shape=[a.rows, a.d], ours_ms=ms, ours_gbs=nbytes / ms / 1e6,
                   ours_frac_of_measured=nbytes / ms / 1e6 / peaks["hbm_gbs"])
        if a.only != "ours":
            ms = time_fn(lambda: torch.nn.functional.layer_norm(x, (a.d,), w, b), a.iters, seconds=a.seconds,
                         flush=flush)
            out.update(lib_ms=ms, lib_gbs=nbytes / ms / 1e6)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    out["peaks"] = {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") if k in peaks}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
