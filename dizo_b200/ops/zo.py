"""Flat parameter arena and the zeroth-order sweeps over it.

All tensors that ZO optimises live in one flat buffer (``ParamArena.data``); a table of
pieces (name, offset, numel, RNG stream id, DiZO slot, position inside the full tensor when
the piece is a shard) lets ONE kernel launch perturb, restore, update, project or measure any
contiguous range of it.  On CUDA the sweeps run ``csrc/zo_kernels.cu`` (z regenerated from
Philox counters in registers, never stored); on CPU the same arithmetic runs in PyTorch with
z from :mod:`dizo_b200.ops.philox`, which is what the tests compare the kernels against.

Reference semantics covered: ``zo_perturb_parameters`` (large_models/trainer.py:1429-1444),
``zo_update`` (:1597-1608), the DiZO norms (:581-584), ``apply_constraints`` (:405-436; the
``reverse_constraints`` pass :439-451 has no counterpart because theta is never overwritten
during the gamma search) and the scalar gamma arithmetic (:545-562, :586-612).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib, philox

CHUNK = 256


@dataclass
class Piece:
    name: str
    shape: tuple
    tensor_id: int
    group: int = 0                 # pieces of one group are contiguous (group = layer, -1 = globals)
    offset: int = 0
    slot: int = -1
    anchor_offset: int = 0
    elem_base: int = 0
    local_cols: int = 0
    full_cols: int = 0
    col0: int = 0
    sq_base: int = -1

    @property
    def numel(self) -> int:
        return int(math.prod(self.shape))


_tables: dict = {}


def gauss_table_dev(device) -> torch.Tensor:
    """The 1024 (a', b) pairs of the inverse-CDF table (int32 bit patterns) on ``device`` (uploaded once per
    device)."""
    dev = torch.device(device)
    key = (dev.type, dev.index)
    t = _tables.get(key)
    if t is None:
        t = torch.from_numpy(philox.gauss_table_entries().view(np.int32).copy()).to(dev)
        _tables[key] = t
    return t


def sr_seed_for(seed: int) -> int:
    """Seed of the stochastic-rounding stream that goes with perturbation seed ``seed`` (the sweep kernel
    derives the same value on the device when it reads the seed from memory)."""
    return (seed * 0x9E3779B97F4A7C15 + 1) & (2 ** 64 - 1)


def fd_eps(eps: float, dtype) -> float:
    """The perturbation scale a forward actually sees: bf16 arenas perturb with the coefficient rounded
    to bf16 (packed ``fma.rn.bf16x2``), so the finite difference divides by that value."""
    if dtype == torch.bfloat16:
        return float(torch.tensor(eps, dtype=torch.float32).to(torch.bfloat16).float())
    return float(eps)


def perturb_reference(theta: torch.Tensor, coef: float, z: torch.Tensor) -> torch.Tensor:
    """Host statement of the packed perturbation: bf16(theta + bf16(coef) * z), rounded once.  ``theta`` is
    bf16, ``z`` holds the stream's (bf16-representable) values; returns bf16 on ``theta``'s device."""
    bits = theta.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    ob = philox.perturb_bf16(bits.reshape(-1), coef, z.detach().cpu().numpy().reshape(-1))
    return torch.from_numpy(ob.view(np.int16).copy()).view(torch.bfloat16).view(theta.shape).to(theta.device)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class ParamArena:
    """One flat buffer + piece table.  ``pieces`` must already be ordered by group."""

    def __init__(self, pieces: list[Piece], device, dtype=torch.bfloat16):
        self.device = torch.device(device)
        self.dtype = dtype
        self.pieces = pieces
        off = 0
        for p in pieces:
            p.offset = off
            off += _round_up(p.numel, CHUNK)
        self.total = off
        self.data = torch.zeros(max(self.total, CHUNK), dtype=dtype, device=self.device)
        self.index = {p.name: i for i, p in enumerate(pieces)}
        self.anchor: torch.Tensor | None = None
        self.n_slots = 0
        self.slot_names: list[str] = []
        self._table_dev: torch.Tensor | None = None
        self._chunk_sq: torch.Tensor | None = None
        self._groups: dict[int, tuple[int, int]] = {}
        for i, p in enumerate(pieces):
            lo, hi = self._groups.get(p.group, (i, i))
            self._groups[p.group] = (min(lo, i), max(hi, i + 1))
        for g, (lo, hi) in self._groups.items():
            assert all(self.pieces[i].group == g for i in range(lo, hi)), "groups must be contiguous"

    # ------------------------------------------------------------------ views
    def view(self, name: str, base: torch.Tensor | None = None, shift: int = 0) -> torch.Tensor:
        p = self.pieces[self.index[name]]
        buf = self.data if base is None else base
        return buf[p.offset - shift: p.offset - shift + p.numel].view(p.shape)

    def views(self) -> dict[str, torch.Tensor]:
        return {p.name: self.view(p.name) for p in self.pieces}

    def group_range(self, group: int) -> tuple[int, int]:
        return self._groups[group]

    def groups(self) -> list[int]:
        return sorted(self._groups)

    def span(self, t_begin: int, t_end: int) -> tuple[int, int]:
        """Element range [begin, end) of pieces [t_begin, t_end) (end is chunk aligned)."""
        a = self.pieces[t_begin].offset
        last = self.pieces[t_end - 1]
        return a, last.offset + _round_up(last.numel, CHUNK)

    def group_numel(self, group: int) -> int:
        lo, hi = self._groups[group]
        a, b = self.span(lo, hi)
        return b - a

    def trainable_numel(self) -> int:
        return sum(p.numel for p in self.pieces)

    # ------------------------------------------------------------------ DiZO anchors
    def set_dizo(self, names: list[str]) -> None:
        """Give every named piece a constraint slot and snapshot it as the anchor theta_0."""
        off = 0
        sq = 0
        self.slot_names = []
        for p in self.pieces:
            p.slot = -1
            p.sq_base = -1
        for n in names:
            p = self.pieces[self.index[n]]
            p.slot = len(self.slot_names)
            p.anchor_offset = off
            p.sq_base = sq
            off += _round_up(p.numel, 8)
            sq += _round_up(p.numel, CHUNK) // CHUNK
            self.slot_names.append(n)
        self._n_sq_chunks = sq
        self._chunk_sq = None
        self.n_slots = len(self.slot_names)
        self.anchor = torch.zeros(max(off, 8), dtype=self.dtype, device=self.device)
        self.snapshot_anchor()
        self._table_dev = None

    def snapshot_anchor(self) -> None:
        for n in self.slot_names:
            p = self.pieces[self.index[n]]
            self.anchor[p.anchor_offset:p.anchor_offset + p.numel].copy_(
                self.data[p.offset:p.offset + p.numel])

    def anchor_view(self, name: str) -> torch.Tensor:
        p = self.pieces[self.index[name]]
        assert p.slot >= 0
        return self.anchor[p.anchor_offset:p.anchor_offset + p.numel].view(p.shape)

    # ------------------------------------------------------------------ device table
    def table(self) -> torch.Tensor:
        if self._table_dev is None:
            dt = np.dtype([("offset", "<i8"), ("numel", "<i8"), ("anchor_offset", "<i8"),
                           ("tensor_id", "<i4"), ("slot", "<i4"), ("elem_base", "<i8"),
                           ("local_cols", "<i8"), ("full_cols", "<i8"), ("col0", "<i8"),
                           ("sq_base", "<i8")])
            arr = np.zeros(len(self.pieces), dtype=dt)
            for i, p in enumerate(self.pieces):
                arr[i] = (p.offset, p.numel, p.anchor_offset, p.tensor_id, p.slot, p.elem_base,
                          p.local_cols, p.full_cols, p.col0, p.sq_base)
            if self.device.type == "cuda":
                assert dt.itemsize == _lib.lib().dz_zo_tensor_struct_bytes()
            raw = torch.from_numpy(arr.view(np.uint8).copy())
            self._table_dev = raw.to(self.device)
        return self._table_dev

    # ------------------------------------------------------------------ z (oracle access)
    def z_for(self, name: str, seed: int) -> torch.Tensor:
        """The perturbation direction of one piece (fp32, on the arena's device)."""
        p = self.pieces[self.index[name]]
        if p.local_cols:
            rows = p.numel // p.local_cols
            z = philox.gaussian_cols(seed, p.tensor_id, rows, p.local_cols, p.full_cols, p.col0,
                                     p.elem_base)
        else:
            z = philox.gaussian(seed, p.tensor_id, p.numel, p.elem_base)
        return torch.from_numpy(z).view(p.shape).to(self.device)

    # ------------------------------------------------------------------ the sweep
    def sweep(self, *, t_begin: int = 0, t_end: int | None = None, dst: torch.Tensor | None = None,
              seed1: int = 0, c1: float = 0.0, c1_dev: torch.Tensor | None = None,
              seed1_dev: torch.Tensor | None = None, seed2: int = 0, c2: float = 0.0, c2_dev: torch.Tensor | None = None,
              alpha: torch.Tensor | None = None, sq_out: torch.Tensor | None = None,
              stochastic_round_seed: int | None = None, small: bool = False,
              dst2: torch.Tensor | None = None) -> None:
        """dst[range] = round(blend(theta) + c1*z(seed1) + c2*z(seed2)); optional norms.

        ``dst2`` (plain perturbation into staging buffers only): a second buffer that receives
        ``theta - c1*z(seed1)`` from the same draw of z - the two forwards of the two-point estimate read the
        two buffers, and z is generated once instead of twice.

        ``dst=None`` writes the arena in place; otherwise ``dst`` is a staging buffer whose
        element 0 corresponds to the first element of the range.  ``c?_dev`` (1-element fp32
        tensors) multiply the host coefficients on the device; ``seed1_dev`` (1-element int64 tensor)
        replaces ``seed1`` by a value read on the device (CUDA-graph replays).  ``alpha`` ([n_slots] fp32)
        switches on the blend ``theta_0 + alpha*(theta - theta_0)`` for slotted pieces;
        ``sq_out`` ([n_slots] fp32) receives ``||stored - theta_0||^2`` per slotted piece of
        the range.  With ``seed1_dev`` a given ``stochastic_round_seed`` only switches stochastic rounding
        on: the stream's seed is then :func:`sr_seed_for` of the device seed.  ``small`` picks the kernel variant
        with a 4 KB table and a bounded register count that fits on an SM beside a GEMM CTA (for sweeps issued
        on a side stream; plain perturbation or blend only)."""
        t_end = len(self.pieces) if t_end is None else t_end
        if t_end <= t_begin:
            return
        begin, end = self.span(t_begin, t_end)
        shift = 0 if dst is None else begin
        out = self.data if dst is None else dst
        if dst is not None:
            assert dst.numel() >= end - begin and dst.dtype == self.dtype
        use_z2 = (c2 != 0.0) or (c2_dev is not None)
        blend = alpha is not None
        norm = sq_out is not None
        if dst2 is not None:
            assert dst is not None and dst2.numel() >= end - begin and dst2.dtype == self.dtype
            assert not (use_z2 or blend or norm or stochastic_round_seed is not None), \
                "the two-sided sweep is the plain perturbation"
        if (blend or norm) and self.anchor is None:
            raise ValueError("blend/norm need set_dizo() first")
        if self.device.type != "cuda":
            if seed1_dev is not None:
                seed1 = int(seed1_dev.item()) & (2 ** 64 - 1)
                if stochastic_round_seed is not None:
                    stochastic_round_seed = sr_seed_for(seed1)
            self._sweep_cpu(t_begin, t_end, out, shift, seed1, c1, c1_dev, seed2, c2, c2_dev,
                            use_z2, alpha, sq_out, stochastic_round_seed)
            if dst2 is not None:
                self._sweep_cpu(t_begin, t_end, dst2, shift, seed1, -c1, c1_dev, seed2, c2, c2_dev,
                                use_z2, alpha, sq_out, stochastic_round_seed)
            return
        assert self.dtype == torch.bfloat16, "the CUDA sweep is bf16"
        L = _lib.lib()
        flags = (1 if use_z2 else 0) | (2 if blend else 0) | (4 if norm else 0) | \
                (8 if stochastic_round_seed is not None else 0)
        if small and not (use_z2 or norm or stochastic_round_seed is not None):
            flags |= 16
        if norm and self._chunk_sq is None:
            self._chunk_sq = torch.zeros(max(self._n_sq_chunks, 1), dtype=torch.float32,
                                         device=self.device)
        if seed1_dev is not None:
            assert seed1_dev.dtype == torch.int64 and seed1_dev.is_cuda and seed1_dev.numel() == 1
        if dst2 is not None:
            rc = L.dz_zo_sweep_dual(
                _lib.ptr(self.data), _lib.ptr(out), _lib.ptr(dst2), ctypes.c_longlong(shift),
                _lib.ptr(self.table()), t_begin, t_end, ctypes.c_longlong(begin // CHUNK),
                ctypes.c_longlong(end // CHUNK), ctypes.c_uint64(seed1 & (2 ** 64 - 1)), _lib.ptr(seed1_dev),
                ctypes.c_float(c1), _lib.ptr(c1_dev), int(bool(small)), _lib.ptr(gauss_table_dev(self.device)),
                _lib.stream_ptr())
            _lib.check(rc, "dz_zo_sweep_dual")
            return
        rc = L.dz_zo_sweep_seeded(
            _lib.ptr(self.data), _lib.ptr(out), ctypes.c_longlong(shift), _lib.ptr(self.anchor),
            _lib.ptr(self.table()), t_begin, t_end, ctypes.c_longlong(begin // CHUNK),
            ctypes.c_longlong(end // CHUNK), ctypes.c_uint64(seed1 & (2 ** 64 - 1)), _lib.ptr(seed1_dev),
            ctypes.c_float(c1), _lib.ptr(c1_dev), ctypes.c_uint64(seed2 & (2 ** 64 - 1)),
            ctypes.c_float(c2 if use_z2 else 0.0), _lib.ptr(c2_dev), _lib.ptr(alpha),
            _lib.ptr(self._chunk_sq), ctypes.c_uint64((stochastic_round_seed or 0) & (2 ** 64 - 1)),
            flags, _lib.ptr(gauss_table_dev(self.device)), _lib.stream_ptr())
        _lib.check(rc, "dz_zo_sweep_seeded")
        if norm:
            rc = L.dz_zo_reduce_chunks(
                ctypes.c_void_p(self.table().data_ptr() + t_begin * self.table_stride()),
                t_end - t_begin, _lib.ptr(self._chunk_sq), _lib.ptr(sq_out), _lib.stream_ptr())
            _lib.check(rc, "dz_zo_reduce_chunks")

    def table_stride(self) -> int:
        return self.table().numel() // len(self.pieces)

    def _sweep_cpu(self, t_begin, t_end, out, shift, seed1, c1, c1_dev, seed2, c2, c2_dev, use_z2,
                   alpha, sq_out, sr_seed):
        c1v = c1 * (float(c1_dev.item()) if c1_dev is not None else 1.0)
        c2v = c2 * (float(c2_dev.item()) if c2_dev is not None else 1.0)
        for i in range(t_begin, t_end):
            p = self.pieces[i]
            src = self.data[p.offset:p.offset + p.numel]
            v = src.float()
            slotted = p.slot >= 0 and self.anchor is not None
            an = None
            if slotted and (alpha is not None or sq_out is not None):
                an = self.anchor[p.anchor_offset:p.anchor_offset + p.numel].float()
            if alpha is not None and slotted:
                v = an + float(alpha[p.slot]) * (v - an)
            packed = (self.dtype == torch.bfloat16 and not use_z2 and alpha is None and sq_out is None
                      and sr_seed is None)
            if packed:
                # the forward-pass perturbation: bf16 coefficient, exact fma, one rounding
                if c1v != 0.0:
                    stored = perturb_reference(src, c1v, self.z_for(p.name, seed1).reshape(-1))
                else:
                    stored = src
                out[p.offset - shift:p.offset - shift + p.numel].copy_(stored)
                continue
            if c1v != 0.0:
                v = v + c1v * self.z_for(p.name, seed1).reshape(-1).to(v.device)
            if use_z2:
                v = v + c2v * self.z_for(p.name, seed2).reshape(-1).to(v.device)
            if sr_seed is not None and self.dtype == torch.bfloat16:
                stored = _stochastic_round_bf16(v, sr_seed, p)
            else:
                stored = v.to(self.dtype)
            out[p.offset - shift:p.offset - shift + p.numel].copy_(stored)
            if sq_out is not None and slotted:
                sq_out[p.slot] = ((stored.float() - an) ** 2).sum()


def _stochastic_round_bf16(v: torch.Tensor, seed: int, p: Piece) -> torch.Tensor:
    """CPU statement of the kernel's stochastic rounding (same Philox stream 1)."""
    n = v.numel()
    ngroups = (n + 7) // 8
    g0 = p.elem_base >> 3
    grp = (np.arange(g0, g0 + ngroups, dtype=np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    c = philox.philox4x32(grp, np.uint32(p.tensor_id), np.uint32(1), np.uint32(0),
                          seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, rounds=philox.Z_PHILOX_ROUNDS)
    words = np.stack(c, axis=-1)                      # [groups, 4]
    lo = (words & np.uint32(0xFFFF)).astype(np.uint32)
    hi = (words >> np.uint32(16)).astype(np.uint32)
    r16 = np.stack([lo, hi], axis=-1).reshape(-1)[:n]  # element 2j -> low half of word j
    bits = v.detach().cpu().numpy().astype(np.float32).view(np.uint32)
    with np.errstate(over="ignore"):
        bits = (bits + r16) & np.uint32(0xFFFF0000)
    return torch.from_numpy(bits.view(np.float32).copy()).to(torch.bfloat16).to(v.device)


# ---------------------------------------------------------------------- gamma search scalars
class GammaState:
    """Device-resident gamma vector of the DiZO projection and its ZO search arithmetic.

    Constants default to the reference's hard-coded values (tau 0.2, zo_eps 0.1, step size 2;
    large_models/trainer.py:590-592)."""

    def __init__(self, n: int, device, tau: float = 0.2, zo_eps: float = 0.1, step_size: float = 2.0):
        self.n = n
        self.device = torch.device(device)
        self.tau, self.zo_eps, self.step_size = tau, zo_eps, step_size
        f = dict(dtype=torch.float32, device=self.device)
        self.sq = torch.zeros(n, **f)
        self.ts = torch.zeros(n, **f)
        self.gamma = torch.zeros(n, **f)
        self.z = torch.zeros(n, **f)
        self.alpha = torch.ones(n, **f)

    def _launch(self, mode, seed=0, it=-1, delta=0.0, loss1=None, loss2=None, reinit=0):
        if self.device.type == "cuda":
            rc = _lib.lib().dz_gamma_step(
                self.n, mode, _lib.ptr(self.sq), _lib.ptr(self.ts), _lib.ptr(self.gamma),
                _lib.ptr(self.z), _lib.ptr(self.alpha), ctypes.c_uint64(seed & (2 ** 64 - 1)), it,
                ctypes.c_float(delta), ctypes.c_float(self.tau), ctypes.c_float(self.zo_eps),
                ctypes.c_float(self.step_size), _lib.ptr(loss1), _lib.ptr(loss2), reinit,
                _lib.ptr(gauss_table_dev(self.device)), _lib.stream_ptr())
            _lib.check(rc, "dz_gamma_step")
            return
        if mode == 0:
            self.ts.copy_(self.sq.sqrt())
            if reinit:
                self.gamma.copy_(self.ts)
        elif mode == 1:
            if delta == 1.0 and it >= 0:
                z = torch.tensor([philox.scalar_gaussian(seed, i, it) for i in range(self.n)],
                                 dtype=torch.float32)
                lim = (self.tau / self.zo_eps) * self.ts
                self.z.copy_(torch.minimum(torch.maximum(z, -lim), lim))
            self.gamma.add_(delta * self.zo_eps * self.z)
        elif mode == 2:
            grad = (float(loss1) - float(loss2)) / (2 * self.zo_eps)
            g = self.gamma - self.step_size * self.ts * grad * self.z
            self.gamma.copy_(torch.minimum(torch.maximum(g, (1 - self.tau) * self.ts),
                                           (1 + self.tau) * self.ts))
        self.alpha.copy_(self.gamma / (self.ts + 1e-8))

    def begin(self, reinit: bool = True) -> None:
        """ts = sqrt(sq); gamma = ts when ``reinit``; alpha refreshed."""
        self._launch(0, reinit=int(reinit))

    def perturb(self, delta: float, seed: int = 0, it: int = -1) -> None:
        """gamma += delta*eps*z; a fresh clipped z is drawn when delta == +1 and it >= 0."""
        self._launch(1, seed=seed, it=it, delta=delta)

    def step(self, loss1: torch.Tensor, loss2: torch.Tensor) -> None:
        self._launch(2, loss1=loss1, loss2=loss2)


def scalar_diff(a: torch.Tensor, b: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
    """out = (a - b) * scale on the device (the projected gradient (L+ - L-) / (2 eps))."""
    if a.is_cuda:
        rc = _lib.lib().dz_scalar_diff(_lib.ptr(a), _lib.ptr(b), ctypes.c_float(scale), _lib.ptr(out),
                                       _lib.stream_ptr())
        _lib.check(rc, "dz_scalar_diff")
    else:
        out.copy_((a.float() - b.float()).reshape(out.shape) * scale)
    return out


def fill_z(numel: int, seed: int, tensor_id: int, device, elem_base: int = 0) -> torch.Tensor:
    """Materialise z (fp32) - for tests and diagnostics only; training never stores z."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return torch.from_numpy(philox.gaussian(seed, tensor_id, numel, elem_base))
    out = torch.empty(numel, dtype=torch.float32, device=dev)
    rc = _lib.lib().dz_zo_fill_z(_lib.ptr(out), ctypes.c_longlong(numel), ctypes.c_longlong(elem_base),
                                 ctypes.c_uint64(seed & (2 ** 64 - 1)), tensor_id,
                                 _lib.ptr(gauss_table_dev(dev)), _lib.stream_ptr())
    _lib.check(rc, "dz_zo_fill_z")
    return out
