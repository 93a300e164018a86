"""Fused compute + collective operations over NVLink peer memory (Python side).

Each operation is ONE launch of ``csrc/comm_gemm.cu`` (tcgen05 GEMM tiles and the peer-memory
transfer in the same kernel) or ``csrc/comm_kernels.cu``:

* :meth:`FusedComm.ag_gemm` - tensor-parallel all-gather -> GEMM.  Activations are sharded by
  rows (sequence parallel).  The producer of the activation writes this rank's rows straight
  into the symmetric ``x_full`` buffer; the kernel's push CTAs store them into every peer's
  ``x_full`` while its GEMM CTAs work own-rows-first and poll the per-source ready flags
  before touching rows that come from a peer.
* :meth:`FusedComm.gemm_rs` + :meth:`FusedComm.rs_reduce_layernorm` - GEMM -> reduce-scatter.
  The GEMM epilogue stores every tile into the slot of the rank that owns those rows; the
  owner's next kernel sums the slots in rank order (deterministic), adds bias and residual and
  applies the following LayerNorm.
* :meth:`FusedComm.fsdp_launch` - FSDP: the row shard of a weight owned by this rank is
  perturbed (theta + c z, z regenerated from the shared seed for the shard's global element
  indices) while it is pushed into every rank's staging weight, in the same launch as a GEMM
  (the one that consumes this weight, or the previous one when prefetching).
* :meth:`FusedComm.norm_allreduce_gamma` - sum over shards of the per-tensor squared distances
  fused with the gamma / alpha arithmetic of the DiZO projection.

Buffer reuse is protected by acks: a pusher waits until every peer has reported consuming the
buffer's previous content.  All device-side waits are bounded; a missing peer surfaces as a
``KernelError`` from :func:`dizo_b200.ops._lib.check_device_errors`, not as a hang.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import ACT
from ..ops.zo import gauss_table_dev
from .symm import SymmRegion

c_ll, c_int, c_uint, c_float, c_void = (ctypes.c_longlong, ctypes.c_int, ctypes.c_uint, ctypes.c_float,
                                         ctypes.c_void_p)


class _Desc(ctypes.Structure):
    _fields_ = [
        ("A", c_void), ("lda", c_ll), ("W", c_void), ("ldw", c_ll),
        ("out", c_void), ("ldo", c_ll), ("bias", c_void), ("residual", c_void), ("ldr", c_ll),
        ("M", c_int), ("N", c_int), ("K", c_int), ("act", c_int), ("out_fp32", c_int), ("out_scale", c_float),
        ("gather", c_int), ("rows_per_src", c_int), ("src_period", c_int), ("wait_self", c_int),
        ("ready_flags", c_void),
        ("ready_epoch", c_uint), ("ack_ptrs", c_void), ("ack_epoch", c_uint),
        ("push_out", c_int), ("out_ptrs", c_void), ("out_slot_stride", c_ll), ("rows_per_owner", c_int),
        ("rs_flag_ptrs", c_void), ("rs_epoch", c_uint),
        ("n_push", c_int), ("push_nseg", c_int), ("push_src", c_void * 3), ("push_ld", c_ll),
        ("push_rows", c_ll), ("push_cols", c_ll),
        ("push_dst_ptrs", c_void), ("push_dst_ld", c_ll), ("push_dst_row0", c_ll * 3), ("push_to_self", c_int),
        ("push_flag_ptrs", c_void), ("push_epoch", c_uint), ("push_wait_acks", c_void),
        ("push_wait_epoch", c_uint),
        ("push_perturb", c_int), ("push_seed", ctypes.c_ulonglong), ("push_coef", c_float),
        ("push_tensor_id", c_int * 3), ("push_elem_base", c_ll * 3), ("gauss_table", c_void),
        ("rank", c_int), ("world", c_int), ("counters", c_void), ("push_target", c_uint),
        ("gemm_target", c_uint), ("two_sm", c_int), ("chunk_rows", c_int), ("join_tiles", c_int),
    ]


_SM_COUNT = 148       # B200
MAX_CHUNKS = 16      # progress chunks per source (CG_MAXC of comm_gemm.cu)


class _Channel:
    """A staging buffer with its ready / ack flag words and epoch counters."""

    def __init__(self, region: SymmRegion, nbytes: int):
        self.region = region
        self.off, self.view, self.ptrs = region.alloc(nbytes)
        _, rv, self.ready_ptrs = region.alloc(4 * region.world * MAX_CHUNKS)
        _, av, self.ack_ptrs = region.alloc(4 * region.world)
        self.ready = rv.view(torch.int32)
        self.ack = av.view(torch.int32)
        self.epoch = 0          # pushes issued into this buffer
        self.ack_epoch = 0      # consumptions of this buffer announced to the peers
        self.nbytes = nbytes


class FusedComm:
    def __init__(self, group=None, device=None, ag_bytes: int = 0, rs_bytes: int = 0, w_bytes: int = 0,
                 n_push: int = 16, norm_slots: int = 256):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        total = 2 * ag_bytes + 2 * rs_bytes + 2 * w_bytes + 64 * 1024 + 8 * norm_slots * (self.world + 1)
        self.region = SymmRegion(total + 16 * 4096, self.group, device)
        self.device = self.region.device
        self.two_sm = True            # use the two-SM (256 x 256 tile) kernel where the shape allows it
        self.push_ctas = 0            # pushing CTAs per launch; 0 = by the number of ranks (see _push_plan)
        self.push_share = 0.0         # their share of a normal CTA's output tiles (0 = they only push)
        self.ag = [_Channel(self.region, ag_bytes) for _ in range(2)] if ag_bytes else []
        self.rs = [_Channel(self.region, rs_bytes) for _ in range(2)] if rs_bytes else []
        self.wst = [_Channel(self.region, w_bytes) for _ in range(2)] if w_bytes else []
        # barrier + norm all-reduce areas
        _, bv, self.bar_ptrs = self.region.alloc(4 * self.world)
        self.bar_epoch = 0
        self.norm_slots = norm_slots
        self.norm_off, nv, self.norm_slot_ptrs = self.region.alloc(4 * norm_slots * self.world)
        self.norm_mc_off, mv, _ = self.region.alloc(4 * norm_slots)
        self.norm_mc_local = mv.view(torch.float32)
        _, fv, self.norm_flag_ptrs = self.region.alloc(4 * self.world)
        self.norm_epoch = 0
        self.counters = torch.zeros(2 + MAX_CHUNKS, dtype=torch.int32, device=self.device)
        self._push_total = 0
        self._gemm_total = 0
        self._calls = {"ag": 0, "rs": 0, "w": 0}
        self._dbg_out = None

    # ------------------------------------------------------------------ helpers
    # what one pushing CTA moves (measured: 8.3 GB/s per CTA with 4 ranks, 13.7 GB/s with 8) and what the tile
    # kernels sustain; both only rank the alternatives of _push_plan
    _PUSH_GBS_PER_CTA = 10.0
    _GEMM_TFLOPS = 1300.0

    def _push_plan(self, d: _Desc, M: int, N: int, consumer_waits: bool, two: int = 0) -> tuple[int, int]:
        """(CTAs that push, ``join_tiles``: tiles left to them; -1 = none, 0 = a full share).

        Measured policy.  Two ranks: every CTA pushes (one destination, half of the bytes stay local; the
        transfer rides along at no visible cost).  More ranks: posted stores from all 148 SMs to seven
        destinations slowed every GEMM tile (8 GPUs: all-gather -> GEMM 0.61 -> 0.71 ms, FSDP 4.45 -> 5.49 ms
        at OPT-66B shapes), so sixteen CTAs only push - as long as sixteen can move the launch's bytes within the
        time of its GEMM.  A launch whose push outweighs its GEMM (the out_proj GEMM beside the fc1 shard push of
        an FSDP block; all-gather -> GEMM at OPT-13B width) is bound by the transfer: with up to four ranks every
        CTA then pushes again (4 GPUs, OPT-13B all-gather -> GEMM: 0.47 ms with sixteen pushers, 0.36 ms with all,
        0.40 ms NCCL + GEMM); with more ranks the number of pushing-only CTAs is the one that balances the
        transfer against the GEMM on the remaining SMs.  ``push_ctas`` / ``push_share`` override the choice."""
        L = _lib.lib()
        if M <= 0:
            return min(_SM_COUNT, 96), 0                                    # push only
        grid0 = L.dz_comm_gemm_grid(M, N, 0, two)
        if self.push_ctas > 0:
            n = self.push_ctas
        elif self.world <= 2:
            n = grid0
        else:
            nbytes = 2.0 * max(int(d.push_nseg), 1) * int(d.push_rows) * int(d.push_cols) * (self.world - 1)
            t_gemm = 2.0 * M * N * int(d.K) / (self._GEMM_TFLOPS * 1e12)
            rate = self._PUSH_GBS_PER_CTA * 1e9
            if nbytes <= 16 * rate * t_gemm:
                n = 16
            elif self.world <= 4:
                n = grid0
            else:
                cost = lambda k: max(nbytes / (k * rate), t_gemm * _SM_COUNT / (_SM_COUNT - k))
                n = min(range(16, 66, 8), key=cost)
        n = max(1, min(n, _SM_COUNT))
        if two:
            n = min((n + 1) & ~1, _SM_COUNT & ~1)      # CTA pairs push together
        if n >= grid0:
            return n, 0
        tiles = L.dz_comm_gemm_tiles(M, N, two)
        units, push_units = (grid0 // 2, n // 2) if two else (grid0, n)     # CTAs or CTA pairs that take tiles
        f = self.push_share
        if f <= 0.0:
            return n, -1
        g = units - push_units
        if f >= 1.0 or tiles <= units:
            return n, 0
        return n, max(1, min(int(tiles * push_units * f / (g + push_units * f)), tiles - 1))

    def _launch(self, d: _Desc, push: bool, M: int, N: int, consumer_waits: bool = True) -> None:
        L = _lib.lib()
        assert ctypes.sizeof(_Desc) == L.dz_comm_gemm_desc_bytes(), "launch descriptor out of step with the library"
        d.rank, d.world = self.rank, self.world
        d.counters = self.counters.data_ptr()
        # the first n_push CTAs carry a slice of the push (four extra warps beside their GEMM warps); every CTA
        # of any launch reports its completion: the counters advance by the pushing CTAs / the grid size
        two = int(self.two_sm and M > 0 and
                  L.dz_comm_gemm_two_sm(M, N, d.gather, d.rows_per_src, d.chunk_rows))
        n_push, join = self._push_plan(d, M, N, consumer_waits, two) if push else (0, 0)
        grid = L.dz_comm_gemm_grid(M, N, n_push, two)
        d.n_push, d.join_tiles, d.two_sm = n_push, join, two
        if push:
            self._push_total += n_push
            d.push_target = self._push_total & 0xFFFFFFFF
        self._gemm_total += grid
        d.gemm_target = self._gemm_total & 0xFFFFFFFF
        if _lib.DEBUG_BOUNDS and self._dbg_out is not None:
            _lib.note(self._dbg_out)              # the local output of this launch
            self._dbg_out = None
        rc = L.dz_comm_gemm(ctypes.byref(d), _lib.ptr(_lib.err_word(self.device)), _lib.stream_ptr())
        _lib.check(rc, "dz_comm_gemm")

    def barrier(self) -> None:
        """All ranks have reached this point of their current streams (P2P flags, bounded wait)."""
        self.bar_epoch += 1
        rc = _lib.lib().dz_peer_barrier(_lib.ptr(self.bar_ptrs), self.rank, self.world,
                                        ctypes.c_uint(self.bar_epoch), _lib.ptr(_lib.err_word(self.device)),
                                        _lib.stream_ptr())
        _lib.check(rc, "dz_peer_barrier")

    # ------------------------------------------------------------------ TP: all-gather -> GEMM
    def ag_input(self, M: int, K: int):
        """(x_full [M, K] symmetric bf16, this rank's row slice to write the local shard into)."""
        ch = self.ag[self._calls["ag"] % 2]
        assert M * K * 2 <= ch.nbytes and M % self.world == 0
        x_full = ch.view[:M * K * 2].view(torch.bfloat16).view(M, K)
        rows = M // self.world
        return x_full, x_full[self.rank * rows:(self.rank + 1) * rows]

    def ag_gemm(self, x_full: torch.Tensor, w: torch.Tensor, bias=None, act=None,
                out: torch.Tensor | None = None) -> torch.Tensor:
        """out[M, N_local] = act(gather_rows(x) @ w.T + bias); the local rows of ``x_full`` must
        already hold this rank's shard (see :meth:`ag_input`)."""
        ch = self.ag[self._calls["ag"] % 2]
        self._calls["ag"] += 1
        M, K = x_full.shape
        N = w.shape[0]
        rows = M // self.world
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        prev = ch.epoch
        ch.epoch += 1
        d = _Desc()
        d.A, d.lda, d.W, d.ldw = x_full.data_ptr(), x_full.stride(0), w.data_ptr(), w.stride(0)
        d.out, d.ldo = out.data_ptr(), out.stride(0)
        self._dbg_out = out
        d.bias = bias.data_ptr() if bias is not None else None
        d.M, d.N, d.K, d.act, d.out_scale = M, N, K, ACT[act], 1.0
        d.gather, d.rows_per_src, d.wait_self = 1, rows, 0
        d.ready_flags, d.ready_epoch = ch.ready.data_ptr(), ch.epoch
        d.ack_ptrs, d.ack_epoch = ch.ack_ptrs.data_ptr(), ch.epoch
        d.push_nseg = 1
        d.push_src[0], d.push_ld = x_full[self.rank * rows:].data_ptr(), x_full.stride(0)
        d.push_rows, d.push_cols = rows, K
        d.push_dst_ptrs, d.push_dst_ld, d.push_to_self = ch.ptrs.data_ptr(), x_full.stride(0), 0
        d.push_dst_row0[0] = self.rank * rows
        d.push_flag_ptrs, d.push_epoch = ch.ready_ptrs.data_ptr(), ch.epoch
        d.push_wait_acks, d.push_wait_epoch = ch.ack.data_ptr(), prev
        # progress chunks: whole row tiles (256 rows where the two-SM kernel can run, else 128), as fine as
        # the flag words allow
        unit = 256 if (self.two_sm and rows % 256 == 0) else 128
        tiles = rows // unit
        ct = next(c for c in range(1, tiles + 1) if tiles % c == 0 and tiles // c <= MAX_CHUNKS)
        d.chunk_rows = ct * unit if self.world > 2 and tiles > 1 else 0
        self._launch(d, True, M, N)
        return out

    # ------------------------------------------------------------------ TP: GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor) -> int:
        """Partial products a @ w.T (K sharded) go to the owners' slots; returns the channel
        index to pass to :meth:`rs_reduce_layernorm`."""
        idx = self._calls["rs"] % 2
        ch = self.rs[idx]
        self._calls["rs"] += 1
        M, K = a.shape
        N = w.shape[0]
        rows = M // self.world
        assert self.world * rows * N * 2 <= ch.nbytes and rows % 128 == 0
        ch.epoch += 1
        d = _Desc()
        d.A, d.lda, d.W, d.ldw = a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0)
        d.ldo = N
        d.M, d.N, d.K, d.act, d.out_scale = M, N, K, 0, 1.0
        d.push_out, d.out_ptrs, d.out_slot_stride, d.rows_per_owner = 1, ch.ptrs.data_ptr(), rows * N, rows
        d.rs_flag_ptrs, d.rs_epoch = ch.ready_ptrs.data_ptr(), ch.epoch
        ch.shape = (rows, N)
        self._launch(d, False, M, N)
        return idx

    @property
    def has_multicast(self) -> bool:
        """The symmetric region is bound to an NVSwitch multicast object (multimem addresses work)."""
        return bool(self.region.multicast_ptr)

    def gemm_rs_pull(self, a: torch.Tensor, w: torch.Tensor) -> int:
        """Pull form of :meth:`gemm_rs`: the partial product a @ w.T stays in this rank's copy of the
        staging buffer (the stand-alone two-SM GEMM, no remote stores), a peer barrier follows, and
        :meth:`rs_reduce_layernorm` lets the switch add the ranks' copies (``multimem.ld_reduce``): the
        owner reads rows x N x 2 bytes once instead of receiving world - 1 partials.  Needs
        :attr:`has_multicast`.  The buffer of call k is written again by call k + 2, after the barrier of
        call k + 1, which every rank passes only once all ranks have finished reducing call k."""
        from ..ops import gemm
        assert self.has_multicast, "no NVSwitch multicast mapping on this region"
        idx = self._calls["rs"] % 2
        ch = self.rs[idx]
        self._calls["rs"] += 1
        M, N = a.shape[0], w.shape[0]
        rows = M // self.world
        assert M * N * 2 <= ch.nbytes and rows * self.world == M
        part = ch.view[:M * N * 2].view(torch.bfloat16).view(M, N)
        gemm.linear(a, w, out=part)
        self.barrier()
        ch.shape = (rows, N)
        ch.pull = True
        return idx

    def rs_reduce_layernorm(self, idx: int, residual: torch.Tensor, bias, ln_w=None, ln_b=None,
                            eps: float = 1e-5, y_out: torch.Tensor | None = None):
        """h = residual + bias + sum_r partial_r (rows this rank owns); y = LayerNorm(h) written to
        ``y_out`` (e.g. the local rows of the next all-gather buffer).  Returns (h, y)."""
        ch = self.rs[idx]
        rows, N = ch.shape
        h = torch.empty((rows, N), dtype=torch.bfloat16, device=self.device)
        y = None
        if ln_w is not None:
            y = y_out if y_out is not None else torch.empty((rows, N), dtype=torch.bfloat16, device=self.device)
        if getattr(ch, "pull", False):
            ch.pull = False
            mc = self.region.multicast_addr(ch.off) + self.rank * rows * N * 2
            rc = _lib.lib().dz_rs_pull_layernorm(
                c_void(mc), c_ll(N), _lib.ptr(residual), c_ll(residual.stride(0)), _lib.ptr(bias), _lib.ptr(ln_w),
                _lib.ptr(ln_b), _lib.ptr(h), c_ll(N), _lib.ptr(y), c_ll(y.stride(0) if y is not None else 0),
                c_ll(rows), N, c_float(eps), _lib.ptr(_lib.err_word(self.device)), _lib.stream_ptr())
            _lib.check(rc, "dz_rs_pull_layernorm")
            return h, y
        rc = _lib.lib().dz_rs_reduce_layernorm(
            _lib.ptr(ch.view), c_ll(rows * N), c_ll(N), _lib.ptr(ch.ready), ctypes.c_uint(ch.epoch), self.world,
            _lib.ptr(residual), c_ll(residual.stride(0)), _lib.ptr(bias), _lib.ptr(ln_w), _lib.ptr(ln_b),
            _lib.ptr(h), c_ll(N), _lib.ptr(y), c_ll(y.stride(0) if y is not None else 0), c_ll(rows), N,
            c_float(eps), _lib.ptr(_lib.err_word(self.device)), _lib.stream_ptr())
        _lib.check(rc, "dz_rs_reduce_layernorm")
        return h, y

    # ------------------------------------------------------------------ FSDP: gather + perturb + GEMM
    def fsdp_launch(self, push: dict | None = None, gemm: dict | None = None):
        """One launch doing either or both of

        ``push = dict(segments=[dict(w_shard=[rows, K] rows owned by this rank, dst_row0=first row
        of that shard inside the staged full weight, tensor_id=, elem_base=index of the shard's
        first element in its full tensor), ...up to 3 equal-shaped segments],
        seed=, coef=, slot=None)``: perturb the shards (theta + coef * z, z regenerated for their
        global element indices; coef 0 = plain copy) while storing them into every rank's staging
        copy of the weight (own copy included).  Uses ``slot`` or the next staging slot; returns it.

        ``gemm = dict(slot=, N=, x=[M, K], rows_per_src=, src_period=0, bias=, act=, residual=, out=)``:
        out = act(x @ W_full.T + bias) (+ residual) with W_full the staged weight in ``slot``.
        Before the first load of a tile the producer polls the ready flags of the ranks that own
        its rows, so a weight pushed in this same launch is consumed as it arrives and one pushed
        by an earlier launch (prefetch) costs no wait.

        Returns (slot pushed into or None, GEMM output or None)."""
        d = _Desc()
        slot = None
        if push is not None:
            slot = push.get("slot")
            if slot is None:
                slot = self._calls["w"] % 2
            self._calls["w"] += 1
            ch = self.wst[slot]
            segs = push["segments"]
            rows_w, K = segs[0]["w_shard"].shape
            prev_ack = ch.ack_epoch
            ch.epoch += 1
            d.push_nseg = len(segs)
            for i, sg in enumerate(segs):
                w = sg["w_shard"]
                assert w.shape == (rows_w, K) and w.stride(0) == segs[0]["w_shard"].stride(0)
                d.push_src[i] = w.data_ptr()
                d.push_dst_row0[i] = int(sg["dst_row0"])
                d.push_tensor_id[i] = int(sg.get("tensor_id", 0))
                d.push_elem_base[i] = int(sg.get("elem_base", 0))
            d.push_ld, d.push_rows, d.push_cols = segs[0]["w_shard"].stride(0), rows_w, K
            d.push_dst_ptrs, d.push_dst_ld = ch.ptrs.data_ptr(), K
            d.push_to_self = 1
            d.push_flag_ptrs, d.push_epoch = ch.ready_ptrs.data_ptr(), ch.epoch
            d.push_wait_acks, d.push_wait_epoch = ch.ack.data_ptr(), prev_ack
            coef = float(push.get("coef", 0.0))
            d.push_perturb, d.push_seed, d.push_coef = int(coef != 0.0), int(push.get("seed", 0)), coef
            d.gauss_table = gauss_table_dev(self.device).data_ptr()
        out = None
        M = Ng = 0
        if gemm is not None:
            ch = self.wst[gemm["slot"]]
            x, N = gemm["x"], gemm["N"]
            M, K = x.shape
            Ng = N
            assert N * K * 2 <= ch.nbytes, "staged weight larger than the staging slot"
            w_full = ch.view[:N * K * 2].view(torch.bfloat16).view(N, K)
            out = gemm.get("out")
            if out is None:
                out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
            d.A, d.lda, d.W, d.ldw = x.data_ptr(), x.stride(0), w_full.data_ptr(), K
            d.out, d.ldo = out.data_ptr(), out.stride(0)
            self._dbg_out = out
            bias, residual = gemm.get("bias"), gemm.get("residual")
            d.bias = bias.data_ptr() if bias is not None else None
            if residual is not None:
                d.residual, d.ldr = residual.data_ptr(), residual.stride(0)
            d.M, d.N, d.K, d.act, d.out_scale = M, N, K, ACT[gemm.get("act")], 1.0
            d.gather, d.rows_per_src, d.wait_self = 2, int(gemm["rows_per_src"]), 1
            d.src_period = int(gemm.get("src_period", 0))
            d.ready_flags, d.ready_epoch = ch.ready.data_ptr(), ch.epoch
            # acks count consumptions of the slot: the next pusher into it waits for this one
            ch.ack_epoch += 1
            d.ack_ptrs, d.ack_epoch = ch.ack_ptrs.data_ptr(), ch.ack_epoch
        same = push is not None and gemm is not None and gemm["slot"] == slot
        self._launch(d, push is not None, M, Ng, consumer_waits=same)
        return slot, out

    def fsdp_weight(self, slot: int, N: int, K: int) -> torch.Tensor:
        """The staging copy of a gathered weight (valid after its consumers' flags are up)."""
        return self.wst[slot].view[:N * K * 2].view(torch.bfloat16).view(N, K)

    # ------------------------------------------------------------------ flag protocol check
    def protocol_report(self) -> list[str]:
        """Host-side check of the flag protocol, to be called when every rank is idle (after a
        synchronise and a barrier): for every staging buffer, each source rank's ready word must equal
        the number of pushes issued into the buffer, the partial-sum words of a reduce-scatter buffer
        the number of GEMMs that filled it, and no ack may run ahead of the consumptions announced.
        Returns the mismatches (empty = consistent)."""
        torch.cuda.synchronize(self.device)
        bad = []
        for kind, chans in (("ag", self.ag), ("w", self.wst)):
            for i, ch in enumerate(chans):
                ready = ch.ready.view(self.world, MAX_CHUNKS)[:, 0].tolist()
                acks = ch.ack.tolist()
                for src in range(self.world):
                    if kind == "ag" and src == self.rank:
                        continue                      # own rows are written in place, never flagged
                    if ready[src] != ch.epoch:
                        bad.append(f"{kind}[{i}] ready[{src}] = {ready[src]}, pushes issued {ch.epoch}")
                want_ack = ch.epoch if kind == "ag" else ch.ack_epoch
                for src in range(self.world):
                    if acks[src] > want_ack:
                        bad.append(f"{kind}[{i}] ack[{src}] = {acks[src]} ahead of {want_ack}")
        for i, ch in enumerate(self.rs):
            flags = ch.ready.view(-1)[:self.world].tolist()
            for src in range(self.world):
                if flags[src] != ch.epoch:
                    bad.append(f"rs[{i}] partials[{src}] = {flags[src]}, GEMMs issued {ch.epoch}")
        return bad

    # ------------------------------------------------------------------ DiZO norms
    def norm_allreduce_gamma(self, partial_sq: torch.Tensor, gs, reinit: bool, use_multimem: bool = False):
        """gs.sq = sum over ranks of ``partial_sq``; gs.ts, gs.gamma (if ``reinit``), gs.alpha
        refreshed - one kernel."""
        n = partial_sq.numel()
        assert n <= self.norm_slots
        self.norm_epoch += 1
        mc = self.region.multicast_addr(self.norm_mc_off) if use_multimem else 0
        rc = _lib.lib().dz_norm_allreduce_gamma(
            _lib.ptr(partial_sq), n, _lib.ptr(self.norm_slot_ptrs), _lib.ptr(self.norm_flag_ptrs),
            _lib.ptr(self.norm_mc_local), c_void(mc), self.rank, self.world, ctypes.c_uint(self.norm_epoch),
            _lib.ptr(gs.sq), _lib.ptr(gs.ts), _lib.ptr(gs.gamma), _lib.ptr(gs.alpha), int(reinit),
            int(bool(mc)), _lib.ptr(_lib.err_word(self.device)), _lib.stream_ptr())
        _lib.check(rc, "dz_norm_allreduce_gamma")
