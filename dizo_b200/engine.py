"""The zeroth-order training step and the DiZO projection, on top of the parameter arena.

``ZOEngine.step`` is the MeZO two-point SPSA estimator + ZO-SGD update of the reference
(``zo_step``/``zo_update``, large_models/trainer.py:1570-1617):

    seed k shared by every rank;  L+ = loss(theta + eps z_k);  L- = loss(theta - eps z_k)
    g = (L+ - L-) / (2 eps)        (kept on the device; one scalar all-reduce under DP)
    theta <- theta - lr * g * z_k  (one sweep; z regenerated, never stored)

Two execution modes with the same mathematics:
  * ``inflight`` (default): theta is never rewritten for a forward; each layer's perturbed
    copy is produced on the fly (:class:`dizo_b200.models.opt.Transform`).  One parameter
    sweep per step writes theta, instead of the reference's four.
  * ``inplace``: the reference's order (+eps, -2eps, +eps, update) with in-place sweeps.

``DiZOProjector`` is the divergence-driven projection (large_models/trainer.py:378-830):
every ``interval`` steps it searches one gamma per constrained tensor (10 ZO iterations on
fresh batches, or first-order steps through the gamma scalars) and projects
theta <- theta_0 + gamma / ||theta - theta_0|| * (theta - theta_0).  The search forwards read
``theta_0 + alpha (theta - theta_0)`` in flight, so the reference's apply/reverse passes
(and their fp16 round-trip error) do not exist here.
"""
from __future__ import annotations

import logging
import os
from typing import Callable

import torch
import torch.distributed as dist

from .models.opt import Batch, OPTModel, Transform
from .ops.zo import GammaState, fd_eps, scalar_diff, sr_seed_for

# DIZO_ZO_PAIRED=0 runs the two forwards of a step one after the other (two draws of z) - for measurements
_PAIRED = os.environ.get("DIZO_ZO_PAIRED", "1") != "0"

logger = logging.getLogger(__name__)


def _dist_on(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


class ZOEngine:
    def __init__(self, model: OPTModel, eps: float = 1e-3, mode: str = "inflight",
                 dp_group=None, stochastic_rounding: bool | None = None):
        """``stochastic_rounding=None`` (default) switches it on for bf16 parameters: at the reference's
        hyper-parameters (lr 1e-6..1e-7, eps 1e-3) an update lr*g*z is about 5e-7, far below half a bf16
        ulp of a typical weight (3e-5 at |w| = 0.01), so round-to-nearest would drop almost every update
        (the reference's fp16 has 8x finer steps).  Stochastic rounding keeps the update unbiased."""
        assert mode in ("inflight", "inplace")
        self.model = model
        self.eps = eps
        # bf16 arenas perturb with bf16(eps); the finite difference divides by what was applied
        self.eps_fd = fd_eps(eps, model.arena.dtype)
        self.mode = mode
        self.dp_group = dp_group          # None: the default group; False: no data parallelism
        if stochastic_rounding is None:
            stochastic_rounding = model.arena.dtype == torch.bfloat16
        self.stochastic_rounding = bool(stochastic_rounding)
        dev = model.device
        f = dict(dtype=torch.float32, device=dev)
        self.loss1 = torch.zeros(1, **f)
        self.loss2 = torch.zeros(1, **f)
        self.projected_grad = torch.zeros(1, **f)   # g of the last step (device)
        self.launches = 0

    # -- pieces of a step, exposed because the trainer API names them ------------------
    def perturb(self, seed: int, scaling: float) -> None:
        """In-place theta += scaling * eps * z(seed) (``zo_perturb_parameters``)."""
        self.model.arena.sweep(seed1=seed, c1=scaling * self.eps)

    def forward(self, batch: Batch, transform: Transform | None = None) -> torch.Tensor:
        return self.model.loss(batch, transform)

    def forward_pair(self, batch: Batch, seed: int, seed_dev: torch.Tensor | None = None,
                     loss_fn: Callable[[Batch, Transform | None], torch.Tensor] | None = None):
        """(L(theta + eps z), L(theta - eps z)) with in-flight perturbation: block by block with one draw of z per
        block where the model supports it (``OPTModel.loss_pair``), else two separate forwards."""
        eps = self.eps
        m = self.model
        if (loss_fn is None and _PAIRED and getattr(m, "pair_supported", None) is not None
                and m.pair_supported()):
            return m.loss_pair(batch, seed, eps, seed_dev=seed_dev)
        fwd = loss_fn or self.forward
        return (fwd(batch, Transform(seed=seed, coef=eps, seed_dev=seed_dev)),
                fwd(batch, Transform(seed=seed, coef=-eps, seed_dev=seed_dev)))

    def reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        """Mean over the data-parallel group of a 1-element device tensor (NCCL / gloo)."""
        if self.dp_group is not False and _dist_on(self.dp_group):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.dp_group)
            t.div_(dist.get_world_size(self.dp_group))
        return t

    def update(self, seed: int, lr: float, sq_out: torch.Tensor | None = None) -> None:
        """theta -= lr * g * z(seed) (``zo_update``); optionally also emit the DiZO norms of
        the updated tensors from the same pass."""
        sr = sr_seed_for(seed) if self.stochastic_rounding else None
        self.model.arena.sweep(seed1=seed, c1=-lr, c1_dev=self.projected_grad, sq_out=sq_out,
                               stochastic_round_seed=sr)

    def step(self, batch: Batch, lr: float, seed: int, sq_out: torch.Tensor | None = None,
             loss_fn: Callable[[Batch, Transform | None], torch.Tensor] | None = None) -> torch.Tensor:
        """One ZO-SGD step; returns L+ (1-element device tensor, like the reference's loss1)."""
        fwd = loss_fn or self.forward
        eps = self.eps
        if self.mode == "inflight":
            l1, l2 = self.forward_pair(batch, seed, loss_fn=loss_fn)
        else:
            self.perturb(seed, 1.0)
            l1 = fwd(batch, None)
            self.perturb(seed, -2.0)
            l2 = fwd(batch, None)
            self.perturb(seed, 1.0)
        self.loss1.copy_(l1.reshape(1))
        self.loss2.copy_(l2.reshape(1))
        scalar_diff(self.loss1, self.loss2, 1.0 / (2.0 * self.eps_fd), self.projected_grad)
        self.reduce_scalar(self.projected_grad)
        self.update(seed, lr, sq_out)
        return self.loss1


def batch_signature(batch: Batch) -> tuple:
    """Shapes of every tensor of a batch (what a captured step is specialised to)."""
    return tuple((k, tuple(v.shape)) if isinstance(v, torch.Tensor) else (k, v)
                 for k, v in sorted(batch.__dict__.items()))


class GraphedZOStep:
    """One whole ZO-SGD step (two forwards with in-flight perturbation, the projected-gradient
    arithmetic, the update sweep) captured in a CUDA graph and replayed with one launch.

    For models whose step is bound by kernel-launch overhead rather than by the kernels (hundreds
    of launches of a few microseconds each on the small OPT sizes).  What changes from step to step
    lives in device memory and is refreshed before each replay: the batch (copied into the captured
    input tensors), the perturbation seed (the sweeps read it through ``seed1_dev``) and the
    learning rate.  One instance serves one batch signature; single-process (the data-parallel
    all-reduce is not captured), ``inflight`` mode.  With stochastic rounding the rounding stream's seed
    is derived from the step's seed on the device."""

    def __init__(self, engine: ZOEngine, example: Batch, warmup: int = 2):
        assert engine.mode == "inflight"
        assert engine.dp_group is False or not _dist_on(engine.dp_group), "single-process only"
        dev = engine.model.device
        assert dev.type == "cuda"
        self.engine = engine
        self.signature = batch_signature(example)
        self.batch = Batch(**{k: (v.to(dev).clone() if isinstance(v, torch.Tensor) else v)
                              for k, v in example.__dict__.items()})
        self.seed = torch.zeros(1, dtype=torch.int64, device=dev)
        self.lr = torch.zeros(1, dtype=torch.float32, device=dev)       # 0 while warming up: theta unchanged
        self._lrg = torch.zeros(1, dtype=torch.float32, device=dev)
        cur = torch.cuda.current_stream(dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._body()
        cur.wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._body()
        self.replays = 0

    def _body(self) -> torch.Tensor:
        e, eps = self.engine, self.engine.eps
        l1, l2 = e.forward_pair(self.batch, 0, seed_dev=self.seed)
        e.loss1.copy_(l1.reshape(1))
        e.loss2.copy_(l2.reshape(1))
        scalar_diff(e.loss1, e.loss2, 1.0 / (2.0 * e.eps_fd), e.projected_grad)
        torch.mul(e.projected_grad, self.lr, out=self._lrg)
        e.model.arena.sweep(seed1_dev=self.seed, c1=-1.0, c1_dev=self._lrg,
                            stochastic_round_seed=1 if e.stochastic_rounding else None)
        return e.loss1

    def __call__(self, batch: Batch, lr: float, seed: int) -> torch.Tensor:
        assert batch_signature(batch) == self.signature, "batch shape differs from the captured one"
        for k, v in batch.__dict__.items():
            if isinstance(v, torch.Tensor):
                getattr(self.batch, k).copy_(v, non_blocking=True)
        self.seed.fill_(int(seed))
        self.lr.fill_(float(lr))
        self.graph.replay()
        self.replays += 1
        return self.loss


class DiZOProjector:
    """gamma search + projection for the constrained tensors of ``model.arena``."""

    def __init__(self, model: OPTModel, include: list[str] | None = None, tau: float = 0.2,
                 zo_eps: float = 0.1, step_size: float = 2.0, max_iters: int = 10,
                 proj_lr: float = 0.1, l1: float = 1e-3, norm_mode: str = "l2norm", dp_group=None):
        if "l2" not in norm_mode:
            raise NotImplementedError("only the l2 norm mode is reachable in the reference "
                                      "(large_models/trainer.py:1168)")
        self.model = model
        self.include = list(model.dizo_include_names() if include is None else include)
        self.max_iters = max_iters
        self.proj_lr = proj_lr
        self.l1 = l1
        self.dp_group = dp_group
        model.arena.set_dizo(self.include)
        self.n = model.arena.n_slots
        self.gs = GammaState(max(self.n, 1), model.device, tau, zo_eps, step_size)
        self._l1 = torch.zeros(1, dtype=torch.float32, device=model.device)
        self._l2 = torch.zeros(1, dtype=torch.float32, device=model.device)
        self.searches = 0
        # FO state persists across searches (large_models/trainer.py:401, :761)
        self.fo_gamma: torch.Tensor | None = None
        self.fo_opt = None
        self.use_kernel_backward = True      # False: always differentiate through the autograd statement
        self._gamma_grad = None

    def _reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.dp_group is not False and _dist_on(self.dp_group):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.dp_group)
            t.div_(dist.get_world_size(self.dp_group))
        return t

    def _begin(self, reinit: bool) -> None:
        """ts = ||theta - theta_0|| per constraint (+ gamma = ts when ``reinit``).  Sharded models
        hold partial sums: their ``reduce_norms`` sums them over the shards and does the gamma
        arithmetic in the same kernel."""
        if hasattr(self.model, "reduce_norms"):
            self.model.reduce_norms(self.gs, reinit)
        else:
            self.gs.begin(reinit=reinit)

    def measure(self) -> None:
        """sq[i] = ||theta_i - theta_0i||^2 for every constrained tensor (one pass)."""
        self.model.arena.sweep(sq_out=self.gs.sq)

    def search_zo(self, next_batch: Callable[[], Batch], seed: int, norms_ready: bool = False) -> None:
        """``dizo_zo_iters``: gamma_i initialised to ts_i, then ``max_iters`` two-point steps."""
        if self.n == 0:
            return
        if not norms_ready:
            self.measure()
        gs = self.gs
        self._begin(reinit=True)
        for it in range(self.max_iters):
            batch = next_batch()
            gs.perturb(+1.0, seed=seed, it=it)
            self._l1.copy_(self.model.loss(batch, Transform(alpha=gs.alpha)).reshape(1))
            gs.perturb(-2.0)
            self._l2.copy_(self.model.loss(batch, Transform(alpha=gs.alpha)).reshape(1))
            gs.perturb(+1.0)
            self._reduce(self._l1)
            self._reduce(self._l2)
            gs.step(self._l1, self._l2)
        self.project()
        self.searches += 1

    def project(self) -> None:
        """theta_i <- theta_0i + alpha_i (theta_i - theta_0i), in place, one pass."""
        if self.n:
            self.model.arena.sweep(alpha=self.gs.alpha)

    def search_fo(self, next_batch: Callable[[], Batch], fo_loss: Callable | None = None) -> None:
        """``dizo_iters``: Adam on gamma through d loss / d gamma (gamma starts at 0 and, like
        its Adam moments, persists across searches; L1 penalty ``l1 * sum |gamma|``).

        d loss / d alpha comes from the kernel backward (:class:`models.gamma_grad.GammaGrad`)
        where the configuration is covered; otherwise from ``fo_loss(batch, alpha)``, an autograd
        statement of the forward (:func:`models.opt_autograd.make_fo_loss`)."""
        if self.n == 0:
            return
        from .models import gamma_grad
        self.measure()
        gs = self.gs
        self._begin(reinit=False)
        if self.fo_gamma is None:
            self.fo_gamma = torch.zeros(self.n, dtype=torch.float32, device=self.model.device,
                                        requires_grad=True)
            self.fo_opt = torch.optim.Adam([self.fo_gamma], lr=self.proj_lr)
        native = fo_loss is None or (self.use_kernel_backward and gamma_grad.supported(self.model))
        if native and self._gamma_grad is None:
            self._gamma_grad = gamma_grad.GammaGrad(self.model)
        for _ in range(self.max_iters):
            batch = next_batch()
            self.fo_opt.zero_grad(set_to_none=True)
            if native:
                with torch.no_grad():
                    ts = gs.ts[:self.n] + 1e-8
                    alpha = torch.zeros_like(gs.alpha)
                    alpha[:self.n] = self.fo_gamma.detach() / ts
                    _, g_alpha = self._gamma_grad.loss_and_grad(batch, alpha)
                    self.fo_gamma.grad = g_alpha / ts + self.l1 * torch.sign(self.fo_gamma.detach())
            else:
                alpha = self.fo_gamma / (gs.ts.detach() + 1e-8)
                loss = fo_loss(batch, alpha) + self.l1 * self.fo_gamma.abs().sum()
                loss.backward()
            self._reduce(self.fo_gamma.grad)
            self.fo_opt.step()
        with torch.no_grad():
            gs.gamma.copy_(self.fo_gamma.detach())
            gs.alpha.copy_(gs.gamma / (gs.ts + 1e-8))
        self.project()
        self.searches += 1

    def state_dict(self) -> dict:
        sd = {"gamma": self.gs.gamma.cpu(), "ts": self.gs.ts.cpu(), "searches": self.searches}
        if self.fo_gamma is not None:
            sd["fo_gamma"] = self.fo_gamma.detach().cpu()
            sd["fo_opt"] = self.fo_opt.state_dict()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        self.gs.gamma.copy_(sd["gamma"])
        self.gs.ts.copy_(sd["ts"])
        self.searches = int(sd.get("searches", 0))
        if "fo_gamma" in sd:
            self.fo_gamma = sd["fo_gamma"].to(self.model.device).requires_grad_(True)
            self.fo_opt = torch.optim.Adam([self.fo_gamma], lr=self.proj_lr)
            self.fo_opt.load_state_dict(sd["fo_opt"])


class DiZO:
    """The reference's ``DiZO(model, norm_mode, exclude_list)`` module (large_models/trainer.py:378-614) as a
    thin facade over :class:`DiZOProjector`, for callers that drive the projection by hand.

    The reference copies ``theta_0 + gamma / ||theta - theta_0|| (theta - theta_0)`` into the weights before a
    forward and divides it out again afterwards (``apply_constraints`` / ``reverse_constraints``); here a forward
    blends the constrained tensors in flight, so theta is only written when ``apply=True``:

    * ``constraints`` - the gamma vector (one entry per constrained tensor, in ``constraints_name`` order),
      ``alpha`` - gamma / (||theta - theta_0|| + 1e-8), ``ts`` - the norms, ``init`` - True until gamma has
      been initialised to the norms;
    * ``apply_constraints(apply=False)`` - measure the norms, initialise gamma on the first call, refresh
      alpha; with ``apply=True`` project theta in place (one sweep);
    * ``reverse_constraints()`` - nothing to undo (kept for call-site compatibility);
    * ``perturb_gamma(random_seed, scaling_factor)`` - gamma += scaling_factor * zo_eps * z(random_seed),
      clipped as the reference clips it, alpha refreshed;
    * ``zo_forward(batch)`` / ``forward(batch, apply=False)`` - the loss under the current alpha.
    """

    def __init__(self, model: OPTModel, norm_mode: str = "l2norm", exclude_list: list[str] | None = None, **kw):
        names = list(model.dizo_include_names())
        if exclude_list:
            drop = set(exclude_list)
            names = [n for n in names if n not in drop]
        self.norm_mode = norm_mode
        self.exclude_list = list(exclude_list or [])
        self.projector = DiZOProjector(model, include=names, norm_mode=norm_mode, **kw)
        self.model = model
        self.constraints_name = list(model.arena.slot_names)
        self.init = True
        self._seed = 0

    @property
    def constraints(self) -> torch.Tensor:
        return self.projector.gs.gamma

    @property
    def alpha(self) -> torch.Tensor:
        return self.projector.gs.alpha

    @property
    def ts(self) -> torch.Tensor:
        return self.projector.gs.ts

    def apply_constraints(self, new=None, pre_trained=None, constraint_iterator=None, apply: bool = False) -> None:
        self.projector.measure()
        self.projector._begin(reinit=self.init)
        self.init = False
        if apply:
            self.projector.project()

    def reverse_constraints(self, new=None, pre_trained=None) -> None:
        return None

    def perturb_gamma(self, random_seed: int | None = None, scaling_factor: float = 1.0) -> None:
        if random_seed is not None:
            self._seed = int(random_seed)
            self.projector.gs.perturb(float(scaling_factor), seed=self._seed, it=0)
        else:
            self.projector.gs.perturb(float(scaling_factor))       # the same z again (restore / flip)

    def zo_forward(self, batch: Batch) -> torch.Tensor:
        return self.model.loss(batch, Transform(alpha=self.projector.gs.alpha))

    def forward(self, batch: Batch, apply: bool = False) -> torch.Tensor:
        self.apply_constraints(apply=apply)
        return self.model.loss(batch) if apply else self.zo_forward(batch)

    __call__ = forward
