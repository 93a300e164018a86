"""``OurTrainer``: the training loop and the ZO / DiZO trainer API.

API and behaviour follow the reference's ``OurTrainer`` (large_models/trainer.py:833-1766):
``train``, ``zo_perturb_parameters``, ``zo_forward``, ``zo_forward_nondiff``, ``zo_step``,
``zo_update``, ``forward``, ``one_step_pred``, ``save_model``, ``add_callback`` and the
attributes ``named_parameters_to_optim``, ``exclude_list``, ``base_model`` (here: the anchor
arena), ``dizo_trainer``, ``projected_grad``, ``zo_random_seed``, ``loss_list``, ``accuracy``,
``best_model_ckpt``.  It does not derive from ``transformers.Trainer``: the loop below is the
part of that class the reference's ZO path exercises - linear-decay-to-half learning rate
(:1100-1102), a log line every 50 steps (:1321-1324), dev evaluation every 100 steps with
``.npy`` curves and a best-dev copy kept in host memory (:1327-1353) - plus what the reference
lacks: real step checkpoints, resume that replays the exact z stream, SIGUSR1 saves, shared-seed
data parallelism with one scalar all-reduce per step, per-phase device timers.
"""
from __future__ import annotations

import json
import logging
import math
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .args import OurArguments
from .data.batching import batch_from_inputs
from .engine import DiZOProjector, ZOEngine
from .metrics import f1
from .models.opt import Batch, OPTModel, Transform
from .utils import TrainerCallback, TrainerControl
from .utils.checkpoint import load_checkpoint, save_checkpoint

logger = logging.getLogger(__name__)


@dataclass
class TrainerState:
    global_step: int = 0
    epoch: float = 0.0
    max_steps: int = 0
    log_history: list = field(default_factory=list)
    best_metric: Optional[float] = None
    best_model_checkpoint: Optional[str] = None

    def save_to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(asdict(self), f, indent=2)

    @classmethod
    def load_from_json(cls, path: str) -> "TrainerState":
        with open(path) as f:
            return cls(**json.load(f))


class DizoTrainerView:
    """The reference's ``dizo_trainer`` object (large_models/trainer.py:744-830) as a thin view
    over :class:`DiZOProjector`: same method names, batches drawn from its own iterator over
    the training loader."""

    def __init__(self, projector: DiZOProjector, next_batch: Callable[[], Batch], seed_fn: Callable[[], int],
                 fo_loss: Optional[Callable] = None):
        self.dizo = projector
        self.projector = projector
        self.proj_lr = projector.proj_lr
        self.max_iters = projector.max_iters
        self._next = next_batch
        self._seed = seed_fn
        self._fo_loss = fo_loss
        self.i = 0

    def dizo_zo_iters(self, model=None, base_model=None, apply: bool = False, norms_ready: bool = False):
        if apply:
            self.projector.project()
        else:
            self.projector.search_zo(self._next, self._seed(), norms_ready=norms_ready)
        self.i += 1

    def dizo_iters(self, model=None, base_model=None, apply: bool = False):
        if apply:
            self.projector.project()
        else:
            self.projector.search_fo(self._next, self._fo_loss)
        self.i += 1


def dizo_trainer(model: OPTModel, pgmloader, norm_mode: str = "l2norm", proj_lr: float = 0.1, max_iters: int = 10,
                 exclude_list: Optional[List[str]] = None, seed: int = 0, to_batch: Optional[Callable] = None,
                 **projector_kw) -> DizoTrainerView:
    """The reference's constructor ``dizo_trainer(base_model, pgmloader, norm_mode, proj_lr, max_iters,
    exclude_list)`` (large_models/trainer.py:744-761) for callers that build the projection loop themselves.
    ``model`` takes the place of ``base_model``: the anchor theta_0 of the constrained tensors lives in the
    model's arena.  ``pgmloader`` is any re-iterable of batches (``to_batch`` converts collated inputs); the
    search draws from its own endless iterator over it, as the reference does (:762-763)."""
    names = [n for n in model.dizo_include_names() if n not in set(exclude_list or [])]
    proj = DiZOProjector(model, include=names, norm_mode=norm_mode, proj_lr=proj_lr, max_iters=max_iters,
                         **projector_kw)
    state = {"it": iter(pgmloader)}

    def next_batch():
        try:
            b = next(state["it"])
        except StopIteration:
            state["it"] = iter(pgmloader)
            b = next(state["it"])
        return to_batch(b) if to_batch is not None else b

    rng = np.random.RandomState(seed + 7919)
    fo_loss = None
    from .models import gamma_grad
    if not gamma_grad.supported(model):
        from .models.opt_autograd import make_fo_loss
        fo_loss = make_fo_loss(model)
    return DizoTrainerView(proj, next_batch, lambda: int(rng.randint(1_000_000_000)), fo_loss)


class OurTrainer:
    def __init__(self, model: OPTModel, args: OurArguments, train_dataset=None, eval_dataset=None,
                 processing_class=None, tokenizer=None, data_collator=None, engine: ZOEngine | None = None,
                 task=None, callbacks: Optional[List[TrainerCallback]] = None, dp_group=None):
        self.model = model
        self.args = args
        self.train_dataset = train_dataset
        self.eval_dataset = eval_dataset
        self.processing_class = processing_class if processing_class is not None else tokenizer
        self.data_collator = data_collator
        self.task = task
        self.dp_group = dp_group
        self.callbacks: List[TrainerCallback] = list(callbacks or [])
        self.control = TrainerControl()
        self.state = TrainerState()
        self.engine = engine or ZOEngine(model, eps=args.zo_eps, mode=args.zo_mode, dp_group=dp_group,
                                         stochastic_rounding=args.zo_stochastic_rounding)
        self.projected_grad = self.engine.projected_grad
        self.zo_random_seed: Optional[int] = None
        self.loss_list: List[float] = []
        self.accuracy: List[float] = []
        self.objective = 0.0
        self.best_model_ckpt: Optional[Dict[str, torch.Tensor]] = None
        self.dizo_trainer: Optional[DizoTrainerView] = None
        self.named_parameters_to_optim = [(p.name, model.arena.view(p.name)) for p in model.arena.pieces]
        self.exclude_list: List[str] = []
        self.base_model = None
        self._train_iter = None
        self._pgm_iter = None
        self._pgm_count = 0          # batches the gamma search has consumed (saved for resume)
        self._phase_ms: Dict[str, float] = {}
        self._metrics_f = None
        self._graphs: dict = {}
        # host-side failure detection: every rank reports its step through the rendezvous store and
        # looks at its peers before it launches the next step (nothing on the device waits for a
        # peer that is known to be gone)
        self._heartbeat = None
        hb_t = float(getattr(args, "heartbeat_timeout", 0.0) or 0.0)
        if hb_t > 0 and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            from .parallel.health import Heartbeat
            self._heartbeat = Heartbeat(dist.distributed_c10d._get_default_store(), dist.get_rank(),
                                        dist.get_world_size(), stale_after=hb_t)
        on = dist.is_available() and dist.is_initialized() and dp_group is not False
        self._rank = dist.get_rank(dp_group) if on else 0
        # the one process that writes files (under tensor parallelism every rank has data rank 0)
        self._writer = (dist.get_rank() == 0) if (dist.is_available() and dist.is_initialized()) else True
        self._sharded = hasattr(model, "gather_state_dict")
        self._world = dist.get_world_size(dp_group) if on else 1

    # ------------------------------------------------------------------ small API
    @property
    def tokenizer(self):
        return self.processing_class

    def add_callback(self, cb) -> None:
        self.callbacks.append(cb() if isinstance(cb, type) else cb)

    def _fire(self, event: str, **kw) -> None:
        for cb in self.callbacks:
            getattr(cb, event)(self.args, self.state, self.control, **kw)

    def _get_learning_rate(self) -> float:
        """ZO runs replace the configured scheduler by lr0 * (1 - step / (2 * max_steps))
        (large_models/trainer.py:1100-1102)."""
        a = self.args
        ms = max(self.state.max_steps, 1)
        if a.trainer == "zo":
            return a.learning_rate * (1.0 - self.state.global_step / (2.0 * ms))
        if a.lr_scheduler_type == "constant":
            return a.learning_rate
        return a.learning_rate * max(0.0, 1.0 - self.state.global_step / ms)

    # ------------------------------------------------------------------ batches
    def _to_batch(self, inputs) -> Batch:
        if isinstance(inputs, Batch):
            b = inputs
        else:
            pad = self.tokenizer.pad_token_id if self.tokenizer is not None else self.model.config.pad_token_id
            b = batch_from_inputs(inputs, pad, classification=self.args.train_as_classification
                                  if "num_options" not in inputs else True,
                                  only_train_option=self.args.only_train_option)
        if b.input_ids.device != self.model.device:
            if self.model.device.type == "cuda" and not b.input_ids.is_pinned():
                b = b.pin()
            b = b.to(self.model.device, non_blocking=True)
        return b

    # ------------------------------------------------------------------ ZO API (reference names)
    def zo_perturb_parameters(self, random_seed: Optional[int] = None, scaling_factor: float = 1) -> None:
        """theta += scaling_factor * eps * z(seed), in place; z is regenerated, never stored."""
        seed = random_seed if random_seed is not None else self.zo_random_seed
        self.engine.perturb(int(seed), float(scaling_factor))

    def zo_forward(self, model, inputs) -> torch.Tensor:
        """Loss of the current parameters on ``inputs`` (no autograd anywhere)."""
        return self.engine.forward(self._to_batch(inputs), None)

    def zo_forward_nondiff(self, model, inputs) -> torch.Tensor:
        """Non-differentiable objective: -mean F1 of greedy generations against ``gold``
        (SQuAD; large_models/trainer.py:1544-1568)."""
        return self._nondiff_loss(inputs, None)

    def _nondiff_loss(self, inputs, transform: Optional[Transform]) -> torch.Tensor:
        from .models.generate import generate
        a = self.args
        ids = torch.as_tensor(inputs["input_ids"])
        mask = torch.as_tensor(inputs["attention_mask"])
        eos = [self.tokenizer.eos_token_id]
        extra = self.tokenizer.encode(a.eos_token, add_special_tokens=False)
        if extra:
            eos.append(extra[-1])
        if transform is not None:
            # decode under theta + c z: perturb in place around the generation, then undo
            self.model.arena.sweep(seed1=transform.seed, c1=transform.coef)
        try:
            out = generate(self.model, ids, attention_mask=mask, max_new_tokens=min(
                a.max_new_tokens, a.max_length - ids.shape[1]), do_sample=a.sampling,
                temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, num_beams=a.num_beams,
                eos_token_id=eos, pad_token_id=self.tokenizer.pad_token_id)
        finally:
            if transform is not None:
                self.model.arena.sweep(seed1=transform.seed, c1=-transform.coef)
        scores = []
        for i in range(ids.shape[0]):
            text = self.tokenizer.decode(out[i][int(mask[i].sum()):], skip_special_tokens=True).strip()
            scores.append(f1(text, inputs["gold"][i]))
        return -torch.tensor([float(np.mean(scores))], dtype=torch.float32, device=self.model.device)

    def zo_step(self, model, inputs) -> torch.Tensor:
        """Two-point estimate of the projected gradient; returns L(theta + eps z).  The update is
        ``zo_update``.  A fresh seed is drawn from NumPy's global generator each step
        (large_models/trainer.py:1577), so ``--seed`` fixes the whole z stream."""
        self.zo_random_seed = int(np.random.randint(1_000_000_000))
        eng = self.engine
        if self.args.non_diff:
            fwd = lambda b, t: self._nondiff_loss(inputs, t)
            batch = None
        else:
            fwd = eng.forward
            batch = self._to_batch(inputs)
        eps, seed = eng.eps, self.zo_random_seed
        if eng.mode == "inflight":
            l1, l2 = eng.forward_pair(batch, seed, loss_fn=fwd if self.args.non_diff else None)
        else:
            self.zo_perturb_parameters(scaling_factor=1)
            l1 = fwd(batch, None)
            self.zo_perturb_parameters(scaling_factor=-2)
            l2 = fwd(batch, None)
            self.zo_perturb_parameters(scaling_factor=1)
        eng.loss1.copy_(l1.reshape(1))
        eng.loss2.copy_(l2.reshape(1))
        from .ops.zo import scalar_diff
        scalar_diff(eng.loss1, eng.loss2, 1.0 / (2.0 * eng.eps_fd), eng.projected_grad)
        eng.reduce_scalar(eng.projected_grad)
        assert self.args.gradient_accumulation_steps == 1, "ZO does not accumulate gradients"
        return eng.loss1

    def zo_update(self, args=None, model=None) -> None:
        """theta -= lr * g * z; every ``dizo_interval`` updates the gamma search + projection
        (large_models/trainer.py:1597-1617)."""
        a = self.args
        due = bool(a.enhanced) and a.enhanced != "None" and \
            (self.state.global_step + 1) % a.dizo_interval == 0 and self.dizo_trainer is not None
        sq = self.dizo_trainer.projector.gs.sq if (due and self.dizo_trainer.projector.n) else None
        self.engine.update(self.zo_random_seed, self._get_learning_rate(), sq_out=sq)
        if due:
            t0 = time.time()
            if a.enhanced == "zo":
                self.dizo_trainer.dizo_zo_iters(self.model, norms_ready=sq is not None)
            else:
                self.dizo_trainer.dizo_iters(self.model)
            if a.verbose or self._metrics_f:
                # gamma / ||theta - theta_0|| per constrained tensor: how far the projection pulled
                pr = self.dizo_trainer.projector
                gs = pr.gs
                al = gs.alpha[:max(pr.n, 1)].float()
                rec = {"projection": self.dizo_trainer.i, "step": self.state.global_step + 1,
                       "alpha_mean": round(al.mean().item(), 5), "alpha_min": round(al.min().item(), 5),
                       "alpha_max": round(al.max().item(), 5),
                       "ts_mean": round(gs.ts[:max(pr.n, 1)].float().mean().item(), 6),
                       "search_s": round(time.time() - t0, 3)}
                if a.verbose:
                    logger.info("DiZO projection %s", rec)
                if self._metrics_f:
                    self._metrics_f.write(json.dumps(rec) + "\n")

    # ------------------------------------------------------------------ CUDA-graph replay
    def _graph_ok(self) -> bool:
        """``--zo_cuda_graph``: replay the step as one CUDA graph when nothing but the plain step is
        due (no projection), on one process, for differentiable objectives."""
        a = self.args
        if not getattr(a, "zo_cuda_graph", False) or self.model.device.type != "cuda" or a.non_diff:
            return False
        if self._world > 1 or self.engine.mode != "inflight":
            return False
        if type(self.model).hidden_states is not OPTModel.hidden_states:
            return False
        due = bool(a.enhanced) and a.enhanced != "None" and self.dizo_trainer is not None and \
            (self.state.global_step + 1) % a.dizo_interval == 0
        return not due

    def _graphed_zo_step(self, inputs) -> torch.Tensor:
        from .engine import GraphedZOStep, batch_signature
        self.zo_random_seed = int(np.random.randint(1_000_000_000))      # same draw as zo_step
        batch = self._to_batch(inputs)
        key = batch_signature(batch)
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= 8:                                   # ragged shapes: keep the cache small
                self._graphs.pop(next(iter(self._graphs)))
            g = self._graphs[key] = GraphedZOStep(self.engine, batch)
        return g(batch, self._get_learning_rate(), self.zo_random_seed)

    def _log_phases(self, ev) -> None:
        """Device time of the two phases of a profiled step (max over the ranks): the two forwards
        with their in-flight perturbation, and the update sweep (+ gamma search when one was due);
        the update's parameter traffic as GB/s when it was a plain update."""
        ev[2].synchronize()
        t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], dtype=torch.float64,
                         device=self.model.device)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        fwd_ms, upd_ms = (float(x) for x in t.tolist())
        a = self.args
        searched = bool(a.enhanced) and a.enhanced != "None" and self.dizo_trainer is not None and \
            (self.state.global_step + 1) % a.dizo_interval == 0
        rec = {"step": self.state.global_step + 1, "forwards_ms": round(fwd_ms, 3), "update_ms": round(upd_ms, 3)}
        if not searched and upd_ms > 0:
            nbytes = 2 * self.model.arena.trainable_numel() * self.model.arena.data.element_size()
            rec["update_gbs"] = round(nbytes / upd_ms / 1e6, 1)
        logger.info("profile %s", rec)
        if self._metrics_f:
            self._metrics_f.write(json.dumps(rec) + "\n")

    def training_step(self, inputs) -> float:
        """One full optimisation step from host inputs: H2D copy, ``zo_step``, ``zo_update``,
        device->host read of the loss."""
        loss = self.zo_step(self.model, inputs)
        self.zo_update(self.args, self.model)
        self.state.global_step += 1
        return float(loss.item())

    # ------------------------------------------------------------------ DiZO wiring
    def _setup_dizo(self) -> None:
        a = self.args
        if not a.enhanced or a.enhanced == "None" or a.trainer != "zo":
            return
        include = self.model.dizo_include_names()
        self.exclude_list = [n for n in self.model.hf_order if n not in set(include)]
        proj = DiZOProjector(self.model, include, tau=a.dizo_tau, zo_eps=a.dizo_zo_eps,
                             step_size=a.dizo_step_size, max_iters=a.dizo_max_iters, proj_lr=a.dizo_proj_lr,
                             l1=a.dizo_l1, norm_mode=a.dizo_norm_mode, dp_group=self.dp_group)
        self.base_model = self.model.arena.anchor
        fo_loss = None
        if a.enhanced == "fo":
            from .models import gamma_grad
            if not gamma_grad.supported(self.model):
                # configurations the kernel backward does not cover (GELU blocks, sharded LoRA, LLaMA-family
                # blocks): autograd statement
                from .models.opt_autograd import make_fo_loss
                fo_loss = make_fo_loss(self.model)
        self._dizo_seed_rng = np.random.RandomState(a.seed + 7919)
        self.dizo_trainer = DizoTrainerView(proj, self._next_pgm_batch,
                                            lambda: int(self._dizo_seed_rng.randint(1_000_000_000)), fo_loss)

    # ------------------------------------------------------------------ data iteration
    def _epoch_order(self, epoch: int) -> List[int]:
        g = torch.Generator().manual_seed(self.args.seed + epoch)
        return torch.randperm(len(self.train_dataset), generator=g).tolist()

    def _batches(self, salt: int = 0, skip_steps: int = 0):
        """Endless stream of collated batches: a seeded permutation per epoch, every rank taking
        its own ``per_device_train_batch_size`` slice of each global batch."""
        bs = self.args.per_device_train_batch_size
        gb = bs * self._world
        epoch = 0
        n = len(self.train_dataset)
        steps_per_epoch = max(1, n // gb) if n >= gb else 1
        epoch, within = divmod(skip_steps, steps_per_epoch)
        while True:
            order = self._epoch_order(epoch * 2 + salt)
            for s in range(within, steps_per_epoch):
                lo = s * gb + self._rank * bs
                idx = [order[(lo + j) % n] for j in range(bs)]
                yield epoch, s, steps_per_epoch, self.data_collator([self.train_dataset[i] for i in idx])
            within = 0
            epoch += 1

    def _next_pgm_batch(self) -> Batch:
        """The gamma search consumes batches from its OWN iterator over the training loader
        (large_models/trainer.py:762-763, :790-796)."""
        if self._pgm_iter is None:
            self._pgm_iter = self._batches(salt=1, skip_steps=self._pgm_count)
        self._pgm_count += 1
        return self._to_batch(next(self._pgm_iter)[3])

    # ------------------------------------------------------------------ evaluation inside the loop
    def forward(self, input_ids, option_len=None, generation=False):
        return self._evaluator().forward(input_ids, option_len, generation)

    def one_step_pred(self, train_samples, eval_sample, verbose=False):
        return self._evaluator().one_step_pred(train_samples, eval_sample, verbose)

    def _evaluator(self):
        from .evaluation import Evaluator
        return Evaluator(self.model, self.tokenizer, self.task, self.args)

    def _in_loop_eval(self) -> None:
        a = self.args
        path = "loss_acc/{}_{}_{}_enhanced_{}".format(a.task_name, a.trainer, "lora" if a.lora else "ft", a.enhanced)
        if self._writer:
            os.makedirs(path, exist_ok=True)
            np.save(f"{path}/loss_list_seed_{a.seed}.npy", self.loss_list)
        if self.eval_dataset is None or len(self.eval_dataset) == 0 or self.task is None:
            return
        name = getattr(self.task, "metric_name", "accuracy")
        metrics = self._evaluator().evaluate([], list(self.eval_dataset))
        metrics["global_step"] = self.state.global_step
        logger.info(f"Eval results: {metrics}")
        self.accuracy.append(metrics[name])
        if self._writer:
            np.save(f"{path}/accuracy_seed_{a.seed}.npy", self.accuracy)
        if metrics[name] >= self.objective:
            logger.info("Best dev result: {}".format(metrics[name]))
            self.objective = metrics[name]
            self.state.best_metric = float(metrics[name])
            # kept in host memory, and actually restorable (load_best_model_at_end)
            if self._sharded:
                # every rank keeps its own shards (a full copy per rank would not fit the host for the
                # model sizes that are sharded in the first place)
                self.best_model_ckpt = {n: self.model.param(n).detach().cpu().clone() for n in self.model.hf_order}
            else:
                self.best_model_ckpt = {k: v.detach().cpu() for k, v in self.model.state_dict().items()}

    # ------------------------------------------------------------------ checkpoints
    def save_model(self, output_dir: Optional[str] = None) -> None:
        """Hugging Face layout: ``model.safetensors`` (or ``pytorch_model.bin``) + ``config.json``."""
        out = output_dir or self.args.output_dir
        if self._writer or self._sharded:
            save_checkpoint(out, self.model, trainer=None, write=self._writer)

    def _save_checkpoint(self) -> str:
        out = os.path.join(self.args.output_dir, f"checkpoint-{self.state.global_step}")
        if self._writer or self._sharded:
            save_checkpoint(out, self.model, trainer=self, write=self._writer)
        if self._writer:
            self._rotate_checkpoints()
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        return out

    def _rotate_checkpoints(self) -> None:
        lim = self.args.save_total_limit
        if not lim:
            return
        d = self.args.output_dir
        cks = sorted((int(x.split("-")[1]), x) for x in os.listdir(d)
                     if x.startswith("checkpoint-") and x.split("-")[1].isdigit())
        import shutil
        for _, name in cks[:-lim]:
            shutil.rmtree(os.path.join(d, name), ignore_errors=True)

    # ------------------------------------------------------------------ the loop
    def train(self, resume_from_checkpoint: Optional[str] = None) -> Dict[str, Any]:
        a = self.args
        assert a.trainer in ("zo", "regular"), "train() needs --trainer zo|regular"
        n = len(self.train_dataset)
        gb = a.per_device_train_batch_size * self._world
        accum = max(1, a.gradient_accumulation_steps) if a.trainer == "regular" else 1
        steps_per_epoch = max(1, n // (gb * accum))
        self.state.max_steps = a.max_steps if a.max_steps > 0 else int(math.ceil(a.num_train_epochs * steps_per_epoch))
        if a.linear_probing:
            from .models.probe import linear_probe
            return linear_probe(self)
        self._setup_dizo()
        if resume_from_checkpoint:
            load_checkpoint(resume_from_checkpoint, self.model, trainer=self)
            logger.info("Resumed from %s at step %d", resume_from_checkpoint, self.state.global_step)
        if a.metrics_jsonl and self._writer:
            self._metrics_f = open(a.metrics_jsonl, "a")
        logger.info("***** Running training *****")
        logger.info(f"  Num examples = {n}")
        logger.info(f"  Instantaneous batch size per device = {a.per_device_train_batch_size}")
        logger.info(f"  Total optimization steps = {self.state.max_steps}")
        logger.info(f"  Number of trainable parameters = {self.model.num_parameters(trainable_only=True)}")
        self._fire("on_train_begin")
        t_start = time.time()
        tokens = 0
        tr_loss = 0.0
        start_step = self.state.global_step
        prof = _parse_range(a.profile_steps)
        stream = self._batches(salt=0, skip_steps=self.state.global_step * accum)
        for epoch, step_in_epoch, spe, inputs in stream:
            if accum > 1:
                # one optimiser step = `accum` micro-batches (large_models/finetune.sh splits the batch
                # this way for the tasks that do not fit)
                micro = [inputs]
                for _ in range(accum - 1):
                    epoch, step_in_epoch, spe, nxt = next(stream)
                    micro.append(nxt)
                inputs = micro
                spe = max(1, spe // accum)
                step_in_epoch = step_in_epoch // accum
            if self.state.global_step >= self.state.max_steps:
                break
            if self._heartbeat is not None:
                self._heartbeat.sync(self.state.global_step)       # raises PeerLost on the host
            profiling = prof is not None and prof[0] <= self.state.global_step < prof[1]
            on_gpu = self.model.device.type == "cuda"
            ev = None
            if profiling and on_gpu:
                torch.cuda.nvtx.range_push(f"zo_step_{self.state.global_step}")
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                ev[0].record()
            if a.trainer == "zo" and self._graph_ok():
                loss_t = self._graphed_zo_step(inputs)
                if ev:
                    ev[1].record()
            elif a.trainer == "zo":
                loss_t = self.zo_step(self.model, inputs)
                if ev:
                    ev[1].record()
                self.zo_update(a, self.model)
            else:
                from .models.opt_autograd import fo_training_step
                loss_t = fo_training_step(self, inputs)
                if ev:
                    ev[1].record()
            if ev:
                ev[2].record()
                torch.cuda.nvtx.range_pop()
                self._log_phases(ev)
            loss = float(loss_t.item())                      # the step's one device->host read
            if a.logging_nan_inf_filter and (math.isnan(loss) or math.isinf(loss)):
                loss = tr_loss / max(1, self.state.global_step - start_step)
            tr_loss += loss
            for one in (inputs if isinstance(inputs, list) else [inputs]):
                tokens += int(torch.as_tensor(one["input_ids"]).numel()) if not isinstance(one, Batch) \
                    else int(one.input_ids.numel())
            self.state.global_step += 1
            self.state.epoch = epoch + (step_in_epoch + 1) / spe
            self._fire("on_step_end")
            log_step = a.zo_log_steps if a.trainer == "zo" else 10
            if self.state.global_step % log_step == 0:
                rec = {"loss": round(loss, 4), "epoch": epoch, "lr": self._get_learning_rate()}
                logger.info(rec)
                self.state.log_history.append({**rec, "step": self.state.global_step})
                if self._metrics_f:
                    el = time.time() - t_start
                    self._metrics_f.write(json.dumps({**rec, "step": self.state.global_step,
                                                      "tokens_per_s": tokens * self._world / max(el, 1e-9)}) + "\n")
                    self._metrics_f.flush()
            self.loss_list.append(loss)
            if a.trainer == "zo" and self.state.global_step % a.zo_eval_steps == 0 and not a.no_eval:
                self._in_loop_eval()
            if a.trainer == "regular" and not a.no_eval and (
                    (a.evaluation_strategy == "epoch" and step_in_epoch + 1 == spe) or
                    (a.evaluation_strategy == "steps" and a.eval_steps and self.state.global_step % a.eval_steps == 0)):
                self._in_loop_eval()
            if a.trainer == "regular" and a.save_strategy == "epoch" and step_in_epoch + 1 == spe \
                    and a.save_total_limit != 0:
                self._save_checkpoint()
            if a.save_strategy == "steps" and a.save_steps > 0 and self.state.global_step % a.save_steps == 0 \
                    and a.save_total_limit != 0:
                self._save_checkpoint()
            if self.control.should_save:
                self._save_checkpoint()
                self.control.should_save = False
            if self.control.should_training_stop:
                break
        if a.load_best_model_at_end and self.best_model_ckpt is not None:
            if self._world > 1:
                dist.barrier(self.dp_group)
            if self._sharded:
                for n, t in self.best_model_ckpt.items():
                    self.model.param(n).copy_(t)
            else:
                self.model.load_state_dict(self.best_model_ckpt)
        runtime = time.time() - t_start
        done = max(1, self.state.global_step - start_step)
        metrics = {"train_runtime": round(runtime, 4),
                   "train_samples_per_second": round(done * gb / max(runtime, 1e-9), 3),
                   "train_steps_per_second": round(done / max(runtime, 1e-9), 3),
                   "train_tokens_per_second": round(tokens * self._world / max(runtime, 1e-9), 1),
                   "train_loss": tr_loss / done, "epoch": self.state.epoch}
        logger.info(metrics)
        self.state.log_history.append(metrics)
        if self._metrics_f:
            self._metrics_f.close()
            self._metrics_f = None
        self._fire("on_train_end")
        return metrics


def _parse_range(spec: Optional[str]):
    if not spec:
        return None
    a, b = spec.split(":")
    return int(a), int(b)
