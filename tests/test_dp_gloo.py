"""Data parallelism on CPU ranks (gloo): shared-seed z, per-rank batch shards, ONE scalar
all-reduce per step; equivalence with a single process on the concatenated batch; a rank that
never joins is detected by the process-group timeout instead of hanging the others."""
import os
import socket
import subprocess
import sys
import textwrap


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_ranks(script: str, world: int, timeout: int = 240, extra_env=None, ranks=None):
    port = _free_port()
    procs = []
    for r in (ranks if ranks is not None else range(world)):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), PYTHONPATH=ROOT,
                   CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<<killed by the test timeout>>"
        outs.append((p.returncode, out))
    return outs


DP_SCRIPT = textwrap.dedent('''
    import os, torch, torch.distributed as dist
    from dizo_b200.data.synthetic import synthetic_batch
    from dizo_b200.engine import ZOEngine, DiZOProjector
    from dizo_b200.models.opt import OPTModel, Batch, preset
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = preset("opt-tiny")
    model = OPTModel(cfg, "cpu", torch.float32).init_random(0)
    eng = ZOEngine(model, eps=1e-3)
    proj = DiZOProjector(model, max_iters=2)
    def shard(step, r): return synthetic_batch(step, 4, 16, cfg.vocab_size, rank=r, cand_ids=(10, 20))
    for step in range(6):
        eng.step(shard(step, rank), 1e-3, seed=100 + step)
    it = iter(range(100))
    proj.search_zo(lambda: shard(50 + next(it), rank), seed=9)
    # replicas stay bit-identical without ever exchanging parameters
    mine = model.arena.data.clone()
    ref = mine.clone(); dist.broadcast(ref, 0)
    assert torch.equal(mine, ref), "replicas diverged"
    if rank == 0:
        # single process on the concatenated batch gives the same trajectory
        solo = OPTModel(cfg, "cpu", torch.float32).init_random(0)
        e2 = ZOEngine(solo, eps=1e-3); e2.dp_group = None
        import dizo_b200.engine as E
        E._dist_on = lambda g=None: False
        def cat(step):
            bs = [shard(step, r) for r in range(world)]
            n, L = bs[0].input_ids.shape
            return Batch(input_ids=torch.cat([b.input_ids for b in bs]), pad_left=torch.cat([b.pad_left for b in bs]),
                         positions=torch.cat([b.positions for b in bs]),
                         rows=torch.cat([b.rows + i * n * L for i, b in enumerate(bs)]),
                         labels=torch.cat([b.labels for b in bs]), cand_ids=bs[0].cand_ids)
        for step in range(6):
            e2.step(cat(step), 1e-3, seed=100 + step)
        p2 = DiZOProjector(solo, max_iters=2)
        p2.gs.gamma.zero_()
        it2 = iter(range(100))
        # anchors: same init, so take them from the DP model's arena
        solo.arena.anchor.copy_(model.arena.anchor)
        p2.search_zo(lambda: cat(50 + next(it2)), seed=9)
        err = (solo.arena.data - mine).abs().max().item()
        assert err < 5e-6, err
        print("DP_OK", err)
    dist.destroy_process_group()
''')


def test_dp_equals_single_process_on_concatenated_batch():
    outs = _run_ranks(DP_SCRIPT, 2)
    for rc, out in outs:
        assert rc == 0, out[-3000:]
    assert "DP_OK" in outs[0][1]


MISSING_RANK_SCRIPT = textwrap.dedent('''
    import datetime, torch, torch.distributed as dist, sys, time
    try:
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
        t = torch.ones(1)
        dist.all_reduce(t)
        print("UNEXPECTED_OK")
    except Exception as e:
        print("DETECTED", type(e).__name__)
        sys.exit(7)
''')


def test_rank_that_never_joins_is_detected_not_hung():
    # world size 2, only rank 0 is started: rendezvous must give up within its timeout
    outs = _run_ranks(MISSING_RANK_SCRIPT, 2, timeout=120, ranks=[0])
    rc, out = outs[0]
    assert rc == 7 and "DETECTED" in out, out[-2000:]


DEAD_PEER_SCRIPT = textwrap.dedent('''
    import datetime, os, sys, torch, torch.distributed as dist
    from dizo_b200.parallel.health import Heartbeat, PeerLost
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=10))
    rank = dist.get_rank()
    hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, dist.get_world_size(), stale_after=3.0)
    hb.beat(0)
    dist.barrier()
    if rank == 1:
        os._exit(0)                       # leaves between steps, nothing in flight
    try:
        import time
        for step in range(1, 40):
            hb.beat(step)
            hb.check(step)                # host-side check before the next launch
            time.sleep(0.25)
        print("NOT_DETECTED")
    except PeerLost as e:
        print("PEER_LOST", e)
        sys.exit(9)
''')


def test_dead_peer_is_reported_by_heartbeat():
    outs = _run_ranks(DEAD_PEER_SCRIPT, 2, timeout=120)
    rc0, out0 = outs[0]
    assert rc0 == 9 and "PEER_LOST" in out0, out0[-2000:]


SILENT_PEER_SCRIPT = textwrap.dedent('''
    import datetime, os, sys, time, torch, torch.distributed as dist
    from dizo_b200.parallel.health import Heartbeat, PeerLost
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    rank = dist.get_rank()
    hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, dist.get_world_size(), stale_after=2.0)
    dist.barrier()
    if rank == 1:
        time.sleep(8)                     # alive but never reports a heartbeat
        os._exit(0)
    t0 = time.time()
    try:
        hb.sync(1)                        # must not block on the missing key until the store times out
        print("NOT_DETECTED")
    except PeerLost as e:
        print("PEER_LOST after %.1f s" % (time.time() - t0), e)
        os._exit(9 if time.time() - t0 < 6.0 else 10)
''')


def test_peer_that_never_reports_is_lost_within_the_stale_limit():
    outs = _run_ranks(SILENT_PEER_SCRIPT, 2, timeout=120)
    rc0, out0 = outs[0]
    assert rc0 == 9 and "PEER_LOST" in out0, out0[-2000:]


TRAINER_PEER_SCRIPT = textwrap.dedent('''
    import datetime, os, sys, time, torch, torch.distributed as dist
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    from dizo_b200.args import OurArguments
    from dizo_b200.models.opt import OPTModel, preset
    from dizo_b200.parallel.health import PeerLost
    from dizo_b200.tasks import SyntheticDataset
    from dizo_b200.trainer import OurTrainer
    from dizo_b200.utils import (DataCollatorWithPaddingAndNesting, StubTokenizer, TrainerCallback,
                                 encode_prompt)
    rank = dist.get_rank()
    tmp = os.environ["HB_TMP"]
    a = OurArguments(trainer="zo", learning_rate=1e-3, max_steps=200, per_device_train_batch_size=2,
                     train_as_classification=True, zo_eval_steps=100000, output_dir=os.path.join(tmp, f"o{rank}"),
                     save_steps=0, task_name="Synthetic", model_name="opt-tiny", max_length=64,
                     heartbeat_timeout=2.0)
    task = SyntheticDataset(n_train=64, n_valid=8)
    tok = StubTokenizer(["terrible", "great", "It", "was", "fine", "dull", "film"])
    model = OPTModel(preset("opt-tiny"), "cpu", torch.float32).init_random(0)
    feats = []
    for smp in task.samples["train"]:
        enc, ol = encode_prompt(task, task.get_template(), [], smp, tok, max_length=64)
        gold = smp.candidates.index(smp.correct_candidate)
        feats.append([{"input_ids": enc[i], "labels": gold, "option_len": ol[i], "num_options": 2} for i in range(2)])

    class Leave(TrainerCallback):
        def on_step_end(self, args, state, control, **kw):
            if rank == 1 and state.global_step == 3:
                os._exit(0)                 # between steps, nothing in flight
            time.sleep(0.05)
    tr = OurTrainer(model, a, train_dataset=feats, processing_class=tok,
                    data_collator=DataCollatorWithPaddingAndNesting(tok, pad_to_multiple_of=8), task=task,
                    callbacks=[Leave()])
    try:
        tr.train()
        print("NOT_DETECTED")
    except PeerLost as e:
        print("PEER_LOST at step", tr.state.global_step, e)
        os._exit(9)
''')


def test_trainer_stops_on_the_host_when_a_peer_leaves(tmp_path):
    outs = _run_ranks(TRAINER_PEER_SCRIPT, 2, timeout=200, extra_env={"HB_TMP": str(tmp_path)})
    rc0, out0 = outs[0]
    assert "PEER_LOST" in out0 and rc0 == 9, out0[-3000:]
