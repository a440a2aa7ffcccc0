"""Failure detection and recovery, injected on the host only: a gloo rank that exits between steps, a rank that raises,
a truncated checkpoint, an incomplete backup, restart from the last complete backup."""
import multiprocessing as mp
import os
import time

import pytest
import torch

from mojodiffusion_b200.parallel.health import DictStore, ElasticRunner, Heartbeat, RankFailure, StepGuard
from mojodiffusion_b200.training import loop
from mojodiffusion_b200.utils.parity import GATE_DEFAULT, ParityHarness, compare, nondegenerate_fill


def test_parity_harness():
    a = nondegenerate_fill((64, 32), 1)
    assert a.std() > 0.3 and not torch.equal(a[0], a[1])
    h = ParityHarness()
    r = h.check("same", a, a.clone())
    assert r.cos == pytest.approx(1.0) and r.max_abs == 0 and r.ok(0.99999999)
    h.check("bf16", a.bfloat16(), a, cos_min=0.9999)
    h.assert_all()
    h.check("bad", -a, a)
    assert h.bit_equal("bits", a, a + 0) == 0
    with pytest.raises(AssertionError) as e:
        h.assert_all()
    assert "bad" in str(e.value) and "cos=-1.0" in str(e.value)
    assert not compare("nan", torch.tensor([float("nan")]), torch.tensor([1.0])).ok(GATE_DEFAULT)
    assert compare("zeros", torch.zeros(3), torch.zeros(3)).cos == 1.0
    with pytest.raises(ValueError):
        compare("shape", torch.zeros(3), torch.zeros(4))


def test_heartbeat_and_step_guard_in_process():
    store, now = DictStore(), [0.0]
    hb0 = Heartbeat(store, 0, 2, timeout_s=5.0, clock=lambda: now[0])
    hb1 = Heartbeat(store, 1, 2, timeout_s=5.0, clock=lambda: now[0])
    hb0.beat(0), hb1.beat(0)
    assert hb0.stale_ranks() == []
    now[0] = 4.0
    hb1.beat(1)
    assert hb0.stale_ranks() == []
    now[0] = 8.0
    assert hb0.stale_ranks() == []                  # 4 s since the value last changed: still inside the limit
    now[0] = 12.0                                   # rank 1 went silent after step 1
    assert hb0.stale_ranks() == [1]
    with pytest.raises(RankFailure):
        hb0.require_all()
    g0, g1 = StepGuard(store, 0, 2), StepGuard(store, 1, 2)
    assert g0.run(0, lambda: 7) == 7
    with pytest.raises(ZeroDivisionError):
        g1.run(1, lambda: 1 / 0)
    with pytest.raises(RankFailure) as e:            # rank 0 learns of it before launching step 1
        g0.run(1, lambda: 7)
    assert e.value.ranks == [1] and "ZeroDivisionError" in e.value.reason

    def bad_status():
        raise RuntimeError("device status: TIMEOUT at 41")
    with pytest.raises(RuntimeError):
        g0.run(2, lambda: 1, bad_status)
    assert store.check([g0.failed_flag(2)])


def _rank_main(rank, world, port, die_at, q):
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, timeout_s=1.0)
    guard = StepGuard(store, rank, world, hb)
    x = torch.ones(4) * (rank + 1)
    done = 0
    try:
        for step in range(6):
            if rank == 1 and step == die_at:
                os._exit(3)                              # leaves between steps, nothing in flight
            def one():
                t = x.clone()
                dist.all_reduce(t)
                return t
            guard.run(step, one)
            done += 1
            time.sleep(0.3)
            if rank == 0 and step >= die_at - 1:
                deadline = time.time() + 6
                while time.time() < deadline:            # wait on the host until the silence is noticed
                    hb.require_all()
                    time.sleep(0.2)
    except RankFailure as e:
        q.put(("rank_failure", rank, done, e.ranks))
        q.close()
        q.join_thread()                                  # flush the message before leaving without teardown
        os._exit(0)                                      # no collective was enqueued for the failed step
    q.put(("finished", rank, done, []))


def test_gloo_rank_exit_is_detected_before_the_next_collective():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    ps = [ctx.Process(target=_rank_main, args=(r, 2, port, 2, q)) for r in range(2)]
    [p.start() for p in ps]
    msg = q.get(timeout=60)
    [p.join(timeout=30) for p in ps]
    assert msg[0] == "rank_failure" and msg[1] == 0 and msg[3] == [1]
    assert msg[2] == 2                                   # two good steps, the third never launched
    assert ps[1].exitcode == 3 and ps[0].exitcode == 0


def test_truncated_checkpoint_and_incomplete_backup(tmp_path):
    from mojodiffusion_b200.io.safetensors_io import load_safetensors, save_safetensors
    p = str(tmp_path / "w.safetensors")
    save_safetensors(p, {"a": torch.randn(64, 64)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(Exception):
        load_safetensors(p)
    ws = str(tmp_path / "ws")
    good = loop.backup_path(ws, "T", loop.TrainProgress(4, 1, 1, 2))
    loop.write_backup(good, loop.TrainProgress(4, 1, 1, 2), {"w": torch.ones(2)}, {"m": torch.zeros(2)}, "flux")
    # a later backup whose writer died before meta.json: it must be ignored
    half = loop.backup_path(ws, "T", loop.TrainProgress(8, 2, 2, 4))
    os.makedirs(os.path.join(half, "lora"))
    save_safetensors(os.path.join(half, "lora", "lora.safetensors"), {"w": torch.ones(2)})
    assert loop.find_last_backup(ws) == good
    with pytest.raises(FileNotFoundError):
        loop.read_backup(half)


def test_elastic_runner_restarts_from_last_backup(tmp_path):
    ws = str(tmp_path)
    calls = []

    def launch(resume):
        calls.append(resume)
        if len(calls) == 1:
            p = loop.TrainProgress(2, 0, 2, 4)
            loop.write_backup(loop.backup_path(ws, "T", p), p, {"w": torch.ones(1)}, {"m": torch.ones(1)}, "flux")
            raise RankFailure([1], "no heartbeat")
        if len(calls) == 2:
            raise RuntimeError("worker exited with code 1")

    r = ElasticRunner(ws, max_restarts=3)
    assert r.run(launch) == 2
    assert calls[0] is None and calls[1].endswith("T-backup-2-0-2") and calls[2] == calls[1]
    r2 = ElasticRunner(ws, max_restarts=1)
    with pytest.raises(ValueError):
        r2.run(lambda resume: (_ for _ in ()).throw(ValueError("always")))
    assert [d.restart for d in r2.history] == [True, False]
