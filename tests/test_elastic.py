"""Process-group generations: a rank leaves between steps, the survivor notices it through the heartbeat store,
opens the next generation, and a replacement process joins it.  CPU ranks on gloo; no GPU is involved."""
import time

import torch
import torch.multiprocessing as mp

from mp_util import _free_port


def _member(rank, world, port, role, q):
    import traceback
    try:
        import torch.distributed as dist

        from slopllm_b200.parallel.dist import Comm
        from slopllm_b200.parallel.elastic import ElasticGroup
        from slopllm_b200.utils.health import HealthMonitor, make_store
        torch.set_num_threads(1)
        store = make_store(rank, world, port=port) if role != "replacement" else make_store(1, world, port=port)
        eg = ElasticGroup(store, rank, world, timeout_s=30.0)
        out = {"role": role}
        if role == "replacement":
            ctx = eg.join()
            out["generation"] = eg.generation
        else:
            ctx = eg.start()
            mon = HealthMonitor(store, rank, world, interval_s=0.05, timeout_s=1.0).start()
            x = torch.full((4,), float(rank + 1))
            out["first"] = Comm(ctx).all_reduce(x).tolist()
            if role == "leaver":
                mon.stop()                                  # leaves between steps: nothing in flight
                eg.shutdown()
                q.put((rank, out, None))
                return
            t0 = time.time()
            while mon.is_healthy() and time.time() - t0 < 20.0:
                time.sleep(0.05)
            out["detected"] = list(mon.state.failed_ranks)
            rebuilt = []
            ctx = eg.recover(on_new_context=lambda c: rebuilt.append(c.world))
            mon.reset()
            out["rebuilt"] = rebuilt
            out["generation"] = eg.generation
        y = torch.full((4,), float(10 * (rank + 1)))
        out["second"] = Comm(ctx).all_reduce(y).tolist()
        dist.barrier()
        eg.shutdown()
        q.put((rank, out, None))
    except Exception:  # noqa: BLE001
        q.put((rank, None, traceback.format_exc()))


def test_survivor_and_replacement_form_the_next_generation():
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = _free_port()
    p0 = mpc.Process(target=_member, args=(0, 2, port, "survivor", q))
    p1 = mpc.Process(target=_member, args=(1, 2, port, "leaver", q))
    p0.start()
    p1.start()
    procs = [p0, p1]
    try:
        rank, left, err = q.get(timeout=60)
        assert err is None, err
        assert rank == 1 and left["first"] == [3.0] * 4
        p1.join(timeout=20)
        p2 = mpc.Process(target=_member, args=(1, 2, port, "replacement", q))
        p2.start()
        procs.append(p2)
        res = {}
        for _ in range(2):
            rank, out, err = q.get(timeout=90)
            assert err is None, err
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    assert res[0]["role"] == "survivor" and res[0]["detected"] == [1] and res[0]["rebuilt"] == [2]
    assert res[0]["generation"] == 1 and res[1]["generation"] == 1
    assert res[0]["second"] == [30.0] * 4 and res[1]["second"] == [30.0] * 4


def test_recovery_times_out_when_nobody_joins():
    """A lone survivor whose peer is never replaced gets a RecoveryTimeout instead of waiting for ever."""
    import pytest

    from slopllm_b200.parallel.elastic import ElasticGroup, RecoveryTimeout
    from slopllm_b200.utils.health import make_store
    store = make_store(0, 1, port=_free_port())
    eg = ElasticGroup(store, 0, 2, timeout_s=1.0)
    eg.generation = 0                      # as if generation 0 had been running
    t0 = time.time()
    with pytest.raises(RecoveryTimeout):
        eg.recover()
    assert time.time() - t0 < 30.0
    assert eg.current_generation() == 1    # the generation was opened; it just never assembled


def test_reattach_swaps_communicator_and_drops_graphs():
    from types import SimpleNamespace

    from slopllm_b200.parallel.dist import Comm, ParallelContext
    from slopllm_b200.parallel.elastic import reattach
    from slopllm_b200.runtime.graphs import CaptureManager, GraphEntry
    old = ParallelContext()
    model = SimpleNamespace(ctx=old, comm=Comm(old), cfg=None, ops=SimpleNamespace(ctx=old))
    graphs = CaptureManager(enabled=False)
    graphs.entries[("decode", 1)] = GraphEntry(calls=3)
    engine = SimpleNamespace(model=model, graphs=graphs)
    new = ParallelContext()
    old_comm = model.comm
    reattach(engine, new)
    assert model.ctx is new and model.ops.ctx is new and model.comm is not old_comm and model.comm.ctx is new
    assert not graphs.entries


def _retry_member(rank, world, port, role, q):
    """Survivor: the first recovery finds nobody (short timeout), the second one meets the replacement."""
    import traceback
    try:
        import torch.distributed as dist

        from slopllm_b200.parallel.dist import Comm
        from slopllm_b200.parallel.elastic import ElasticGroup, RecoveryTimeout
        from slopllm_b200.utils.health import make_store
        torch.set_num_threads(1)
        out = {"role": role}
        if role == "survivor":
            store = make_store(0, world, port=port)
            eg = ElasticGroup(store, 0, world, timeout_s=2.0)
            eg.generation = eg._tried = 0                  # generation 0 was running; rank 1 is gone
            try:
                eg.recover()
                out["first_attempt"] = "assembled"
            except RecoveryTimeout:
                out["first_attempt"] = "timeout"
            out["after_timeout"] = eg.current_generation()
            store.set("retry/go", "1")                     # now the replacement may come
            eg.timeout_s = 30.0
            ctx = eg.recover()
        else:
            store = make_store(1, world, port=port)
            store.wait(["retry/go"])
            eg = ElasticGroup(store, 1, world, timeout_s=30.0)
            store.set("elastic/member/0/1", "1")           # this rank number lived in generation 0
            ctx = eg.join()
        out["generation"] = eg.generation
        out["sum"] = Comm(ctx).all_reduce(torch.full((2,), float(rank + 1))).tolist()
        dist.barrier()
        eg.shutdown()
        q.put((rank, out, None))
    except Exception:  # noqa: BLE001
        q.put((rank, None, traceback.format_exc()))


def test_second_recovery_uses_a_fresh_generation_after_a_timeout():
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = _free_port()
    procs = [mpc.Process(target=_retry_member, args=(0, 2, port, "survivor", q)),
             mpc.Process(target=_retry_member, args=(1, 2, port, "replacement", q))]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            rank, out, err = q.get(timeout=120)
            assert err is None, err
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    assert res[0]["first_attempt"] == "timeout" and res[0]["after_timeout"] == 1
    # generation 1 was spent by the failed attempt: both meet in generation 2
    assert res[0]["generation"] == 2 and res[1]["generation"] == 2
    assert res[0]["sum"] == [3.0, 3.0] and res[1]["sum"] == [3.0, 3.0]
