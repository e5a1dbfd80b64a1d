"""Failure detection without touching a GPU: heartbeats over a TCP store between CPU processes, a rank
that leaves between steps, a rank that stops beating, and host-side fault injection in the scheduler
and the page allocator."""
import time

import pytest

from slopllm_b200.utils.health import FaultInjector, HealthMonitor, HealthState, RankFailure, make_store
from slopllm_b200.utils.tracing import PhaseTimers, nvtx_range

from mp_util import _free_port, run_ranks


class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode()

    def get(self, k):
        return self.d[k]


def test_monitor_detects_stale_peer_with_fake_clock():
    store, now = DictStore(), [100.0]
    events = []
    a = HealthMonitor(store, 0, 2, timeout_s=2.0, on_failure=events.append, clock=lambda: now[0])
    b = HealthMonitor(store, 1, 2, timeout_s=2.0, clock=lambda: now[0])
    a.beat(); b.beat()
    assert a.check_peers().healthy
    now[0] += 1.5
    b.beat()
    assert a.check_peers().healthy
    b.pause()                                    # injected fault: rank 1 stops beating
    now[0] += 2.5
    b.beat()
    st = a.check_peers()
    assert not st.healthy and st.failed_ranks == [1] and len(events) == 1
    with pytest.raises(RankFailure):
        a.raise_if_unhealthy()
    a.reset()
    assert a.is_healthy()


def _rank(rank, world, port):
    store = make_store(rank, world, port=port)
    # the ranks start their monitors together: a process that is still importing must not look like a dead peer
    store.set(f"ready/{rank}", "1")
    store.wait([f"ready/{r}" for r in range(world)])
    mon = HealthMonitor(store, rank, world, interval_s=0.05, timeout_s=1.5).start()
    steps = 0
    t0 = time.time()
    while time.time() - t0 < 12.0:
        if rank == 2 and steps == 5:
            mon.stop()                           # rank 2 leaves between steps (no work in flight)
            return {"left_after": steps}
        if not mon.is_healthy():
            mon.stop()
            return {"detected": mon.state.failed_ranks, "steps": steps, "seconds": time.time() - t0}
        steps += 1
        time.sleep(0.05)
    mon.stop()
    return {"detected": [], "steps": steps}


def test_ranks_notice_a_peer_that_left():
    res = run_ranks(_rank, 3, _free_port(), timeout=60)
    assert res[2] == {"left_after": 5}
    for r in (0, 1):
        assert res[r]["detected"] == [2] and res[r]["seconds"] < 10.0


def test_fault_injector_counts_down():
    fi = FaultInjector()
    fi.arm("page_alloc", after=2)
    assert [fi.hit("page_alloc") for _ in range(4)] == [False, False, True, False]
    fi.arm("send")
    with pytest.raises(ConnectionError):
        fi.maybe_raise("send", ConnectionError("dropped"))
    assert fi.fired == ["page_alloc", "send"]


def test_scheduler_fails_requests_fast_when_unhealthy():
    """An engine whose step raises RankFailure: the scheduler ends every admitted request with an error and
    stays usable (per-batch rollback, `src/generation-scheduler.ts:669-689`)."""
    import torch
    from slopllm_b200.config import GlmMoeDsaConfig, SamplingParams
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.runtime.engine import Engine
    from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler
    cfg = GlmMoeDsaConfig.tiny()
    eng = Engine(cfg, GlmMoeDsaModel(cfg, random_model(cfg, 0)), num_pages=16, max_batch=2, max_seq_len=256, cuda_graph=False)
    fi = FaultInjector()
    real = eng.decode_step

    def decode_step(*a, **k):
        fi.maybe_raise("peer_lost", RankFailure("no heartbeat from rank(s) [1]"))
        return real(*a, **k)

    eng.decode_step = decode_step
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=64)
    fi.arm("peer_lost", after=1)
    done = []
    req = GenerationRequest(id="a", input_ids=list(range(3, 30)), max_tokens=8, sampling=SamplingParams(temperature=0.0),
                            on_finish=done.append)
    sched.submit(req)
    for _ in range(20):
        sched.step()
        if done:
            break
    assert done and req.error and "heartbeat" in req.error and req.finish_reason == "error"
    ok = GenerationRequest(id="b", input_ids=list(range(3, 20)), max_tokens=3, sampling=SamplingParams(temperature=0.0),
                           on_finish=done.append)
    sched.submit(ok)
    for _ in range(20):
        sched.step()
        if len(done) == 2:
            break
    assert ok.finish_reason == "length" and len(ok.generated) == 3
    assert torch.is_tensor(torch.zeros(1))


def test_phase_timers_and_nvtx_noop():
    t = PhaseTimers()
    with t.phase("decode", 4):
        with nvtx_range("layer0"):
            pass
    t.record("decode", 4, 0.5)
    text = t.prometheus()
    assert 'phase="decode",batch_size="4"' in text and "phase_seconds_count" in text and t.count[("decode", 4)] == 2


def test_scheduler_thread_refuses_to_step_while_a_peer_is_lost():
    """With a monitor attached, the scheduler loop launches nothing while the monitor reports a lost rank: running and
    queued requests end with an error at once, pending cache flushes are answered, and service resumes after reset()."""
    import threading
    from slopllm_b200.config import SamplingParams
    from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler
    from test_scheduler import FakeEngine

    class Mon:
        def __init__(self):
            self.ok = True
            self.state = HealthState(False, [1], "no heartbeat from rank(s) [1]")

        def is_healthy(self):
            return self.ok

    mon, eng = Mon(), FakeEngine()
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=64, health=mon)
    sched.start()
    try:
        def req(i, n):
            done = threading.Event()
            r = GenerationRequest(id=str(i), input_ids=list(range(5, 15)), max_tokens=n, sampling=SamplingParams(temperature=0.0),
                                  on_finish=lambda r: done.set())
            r.done = done
            return r
        a = req(0, 3)
        sched.submit(a)
        assert a.done.wait(10) and a.finish_reason == "length"
        mon.ok = False
        time.sleep(0.1)
        steps_before = len(eng.decode_batches)
        b = req(1, 3)
        sched.submit(b)
        flush = sched.flush_gpu_cache()
        assert b.done.wait(10) and b.finish_reason == "error" and "heartbeat" in b.error
        assert flush.done.wait(10)
        assert len(eng.decode_batches) == steps_before and sched.metrics.rank_failures_total == 1
        mon.ok = True
        c = req(2, 3)
        sched.submit(c)
        assert c.done.wait(10) and c.finish_reason == "length"
    finally:
        sched.stop()


def test_nvtx_ranges_cover_engine_steps_and_layers(monkeypatch):
    """With the switch on, prefill / decode steps, every layer and its attention / MLP halves run inside named ranges."""
    from contextlib import contextmanager

    import torch
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.runtime.engine import Engine
    from slopllm_b200.utils import tracing
    seen, depth = [], [0]

    @contextmanager
    def record(name):
        seen.append((depth[0], name))
        depth[0] += 1
        try:
            yield
        finally:
            depth[0] -= 1
    cfg = GlmMoeDsaConfig.tiny()
    eng = Engine(cfg, GlmMoeDsaModel(cfg, random_model(cfg, 0)), num_pages=8, max_batch=1, max_seq_len=256, cuda_graph=False)
    s = eng.kv.new_sequence()
    prompt = list(range(3, 40))
    last, _ = eng.prefill([s], [prompt], chunk_size=64)
    assert not seen                                              # off by default: nothing is recorded
    monkeypatch.setattr(tracing, "NVTX", True)
    monkeypatch.setattr(tracing, "nvtx_range", record)
    eng.decode_step([s], last)
    names = [n for _, n in seen]
    assert names[0] == "decode_step" and seen[0][0] == 0
    for i in range(cfg.num_hidden_layers):
        at = names.index(f"layer{i}")
        assert names[at + 1] == "attention" and "mlp" in names[at + 1:at + 4] and seen[at + 1][0] == seen[at][0] + 1
    assert torch.is_tensor(torch.zeros(1))


def test_health_endpoint_reports_the_lost_ranks():
    import asyncio
    import json
    from slopllm_b200.config import EngineConfig
    from slopllm_b200.scheduler.scheduler import GenerationScheduler
    from slopllm_b200.server.openai import OpenAIServer
    from slopllm_b200.server.tokenizer import ByteTokenizer
    from test_scheduler import FakeEngine

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self[k]
    now = [100.0]
    store = Store()
    mon = HealthMonitor(store, 0, 2, timeout_s=2.0, clock=lambda: now[0])
    store.set("hb/1", repr(100.0))
    sched = GenerationScheduler(FakeEngine(), max_batch=1, chunk_size=64, health=mon)

    async def run():
        srv = OpenAIServer(sched, ByteTokenizer(), EngineConfig(host="127.0.0.1", port=0), healthy=mon.is_healthy)
        await srv.start()

        async def get():
            r, w = await asyncio.open_connection("127.0.0.1", srv.port)
            w.write(b"GET /health HTTP/1.1\r\nHost: x\r\n\r\n")
            await w.drain()
            raw = await r.read()
            w.close()
            head, _, payload = raw.partition(b"\r\n\r\n")
            return int(head.split()[1]), json.loads(payload)
        mon.check_peers()
        assert await get() == (200, {"status": "ok"})
        now[0] = 110.0                                   # rank 1 has been silent for 10 s
        mon.check_peers()
        st, body = await get()
        assert st == 503 and body["status"] == "unhealthy" and body["failed_ranks"] == [1] and "heartbeat" in body["reason"]
        await srv.close()
    asyncio.run(run())
