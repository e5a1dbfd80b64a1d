"""Data-parallel serving: replicas behind one front end, requests and tokens carried over store mailboxes.
Fake engines (no model, no GPU); the remote replica runs in a thread over a HashStore and in a second process over a
TCPStore."""
import threading
import time

import torch.distributed as dist
import torch.multiprocessing as mp

from mp_util import _free_port
from test_scheduler import FakeEngine

from slopllm_b200.config import SamplingParams
from slopllm_b200.scheduler.data_parallel import DataParallelRouter, Mailbox, ReplicaAgent, ReplicaProxy
from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler


def _req(i, prompt, n=4):
    got, done = [], threading.Event()
    r = GenerationRequest(id=str(i), input_ids=list(prompt), max_tokens=n, sampling=SamplingParams(temperature=0),
                          on_token=got.append, on_finish=lambda r: done.set())
    r.got, r.done = got, done
    return r


def test_mailbox_keeps_order_across_producers():
    store = dist.HashStore()
    a, b, rx = Mailbox(store, "q"), Mailbox(store, "q"), Mailbox(store, "q")
    a.put({"n": 1})
    b.put({"n": 2})
    a.put({"n": 3})
    assert [m["n"] for m in rx.drain()] == [1, 2, 3]
    assert rx.drain() == []
    b.put({"n": 4})
    assert [m["n"] for m in rx.drain()] == [4]


def test_router_places_by_load_and_prefix_affinity():
    class Stub:
        def __init__(self):
            self.got = []
            self.metrics = None
            self.engine = None

        def submit(self, r):
            self.got.append(r)
    reps = [Stub(), Stub(), Stub()]
    router = DataParallelRouter(reps, page_tokens=4)
    short = [_req(i, [1, 2]) for i in range(3)]
    for r in short:
        router.submit(r)
    assert [len(s.got) for s in reps] == [1, 1, 1] and router.load == [1, 1, 1]     # idlest first, ties by index
    a = _req(10, [9, 9, 9, 9, 5, 6])
    router.submit(a)                                                                # first sight of this first page
    home = next(i for i, s in enumerate(reps) if a in s.got)
    b = _req(11, [9, 9, 9, 9, 7, 8, 1])
    router.submit(b)
    assert b in reps[home].got                                                      # same first page: same replica
    for _ in range(DataParallelRouter.AFFINITY_SLACK + 1):                          # until that replica is clearly busier
        router.submit(_req(12, [9, 9, 9, 9, 0, 0]))
    assert max(router.load) - min(router.load) <= DataParallelRouter.AFFINITY_SLACK + 1
    a.on_finish(a)                                                                  # a finished request frees its slot
    assert router.load[home] == len(reps[home].got) - 1 and a.done.is_set()


def test_remote_replica_over_mailboxes_in_process():
    store = dist.HashStore()
    local = GenerationScheduler(FakeEngine(), max_batch=2, chunk_size=64, eos_token_ids=[])
    remote = GenerationScheduler(FakeEngine(), max_batch=2, chunk_size=64, eos_token_ids=[])
    local.start()
    remote.start()
    agent = ReplicaAgent(store, 1, remote, poll_s=0.002, metrics_every_s=0.05).start()
    proxy = ReplicaProxy(store, 1, poll_s=0.002).start()
    router = DataParallelRouter([local, proxy])
    try:
        reqs = [_req(i, range(10 * i, 10 * i + 5), 4) for i in range(6)]
        for r in reqs:
            router.submit(r)
        for r in reqs:
            assert r.done.wait(20), r.id
            first = (10 * int(r.id) + 5) % 1000
            assert r.generated == r.got == [first, first + 1, first + 2, first + 3] and r.finish_reason == "length"
            assert r.prompt_tokens == 5
        # placement follows the live load at submit time, so a request that has already finished frees its replica
        assert sum(router.routed) == 6 and min(router.routed) >= 1 and router.load == [0, 0]
        t0 = time.time()
        while router.metrics.request_success_total < 6 and time.time() - t0 < 10:   # the remote snapshot is periodic
            time.sleep(0.02)
        m = router.metrics
        assert m.request_success_total == 6 and m.generation_tokens_total == 24
        assert router.engine.kv.num_pages == 64 and router.engine.kv.tokens_per_page == 64
        ev = router.flush_gpu_cache()
        assert ev.done.wait(20)
        # a client that goes away: the proxy forwards the cancellation and the replica retires the row
        slow = _req(99, range(500, 505), 100000)
        proxy.submit(slow)
        t0 = time.time()
        while not slow.got and time.time() - t0 < 10:
            time.sleep(0.005)
        slow.cancel()
        assert slow.done.wait(20) and slow.finish_reason
    finally:
        proxy.stop()
        agent.stop()
        local.stop()
        remote.stop()


def _remote_process(port):
    import sys
    import os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_scheduler import FakeEngine as FE

    from slopllm_b200.utils.health import make_store
    store = make_store(1, 2, port=port)
    sched = GenerationScheduler(FE(), max_batch=2, chunk_size=64, eos_token_ids=[])
    sched.start()
    agent = ReplicaAgent(store, 1, sched, poll_s=0.002, metrics_every_s=0.05).start()
    agent._thread.join(timeout=60)            # ends when the front end sends "stop"
    sched.stop()


def test_remote_replica_in_another_process():
    from slopllm_b200.utils.health import make_store
    port = _free_port()
    store = make_store(0, 2, port=port)
    p = mp.get_context("spawn").Process(target=_remote_process, args=(port,))
    p.start()
    proxy = ReplicaProxy(store, 1, poll_s=0.002).start()
    try:
        reqs = [_req(i, range(100 + i, 110 + i), 3) for i in range(3)]
        for r in reqs:
            proxy.submit(r)
        for r in reqs:
            assert r.done.wait(60), r.id
            first = 110 + int(r.id)
            assert r.generated == [first, first + 1, first + 2]
    finally:
        proxy.stop()
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert p.exitcode == 0


def _dp_job(rank, world, store_port):
    """4 CPU ranks = 2 replicas x TP 2 of the tiny model: job rank 0 is the front end, rank 2 leads the second replica."""
    import torch

    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.parallel.dist import init_from_env
    from slopllm_b200.runtime.engine import Engine
    from slopllm_b200.scheduler.replicated import make_channel
    from slopllm_b200.utils.health import make_store
    ctx = init_from_env("gloo", dp=2)
    assert (ctx.world, ctx.dp_world, ctx.global_rank, ctx.global_world) == (2, 2, rank, 4)
    assert ctx.rank == rank % 2 and ctx.dp_rank == rank // 2 and ctx.peer(1) == 2 * ctx.dp_rank + 1
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0, tp_rank=ctx.rank, tp_world=ctx.world)
    eng = Engine(cfg, GlmMoeDsaModel(cfg, w, ctx), num_pages=32, max_batch=2, max_seq_len=512, cuda_graph=False)
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=64, eos_token_ids=[], replica_channel=make_channel(ctx, idle_wait_s=0.01))
    sched.start()
    if ctx.rank != 0:
        sched._thread.join(timeout=120)
        return None
    store = make_store(rank, world, port=store_port)
    if ctx.dp_rank != 0:
        agent = ReplicaAgent(store, ctx.dp_rank, sched, poll_s=0.002).start()
        agent._thread.join(timeout=120)
        sched.stop()
        return {"served": sched.metrics.request_success_total}
    proxy = ReplicaProxy(store, 1, poll_s=0.002).start()
    router = DataParallelRouter([sched, proxy])
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist()
    reqs = [_req(i, prompt, 5) for i in range(2)]            # the same prompt on both replicas: same weights, same tokens
    for r in reqs:
        router.submit(r)
    for r in reqs:
        assert r.done.wait(90), r.id
    proxy.stop()
    sched.stop()
    return {"routed": router.routed, "tokens": [r.generated for r in reqs], "local_served": sched.metrics.request_success_total}


def test_two_replicas_of_two_ranks_serve_one_front_end():
    from mp_util import run_ranks
    res = run_ranks(_dp_job, 4, _free_port(), timeout=240)
    front, leader1 = res[0], res[2]
    assert front["routed"] == [1, 1] and front["local_served"] == 1 and leader1["served"] == 1
    assert len(front["tokens"][0]) == 5 and front["tokens"][0] == front["tokens"][1]


def test_serve_cli_with_two_replicas_on_cpu():
    """`serve --dp 2` under torchrun on two CPU ranks: both replicas answer chat completions through the one front end,
    the metrics page adds the replicas up, and the rank-failure monitor runs alongside."""
    import json
    import subprocess
    import sys
    import urllib.request
    port, dp_port, health_port, master = _free_port(), _free_port(), _free_port(), _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(master), "-m", "slopllm_b200.cli.serve", "--random-init", "tiny", "--cpu", "--dp", "2",
           "--gpus", "0,1", "--batch-size", "2", "--chunk-size", "64", "--max-pages", "64", "--port", str(port),
           "--dp-port", str(dp_port), "--health-port", str(health_port)]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        up = False
        for _ in range(240):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    up = r.status == 200
                    break
            except Exception:  # noqa: BLE001
                assert proc.poll() is None, proc.stdout.read()
                time.sleep(0.5)
        assert up

        def chat(i, out):
            body = {"model": "tiny", "messages": [{"role": "user", "content": f"hello {i}"}], "max_tokens": 4, "temperature": 0}
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=120) as r:
                out[i] = json.loads(r.read())
        out = {}
        threads = [threading.Thread(target=chat, args=(i, out)) for i in range(4)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(150)
        assert len(out) == 4 and all(o["usage"]["completion_tokens"] == 4 for o in out.values())
        time.sleep(1.0)                                     # the remote replica's metric snapshot is periodic
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10) as r:
            metrics = r.read().decode()
        assert 'num_gpu_blocks="128"' in metrics            # 64 pages on each of the two replicas
        success = int(float([ln for ln in metrics.splitlines() if ln.startswith("vllm:request_success_total")][0].split()[1]))
        assert success >= 4
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
