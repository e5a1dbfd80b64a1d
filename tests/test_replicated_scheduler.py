"""Two CPU ranks (gloo) serve the tiny TP=2 model in lock step: rank 0 takes the requests, both
ranks must admit, cancel and finish them in the same steps and agree on every token."""
import time

import torch

from slopllm_b200.config import GlmMoeDsaConfig, SamplingParams
from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
from slopllm_b200.models.weights import random_model
from slopllm_b200.parallel.dist import ParallelContext, init_from_env
from slopllm_b200.runtime.engine import Engine
from slopllm_b200.scheduler.replicated import ReplicaChannel, make_channel
from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler

from mp_util import run_ranks


def _serve(rank, world):
    ctx = init_from_env("gloo") if world > 1 else ParallelContext()
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0, tp_rank=ctx.rank, tp_world=ctx.world)
    eng = Engine(cfg, GlmMoeDsaModel(cfg, w, ctx), num_pages=32, max_batch=2, max_seq_len=512, cuda_graph=False)
    chan = make_channel(ctx, idle_wait_s=0.01) if world > 1 else ReplicaChannel(0, 1)
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=64, eos_token_ids=[], replica_channel=chan)
    finished = []
    sched.start()
    reqs = []
    if rank == 0:
        g = torch.Generator().manual_seed(1)
        for i in range(3):                       # 3 requests on 2 rows: the third waits for a free row
            prompt = torch.randint(0, cfg.vocab_size, (40 + 10 * i,), generator=g).tolist()
            r = GenerationRequest(id=f"r{i}", input_ids=prompt, max_tokens=6 if i != 1 else 200, sampling=SamplingParams(temperature=0.0),
                                  on_finish=lambda q: finished.append(q.id))
            reqs.append(r)
            sched.submit(r)
        time.sleep(0.3)
        reqs[1].cancel()                         # long request: cancelled while running
        t0 = time.time()
        while len(finished) < 3 and time.time() - t0 < 60:
            time.sleep(0.02)
        sched.stop()
        out = {r.id: (list(r.generated), r.finish_reason) for r in reqs}
    else:
        sched._thread.join(timeout=90)
        out = None
    # every rank saw the same requests retire in the same way
    return out, dict(sched.metrics.__dict__), eng.kv.free_pages


def test_two_ranks_stay_in_lock_step():
    res = run_ranks(_serve, 2)
    out0, m0, free0 = res[0]
    _, m1, free1 = res[1]
    assert out0["r0"][1] == "length" and len(out0["r0"][0]) == 6
    assert out0["r2"][1] == "length" and len(out0["r2"][0]) == 6
    assert out0["r1"][1] == "cancelled"
    assert m0["generation_tokens_total"] == m1["generation_tokens_total"] > 0
    assert m0["prompt_tokens_total"] == m1["prompt_tokens_total"]
    assert free0 == free1


def test_single_rank_channel_matches_plain_scheduler():
    out, _, _ = _serve(0, 1)
    assert out["r0"][1] == "length" and out["r1"][1] == "cancelled"


def _serve_stop_string(rank, world):
    """Rank 0's front end sees a stop string for a running request at the worst moment: after the step's events were
    collected for the broadcast, before the step runs."""
    ctx = init_from_env("gloo")
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0, tp_rank=ctx.rank, tp_world=ctx.world)
    eng = Engine(cfg, GlmMoeDsaModel(cfg, w, ctx), num_pages=32, max_batch=2, max_seq_len=512, cuda_graph=False)
    chan = make_channel(ctx, idle_wait_s=0.01)
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=64, eos_token_ids=[], replica_channel=chan)
    finished, reqs, fired = [], [], []
    if rank == 0:
        g = torch.Generator().manual_seed(2)
        for i in range(2):
            prompt = torch.randint(0, cfg.vocab_size, (40 + 10 * i,), generator=g).tolist()
            reqs.append(GenerationRequest(id=f"s{i}", input_ids=prompt, max_tokens=12 if i == 0 else 200,
                                          sampling=SamplingParams(temperature=0.0), on_finish=lambda q: finished.append(q.id)))
        collect = chan._collect

        def collect_then_stop(s):
            wire = collect(s)
            if not fired and len(reqs[1].generated) >= 3:
                fired.append(len(reqs[1].generated))
                reqs[1].cancel(reason="stop")            # what the HTTP handler does when the text hits a stop string
            return wire
        chan._collect = collect_then_stop
    sched.start()
    if rank == 0:
        for r in reqs:
            sched.submit(r)
        t0 = time.time()
        while len(finished) < 2 and time.time() - t0 < 60:
            time.sleep(0.02)
        sched.stop()
        out = {r.id: (len(r.generated), r.finish_reason, r.retired) for r in reqs}
    else:
        sched._thread.join(timeout=90)
        out = None
    return out, dict(sched.metrics.__dict__), eng.kv.free_pages, len(chan.live), fired


def test_stop_string_between_collect_and_step_keeps_ranks_in_lock_step():
    res = run_ranks(_serve_stop_string, 2)
    out0, m0, free0, live0, fired = res[0]
    _, m1, free1, live1, _ = res[1]
    assert fired, "the stop never fired"
    assert out0["s0"][1] == "length" and out0["s0"][0] == 12
    assert out0["s1"][1] == "stop" and out0["s1"][2]
    # both ranks decoded the stopped row for the same number of steps and released the same pages
    assert m0["generation_tokens_total"] == m1["generation_tokens_total"]
    assert m0["request_success_total"] == 2
    assert free0 == free1
    assert live0 == live1 == 0
